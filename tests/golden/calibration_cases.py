"""Models, batches and settings shared by the calibration fixture generator and its test."""
import torch

MODELS = ["mlp", "convnet"]
KINDS = [
    ("Max", {}),
    ("CacheQuantile", dict(quantile=0.99, max_samples=100000)),
    ("MovingQuantile", dict(quantile=0.99)),
    ("MovingQuantile", dict(quantile=1.0)),
    ("MovingStd", dict(std_alpha=2.5)),
]


def make_rpu_config(cls):
    rpu = cls()
    rpu.mapping.max_input_size = 16
    rpu.forward.inp_res = -1
    rpu.forward.out_noise = 0.03          # calibration must run without it
    rpu.pre_post.input_range.enable = False
    return rpu


def build_model(name):
    torch.manual_seed(7)
    if name == "mlp":
        return torch.nn.Sequential(torch.nn.Linear(40, 24), torch.nn.ReLU(), torch.nn.Linear(24, 10))
    return torch.nn.Sequential(torch.nn.Conv2d(3, 4, 3, padding=1), torch.nn.ReLU(), torch.nn.Flatten(),
                               torch.nn.Linear(4 * 6 * 6, 5))


def make_batches(name):
    gen = torch.Generator().manual_seed(11)
    shape = (12, 40) if name == "mlp" else (4, 3, 6, 6)
    batches = [torch.randn(*shape, generator=gen) * (1.0 + 0.5 * i) for i in range(3)]
    if name == "mlp":
        batches[1][3] = 0.0               # an all-zero row is ignored by the statistics
    return batches
