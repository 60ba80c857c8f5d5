"""Helpers shared by the test modules."""
import os
from types import SimpleNamespace

import torch

import analog_oracle as O
import cases as C
from aihwkit_lightning_b200.simulator import configs as product_cfg

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")

NS = SimpleNamespace(
    TorchInferenceRPUConfig=product_cfg.TorchInferenceRPUConfig,
    WeightNoiseInjectionType=product_cfg.WeightNoiseInjectionType,
    WeightQuantizationType=product_cfg.WeightQuantizationType,
    WeightClipType=product_cfg.WeightClipType,
)


def load_golden(name):
    return torch.load(os.path.join(GOLDEN, name + ".pt"), weights_only=False)


def rel_fro(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    denom = b.norm().item()
    return (a - b).norm().item() / (denom if denom > 0 else 1.0)


def frac_equal(a, b):
    return (a.cpu() == b.cpu()).float().mean().item()


def run_product_layer(case, data, device="cuda", engine="auto", capture=None):
    """Build the product's AnalogLinear for ``case``, replay the case's noise, run its steps
    and one backward.  Returns (layer, x, out)."""
    from aihwkit_lightning_b200.nn import AnalogLinear
    from aihwkit_lightning_b200.nn import functional as F

    rpu = C.build_rpu_config(NS, case)
    layer = AnalogLinear(data["k"], data["n"], bias=case["bias"], rpu_config=rpu)
    layer = layer.to(device=device, dtype=data["dtype"])
    layer.set_weights_and_biases(data["w"].to(device), None if data["b"] is None else data["b"].to(device))
    layer.train(case["training"])
    if layer.learnable_weight_clip is not None:
        layer.learnable_weight_clip.data.mul_(case["lwc_scale"])
    for step in range(case["steps"]):
        x = data["xs"][step].to(device).clone().requires_grad_(True)
        layer.zero_grad()
        with F.operator_settings(w_noise=data["w_noise"][step], out_noise=data["out_noise"][step],
                                 engine=engine, capture=capture):
            out = layer(x)
    out.backward(data["g"].to(device))
    torch.cuda.synchronize()
    return layer, x, out


def oracle_run(case, data, x=None, w=None, b=None, g=None, w_noise=None, out_noise=None, training=None):
    """Oracle forward+backward for one step on CPU with the given (or the case's) tensors."""
    rpu = C.build_rpu_config(NS, case)
    x = data["xs"][-1] if x is None else x
    w = data["w"] if w is None else w
    b = data["b"] if b is None else b
    g = data["g"] if g is None else g
    training = case["training"] if training is None else training
    in_sizes = O.split_sizes(x.shape[-1], case["max_input_size"])
    static = case["ir_enable"] and not case["ir_dynamic"]
    ir = idx = x_min = x_max = None
    if static:
        ir = torch.full((len(in_sizes),), case["ir_init_value"], dtype=x.dtype)
        idx = torch.zeros(len(in_sizes), dtype=x.dtype)
        x_min = torch.zeros(len(in_sizes), dtype=x.dtype) - 1e-5
        x_max = torch.zeros(len(in_sizes), dtype=x.dtype) + 1e-5
    lwc = None
    if case["clip_type"] == "LearnablePerChannel":
        lwc = O.sliced_abs_max(in_sizes, w) * case["lwc_scale"]
    rec = O.forward(x, w, b, ir, idx, x_min, x_max, in_sizes, training, rpu,
                    O.NoiseReplay(w_noise, out_noise), learnable_weight_clip=lwc)
    grads = O.backward(rec, g, w, b is not None, ir, rpu)
    return rec, grads
