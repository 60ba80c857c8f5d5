"""The oracle against the golden vectors generated from the unmodified reference.

``tests/golden/make_golden.py`` wrote, for every case, what the reference's torch backend
returns (output, all gradients, updated input ranges) when its noise draws are replayed from
the seeded tensors of ``cases.make_inputs``.  The oracle has to reproduce them bit for bit.
"""
import os
from types import SimpleNamespace

import pytest
import torch

import analog_oracle as O
import cases as C
from aihwkit_lightning_b200.simulator import configs as product_cfg

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
NS = SimpleNamespace(
    TorchInferenceRPUConfig=product_cfg.TorchInferenceRPUConfig,
    WeightNoiseInjectionType=product_cfg.WeightNoiseInjectionType,
    WeightQuantizationType=product_cfg.WeightQuantizationType,
    WeightClipType=product_cfg.WeightClipType,
)


def same(a, b):
    if a is None or b is None:
        return a is None and b is None
    return a.shape == b.shape and a.dtype == b.dtype and bool((a == b).all())


def run_oracle(case, data):
    rpu = C.build_rpu_config(NS, case)
    in_sizes = O.split_sizes(data["k"], case["max_input_size"])
    static = case["ir_enable"] and not case["ir_dynamic"]
    ir = idx = x_min = x_max = None
    if static:
        ir = torch.full((len(in_sizes),), case["ir_init_value"], dtype=data["dtype"])
        idx = torch.zeros(len(in_sizes), dtype=data["dtype"])
        x_min = torch.zeros(len(in_sizes), dtype=data["dtype"]) - 1e-5
        x_max = torch.zeros(len(in_sizes), dtype=data["dtype"]) + 1e-5
    lwc = None
    if case["clip_type"] == "LearnablePerChannel":
        lwc = O.sliced_abs_max(in_sizes, data["w"]) * case["lwc_scale"]
    for step in range(case["steps"]):
        rec = O.forward(
            data["xs"][step], data["w"], data["b"], ir, idx, x_min, x_max, in_sizes,
            case["training"], rpu, O.NoiseReplay(data["w_noise"][step], data["out_noise"][step]),
            learnable_weight_clip=lwc,
        )
    grads = O.backward(rec, data["g"], data["w"], case["bias"], ir, rpu)
    if static and not case["ir_learn"]:
        grads["grad_ir"] = None
    return rec, grads, ir, idx, x_min, x_max


@pytest.mark.parametrize("name", [c["name"] for c in C.CASES])
def test_oracle_reproduces_reference(name):
    case = C.CASES_BY_NAME[name]
    want = torch.load(os.path.join(GOLDEN, name + ".pt"), weights_only=False)
    assert want["case"] == case, "golden file is stale: re-run tests/golden/make_golden.py"
    data = C.make_inputs(case)
    rec, grads, ir, idx, x_min, x_max = run_oracle(case, data)
    assert same(want["out"], rec.out)
    for key in ("grad_x", "grad_w", "grad_bias", "grad_ir", "grad_clip"):
        assert same(want[key], grads[key]), key
    assert same(want["input_range"], ir)
    assert same(want["input_range_update_idx"], idx)
    assert same(want["x_min"], x_min) and same(want["x_max"], x_max)
    assert want["in_sizes"] == O.split_sizes(data["k"], case["max_input_size"])


def test_split_sizes_known_answers():
    # `linear.py:155-170`: ceil(size/max) tiles whose sizes differ by at most one
    assert O.split_sizes(10, 9) == [5, 5]
    assert O.split_sizes(10, 11) == [10]
    assert O.split_sizes(43, 10) == [9, 9, 9, 8, 8]
    assert O.split_sizes(4096, 512) == [512] * 8
    assert O.split_sizes(576, 256) == [192, 192, 192]
    assert O.split_sizes(7, -1) == [7]


def test_weight_discretiser_closed_form():
    """Closed form the reference's own test expects of the discretiser
    (`tests/test_correctness_against_aihwkit.py:934-946`): step = abs-max / (res/2)."""
    torch.manual_seed(0)
    w = torch.randn(1, 10)
    for res in (30.0, 1 / 30.0):
        n_half = res / 2 if res > 1.0 else 1 / (2 * res)
        for per_channel in (False, True):
            scale = w.abs().amax(dim=1, keepdim=True) if per_channel else w.abs().max()
            step = (1 / n_half) * scale
            want = (w / step).round() * step
            got = O.discretize_weight(w, scale, res)
            assert torch.allclose(got, want, atol=1e-6)


def test_clip_weights_matches_direct_formula():
    torch.manual_seed(0)
    w = torch.randn(8, 33)
    got = O.clip_weights(w, "LayerGaussian", 2.0)
    lim = 2.0 * w.std()
    assert torch.equal(got, w.clamp(-lim, lim))
    got = O.clip_weights(w, "LayerGaussianPerChannel", 2.0)
    lim = 2.0 * w.std(1, keepdim=True)
    assert torch.equal(got, torch.minimum(torch.maximum(w, -lim), lim))
