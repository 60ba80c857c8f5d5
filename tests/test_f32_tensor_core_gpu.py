"""fp32 layers on the tensor cores: DAC codes as exact bf16 integers, weights and upstream gradients as
three bf16 planes, fp32 accumulation -- against the CPU oracle to the fp32 bar (1e-5 relative), with the
noise replayed.  Static and dynamic input ranges, ADC clamp masks folded into the gradient planes, bias,
per-channel scales, multi-dimensional inputs, row counts and widths that are not multiples of the block
sizes; benchmark configuration 1 at its own size; both backward kernels (single CTAs and CTA pairs)."""
import pytest
import torch

import cases as C
from test_parity_gpu import check_close
from util import oracle_run, rel_fro, run_product_layer

pytestmark = pytest.mark.gpu

CASES = [
    ("static_train_noise", dict(in_shape=(512, 1024), out_features=1024, max_input_size=512, ir_init_value=3.0,
                                weight_scale=1 / 32)),                       # configuration 1
    ("static_train_noise_pc", dict(in_shape=(512, 1024), out_features=1024, max_input_size=512, ir_init_value=3.0,
                                   weight_scale=1 / 32, out_noise_per_channel=False)),
    ("static_train_noise_pc", dict(in_shape=(192, 640), out_features=320, max_input_size=160, ir_init_value=2.0)),
    ("dynamic_adc_noise", dict(in_shape=(256, 1024), out_features=512, max_input_size=256)),
    ("dynamic_adc_gauss_pc_clip", dict(in_shape=(200, 512), out_features=264, max_input_size=128)),
    ("static_adc", dict(in_shape=(130, 512), out_features=520, max_input_size=128, ir_init_value=2.0)),
    ("dynamic_3d_input", dict(in_shape=(3, 50, 256), out_features=136, max_input_size=64)),
    ("dynamic_plain_eval", dict(in_shape=(300, 384), out_features=200, max_input_size=128)),
    ("static_init_from_data", dict(in_shape=(256, 512), out_features=256, max_input_size=256)),
    ("no_bias", dict(in_shape=(128, 256), out_features=128, max_input_size=-1)),
]


@pytest.mark.parametrize("base,over", CASES, ids=[f"{b}-{'x'.join(map(str, o['in_shape']))}x{o['out_features']}" for b, o in CASES])
@pytest.mark.parametrize("engine", ["tcgen05_single", "tcgen05_pair"])
def test_fp32_layer_on_tensor_cores_matches_oracle(base, over, engine):
    case = dict(C.CASES_BY_NAME[base])
    case.setdefault("weight_scale", 0.05)
    case["weight_scale"] = 0.05
    case.update(over)
    case["steps"] = 1
    data = C.make_inputs(case)
    rec, grads = oracle_run(case, data, w_noise=data["w_noise"][-1], out_noise=data["out_noise"][-1])
    capture = {}
    layer, x, out = run_product_layer(case, data, engine=engine, capture=capture)
    assert capture["uses_tcgen05"]
    dtype = data["dtype"]
    assert dtype == torch.float32
    check_close("out", out, rec.out, dtype, case)
    check_close("grad_x", x.grad, grads["grad_x"], dtype, case)
    check_close("grad_w", layer.weight.grad, grads["grad_w"], dtype, case)
    if case["bias"]:
        check_close("grad_bias", layer.bias.grad, grads["grad_bias"], dtype, case)
    if grads["grad_ir"] is not None and case["ir_learn"]:
        assert torch.allclose(layer.input_range.grad.cpu(), grads["grad_ir"], rtol=1e-4, atol=1e-5)


def test_auto_engine_picks_the_tensor_cores_for_a_large_fp32_layer_and_agrees_with_the_cuda_cores():
    from aihwkit_lightning_b200.nn import AnalogLinear
    from aihwkit_lightning_b200.nn import functional as F
    from util import NS

    case = dict(C.DEFAULTS)
    case.update(ir_dynamic=True, inp_res=254.0, max_input_size=512, out_bound=10.0, out_res=254.0)
    rpu = C.build_rpu_config(NS, case)
    torch.manual_seed(0)
    layer = AnalogLinear(1024, 768, bias=True, rpu_config=rpu).cuda().eval()
    x = torch.randn(640, 1024, device="cuda", requires_grad=True)
    g = torch.randn(640, 768, device="cuda")
    results = {}
    for engine in ("auto", "simt"):
        cap = {}
        layer.zero_grad(set_to_none=True)
        x.grad = None
        with F.operator_settings(engine=engine, capture=cap):
            out = layer(x)
        out.backward(g)
        results[engine] = (cap["uses_tcgen05"], out.detach(), x.grad.clone(), layer.weight.grad.clone())
    assert results["auto"][0] and not results["simt"][0]
    # ADC on: a last-ulp difference of an accumulator may move an output by one converter level
    flips = (results["auto"][1] != results["simt"][1]).float().mean().item()
    assert flips < 5e-3 or rel_fro(results["auto"][1], results["simt"][1]) < 1e-5
    assert rel_fro(results["auto"][2], results["simt"][2]) < 2e-3
    assert rel_fro(results["auto"][3], results["simt"][3]) < 2e-3
