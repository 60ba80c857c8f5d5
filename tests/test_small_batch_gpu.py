"""The few-rows forward (M <= 16, eval / no autograd): one sweep over the weights yields abs-max
and tile products, a second small kernel runs the per-tile output stage.  Checked against the CPU
oracle and against the regular tcgen05 path of the same layer."""
import pytest
import torch

import cases as C
from util import NS, frac_equal, oracle_run, rel_fro

pytestmark = pytest.mark.gpu

BF16_REL = 1e-2

CASES = [
    dict(in_shape=(1, 1024), out_features=512, max_input_size=256, ir_dynamic=True, out_bound=10.0, out_res=254.0),
    dict(in_shape=(5, 1024), out_features=520, max_input_size=512, ir_dynamic=True, out_bound=3.0, out_res=254.0),
    dict(in_shape=(16, 768), out_features=264, max_input_size=96, ir_dynamic=True, out_bound=2.0, out_res=254.0,
         clip_type="LayerGaussianPerChannel", clip_sigma=2.5),
    dict(in_shape=(2, 4, 512), out_features=128, max_input_size=-1, ir_dynamic=False, ir_init_value=2.0,
         out_bound=4.0, out_res=254.0),
    dict(in_shape=(16, 640), out_features=72, max_input_size=320, ir_dynamic=True),
    dict(in_shape=(3, 256), out_features=64, max_input_size=128, ir_enable=False, inp_res=-1.0, bias=False),
]


@pytest.mark.parametrize("over", CASES, ids=[f"{'x'.join(map(str, c['in_shape']))}x{c['out_features']}" for c in CASES])
def test_few_rows_forward_matches_oracle_and_regular_path(over):
    from aihwkit_lightning_b200 import _lib
    from aihwkit_lightning_b200.nn import AnalogLinear
    from aihwkit_lightning_b200.nn import functional as F

    case = dict(C.DEFAULTS)
    case.update(dtype="bf16", training=False, weight_scale=0.05)
    case.update(over)
    data = C.make_inputs(case)
    rec, _ = oracle_run(case, data)
    rpu = C.build_rpu_config(NS, case)
    layer = AnalogLinear(data["k"], data["n"], bias=case["bias"], rpu_config=rpu).to(device="cuda", dtype=torch.bfloat16)
    layer.set_weights_and_biases(data["w"].cuda(), None if data["b"] is None else data["b"].cuda())
    layer.eval()
    x = data["xs"][-1].cuda()
    lib = _lib.load()
    with torch.no_grad():
        _lib.profile_read(True)
        out = layer(x)                                   # few-rows path
        launches = {k: v[0] for k, v in _lib.profile_read(True).items() if v[0]}
        with F.operator_settings(engine="tcgen05"):
            regular = layer(x)                           # forced onto the regular kernels
    # the few-rows path replaces the weight pre-pass and the GEMM by its two kernels
    assert launches.get("fwd_gemm") == 2 and "weight_modify" not in launches, launches
    assert out.shape == rec.out.shape
    assert torch.isfinite(out.float()).all()
    assert rel_fro(out, rec.out) <= BF16_REL
    assert rel_fro(out, regular) <= BF16_REL
    assert frac_equal(out, rec.out) >= 0.95
    assert lib.al_smallm_scratch_floats(17, 64, 2) == 0


def test_few_rows_path_is_not_taken_under_autograd():
    from aihwkit_lightning_b200 import _lib
    from aihwkit_lightning_b200.nn import AnalogLinear

    case = dict(C.DEFAULTS)
    case.update(dtype="bf16", ir_dynamic=True, in_shape=(4, 256), out_features=64, max_input_size=128)
    rpu = C.build_rpu_config(NS, case)
    layer = AnalogLinear(256, 64, rpu_config=rpu).to(device="cuda", dtype=torch.bfloat16)
    x = torch.randn(4, 256, device="cuda").bfloat16().requires_grad_(True)
    _lib.profile_read(True)
    layer(x).sum().backward()
    launches = {k: v[0] for k, v in _lib.profile_read(True).items() if v[0]}
    assert launches.get("fwd_gemm") == 1 and launches.get("dgrad_gemm") == 1
    assert x.grad is not None and torch.isfinite(x.grad.float()).all()


@pytest.mark.parametrize("rows", [1, 64])
def test_forward_can_be_captured_in_a_cuda_graph(rows):
    """Inference loops replay the layer from a CUDA graph: nothing in the forward may synchronise,
    allocate outside PyTorch's allocator or depend on host state that changes between replays.
    rows = 1 takes the few-rows kernels, rows = 64 the DAC / weight pre-pass / tcgen05 kernels."""
    from aihwkit_lightning_b200.nn import AnalogLinear

    case = dict(C.DEFAULTS)
    case.update(dtype="bf16", ir_dynamic=True, out_bound=10.0, out_res=254.0, max_input_size=256)
    rpu = C.build_rpu_config(NS, case)
    torch.manual_seed(0)
    layer = AnalogLinear(512, 256, bias=True, rpu_config=rpu).to(device="cuda", dtype=torch.bfloat16).eval()
    static_x = torch.randn(rows, 512, device="cuda").bfloat16()
    with torch.no_grad():
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                layer(static_x)                       # warm-up outside the capture
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            static_out = layer(static_x)
        for seed in (1, 2):
            new_x = torch.randn(rows, 512, device="cuda", generator=torch.Generator("cuda").manual_seed(seed)).bfloat16()
            static_x.copy_(new_x)
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(static_out, layer(new_x))
