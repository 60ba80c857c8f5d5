"""abs-max (bit-exact), std (1e-5 relative) and weight-clipping kernels against torch on CPU."""
import pytest
import torch

import analog_oracle as O

pytestmark = pytest.mark.gpu

# the reference benchmarks its abs-max kernel on these odd sizes (`triton_abs_max.py:405`)
SIZES = [1, 10, 25, 255, 257, 1023, 1025]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cols", SIZES)
@pytest.mark.parametrize("max_in", [-1, 7, 128, 512])
def test_sliced_abs_max_bit_exact(dtype, cols, max_in):
    from aihwkit_lightning_b200.nn import functional as F

    torch.manual_seed(cols)
    rows = 37
    a = torch.randn(rows, cols).to(dtype)
    in_sizes = O.split_sizes(cols, max_in)
    want = O.sliced_abs_max(in_sizes, a)
    got = F.sliced_abs_max(in_sizes, a.cuda())
    assert torch.equal(got.cpu(), want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,max_in", [((1000, 1024), 256), ((7, 33), 10), ((513, 300), -1)])
def test_sliced_std(dtype, shape, max_in):
    from aihwkit_lightning_b200.nn import functional as F

    torch.manual_seed(0)
    a = (torch.randn(shape) * 1.7 + 0.3).to(dtype)
    in_sizes = O.split_sizes(shape[1], max_in)
    got = F.sliced_std(in_sizes, a.cuda()).cpu()
    lo = 0
    for t, size in enumerate(in_sizes):
        want = a[:, lo:lo + size].std().float()
        tol = 1e-5 if dtype == torch.float32 else 4e-3  # bf16: the result itself is rounded to bf16
        assert abs(got[t].item() - want.item()) <= tol * abs(want.item()), (t, got[t].item(), want.item())
        lo += size


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("clip", ["LayerGaussian", "LayerGaussianPerChannel"])
def test_clip_weights(dtype, clip):
    from aihwkit_lightning_b200.nn import functional as F
    from aihwkit_lightning_b200.simulator.enums import WeightClipType

    torch.manual_seed(1)
    w = torch.randn(64, 300).to(dtype)
    want = O.clip_weights(w, clip, 2.0)
    wc = w.cuda()
    F.clip_weights_(wc, WeightClipType(clip), 2.0)
    if dtype == torch.float32:
        assert torch.allclose(wc.cpu(), want, rtol=1e-5, atol=1e-6)
    else:
        assert (wc.cpu() == want).float().mean().item() > 0.99
        assert torch.allclose(wc.cpu().float(), want.float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("tile,static", [(256, False), (512, False), (1024, True), (2048, False), (512, True)])
def test_batched_dac_is_bit_exact(tile, static):
    """Tiles of 256 * Q bf16 elements take the DAC kernel that handles several tiles per warp from
    registers: dequantised inputs and per-row ranges against the oracle, bit for bit, with a row
    count that leaves the last warps partly idle and a tile count that does not fill a batch."""
    from aihwkit_lightning_b200.nn import AnalogLinear
    from aihwkit_lightning_b200.nn import functional as F

    import cases as C
    from util import NS

    k = tile * 3
    case = dict(C.DEFAULTS)
    case.update(dtype="bf16", in_shape=(37, k), out_features=16, max_input_size=tile, training=False,
                ir_dynamic=not static, ir_init_value=1.5, bias=False)
    rpu = C.build_rpu_config(NS, case)
    torch.manual_seed(3)
    x = (torch.randn(37, k) * 1.3).bfloat16()
    x[5] = 0.0                                     # an all-zero row: range 0, step clamped to tiny
    layer = AnalogLinear(k, 16, bias=False, rpu_config=rpu).to(device="cuda", dtype=torch.bfloat16).eval()
    cap = {}
    with torch.no_grad(), F.operator_settings(capture=cap, capture_codes=False):
        layer(x.cuda())
    assert cap["codes"] is None                    # the call took the path without the debug output
    ir_param = None if not static else torch.full((3,), 1.5, dtype=torch.bfloat16)
    idx = None if not static else torch.zeros(3, dtype=torch.bfloat16)
    rec = O.forward(x, layer.weight.detach().cpu(), None, ir_param, idx, None, None, [tile] * 3, False, rpu)
    for t, tr in enumerate(rec.tiles):
        assert torch.equal(cap["xq"][:, t * tile:(t + 1) * tile].cpu(), tr.q), f"xq tile {t}"
        if not static:
            assert torch.equal(cap["ir_rows"][t].cpu(), tr.ir.reshape(-1)), f"ir tile {t}"
