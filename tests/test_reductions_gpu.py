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
