"""Parity at the sizes the benchmark configurations name.

The CPU oracle cannot run 8192 x 4096 x 4096 in seconds, but the path is row-local: with
dynamic (per-token) input ranges every output row and every input-gradient row depends only on
its own input row, the weights and its own noise draws.  So the CUDA path runs at full size and
(a) a random subset of rows is compared with the oracle run on just those rows (same seeded
inputs, replayed noise), (b) the weight gradient -- a sum over all rows -- is compared with a
plain PyTorch fp32 matmul over the captured operands (de-quantised inputs, clamp masks), and
(c) it is checked to be additive over a split of the batch.
"""
import pytest
import torch

import analog_oracle as O
import cases as C
from util import NS, frac_equal, rel_fro

pytestmark = pytest.mark.gpu

BF16_REL = 1e-2


def build_layer(k, n, case, w):
    from aihwkit_lightning_b200.nn import AnalogLinear

    rpu = C.build_rpu_config(NS, case)
    layer = AnalogLinear(k, n, bias=False, rpu_config=rpu).to(device="cuda", dtype=w.dtype)
    layer.set_weights(w.cuda())
    return layer, rpu


def test_config2_training_step_at_full_size():
    from aihwkit_lightning_b200.nn import functional as F

    m, k, n, tile = 8192, 4096, 4096, 512
    t_count = k // tile
    case = dict(C.DEFAULTS)
    case.update(dtype="bf16", max_input_size=tile, ir_dynamic=True, inp_res=254.0, out_res=254.0,
                out_bound=10.0, out_noise=0.04, noise_type="AddNormalPerChannel", std_dev=0.02, bias=False)
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(m, k, generator=gen).bfloat16()
    w = ((torch.rand(n, k, generator=gen) * 2 - 1) / 64).bfloat16()  # nn.Linear's default init range
    g = torch.randn(m, n, generator=gen).bfloat16()
    w_noise = torch.randn(n, k, generator=gen).bfloat16()
    rows = torch.randperm(m, generator=gen)[:24].sort().values
    # output noise: replayed rows carry seeded draws, the rest zeros (saves host memory)
    out_noise = torch.zeros(t_count, m, n, dtype=torch.bfloat16)
    out_noise[:, rows] = torch.randn(t_count, len(rows), n, generator=gen).bfloat16()

    layer, rpu = build_layer(k, n, case, w)
    layer.train()
    cap = {}
    xin = x.cuda().requires_grad_(True)
    with F.operator_settings(w_noise=w_noise, out_noise=out_noise, capture=cap):
        out = layer(xin)
    out.backward(g.cuda())
    torch.cuda.synchronize()
    assert cap["uses_tcgen05"]

    # (a) row subset against the oracle
    rec = O.forward(x[rows], w, None, None, None, None, None, [tile] * t_count, True, rpu,
                    O.NoiseReplay(w_noise, out_noise[:, rows]))
    grads = O.backward(rec, g[rows], w, False, None, rpu)
    got_out, got_gx = out.detach()[rows.cuda()].cpu(), xin.grad[rows.cuda()].cpu()
    assert rel_fro(got_out, rec.out) <= BF16_REL
    assert frac_equal(got_out, rec.out) >= 0.95
    assert rel_fro(got_gx, grads["grad_x"]) <= BF16_REL
    clipped = sum(int(((tr.pre_clamp < -tr.bound) | (tr.pre_clamp > tr.bound)).sum()) for tr in rec.tiles)
    assert clipped > 0, "the ADC clamp should be active on this workload"

    # (b) weight / input gradient against fp32 matmuls over the captured operands
    xq, w_mod, mask = cap["xq"].float(), cap["w_mod"].float(), cap["keep_mask"]
    gg = g.cuda().float()
    bits = torch.arange(32, device="cuda", dtype=torch.int32)
    for t in (0, t_count - 1):
        keep = ((mask[t].T.unsqueeze(-1) >> bits) & 1).reshape(m, -1)[:, :n].float()  # mask is [T, N/32, M]
        g_t = gg * keep
        want_w = g_t.T @ xq[:, t * tile:(t + 1) * tile]
        want_x = g_t @ w_mod[:, t * tile:(t + 1) * tile]
        assert rel_fro(layer.weight.grad[:, t * tile:(t + 1) * tile], want_w) <= 5e-3
        assert rel_fro(xin.grad[:, t * tile:(t + 1) * tile], want_x) <= 5e-3

    # (c) additivity of the weight gradient over a split of the batch (same noise replayed)
    total = torch.zeros(n, k, device="cuda")
    for lo, hi in ((0, m // 2), (m // 2, m)):
        layer.weight.grad = None
        xs = x[lo:hi].cuda().requires_grad_(True)
        with F.operator_settings(w_noise=w_noise, out_noise=out_noise[:, lo:hi].contiguous()):
            layer(xs).backward(g[lo:hi].cuda())
        total += layer.weight.grad.float()
    layer.weight.grad = None
    xs = x.cuda().requires_grad_(True)
    with F.operator_settings(w_noise=w_noise, out_noise=out_noise):
        layer(xs).backward(g.cuda())
    assert rel_fro(layer.weight.grad, total) <= 5e-3


SWEEP = [
    # (M, K=N, max_input_size): points of the inference shape sweep (noise off, exact compare):
    # every M at K = N = 4096 and 8192, the corners of the other sizes and tilings
    (1, 2048, 256), (4096, 2048, 512), (4096, 4096, 256), (256, 4096, 1024),
    (1, 4096, 512), (16, 4096, 512), (256, 4096, 512), (4096, 4096, 512), (16384, 4096, 512),
    (1, 8192, 512), (16, 8192, 1024), (256, 8192, 512), (4096, 8192, 512), (16384, 8192, 256),
    (256, 16384, 512), (16384, 16384, 1024),
]


@pytest.mark.parametrize("m,kn,max_in", SWEEP, ids=[f"M{m}-K{kn}-tile{t}" for m, kn, t in SWEEP])
def test_inference_sweep_point(m, kn, max_in):
    case = dict(C.DEFAULTS)
    case.update(dtype="bf16", max_input_size=max_in, ir_dynamic=True, inp_res=254.0, out_res=254.0,
                out_bound=10.0, bias=False, training=False)
    gen = torch.Generator().manual_seed(m + kn)
    x = torch.randn(m, kn, generator=gen).bfloat16()
    w = (0.02 * torch.randn(kn, kn, generator=gen)).bfloat16()
    layer, rpu = build_layer(kn, kn, case, w)
    layer.eval()
    with torch.no_grad():
        out = layer(x.cuda())
    torch.cuda.synchronize()
    rows = torch.arange(m) if m <= 16 else torch.randperm(m, generator=gen)[:16].sort().values
    in_sizes = O.split_sizes(kn, max_in)
    rec = O.forward(x[rows], w, None, None, None, None, None, in_sizes, False, rpu)
    got = out[rows.cuda()].cpu()
    assert rel_fro(got, rec.out) <= BF16_REL
    assert frac_equal(got, rec.out) >= 0.95
