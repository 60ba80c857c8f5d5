"""The decoder-layer element-wise operators (gated activation, rotary embedding of a fused qkv) against
their PyTorch formulations, forward and backward."""
import pytest
import torch
from torch.nn import functional as TF

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("shape", [(3, 40, 64), (257, 8192)])
def test_swiglu_matches_torch(dtype, tol, shape):
    from aihwkit_lightning_b200.nn.decoder_ops import swiglu

    gen = torch.Generator(device="cuda").manual_seed(sum(shape))
    width = shape[-1]
    gu = torch.randn(*shape[:-1], 2 * width, device="cuda", generator=gen).to(dtype)
    g = torch.randn(*shape, device="cuda", generator=gen).to(dtype)
    a = gu.clone().requires_grad_(True)
    out = swiglu(a)
    out.backward(g)
    b = gu.double().requires_grad_(True)
    gate, up = b.chunk(2, dim=-1)
    want = TF.silu(gate) * up
    want.backward(g.double())
    rel = lambda x, y: ((x.double() - y).norm() / y.norm()).item()
    assert out.shape == want.shape and out.dtype == dtype
    assert rel(out, want) <= tol
    assert rel(a.grad, b.grad) <= tol


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("b,s,heads,hd", [(2, 17, 3, 16), (2, 128, 32, 96)])
def test_rotary_qkv_matches_torch(dtype, tol, b, s, heads, hd):
    from aihwkit_lightning_b200.nn.decoder_ops import rotary_qkv

    gen = torch.Generator(device="cuda").manual_seed(b + s + heads + hd)
    qkv = torch.randn(b, s, 3, heads, hd, device="cuda", generator=gen).to(dtype)
    gq, gk, gv = (torch.randn(b, s, heads, hd, device="cuda", generator=gen).to(dtype) for _ in range(3))
    pos = torch.arange(s, device="cuda", dtype=torch.float32)
    inv = 1.0 / (10000 ** (torch.arange(0, hd, 2, device="cuda", dtype=torch.float32) / hd))
    ang = pos[:, None] * inv[None, :]
    cos, sin = ang.cos(), ang.sin()

    a = qkv.clone().requires_grad_(True)
    q, k, v = rotary_qkv(a, cos, sin)
    (q * gq).sum().backward(retain_graph=True)
    torch.autograd.backward([k, v], [gk, gv])

    x = qkv.double().requires_grad_(True)
    c = torch.cat([cos, cos], -1).double()[None, :, None, :]
    sn = torch.cat([sin, sin], -1).double()[None, :, None, :]

    def rope(t):
        t1, t2 = t[..., : hd // 2], t[..., hd // 2:]
        return t * c + torch.cat([-t2, t1], -1) * sn

    wq, wk, wv = rope(x[:, :, 0]), rope(x[:, :, 1]), x[:, :, 2]
    torch.autograd.backward([wq, wk, wv], [gq.double(), gk.double(), gv.double()])
    rel = lambda p, r: ((p.double() - r).norm() / r.norm()).item()
    assert rel(q, wq) <= tol and rel(k, wk) <= tol
    assert torch.equal(v, qkv[:, :, 2])
    assert rel(a.grad, x.grad) <= tol


def test_bad_arguments_are_refused():
    from aihwkit_lightning_b200.nn.decoder_ops import rotary_qkv, swiglu

    with pytest.raises(TypeError):
        swiglu(torch.randn(4, 16))  # CPU tensor
    with pytest.raises(Exception):
        swiglu(torch.randn(4, 12, device="cuda", dtype=torch.bfloat16))  # width 6: not a multiple of 8
    qkv = torch.randn(1, 4, 3, 2, 16, device="cuda")
    with pytest.raises(ValueError):
        rotary_qkv(qkv, torch.ones(4, 16, device="cuda"), torch.ones(4, 16, device="cuda"))  # tables of the wrong width
