"""Element-wise operators of a decoder layer around its analog linear layers.

``swiglu`` (the gated activation behind a fused gate / up projection) and ``rotary_qkv`` (the rotary
embedding behind a fused qkv projection) as single passes of the library (``csrc/decoder_glue_kernels.cu``)
with hand-written backward passes.  The reference leaves both to PyTorch; on the strided views of the fused
activations they are chains of element-wise kernels that cost more than the attention between them.
"""
import torch
from torch import Tensor

from .. import _lib
from .functional import _DTYPE, _OnDevice, _stream


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up: Tensor) -> Tensor:  # type: ignore[override]
        lib = _lib.load()
        gu = gate_up.contiguous()
        width = gu.shape[-1] // 2
        rows = gu.numel() // (2 * width)
        out = torch.empty(*gu.shape[:-1], width, device=gu.device, dtype=gu.dtype)
        with _OnDevice(gu.device):
            _lib.check(lib.al_swiglu_forward(_DTYPE[gu.dtype], gu.data_ptr(), rows, width, out.data_ptr(),
                                             _stream(gu.device)))
        ctx.save_for_backward(gu)
        return out

    @staticmethod
    def backward(ctx, grad_out: Tensor):  # type: ignore[override]
        lib = _lib.load()
        (gu,) = ctx.saved_tensors
        g = grad_out.contiguous()
        width = gu.shape[-1] // 2
        rows = gu.numel() // (2 * width)
        dgu = torch.empty_like(gu)
        with _OnDevice(gu.device):
            _lib.check(lib.al_swiglu_backward(_DTYPE[gu.dtype], gu.data_ptr(), g.data_ptr(), rows, width,
                                              dgu.data_ptr(), _stream(gu.device)))
        return dgu


def swiglu(gate_up: Tensor) -> Tensor:
    """``silu(gate) * up`` of ``gate_up = [..., gate | up]`` (CUDA tensor, fp32 or bf16, width a multiple of 8)."""
    if gate_up.dtype not in _DTYPE or not gate_up.is_cuda:
        raise TypeError("swiglu needs a CUDA tensor in float32 or bfloat16")
    return _SwiGLU.apply(gate_up)


class _RotaryQKV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv: Tensor, cos: Tensor, sin: Tensor):  # type: ignore[override]
        lib = _lib.load()
        x = qkv.contiguous()  # [b, s, 3, heads, hd]
        b, s, three, heads, hd = x.shape
        assert three == 3, "qkv must be [batch, seq, 3, heads, head_dim]"
        rows, es = b * s, x.element_size()
        q = torch.empty(b, s, heads, hd, device=x.device, dtype=x.dtype)
        k, v = torch.empty_like(q), torch.empty_like(q)
        part = heads * hd * es
        with _OnDevice(x.device):
            _lib.check(lib.al_rotary_qkv(_DTYPE[x.dtype], 0, x.data_ptr(), x.data_ptr() + part, x.data_ptr() + 2 * part,
                                         3 * heads * hd, cos.data_ptr(), sin.data_ptr(), rows, s, heads, hd,
                                         q.data_ptr(), k.data_ptr(), v.data_ptr(), heads * hd, _stream(x.device)))
        ctx.save_for_backward(cos, sin)
        return q, k, v

    @staticmethod
    def backward(ctx, gq: Tensor, gk: Tensor, gv: Tensor):  # type: ignore[override]
        lib = _lib.load()
        cos, sin = ctx.saved_tensors
        gq, gk, gv = gq.contiguous(), gk.contiguous(), gv.contiguous()
        b, s, heads, hd = gq.shape
        dqkv = torch.empty(b, s, 3, heads, hd, device=gq.device, dtype=gq.dtype)
        part = heads * hd * gq.element_size()
        with _OnDevice(gq.device):
            _lib.check(lib.al_rotary_qkv(_DTYPE[gq.dtype], 1, gq.data_ptr(), gk.data_ptr(), gv.data_ptr(), heads * hd,
                                         cos.data_ptr(), sin.data_ptr(), b * s, s, heads, hd, dqkv.data_ptr(),
                                         dqkv.data_ptr() + part, dqkv.data_ptr() + 2 * part, 3 * heads * hd,
                                         _stream(gq.device)))
        return dqkv, None, None


def rotary_qkv(qkv: Tensor, cos: Tensor, sin: Tensor):
    """``[batch, seq, 3, heads, head_dim]`` -> rotated ``q``, ``k`` and ``v``, each ``[batch, seq, heads, head_dim]``.

    ``cos`` / ``sin``: float32 ``[seq, head_dim / 2]`` tables; element ``j`` of a head's first half is rotated
    with element ``j`` of its second half (the HF "rotate_half" convention)."""
    if qkv.dtype not in _DTYPE or not qkv.is_cuda:
        raise TypeError("rotary_qkv needs a CUDA tensor in float32 or bfloat16")
    half = qkv.shape[-1] // 2
    if cos.dtype != torch.float32 or sin.dtype != torch.float32 or tuple(cos.shape) != (qkv.shape[1], half) \
            or tuple(sin.shape) != (qkv.shape[1], half):
        raise ValueError("cos / sin must be float32 [seq, head_dim / 2]")
    return _RotaryQKV.apply(qkv, cos.contiguous(), sin.contiguous())
