"""CPU oracle for the noisy, quantised, input-tiled analog linear path.

THIS FILE IS TEST INFRASTRUCTURE.  It is a restatement, in plain torch CPU ops, of the
algorithm of the reference's torch backend.  Only the tests, the smoke check and the CPU
baseline leg of the benchmark may import it; the product (the CUDA library and the Python
package around it) never does.

Parity status: PINNED.  ``tests/golden/make_golden.py`` imports the unmodified reference
(`src/aihwkit_lightning`) in a container that has it, replays a shared noise stream into both
and asserts that this oracle reproduces the reference's outputs and gradients bit for bit
(fp32 and bf16); the resulting vectors are committed under ``tests/golden/`` and checked by
``tests/test_oracle_golden.py`` wherever the reference itself is not present.

The arithmetic itself lives in PyTorch (ATen CPU kernels), which the reference depends on
without pinning a version (`pyproject.toml:22-26`, ``torch>=1.10.0``); the oracle uses the same
ATen ops so that reduced-precision rounding (every op rounds to the tensor dtype) is inherited
rather than re-derived.

Reference locations restated here (paths inside the reference project):

* tiling              ``src/aihwkit_lightning/nn/modules/linear.py:155-170``
* per-tile loop       ``src/aihwkit_lightning/nn/modules/torch_utils/torch_linear.py:116-314``
* static input range  ``.../torch_utils/torch_linear.py:317-358`` (+ ``:29-108`` for the backward)
* fast-mode range     ``.../torch_utils/torch_linear.py:361-423``
* weight noise        ``.../torch_utils/torch_linear.py:426-462``
* uniform quantiser   ``.../torch_utils/quant_utils.py:35-109``
* weight discretiser  ``.../torch_utils/quant_utils.py:159-237``
* sliced abs-max      ``.../torch_utils/torch_abs_max.py:17-39``
* weight clipping     ``src/aihwkit_lightning/nn/modules/linear.py:269-283``
"""
from __future__ import annotations

from dataclasses import dataclass, field
from math import sqrt
from typing import Callable, Dict, List, Optional, Tuple

import torch
from torch import Tensor

# String values of the reference enums (`simulator/parameters/enums.py:22-90`); the oracle
# compares on ``.value`` so that it accepts the reference's enums and the product's alike.
NOISE_NONE, NOISE_ADD, NOISE_ADD_PC = "None", "AddNormal", "AddNormalPerChannel"
QUANT_NONE, QUANT_DISC, QUANT_DISC_PC = "None", "Discretize", "DiscretizePerChannel"
CLIP_NONE, CLIP_GAUSS, CLIP_GAUSS_PC, CLIP_LEARN_PC = (
    "None",
    "LayerGaussian",
    "LayerGaussianPerChannel",
    "LearnablePerChannel",
)


def _ev(enum_or_str) -> str:
    return getattr(enum_or_str, "value", enum_or_str)


def split_sizes(size: int, split_max_size: int) -> List[int]:
    """Tile widths (`linear.py:155-170`): ``ceil(size/max)`` tiles, sizes differ by at most 1."""
    if split_max_size <= 0:
        return [size]
    n_splits = (size + split_max_size - 1) // split_max_size
    base, extra = divmod(size, n_splits)
    return [base + (i < extra) for i in range(n_splits)]


def sliced_abs_max(in_sizes: List[int], weights: Tensor) -> Tensor:
    """Per-tile, per-row abs-max ``[T, rows]`` (`torch_abs_max.py:17-39`)."""
    out = []
    lo = 0
    for size in in_sizes:
        out.append(weights[:, lo : lo + size].abs().amax(dim=1))
        lo += size
    return torch.stack(out)


def quant_step(bound, res: float):
    """Step of the uniform quantiser: ``2*bound/res`` for ``res > 1`` else ``2*bound*res``
    (`quant_utils.py:63-77`, scalar ``res``)."""
    alpha = 2 * bound
    return alpha / res if res > 1.0 else alpha * res


def uniform_quantize(inp: Tensor, res: float, bound, no_rounding: bool = False) -> Tensor:
    """``round(inp / max(step, tiny)) * step`` (`quant_utils.py:78-99`), every op in ``inp.dtype``."""
    step = quant_step(bound, res)
    tiny = torch.finfo(inp.dtype).tiny
    clamped = step.clamp_min(tiny) if isinstance(step, Tensor) else max(tiny, step)
    out = inp / clamped
    if not no_rounding:
        out = out.round()
    out = out * step
    return out


def discretize_weight(w_t: Tensor, scale: Tensor, mod_res: float, no_rounding: bool = False) -> Tensor:
    """Weight discretisation of one tile (`quant_utils.py:204-233`, non-learnable branch).

    ``scale`` is the tile's scalar abs-max (DISCRETIZE) or the ``[N,1]`` row abs-max
    (DISCRETIZE_PER_CHANNEL).  The quantiser is entered with ``res = scale / n_states`` as a
    tensor and ``bound = 1.0`` (`quant_utils.py:225-233`), hence the ``(res > 1).all()``
    switch, the zero guard and the clamp to ``n_states / 2`` below (`quant_utils.py:63-86`).
    """
    n_states = max(mod_res, 1 / mod_res)
    max_state = n_states / 2
    res = scale / n_states
    alpha = 2 * 1.0
    res = alpha / res if bool((res > 1.0).all()) else alpha * res
    res = res.clone()
    res[res == 0.0] = 1.0
    clamped = res.clamp_min(torch.finfo(w_t.dtype).tiny)
    out = w_t / clamped
    out = torch.clamp(out, min=-max_state, max=max_state)
    if not no_rounding:
        out = out.round()
    out = out * res
    return out


def learnable_quantize(w_t: Tensor, res_arg: Tensor, bound: float, max_state: float, skip_rounding: bool):
    """``UniformQuantize.forward`` with ``learn_res=True`` (`quant_utils.py:63-109`) as
    `clip_and_quantize` enters it for LEARNABLE_PER_CHANNEL clipping (`quant_utils.py:184-233`):
    ``res_arg`` is the ``[N,1]`` tensor handed in as ``res`` (the clip values, or clip / n_states
    when the weights are also discretised).  Returns the output and the clamped step that the
    backward divides by."""
    alpha = 2 * bound
    res = alpha / res_arg if bool((res_arg > 1.0).all()) else alpha * res_arg
    res = res.clone()
    res[res == 0.0] = 1.0
    clamped = res.clamp_min(torch.finfo(w_t.dtype).tiny)
    out = w_t / clamped
    out = torch.clamp(out, min=-max_state, max=max_state)
    if not skip_rounding:
        out = out.round()
    out = out * res
    return out, clamped


@dataclass
class TileRecord:
    """Everything the backward and the parity tests want to see of one tile."""

    lo: int
    hi: int
    ir: Optional[Tensor] = None  # [M,1] (dynamic) or 0-d (static); None when IR is off
    upper: Optional[Tensor] = None  # x >= ir (static IR)
    lower: Optional[Tensor] = None  # x <= -ir (static IR)
    codes: Optional[Tensor] = None  # rint(x/step) as produced in the layer dtype
    q: Optional[Tensor] = None  # de-quantised DAC output fed to the GEMM  [M, tile]
    amax_rows: Optional[Tensor] = None  # [N,1]
    w_mod: Optional[Tensor] = None  # [N, tile]
    bound: Optional[Tensor] = None  # ADC bound, broadcastable to [M,N]
    pre_clamp: Optional[Tensor] = None  # ADC-quantised tile output before the clamp
    out_t: Optional[Tensor] = None  # tile contribution after everything
    learn: Optional[dict] = None  # learnable weight clip: what its backward needs


@dataclass
class ForwardRecord:
    out: Tensor
    tiles: List[TileRecord] = field(default_factory=list)
    x2d: Optional[Tensor] = None
    in_shape: Tuple[int, ...] = ()


class NoiseReplay:
    """Hands out pre-drawn standard normals in the order the per-tile loop asks for them.

    Per tile the order is: weight noise ``[N, tile]`` first (`torch_linear.py:453/456`), then
    output noise ``[M, N]`` (`torch_linear.py:281`).  ``w_noise`` is ``[N, K]``, ``out_noise``
    ``[T, M, N]``; both may be ``None`` when the respective noise is off.
    """

    def __init__(self, w_noise: Optional[Tensor], out_noise: Optional[Tensor]):
        self.w_noise = w_noise
        self.out_noise = out_noise

    def weight(self, lo: int, hi: int, like: Tensor) -> Tensor:
        if self.w_noise is None:
            return torch.randn_like(like)
        return self.w_noise[:, lo:hi].to(like.dtype)

    def output(self, tile: int, like: Tensor) -> Tensor:
        if self.out_noise is None:
            return torch.randn_like(like)
        return self.out_noise[tile].to(like.dtype).reshape(like.shape)


def update_input_range_from_data(
    x_t: Tensor, slice_idx: int, ir_params, input_range: Tensor, input_range_update_idx: Tensor
) -> None:
    """Running mean of ``init_std_alpha * std(x_tile)`` for the first ``init_from_data`` calls
    (`torch_linear.py:338-352`); mutates ``input_range`` and ``input_range_update_idx``."""
    idx = input_range_update_idx[slice_idx]
    if idx < ir_params.init_from_data:
        std = x_t.std()
        if std > 0.0:
            input_range.data[slice_idx] = (
                (input_range.data[slice_idx].float() * idx + ir_params.init_std_alpha * std.float())
                / (idx + 1)
            ).to(dtype=input_range.dtype)
            input_range_update_idx[slice_idx] += 1
        input_range.data[slice_idx] = input_range.data[slice_idx].abs()


def update_input_range_fast(
    x_t: Tensor,
    slice_idx: int,
    ir_params,
    input_range: Tensor,
    input_range_update_idx: Tensor,
    x_min: Tensor,
    x_max: Tensor,
) -> None:
    """Min/max tracking of the fast mode (`torch_linear.py:386-420`)."""
    idx = input_range_update_idx[slice_idx]
    if idx < ir_params.init_from_data:
        act_min = x_t.min()
        act_max = x_t.max()
        if x_min[slice_idx].min() > -1.1e-5 and x_max[slice_idx].max() < 1.1e-5:
            x_min[slice_idx] = x_min[slice_idx] + act_min
            x_max[slice_idx] = x_max[slice_idx] + act_max
        elif ir_params.act_range_momentum == -1:
            x_min[slice_idx] = min(x_min[slice_idx], act_min)
            x_max[slice_idx] = max(x_max[slice_idx], act_max)
        else:
            mom = ir_params.act_range_momentum
            x_min[slice_idx] = x_min[slice_idx] * mom + act_min * (1 - mom)
            x_max[slice_idx] = x_max[slice_idx] * mom + act_max * (1 - mom)
        input_range_update_idx[slice_idx] += 1
        input_range.data[slice_idx] = max(x_min[slice_idx].abs(), x_max[slice_idx].abs())


@torch.no_grad()
def forward(
    inp: Tensor,
    weights: Tensor,
    bias: Optional[Tensor],
    input_range: Optional[Tensor],
    input_range_update_idx: Optional[Tensor],
    x_min: Optional[Tensor],
    x_max: Optional[Tensor],
    in_sizes: List[int],
    training: bool,
    rpu_config,
    noise: Optional[NoiseReplay] = None,
    no_rounding: bool = False,
    learnable_weight_clip: Optional[Tensor] = None,
) -> ForwardRecord:
    """Restated ``TorchLinear.linear`` (`torch_linear.py:116-314`) that also records every
    intermediate.  ``learnable_weight_clip`` is the ``[T, N]`` parameter of LEARNABLE_PER_CHANNEL
    clipping (`base.py:104-118`)."""
    noise = noise or NoiseReplay(None, None)
    fwd, mod, clip = rpu_config.forward, rpu_config.modifier, rpu_config.clip
    irp = rpu_config.pre_post.input_range
    noise_type, quant_type, clip_type = _ev(mod.noise_type), _ev(mod.quantization_type), _ev(clip.type)
    learnable = clip_type == CLIP_LEARN_PC
    if learnable:
        assert learnable_weight_clip is not None, "learnable_weight_clip should not be None"
        assert quant_type in (QUANT_NONE, QUANT_DISC_PC), (
            "You can't learn weight ranges per column but quantize per tensor"
        )
    apply_out_quant = fwd.out_res > 0
    if apply_out_quant:
        assert fwd.out_bound > 0, "Out quant. without a bound."
        assert irp.enable, "Out quant. without IR."

    in_shape = tuple(inp.shape)
    x2d = inp.reshape(-1, in_shape[-1])
    n_tiles = len(in_sizes)
    rec = ForwardRecord(out=None, x2d=x2d, in_shape=in_shape)  # type: ignore[arg-type]
    out = 0.0
    lo = 0
    for t, size in enumerate(in_sizes):
        hi = lo + size
        tr = TileRecord(lo=lo, hi=hi)
        x_t = x2d[:, lo:hi]
        ir = None
        if irp.enable:
            if irp.fast_mode:
                if training:
                    update_input_range_fast(
                        x_t, t, irp, input_range, input_range_update_idx, x_min, x_max
                    )
                ir = input_range[t].detach().clone()
                x_t = torch.clamp(x_t, min=-ir, max=ir)
            elif irp.dynamic:
                ir = x_t.abs().max(dim=-1, keepdim=True)[0]
            else:
                if training:
                    update_input_range_from_data(x_t, t, irp, input_range, input_range_update_idx)
                ir = input_range[t].detach().clone()
                tr.upper = x_t >= ir
                tr.lower = x_t <= -ir
                x_t = torch.clamp(x_t, min=-ir, max=ir)
            tr.ir = ir

        if fwd.inp_res > 0:
            assert ir is not None, "Input range must be provided"
            step = quant_step(ir, fwd.inp_res)
            tiny = torch.finfo(x_t.dtype).tiny
            codes = x_t / step.clamp_min(tiny)
            if not no_rounding:
                codes = codes.round()
            tr.codes = codes
            x_t = codes * step
        tr.q = x_t

        w_t = weights[:, lo:hi]
        need_wmax = (
            apply_out_quant
            or fwd.out_bound > 0
            or (training and fwd.out_noise > 0)
            or (training and noise_type in (NOISE_ADD, NOISE_ADD_PC))
            or quant_type in (QUANT_DISC, QUANT_DISC_PC)
            or learnable
        )
        amax_rows = w_t.abs().amax(dim=-1, keepdim=True) if need_wmax else None

        if learnable:
            # `quant_utils.py:184-233`: clamp to the learned range (no rounding), or discretise with
            # the learned range as the scale; afterwards the learned range stands in for the
            # abs-max everywhere (`torch_linear.py:236-246`)
            lwc_t = learnable_weight_clip[t].detach().unsqueeze(-1)
            numel = w_t.numel()
            if quant_type == QUANT_NONE:
                w_q, clamped = learnable_quantize(w_t, lwc_t, 0.5, 1.0, True)
                tr.learn = dict(w=w_t, res=clamped, qmax=1.0, skip=True, grad_scale=1 / sqrt(numel), n_states=None)
            else:
                n_states = max(mod.res, 1 / mod.res)
                qmax = n_states / 2
                skip = bool(no_rounding)
                w_q, clamped = learnable_quantize(w_t, lwc_t / n_states, 1.0, qmax, skip)
                tr.learn = dict(w=w_t, res=clamped, qmax=qmax, skip=skip, n_states=n_states,
                                grad_scale=1 / sqrt(numel) if skip else 2 * sqrt(qmax / numel))
            w_t = w_q
            amax_rows = lwc_t.view_as(amax_rows)
        elif quant_type in (QUANT_DISC, QUANT_DISC_PC):
            scale = amax_rows.max() if quant_type == QUANT_DISC else amax_rows
            w_t = discretize_weight(w_t, scale, mod.res, no_rounding)
        tr.amax_rows = amax_rows

        if training and noise_type != NOISE_NONE:
            s = amax_rows.max() if noise_type == NOISE_ADD else amax_rows
            w_t = w_t + mod.std_dev * s * noise.weight(lo, hi, w_t)
        tr.w_mod = w_t

        out_t = x_t @ w_t.T

        if training and fwd.out_noise > 0:
            assert irp.enable, "Input range must be enabled"
            s = amax_rows if fwd.out_noise_per_channel else amax_rows.max()
            s = s if s.numel() == 1 else s.view(-1, out_t.size(-1))
            out_t = out_t + s * (fwd.out_noise / sqrt(n_tiles) * ir) * noise.output(t, out_t)

        if fwd.out_bound > 0 or apply_out_quant:
            assert ir is not None, "Input range must be provided when using an out_bound"
            s = amax_rows if clip_type in (CLIP_GAUSS_PC, CLIP_LEARN_PC) else amax_rows.max()
            bound = (ir * fwd.out_bound) * s.view(1, -1)
            tr.bound = bound
            if apply_out_quant:
                out_t = uniform_quantize(out_t, fwd.out_res, bound, no_rounding)
            if fwd.out_bound > 0:
                tr.pre_clamp = out_t
                out_t = torch.clamp(out_t, min=-bound, max=bound)
        tr.out_t = out_t
        out = out + out_t
        rec.tiles.append(tr)
        lo = hi

    out = out + bias if bias is not None else out
    rec.out = out.reshape(*in_shape[:-1], weights.shape[0])
    return rec


@torch.no_grad()
def backward(
    rec: ForwardRecord,
    grad_out: Tensor,
    weights: Tensor,
    has_bias: bool,
    input_range: Optional[Tensor],
    rpu_config,
) -> Dict[str, Optional[Tensor]]:
    """What autograd derives from the reference forward, written out per tile.

    ADC clamp: gradient passes where ``-bound <= o <= bound`` (torch ``clamp`` backward).
    Quantisers and noise are straight-through (`quant_utils.py:152-156`,
    `torch_linear.py:450-460`).  Static input range: range gradient and decay term
    (`torch_linear.py:98-106`), then zeroing of clipped positions that are not exactly on the
    range (`torch_linear.py:44-54`).
    """
    irp = rpu_config.pre_post.input_range
    g = grad_out.reshape(-1, grad_out.shape[-1])
    x2d = rec.x2d
    grad_x = torch.zeros_like(x2d)
    grad_w = torch.zeros_like(weights)
    static_ir = irp.enable and not irp.dynamic and not irp.fast_mode
    fast_ir = irp.enable and irp.fast_mode
    grad_ir = torch.zeros_like(input_range) if ((static_ir or fast_ir) and input_range is not None) else None
    grad_clip = None
    if rec.tiles and rec.tiles[0].learn is not None:
        grad_clip = torch.zeros(len(rec.tiles), weights.shape[0], dtype=weights.dtype)
    for t, tr in enumerate(rec.tiles):
        g_t = g
        if tr.pre_clamp is not None:
            keep = (tr.pre_clamp >= -tr.bound) & (tr.pre_clamp <= tr.bound)
            g_t = g * keep
        gw_t = g_t.T @ tr.q
        if tr.learn is not None:
            # `UniformQuantize.backward`, learn_res branch (`quant_utils.py:125-151`): indicator
            # tensors are fp32 (`.float()`), which promotes the products and the row sum to fp32;
            # autograd then casts both gradients back to the dtype of their inputs
            L = tr.learn
            q_w = L["w"] / L["res"]
            small = (q_w < -L["qmax"]).float()
            big = (q_w > L["qmax"]).float()
            middle = 1.0 - small - big
            if L["skip"]:
                g_res = (small * (-L["qmax"]) + big * L["qmax"]) * gw_t * L["grad_scale"]
            else:
                g_res = (small * (-L["qmax"]) + big * L["qmax"] + middle * (-q_w + q_w.round())) * gw_t * L["grad_scale"]
            g_res = g_res.sum(dim=-1, keepdim=True).to(weights.dtype)
            if L["n_states"] is not None:
                g_res = g_res / L["n_states"]  # res argument was clip / n_states
            grad_clip[t] = g_res.view(-1)
            gw_t = (middle * gw_t).to(weights.dtype)
        grad_w[:, tr.lo : tr.hi] = gw_t
        gx = g_t @ tr.w_mod
        x_t = x2d[:, tr.lo : tr.hi]
        if static_ir:
            ir = tr.ir
            acc = torch.zeros_like(ir)
            acc += torch.clamp(gx[tr.upper], min=None, max=0.0).sum()
            acc -= torch.clamp(gx[tr.lower], min=0.0, max=None).sum()
            acc *= ir
            if irp.decay > 0:
                percentage = 1.0 - (tr.upper | tr.lower).sum().div(tr.upper.numel())
                acc += irp.decay * ir * (percentage > irp.input_min_percentage)
            grad_ir[t] = acc
            zero = (tr.upper | tr.lower) & ~(x_t.abs() == ir)
            gx = gx.clone()
            gx[zero] = 0.0
        elif fast_ir:
            # plain torch.clamp with tensor bounds (`torch_linear.py:422`): the gradient passes
            # inside [-ir, ir]; the upper bound receives the gradient mass above it, the lower
            # bound (= -ir) the mass below it
            ir = tr.ir
            if grad_ir is not None:
                acc = torch.zeros_like(ir)
                zero = torch.zeros((), dtype=gx.dtype)
                acc = acc + torch.where(x_t > ir, gx, zero).sum()
                acc = acc + (-torch.where(x_t < -ir, gx, zero).sum())
                grad_ir[t] = acc
            gx = gx * ((x_t >= -ir) & (x_t <= ir))
        grad_x[:, tr.lo : tr.hi] = gx
    return {
        "grad_x": grad_x.reshape(rec.in_shape),
        "grad_w": grad_w,
        "grad_bias": g.sum(0) if has_bias else None,
        "grad_ir": grad_ir,
        "grad_clip": grad_clip,
    }


def clip_weights(weight: Tensor, clip_type, sigma: float) -> Tensor:
    """``clamp(W, +-sigma*std(W))`` per tensor or per row (`linear.py:269-283`); returns a copy."""
    clip_type = _ev(clip_type)
    if clip_type in (CLIP_NONE, CLIP_LEARN_PC):
        return weight.clone()
    assert sigma > 0, "Clip sigma must be greater than 0"
    w2d = weight.reshape(weight.shape[0], -1)
    sigma_std = sigma * w2d.std(None if clip_type == CLIP_GAUSS else 1, keepdim=True)
    return w2d.clamp(-sigma_std, sigma_std).reshape(weight.shape)


# --------------------------------------------------------------------------------------------
# Autograd flavour: the same per-tile op sequence expressed with torch autograd, used only to
# time the CPU path the way a user of the reference would run it (forward, then ``.backward()``).
# --------------------------------------------------------------------------------------------
class _SteClamp(torch.autograd.Function):
    """Clamp with the straight-through rule of `torch_linear.py:29-54`."""

    @staticmethod
    def forward(ctx, x, upper, lower, ir):  # type: ignore[override]
        ctx.save_for_backward((upper | lower) & ~(x.abs() == ir))
        return torch.clamp(x, min=-ir, max=ir)

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        (mask,) = ctx.saved_tensors
        g = g.clone()
        g[mask] = 0.0
        return g, None, None, None


class _RangeGrad(torch.autograd.Function):
    """Identity whose backward emits the range gradient of `torch_linear.py:57-108`."""

    @staticmethod
    def forward(ctx, x, ir, upper, lower, decay, min_pct):  # type: ignore[override]
        ctx.save_for_backward(upper, lower, ir)
        ctx.decay, ctx.min_pct = decay, min_pct
        return x

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        upper, lower, ir = ctx.saved_tensors
        acc = torch.zeros_like(ir)
        acc += torch.clamp(g[upper], min=None, max=0.0).sum()
        acc -= torch.clamp(g[lower], min=0.0, max=None).sum()
        acc *= ir
        if ctx.decay > 0:
            pct = 1.0 - (upper | lower).sum().div(upper.numel())
            acc += ctx.decay * ir * (pct > ctx.min_pct)
        return g, acc, None, None, None, None


class _SteQuant(torch.autograd.Function):
    """Uniform quantiser with identity gradient (`quant_utils.py:35-109,152-156`)."""

    @staticmethod
    def forward(ctx, x, res, bound):  # type: ignore[override]
        return uniform_quantize(x, res, bound)

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        return g, None, None


def linear_autograd(
    inp: Tensor,
    weights: Tensor,
    bias: Optional[Tensor],
    input_range: Optional[Tensor],
    input_range_update_idx: Optional[Tensor],
    in_sizes: List[int],
    training: bool,
    rpu_config,
) -> Tensor:
    """Differentiable per-tile loop with the op sequence of `torch_linear.py:116-314`
    (dynamic or static input range, DAC, additive weight noise, output noise, ADC)."""
    fwd, mod, clip = rpu_config.forward, rpu_config.modifier, rpu_config.clip
    irp = rpu_config.pre_post.input_range
    noise_type, clip_type = _ev(mod.noise_type), _ev(clip.type)
    n_tiles = len(in_sizes)
    out = 0.0
    lo = 0
    for t, size in enumerate(in_sizes):
        x_t = inp[..., lo : lo + size]
        ir = None
        if irp.enable:
            if irp.dynamic:
                ir = x_t.abs().max(dim=-1, keepdim=True)[0]
            else:
                if training:
                    update_input_range_from_data(
                        x_t.detach(), t, irp, input_range, input_range_update_idx
                    )
                ir = input_range[t]
                upper, lower = x_t >= ir, x_t <= -ir
                x_t = _SteClamp.apply(x_t, upper, lower, ir)
                x_t = _RangeGrad.apply(x_t, ir, upper, lower, irp.decay, irp.input_min_percentage)
        if fwd.inp_res > 0:
            x_t = _SteQuant.apply(x_t, fwd.inp_res, ir)
        w_t = weights[:, lo : lo + size]
        amax_rows = w_t.abs().amax(dim=-1, keepdim=True)
        if training and noise_type != NOISE_NONE:
            with torch.no_grad():
                s = amax_rows.max() if noise_type == NOISE_ADD else amax_rows
                w_noise = mod.std_dev * s * torch.randn_like(w_t)
            w_t = w_t.clone() + w_noise
        out_t = x_t @ w_t.T
        if training and fwd.out_noise > 0:
            with torch.no_grad():
                s = amax_rows if fwd.out_noise_per_channel else amax_rows.max()
                s = s if s.numel() == 1 else s.view(-1, out_t.size(-1))
                o_noise = s * (fwd.out_noise / sqrt(n_tiles) * ir) * torch.randn_like(out_t)
            out_t = out_t + o_noise
        if fwd.out_bound > 0 or fwd.out_res > 0:
            with torch.no_grad():
                s = amax_rows if clip_type in (CLIP_GAUSS_PC, CLIP_LEARN_PC) else amax_rows.max()
                bound = (ir * fwd.out_bound) * s.view(1, -1)
            if fwd.out_res > 0:
                out_t = _SteQuant.apply(out_t, fwd.out_res, bound)
            if fwd.out_bound > 0:
                out_t = torch.clamp(out_t, min=-bound, max=bound)
        out = out + out_t
        lo += size
    return out + bias if bias is not None else out
