"""The analog linear operator: one ``torch.autograd.Function`` around the C-ABI calls.

It stands where the reference has ``TorchLinear.linear`` / ``TritonLinear.apply``
(`nn/modules/torch_utils/torch_linear.py:116-129`, `nn/modules/triton_utils/triton_linear.py:446-456`):
same arguments, same results, same in-place update of ``input_range`` /
``input_range_update_idx`` during the init-from-data phase.  PyTorch only supplies device
memory and the current stream here.
"""
from contextlib import contextmanager
from typing import List, Optional

import torch
from torch import Tensor

from .. import _lib
from ..exceptions import ConfigError
from ..simulator.enums import WeightClipType, WeightNoiseInjectionType, WeightQuantizationType

_NOISE = {
    WeightNoiseInjectionType.NONE: 0,
    WeightNoiseInjectionType.ADD_NORMAL: 1,
    WeightNoiseInjectionType.ADD_NORMAL_PER_CHANNEL: 2,
}
_QUANT = {
    WeightQuantizationType.NONE: 0,
    WeightQuantizationType.DISCRETIZE: 1,
    WeightQuantizationType.DISCRETIZE_PER_CHANNEL: 2,
}
_CLIP = {
    WeightClipType.NONE: 0,
    WeightClipType.LAYER_GAUSSIAN: 1,
    WeightClipType.LAYER_GAUSSIAN_PER_CHANNEL: 2,
    WeightClipType.LEARNABLE_PER_CHANNEL: 3,
}
_DTYPE = {torch.float32: _lib.AL_F32, torch.bfloat16: _lib.AL_BF16}
_ENGINE = {"auto": _lib.AL_ENGINE_AUTO, "simt": _lib.AL_ENGINE_SIMT, "tcgen05": _lib.AL_ENGINE_TCGEN05,
           "tcgen05_pair": _lib.AL_ENGINE_TCGEN05_PAIR, "tcgen05_single": _lib.AL_ENGINE_TCGEN05_SINGLE}


class _Settings:
    """Process-wide switches of the operator (debug and parity aids)."""

    engine = "auto"
    capture_codes = True       # with ``capture``: also ask for the integer DAC codes (debug output)
    reference_rounding = True  # bf16: round after every op like the reference's torch path
    no_rounding = False  # the reference's `_AIHWKIT_NO_ROUNDING` test switch (`quant_utils.py:60`)
    w_noise: Optional[Tensor] = None  # shared-noise parity mode: [N,K] standard normals
    out_noise: Optional[Tensor] = None  # [T,M,N] standard normals
    capture: Optional[dict] = None  # when a dict: filled with the intermediates of each call
    # callable(weight_grad) run inside backward as soon as the weight-gradient kernels are enqueued and
    # before the input-gradient ones (data-parallel training starts the gradient exchange there)
    after_wgrad = None
    # with ``after_wgrad``: SMs the GEMM that runs beside the exchange leaves unoccupied for it
    comm_sms = 0
    # with ``after_wgrad``: SMs the weight-gradient GEMM leaves unoccupied as well (for the exchanges of
    # the layers before it that are still in flight when it starts)
    comm_sms_wgrad = 0
    # callable(weight_address, shape, dtype) -> Tensor or None: where the backward writes a layer's weight
    # gradient (``distributed.PeerGradientSync`` hands out views of a buffer that all replicas have mapped,
    # so that the exchange kernel can reduce it in place); None: a fresh tensor
    grad_w_alloc = None
    # callable(std [T] float32 tensor) -> tensor: data-parallel training averages the per-tile standard
    # deviations of the init-from-data phase over the replicas here (``distributed.mean_over_replicas``),
    # so that every replica keeps the same input ranges
    sync_tile_std = None
    # a ``GraphNoise``: the calls draw their noise counters from it instead of torch's generator, so
    # that a training step can be captured in a CUDA graph and still see fresh noise on every replay
    graph_noise = None
    # fp32 convolutions with fewer than 64 output channels and no ADC compute their input gradient straight
    # from the output gradient (``al_conv2d_input_grad``) instead of a patch gradient that is folded afterwards
    conv_direct_input_grad = True


settings = _Settings()


class GraphNoise:
    """Noise counters for analog calls that are captured in a CUDA graph.

    A captured call replays with the arguments it was captured with, so a call counter passed by
    value would repeat the same noise on every replay.  With ``settings.graph_noise`` set, every call
    gets a distinct host-side offset (fixed at capture) plus the address of one counter in device
    memory that the noise kernels add to it; ``advance()`` (capturable itself, so it can be the first
    node of the graph) moves that counter on by 2**32 and with it every call's noise.

        noise = F.GraphNoise(device)
        F.settings.graph_noise = noise
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            noise.advance()
            loss = model(x).sum(); loss.backward(); optimizer.step()
        graph.replay()  # fresh noise each time
    """

    def __init__(self, device):
        device = torch.device(device)
        index = device.index if device.index is not None else torch.cuda.current_device()
        self.counter = torch.zeros(1, dtype=torch.int64, device=device)
        self.seed = torch.cuda.default_generators[index].initial_seed() & 0xFFFFFFFFFFFFFFFF
        self.calls = 0

    def advance(self) -> None:
        self.counter.add_(1 << 32)

    def next(self):
        offset = self.calls
        self.calls += 4
        return self.seed, offset


@contextmanager
def operator_settings(**kwargs):
    """Temporarily override fields of ``settings`` (engine, reference_rounding, no_rounding,
    w_noise, out_noise, capture)."""
    old = {k: getattr(settings, k) for k in kwargs}
    for k, v in kwargs.items():
        if not hasattr(_Settings, k):
            raise AttributeError(k)
        setattr(settings, k, v)
    try:
        yield settings
    finally:
        for k, v in old.items():
            setattr(settings, k, v)


def _ptr(t: Optional[Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)  # pylint: disable=protected-access


def _stream(device) -> int:
    """Handle of the current CUDA stream of ``device`` (the raw getter skips building a Stream object)."""
    if _raw_stream is not None:
        return _raw_stream(device.index if device.index is not None else torch.cuda.current_device())
    return torch.cuda.current_stream(device).cuda_stream


class _OnDevice:
    """``with torch.cuda.device(dev)`` that costs nothing when ``dev`` is already current."""

    __slots__ = ("guard",)

    def __init__(self, device):
        index = device.index
        self.guard = None if index is None or index == torch.cuda.current_device() else torch.cuda.device(device)

    def __enter__(self):
        if self.guard is not None:
            self.guard.__enter__()

    def __exit__(self, *exc):
        if self.guard is not None:
            self.guard.__exit__(*exc)
        return False


def _next_seed(device):
    """(seed, offset) from torch's CUDA generator so that ``torch.manual_seed`` governs the
    analog noise; advances the generator like a kernel drawing 4 values per thread would."""
    gen = torch.cuda.default_generators[device.index if device.index is not None else torch.cuda.current_device()]
    seed, offset = gen.initial_seed(), gen.get_offset()
    gen.set_offset(offset + 4)
    return seed & 0xFFFFFFFFFFFFFFFF, offset


_DESC_CACHE: dict = {}


def make_desc(rpu_config, m: int, k: int, n: int, t: int, dtype, training: bool) -> "_lib.AlDesc":
    """Flattened configuration of one call.  Descriptors are cached by VALUE of every field that
    goes into them (the configuration objects are mutable), and handed out as copies."""
    fwd, mod, clip = rpu_config.forward, rpu_config.modifier, rpu_config.clip
    irp = rpu_config.pre_post.input_range
    key = (m, k, n, t, dtype, training, irp.enable, irp.fast_mode, irp.dynamic, irp.init_from_data,
           irp.init_std_alpha, irp.decay, irp.input_min_percentage, irp.act_range_momentum, fwd.inp_res,
           fwd.out_res, fwd.out_bound, fwd.out_noise, fwd.out_noise_per_channel, mod.noise_type,
           mod.quantization_type, mod.std_dev, mod.res, clip.type, settings.no_rounding,
           settings.reference_rounding, settings.engine)
    cached = _DESC_CACHE.get(key)
    if cached is not None:
        return _lib.AlDesc.from_buffer_copy(cached)
    if len(_DESC_CACHE) > 4096:
        _DESC_CACHE.clear()
    d = _build_desc(rpu_config, m, k, n, t, dtype, training)
    _DESC_CACHE[key] = _lib.AlDesc.from_buffer_copy(d)
    return d


def _build_desc(rpu_config, m: int, k: int, n: int, t: int, dtype, training: bool) -> "_lib.AlDesc":
    fwd, mod, clip = rpu_config.forward, rpu_config.modifier, rpu_config.clip
    irp = rpu_config.pre_post.input_range
    if dtype not in _DTYPE:
        raise ConfigError(f"analog layers run in float32 or bfloat16, got {dtype}")
    d = _lib.AlDesc()
    d.M, d.K, d.N, d.T = m, k, n, t
    d.dtype = _DTYPE[dtype]
    d.training = int(training)
    if not irp.enable:
        d.ir_mode = _lib.AL_IR_OFF
    elif irp.fast_mode:
        d.ir_mode = _lib.AL_IR_FAST
    else:
        d.ir_mode = _lib.AL_IR_DYNAMIC if irp.dynamic else _lib.AL_IR_STATIC
    d.init_from_data = int(irp.init_from_data)
    d.init_std_alpha = float(irp.init_std_alpha)
    d.decay = float(irp.decay)
    d.input_min_percentage = float(irp.input_min_percentage)
    d.act_range_momentum = float(irp.act_range_momentum)
    d.inp_res = float(fwd.inp_res)
    d.out_res = float(fwd.out_res)
    d.out_bound = float(fwd.out_bound)
    d.out_noise = float(fwd.out_noise)
    d.out_noise_per_channel = int(bool(fwd.out_noise_per_channel))
    d.noise_type = _NOISE[mod.noise_type]
    d.quant_type = _QUANT[mod.quantization_type]
    d.std_dev = float(mod.std_dev)
    d.mod_res = float(mod.res)
    d.clip_type = _CLIP[clip.type]
    d.no_rounding = int(settings.no_rounding)
    d.ref_rounding = int(settings.reference_rounding)
    d.engine = _ENGINE[settings.engine]
    d.save_for_backward = 0
    return d


class _NoGradCtx:
    """Stands in for the autograd context when a call records nothing for a backward pass."""

    needs_input_grad = (False,) * 13

    def save_for_backward(self, *_):
        return None


class AnalogLinearFunction(torch.autograd.Function):
    """out = analog_linear(x, weight, bias) with the noisy / quantised tile model."""

    @staticmethod
    def forward(ctx, inp, weight, bias, input_range, input_range_update_idx, in_sizes, training,
                rpu_config, x_min=None, x_max=None, learnable_weight_clip=None,
                grad_enabled=True):  # type: ignore[override]
        return _analog_forward(ctx, inp, weight, bias, input_range, input_range_update_idx, in_sizes, training,
                               rpu_config, x_min, x_max, learnable_weight_clip, grad_enabled)

    @staticmethod
    def backward(ctx, grad_out):  # type: ignore[override]
        return _analog_backward(ctx, grad_out)


def _analog_forward(ctx, inp, weight, bias, input_range, input_range_update_idx, in_sizes, training,
                    rpu_config, x_min, x_max, learnable_weight_clip, grad_enabled, prequant=None):
    """One forward call of the library; ``ctx`` receives what the backward pass needs.
    ``prequant``: (xq [M,K], ir_rows [T,M]) when the DAC already ran (convolutions: fused into the patch
    extraction); ``inp`` is then ``xq`` itself."""
    lib = _lib.load()
    if not inp.is_cuda or not weight.is_cuda:
        raise ValueError(
            "analog layers of this package run on CUDA tensors only (no CPU fallback): "
            f"input on {inp.device}, weight on {weight.device}"
        )
    if inp.dtype != weight.dtype:
        raise RuntimeError(f"input dtype {inp.dtype} and weight dtype {weight.dtype} differ")
    n, k = weight.shape
    if prequant is None:
        if inp.shape[-1] != k:
            raise RuntimeError(f"input has {inp.shape[-1]} features, the layer expects {k}")
        x2d = inp.reshape(-1, k).contiguous()
        m = x2d.shape[0]
        pre_codes = None
    else:
        # (xq or None, ir_rows, codes16 or None, rows, patch length): the DAC already ran (``al_unfold2d_dac``)
        x2d, _, pre_codes, m, pre_k = prequant
        if pre_k != k:
            raise RuntimeError(f"patches have {pre_k} features, the layer expects {k}")
    w = weight.contiguous()
    t = len(in_sizes)
    dev, dtype = inp.device, inp.dtype
    # needs_input_grad mirrors requires_grad of the inputs even under torch.no_grad(); the
    # caller's grad mode arrives as an argument (inside forward it is always off)
    needs_grad = grad_enabled and (any(ctx.needs_input_grad[:4]) or ctx.needs_input_grad[10])
    desc = make_desc(rpu_config, m, k, n, t, dtype, training)
    desc.save_for_backward = int(needs_grad)
    ends = _lib.tile_ends_array(in_sizes)
    static = desc.ir_mode in (_lib.AL_IR_STATIC, _lib.AL_IR_FAST)  # one stored range per tile
    if static:
        assert input_range is not None, "Input range must be provided"
        assert input_range_update_idx is not None, "Input range update index must be provided"
    if m == 0:
        ctx.empty = True
        return inp.new_zeros(*inp.shape[:-1], n) + (bias if bias is not None else 0)
    ctx.empty = False

    with _OnDevice(dev):
        out = torch.empty(m, n, device=dev, dtype=dtype)
        args = _lib.AlForwardArgs()
        args.x, args.w, args.bias, args.out = _ptr(x2d), _ptr(w), _ptr(bias), _ptr(out)
        if prequant is not None:
            args.x, args.x_prequantised = None, (2 if pre_codes is not None else 1)
        args.tile_ends = ends
        ir_data = iridx_data = None
        if static:
            ir_data = input_range.data if input_range.is_contiguous() else input_range.data.contiguous()
            iridx_data = input_range_update_idx
            args.input_range, args.input_range_update_idx = _ptr(ir_data), _ptr(iridx_data)
            if desc.ir_mode == _lib.AL_IR_FAST:
                assert x_min is not None and x_max is not None, "x_min and x_max must be provided"
                args.x_min, args.x_max = _ptr(x_min), _ptr(x_max)
        learn_clip = desc.clip_type == _CLIP[WeightClipType.LEARNABLE_PER_CHANNEL]
        lwc = None
        if learn_clip:
            assert learnable_weight_clip is not None, "learnable_weight_clip should not be None"
            assert tuple(learnable_weight_clip.shape) == (t, n), f"learnable_weight_clip.shape must be ({t}, {n})"
            lwc = learnable_weight_clip.detach().to(dtype).contiguous()
            args.learnable_weight_clip = _ptr(lwc)
        modifies = desc.quant_type != 0 or (training and desc.noise_type != 0) or learn_clip
        need_std = static and training and desc.init_from_data > 0
        few_rows = m <= 16 and not needs_grad and dtype == torch.bfloat16 and settings.capture is None
        xq = x2d
        ir_rows = w_amax = w_tile_max = keep_mask = None
        w_mod = w
        # fp32 layer on the tensor cores: the GEMMs read the DAC codes and the weights as bf16 planes
        planes = dtype == torch.float32 and bool(lib.al_uses_tcgen05(desc, ends))
        codes16 = w_planes = None
        if not needs_grad and settings.capture is None:
            # nothing of the workspace outlives the call: one allocation, carved by offset
            es = w.element_size()
            plan = [("w_amax", t * n * es), ("w_tile_max", 2 * t * 4)]
            if desc.ir_mode != _lib.AL_IR_OFF and prequant is None:
                plan += [("xq", m * k * es), ("ir_rows", (t if static else t * m) * es)]
            if modifies:
                plan.append(("w_mod", n * k * es))
            if need_std:
                plan.append(("std_scratch", lib.al_std_scratch_floats(m, t) * 4))
            if few_rows:
                plan.append(("smallm_scratch", lib.al_smallm_scratch_floats(m, n, t) * 4))
            if planes:
                plan.append(("w_planes", lib.al_f32_planes() * n * k * 2))
                if pre_codes is None:
                    plan.append(("codes16", m * k * 2))
            total = 0
            for _, nbytes in plan:
                total += (nbytes + 255) & ~255
            arena = torch.empty(total, device=dev, dtype=torch.uint8)
            cursor = arena.data_ptr()
            args.xq, args.w_mod = _ptr(x2d), _ptr(w)
            for field, nbytes in plan:
                setattr(args, field, cursor)
                cursor += (nbytes + 255) & ~255
            if prequant is not None:
                args.xq, args.ir_rows, args.codes16 = _ptr(prequant[0]), _ptr(prequant[1]), _ptr(pre_codes)
        else:
            if prequant is not None:
                xq, ir_rows = prequant[0], prequant[1]
            elif desc.ir_mode != _lib.AL_IR_OFF:
                xq = torch.empty_like(x2d)
                ir_rows = torch.empty((t, m) if not static else (t,), device=dev, dtype=dtype)
            args.xq, args.ir_rows = _ptr(xq), _ptr(ir_rows)
            w_amax = torch.empty(t, n, device=dev, dtype=dtype)
            w_tile_max = torch.empty(2 * t, device=dev, dtype=torch.float32)
            args.w_amax, args.w_tile_max = _ptr(w_amax), _ptr(w_tile_max)
            w_mod = torch.empty_like(w) if modifies else w
            args.w_mod = _ptr(w_mod)
            if desc.out_bound > 0 and needs_grad:
                keep_mask = torch.empty(t, (n + 31) // 32, m, device=dev, dtype=torch.int32)
            args.keep_mask = _ptr(keep_mask)
            std_scratch = None
            if need_std:
                std_scratch = torch.empty(lib.al_std_scratch_floats(m, t), device=dev, dtype=torch.float32)
            args.std_scratch = _ptr(std_scratch)
            smallm_scratch = None
            if few_rows:
                smallm_scratch = torch.empty(lib.al_smallm_scratch_floats(m, n, t), device=dev, dtype=torch.float32)
            args.smallm_scratch = _ptr(smallm_scratch)
            if planes:
                codes16 = pre_codes if pre_codes is not None else torch.empty(m, k, device=dev, dtype=torch.bfloat16)
                w_planes = torch.empty(lib.al_f32_planes(), n, k, device=dev, dtype=torch.bfloat16)
                args.codes16, args.w_planes = _ptr(codes16), _ptr(w_planes)
        std_shared = None
        if need_std and desc.ir_mode == _lib.AL_IR_STATIC and settings.sync_tile_std is not None:
            std_shared = settings.sync_tile_std(sliced_std(in_sizes, x2d)).to(torch.float32).contiguous()
            args.std_override = _ptr(std_shared)
        w_noise, out_noise = settings.w_noise, settings.out_noise
        if w_noise is not None:
            w_noise = w_noise.to(device=dev, dtype=dtype).contiguous()
            assert w_noise.shape == w.shape, "replayed weight noise must be [N,K]"
        if out_noise is not None:
            out_noise = out_noise.to(device=dev, dtype=dtype).contiguous()
            assert out_noise.numel() == t * m * n, "replayed output noise must be [T,M,N]"
        args.w_noise, args.out_noise = _ptr(w_noise), _ptr(out_noise)
        codes = None
        if settings.capture is not None and settings.capture_codes and desc.ir_mode != _lib.AL_IR_OFF:
            codes = torch.empty_like(x2d)
        args.codes = _ptr(codes)
        if training and (desc.noise_type != 0 or desc.out_noise > 0):
            if settings.graph_noise is not None:
                args.seed, args.offset = settings.graph_noise.next()
                args.offset_base = settings.graph_noise.counter.data_ptr()
            else:
                args.seed, args.offset = _next_seed(dev)
        _lib.check(lib.al_forward(desc, args, _stream(dev)))
        if static and ir_data is not input_range.data:
            input_range.data.copy_(ir_data)

    if settings.capture is not None:
        settings.capture.update(
            codes=codes, xq=xq, ir_rows=ir_rows, w_amax=w_amax, w_tile_max=w_tile_max[:t],
            w_mod=w_mod, keep_mask=keep_mask,
            uses_tcgen05=bool(lib.al_uses_tcgen05(desc, ends)),
        )
    ctx.desc, ctx.in_sizes, ctx.dtype = desc, list(in_sizes), dtype
    ctx.weight_address = weight.data_ptr()
    ctx.shape = tuple(inp.shape) if prequant is None else (m, k)
    ctx.has_bias = bias is not None
    ctx.ir_needs_grad = static and input_range is not None and input_range.requires_grad
    ctx.learn_clip = learn_clip
    if needs_grad:
        # with bf16 planes the backward GEMMs read those: the fp32 copies need not be kept, except the (small)
        # modified weights of a layer with fewer than 64 channels, whose input gradient runs on the CUDA cores
        ctx.save_for_backward(x2d if static else None, None if planes else xq,
                              None if (planes and n >= 64) else w_mod, ir_rows,
                              keep_mask, w if learn_clip else None, lwc, codes16, w_planes)
    return out.view(*inp.shape[:-1], n) if prequant is None else out


def _analog_backward(ctx, grad_out, skip_input_grad=False):
    """The matching backward call: gradients of input, weight, bias, input range and weight ranges.
    ``skip_input_grad``: the caller computes the input gradient itself (a convolution that never forms the
    patch gradient)."""
    if ctx.empty:
        return (None,) * 12
    lib = _lib.load()
    x2d, xq, w_mod, ir_rows, keep_mask, w_saved, lwc, codes16, w_planes = ctx.saved_tensors
    desc = ctx.desc
    m, k, n, t = desc.M, desc.K, desc.N, desc.T
    dev, dtype = grad_out.device, ctx.dtype
    g = grad_out.reshape(m, n).to(dtype).contiguous()
    need_x, need_w, need_b, need_ir = ctx.needs_input_grad[:4]
    need_x = need_x and not skip_input_grad
    need_b = need_b and ctx.has_bias
    need_ir = need_ir and ctx.ir_needs_grad
    need_clip = ctx.learn_clip and (ctx.needs_input_grad[10] or need_w)
    need_w = need_w or need_clip
    with _OnDevice(dev):
        args = _lib.AlBackwardArgs()
        ends = _lib.tile_ends_array(ctx.in_sizes)
        args.tile_ends = ends
        args.grad_out, args.x, args.xq, args.w_mod = _ptr(g), _ptr(x2d), _ptr(xq), _ptr(w_mod)
        args.ir_rows, args.keep_mask = _ptr(ir_rows), _ptr(keep_mask)
        grad_x = torch.empty(m, k, device=dev, dtype=dtype) if (need_x or need_ir) else None
        grad_w = None
        if need_w:
            if settings.grad_w_alloc is not None and ctx.needs_input_grad[1] and not need_clip:
                grad_w = settings.grad_w_alloc(ctx.weight_address, (n, k), dtype)
            if grad_w is None:
                grad_w = torch.empty(n, k, device=dev, dtype=dtype)
        grad_b = torch.empty(n, device=dev, dtype=dtype) if need_b else None
        grad_ir = torch.empty(t, device=dev, dtype=dtype) if need_ir else None
        scratch = torch.empty(lib.al_backward_scratch_floats(m, k, n, t), device=dev, dtype=torch.float32)
        args.grad_x, args.grad_w, args.grad_bias = _ptr(grad_x), _ptr(grad_w), _ptr(grad_b)
        args.grad_input_range, args.reduce_scratch = _ptr(grad_ir), _ptr(scratch)
        args.reduce_scratch_floats = scratch.numel()
        g_planes = None
        if codes16 is not None:
            g_planes = torch.empty(lib.al_backward_plane_elems(desc, ends), device=dev, dtype=torch.bfloat16)
            args.codes16, args.w_planes, args.g_planes = _ptr(codes16), _ptr(w_planes), _ptr(g_planes)
            args.g_planes_elems = g_planes.numel()
        grad_clip = None
        if need_clip:
            grad_clip = torch.empty(t, n, device=dev, dtype=dtype)
            args.w, args.learnable_weight_clip = _ptr(w_saved), _ptr(lwc)
            args.grad_weight_clip = _ptr(grad_clip)
        hook = settings.after_wgrad
        if hook is not None and grad_w is not None and grad_x is not None:
            # weight-side gradients first: their exchange between replicas can then run while the
            # input gradient is still being computed
            args.grad_x = args.grad_input_range = None
            if settings.comm_sms_wgrad > 0:
                lib.al_reserve_sms(int(settings.comm_sms_wgrad))
                try:
                    _lib.check(lib.al_backward(desc, args, _stream(dev)))
                finally:
                    lib.al_reserve_sms(0)
            else:
                _lib.check(lib.al_backward(desc, args, _stream(dev)))
            hook(grad_w)
            args.grad_x, args.grad_input_range = _ptr(grad_x), _ptr(grad_ir)
            args.grad_w = args.grad_bias = args.grad_weight_clip = None
            if settings.comm_sms > 0:
                lib.al_reserve_sms(int(settings.comm_sms))
                try:
                    _lib.check(lib.al_backward(desc, args, _stream(dev)))
                finally:
                    lib.al_reserve_sms(0)
            else:
                _lib.check(lib.al_backward(desc, args, _stream(dev)))
        else:
            _lib.check(lib.al_backward(desc, args, _stream(dev)))
            if hook is not None and grad_w is not None:
                hook(grad_w)
    if grad_x is not None:
        grad_x = grad_x.view(ctx.shape) if need_x else None
    if not ctx.needs_input_grad[1]:
        grad_w = None
    if not ctx.needs_input_grad[10]:
        grad_clip = None
    return grad_x, grad_w, grad_b, grad_ir, None, None, None, None, None, None, grad_clip, None


def analog_linear(inp: Tensor, weight: Tensor, bias: Optional[Tensor], input_range: Optional[Tensor],
                  input_range_update_idx: Optional[Tensor], in_sizes: List[int], training: bool,
                  rpu_config, x_min: Optional[Tensor] = None, x_max: Optional[Tensor] = None,
                  learnable_weight_clip: Optional[Tensor] = None) -> Tensor:
    """Functional form used by ``AnalogLinear`` and ``AnalogConv2d``."""
    grad = torch.is_grad_enabled()
    if not grad or not (inp.requires_grad or weight.requires_grad
                        or (bias is not None and bias.requires_grad)
                        or (input_range is not None and input_range.requires_grad)
                        or (learnable_weight_clip is not None and learnable_weight_clip.requires_grad)):
        # nothing to differentiate: skip the autograd machinery altogether
        return _analog_forward(_NoGradCtx(), inp, weight, bias, input_range, input_range_update_idx, in_sizes,
                               training, rpu_config, x_min, x_max, learnable_weight_clip, False)
    return AnalogLinearFunction.apply(inp, weight, bias, input_range, input_range_update_idx,
                                      in_sizes, training, rpu_config, x_min, x_max, learnable_weight_clip,
                                      torch.is_grad_enabled())


def sliced_abs_max(in_sizes: List[int], weights: Tensor) -> Tensor:
    """Per-tile, per-row abs-max ``[T, rows]`` of a 2-D CUDA tensor
    (`nn/modules/torch_utils/torch_abs_max.py:17-39`)."""
    lib = _lib.load()
    assert weights.ndim == 2, "Weight must be 2D"
    if not weights.is_cuda:
        raise ValueError("sliced_abs_max runs on CUDA tensors only")
    w = weights.detach().contiguous()
    out = torch.empty(len(in_sizes), w.shape[0], device=w.device, dtype=w.dtype)
    with _OnDevice(w.device):
        _lib.check(lib.al_abs_max_tiles(_DTYPE[w.dtype], w.data_ptr(), w.shape[0], w.shape[1],
                                        _lib.tile_ends_array(in_sizes), len(in_sizes), out.data_ptr(),
                                        _stream(w.device)))
    return out


def sliced_std(in_sizes: List[int], values: Tensor) -> Tensor:
    """Per-tile unbiased std over all rows ``[T]`` (float32) of a 2-D CUDA tensor."""
    lib = _lib.load()
    assert values.ndim == 2, "values must be 2D"
    v = values.detach().contiguous()
    t = len(in_sizes)
    out = torch.empty(t, device=v.device, dtype=torch.float32)
    scratch = torch.empty(lib.al_std_scratch_floats(v.shape[0], t), device=v.device, dtype=torch.float32)
    with _OnDevice(v.device):
        _lib.check(lib.al_std_tiles(_DTYPE[v.dtype], v.data_ptr(), v.shape[0], v.shape[1],
                                    _lib.tile_ends_array(in_sizes), t, out.data_ptr(), scratch.data_ptr(),
                                    _stream(v.device)))
    return out


def clip_weights_(weight: Tensor, clip_type: WeightClipType, sigma: float) -> None:
    """In-place Gaussian weight clipping of a CUDA parameter (`nn/modules/linear.py:269-283`)."""
    if clip_type in (WeightClipType.NONE, WeightClipType.LEARNABLE_PER_CHANNEL):
        return
    assert sigma > 0, "Clip sigma must be greater than 0"
    if clip_type not in (WeightClipType.LAYER_GAUSSIAN, WeightClipType.LAYER_GAUSSIAN_PER_CHANNEL):
        raise ValueError(f"Unknown clip type {clip_type}")
    lib = _lib.load()
    if not weight.is_cuda:
        raise ValueError("clip_weights runs on CUDA tensors only")
    w = weight.data
    assert w.is_contiguous(), "weight must be contiguous"
    rows = w.shape[0]
    cols = w.numel() // rows
    scratch = torch.empty(2 * rows + 8, device=w.device, dtype=torch.float32)
    with _OnDevice(w.device):
        _lib.check(lib.al_clip_weights(_DTYPE[w.dtype], w.data_ptr(), rows, cols, _CLIP[clip_type],
                                       float(sigma), scratch.data_ptr(), _stream(w.device)))


class Unfold2dFunction(torch.autograd.Function):
    """Patch matrix ``[B, L, C*kh*kw]`` of a ``[B, C, H, W]`` CUDA tensor; the same values as
    ``unfold(x, ...).transpose(-1, -2).contiguous()`` in the reference's conv forward
    (`nn/modules/conv.py:312-322`), produced and differentiated by the library's kernels."""

    @staticmethod
    def forward(ctx, x, kernel_size, dilation, padding, stride):  # type: ignore[override]
        lib = _lib.load()
        if not x.is_cuda:
            raise ValueError("analog convolutions of this package run on CUDA tensors only")
        if x.dtype not in _DTYPE:
            raise ConfigError(f"analog layers run in float32 or bfloat16, got {x.dtype}")
        xc = x.contiguous()
        b, c, h, w = xc.shape
        (kh, kw), (dh, dw), (ph, pw), (sh, sw) = kernel_size, dilation, padding, stride
        ho = (h + 2 * ph - dh * (kh - 1) - 1) // sh + 1
        wo = (w + 2 * pw - dw * (kw - 1) - 1) // sw + 1
        out = torch.empty(b, max(ho, 0) * max(wo, 0), c * kh * kw, device=x.device, dtype=x.dtype)
        geom = (b, c, h, w, kh, kw, sh, sw, ph, pw, dh, dw)
        with _OnDevice(x.device):
            _lib.check(lib.al_unfold2d(_DTYPE[x.dtype], xc.data_ptr(), *geom, out.data_ptr(), _stream(x.device)))
        ctx.geom, ctx.dtype_code = geom, _DTYPE[x.dtype]
        return out

    @staticmethod
    def backward(ctx, grad_patches):  # type: ignore[override]
        lib = _lib.load()
        gp = grad_patches.contiguous()
        b, c, h, w = ctx.geom[:4]
        gx = torch.empty(b, c, h, w, device=gp.device, dtype=gp.dtype)
        with _OnDevice(gp.device):
            _lib.check(lib.al_fold2d(ctx.dtype_code, gp.data_ptr(), *ctx.geom, gx.data_ptr(), _stream(gp.device)))
        return gx, None, None, None, None


def _direct_input_grad_applies(ctx) -> bool:
    """Whether the input gradient of this convolution comes straight from ``grad_out`` and the modified weights
    (``al_conv2d_input_grad``) instead of the general route (patch gradient + fold).  Not with an ADC clamp
    mask, strides, bf16, fewer than 4 or at least 64 output channels (from 64 on the patch gradient is a
    tensor-core GEMM)."""
    if ctx.empty or not ctx.needs_input_grad[0] or not settings.conv_direct_input_grad:
        return False
    w_mod, keep_mask = ctx.saved_tensors[2], ctx.saved_tensors[4]
    if w_mod is None or keep_mask is not None or ctx.dtype != torch.float32 or ctx.desc.N >= 64:
        return False
    if ctx.ir_needs_grad:
        return False
    return bool(_lib.load().al_conv2d_input_grad_supported(ctx.dtype_code, ctx.desc.N, *ctx.geom))


def _direct_input_grad(ctx, grad_out):
    lib = _lib.load()
    desc, w_mod = ctx.desc, ctx.saved_tensors[2]
    b, c, h, w = ctx.geom[:4]
    g = grad_out.reshape(desc.M, desc.N).to(ctx.dtype).contiguous()
    grad_img = torch.empty(b, c, h, w, device=g.device, dtype=g.dtype)
    with _OnDevice(g.device):
        _lib.check(lib.al_conv2d_input_grad(ctx.dtype_code, g.data_ptr(), w_mod.data_ptr(), desc.N, *ctx.geom,
                                            grad_img.data_ptr(), _stream(g.device)))
    return grad_img


class AnalogConv2dFunction(torch.autograd.Function):
    """Analog convolution with a dynamic input range as ONE operator: the patch extraction quantises on
    the way (``al_unfold2d_dac``), the tiled GEMM consumes the quantised patches, and the backward folds
    the patch gradients back into the image.  Same values as ``unfold2d`` followed by ``analog_linear``;
    the unquantised patch matrix is never written.  Returns ``[B * Ho * Wo, out_channels]``."""

    @staticmethod
    def forward(ctx, inp, weight, bias, input_range, input_range_update_idx, in_sizes, training, rpu_config,
                x_min, x_max, learnable_weight_clip, grad_enabled, geometry):  # type: ignore[override]
        lib = _lib.load()
        xc = inp.contiguous()
        b, c, h, w = xc.shape
        (kh, kw), (dh, dw), (ph, pw), (sh, sw) = geometry
        ho = (h + 2 * ph - dh * (kh - 1) - 1) // sh + 1
        wo = (w + 2 * pw - dw * (kw - 1) - 1) // sw + 1
        rows, t, k = b * ho * wo, len(in_sizes), c * kh * kw
        geom = (b, c, h, w, kh, kw, sh, sw, ph, pw, dh, dw)
        ends = _lib.tile_ends_array(in_sizes)
        with _OnDevice(xc.device):
            # an fp32 layer whose GEMMs run on the tensor cores takes the DAC codes as bf16 (half the bytes
            # of the quantised patch matrix, and its exact content: the GEMMs multiply codes, the step
            # comes in afterwards)
            desc = make_desc(rpu_config, rows, k, weight.shape[0], t, xc.dtype, training)
            as_codes = xc.dtype == torch.float32 and bool(lib.al_uses_tcgen05(desc, ends))
            xq = None if as_codes else torch.empty(rows, k, device=xc.device, dtype=xc.dtype)
            codes16 = torch.empty(rows, k, device=xc.device, dtype=torch.bfloat16) if as_codes else None
            ir_rows = torch.empty(t, rows, device=xc.device, dtype=xc.dtype)
            status = lib.al_unfold2d_dac(_DTYPE[xc.dtype], xc.data_ptr(), *geom, ends, t,
                                         float(rpu_config.forward.inp_res), _ptr(xq), ir_rows.data_ptr(), _ptr(codes16),
                                         _stream(xc.device))
        if status == _lib.AL_ERR_UNSUPPORTED:
            raise _PatchTooLarge()
        _lib.check(status)
        ctx.geom, ctx.dtype_code = geom, _DTYPE[xc.dtype]
        return _analog_forward(ctx, xc, weight, bias, input_range, input_range_update_idx, in_sizes, training,
                               rpu_config, x_min, x_max, learnable_weight_clip, grad_enabled,
                               prequant=(xq, ir_rows, codes16, rows, k))

    @staticmethod
    def backward(ctx, grad_out):  # type: ignore[override]
        direct = _direct_input_grad_applies(ctx)
        grads = _analog_backward(ctx, grad_out, skip_input_grad=direct)  # weight-side gradients first
        grad_img = _direct_input_grad(ctx, grad_out) if direct else None
        if grads[0] is not None:
            lib = _lib.load()
            gp = grads[0]
            b, c, h, w = ctx.geom[:4]
            grad_img = torch.empty(b, c, h, w, device=gp.device, dtype=gp.dtype)
            with _OnDevice(gp.device):
                _lib.check(lib.al_fold2d(ctx.dtype_code, gp.data_ptr(), *ctx.geom, grad_img.data_ptr(), _stream(gp.device)))
        return (grad_img,) + tuple(grads[1:]) + (None,)


class _PatchTooLarge(Exception):
    """The fused patch extraction cannot stage a whole patch: the caller takes the two-step route."""


def analog_conv2d_rows(inp: Tensor, weight2d: Tensor, bias, input_range, input_range_update_idx, in_sizes, training,
                       rpu_config, x_min, x_max, learnable_weight_clip, kernel_size, dilation, padding, stride):
    """``[B, C, H, W] -> [B * Ho * Wo, out_channels]`` (or ``[Ho * Wo, out]`` for a 3-D input): patches through the
    analog linear operator.  Dynamic input ranges with the DAC on take the fused operator."""
    irp = rpu_config.pre_post.input_range
    fused = (inp.dim() == 4 and inp.is_cuda and irp.enable and irp.dynamic and not irp.fast_mode
             and rpu_config.forward.inp_res > 0 and not settings.no_rounding and settings.capture is None
             and inp.dtype in _DTYPE and inp.shape[0] > 0)
    if fused:
        grad = torch.is_grad_enabled()
        geometry = (tuple(kernel_size), tuple(dilation), tuple(padding), tuple(stride))
        try:
            if not grad or not (inp.requires_grad or weight2d.requires_grad or (bias is not None and bias.requires_grad)):
                ctx = _NoGradCtx()
                return AnalogConv2dFunction.forward(ctx, inp, weight2d, bias, input_range, input_range_update_idx,
                                                    in_sizes, training, rpu_config, x_min, x_max, learnable_weight_clip,
                                                    False, geometry)
            return AnalogConv2dFunction.apply(inp, weight2d, bias, input_range, input_range_update_idx, in_sizes,
                                              training, rpu_config, x_min, x_max, learnable_weight_clip, grad, geometry)
        except _PatchTooLarge:
            pass
    patches = unfold2d(inp, kernel_size, dilation, padding, stride)
    out = analog_linear(patches, weight2d, bias, input_range, input_range_update_idx, in_sizes, training, rpu_config,
                        x_min, x_max, learnable_weight_clip)
    return out.reshape(-1, out.shape[-1])


def unfold2d(x: Tensor, kernel_size, dilation, padding, stride) -> Tensor:
    """``[B, C, H, W]`` (or ``[C, H, W]``) -> ``[B, L, C*kh*kw]`` (or ``[L, C*kh*kw]``)."""
    if x.dim() == 3:
        return Unfold2dFunction.apply(x.unsqueeze(0), kernel_size, dilation, padding, stride).squeeze(0)
    return Unfold2dFunction.apply(x, kernel_size, dilation, padding, stride)
