"""Forward + backward of the analog operator at the real layer shapes of the ResNet-32 configuration
(batch 256, ``max_input_size=256``, no ADC): the patch matrices of the stage-2 and stage-3
convolutions have few output channels and very many rows, which is where the CUDA-core weight
gradient splits its reduction over CTAs and keeps partial sums in the caller's scratch.  The
scratch is handed over with guard words behind it that must be intact afterwards, and the
gradients are compared with fp32 matrix products over the operands the forward saved."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

GUARD = 1 << 18  # floats behind the scratch (1 MiB)


@pytest.mark.parametrize("m,k,n,max_in", [
    (65536, 288, 32, 256),   # stage 2: T = 2 (2 x 144); the shape whose split counts once disagreed
    (65536, 144, 32, 256),   # stage 2, first convolution
    (16384, 576, 64, 256),   # stage 3: T = 3 (3 x 192)
    (16384, 288, 64, 256),
    (262144, 144, 16, 256),  # stage 1
])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_weight_gradient_partials_stay_inside_the_scratch(m, k, n, max_in, dtype):
    from aihwkit_lightning_b200 import _lib
    from aihwkit_lightning_b200.nn import functional as F
    from aihwkit_lightning_b200.nn.modules.base import split_sizes
    from aihwkit_lightning_b200.simulator.configs import TorchInferenceRPUConfig

    lib = _lib.load()
    rpu = TorchInferenceRPUConfig()
    rpu.mapping.max_input_size = max_in
    rpu.forward.inp_res = 254
    rpu.forward.out_noise = 0.0
    rpu.pre_post.input_range.enable = True
    rpu.pre_post.input_range.dynamic = True
    in_sizes = split_sizes(k, max_in)
    t = len(in_sizes)
    ends = _lib.tile_ends_array(in_sizes)
    gen = torch.Generator(device="cuda").manual_seed(m + k + n)
    x = torch.randn(m, k, device="cuda", generator=gen).to(dtype)
    w = (torch.rand(n, k, device="cuda", generator=gen) * 0.2 - 0.1).to(dtype)
    g = torch.randn(m, n, device="cuda", generator=gen).to(dtype)
    stream = torch.cuda.current_stream().cuda_stream

    desc = F.make_desc(rpu, m, k, n, t, dtype, True)
    desc.save_for_backward = 1
    fa = _lib.AlForwardArgs()
    out = torch.empty(m, n, device="cuda", dtype=dtype)
    xq = torch.empty_like(x)
    ir_rows = torch.empty(t, m, device="cuda", dtype=dtype)
    w_amax = torch.empty(t, n, device="cuda", dtype=dtype)
    w_tile_max = torch.empty(2 * t, device="cuda", dtype=torch.float32)
    fa.x, fa.w, fa.out, fa.tile_ends = x.data_ptr(), w.data_ptr(), out.data_ptr(), ends
    fa.xq, fa.ir_rows, fa.w_amax, fa.w_tile_max, fa.w_mod = (xq.data_ptr(), ir_rows.data_ptr(), w_amax.data_ptr(),
                                                            w_tile_max.data_ptr(), w.data_ptr())
    _lib.check(lib.al_forward(desc, fa, stream))

    need = lib.al_backward_scratch_floats(m, k, n, t)
    splits, rows = ctypes.c_int32(), ctypes.c_int32()
    _lib.check(lib.al_wgrad_split_plan(m, k, n, t, ctypes.byref(splits), ctypes.byref(rows)))
    if dtype == torch.float32:
        assert splits.value > 1  # these shapes are the ones that split
    arena = torch.full((need + GUARD,), float("nan"), device="cuda", dtype=torch.float32)
    arena[need:] = 12345.0
    ba = _lib.AlBackwardArgs()
    grad_x = torch.empty(m, k, device="cuda", dtype=dtype)
    grad_w = torch.empty(n, k, device="cuda", dtype=dtype)
    ba.grad_out, ba.xq, ba.w_mod, ba.ir_rows, ba.tile_ends = g.data_ptr(), xq.data_ptr(), w.data_ptr(), ir_rows.data_ptr(), ends
    ba.grad_x, ba.grad_w = grad_x.data_ptr(), grad_w.data_ptr()
    ba.reduce_scratch, ba.reduce_scratch_floats = arena.data_ptr(), need
    _lib.check(lib.al_backward(desc, ba, stream))
    torch.cuda.synchronize()

    assert bool((arena[need:] == 12345.0).all()), "the backward wrote behind its scratch buffer"
    want_w = g.float().t() @ xq.float()
    want_x = g.float() @ w.float()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert ((grad_w.float() - want_w).norm() / want_w.norm()).item() <= tol
    assert ((grad_x.float() - want_x).norm() / want_x.norm()).item() <= tol
    assert ((out.float() - xq.float() @ w.float().t()).norm() / out.float().norm()).item() <= tol


@pytest.mark.parametrize("m,k,n,max_in", [
    (65536, 288, 32, 256),   # T = 2, input gradient on the CUDA cores (fewer than 64 channels)
    (16384, 576, 64, 256),   # T = 3, all three GEMMs on the tensor cores
    (262144, 144, 16, 256),  # one output block, 296 copies of it over the batch rows
])
def test_tensor_core_weight_gradient_split_stays_inside_the_scratch(m, k, n, max_in):
    """The same layer shapes in fp32 with the bf16-plane workspaces given: forward and weight gradient run
    on the tcgen05 kernels, and the weight gradient splits its reduction over CTAs into the caller's scratch."""
    from aihwkit_lightning_b200 import _lib
    from aihwkit_lightning_b200.nn import functional as F
    from aihwkit_lightning_b200.nn.modules.base import split_sizes
    from aihwkit_lightning_b200.simulator.configs import TorchInferenceRPUConfig

    lib = _lib.load()
    rpu = TorchInferenceRPUConfig()
    rpu.mapping.max_input_size = max_in
    rpu.forward.inp_res = 254
    rpu.forward.out_noise = 0.0
    rpu.pre_post.input_range.enable = True
    rpu.pre_post.input_range.dynamic = True
    in_sizes = split_sizes(k, max_in)
    t = len(in_sizes)
    ends = _lib.tile_ends_array(in_sizes)
    dtype = torch.float32
    gen = torch.Generator(device="cuda").manual_seed(m + k + n)
    x = torch.randn(m, k, device="cuda", generator=gen)
    w = torch.rand(n, k, device="cuda", generator=gen) * 0.2 - 0.1
    g = torch.randn(m, n, device="cuda", generator=gen)
    stream = torch.cuda.current_stream().cuda_stream

    desc = F.make_desc(rpu, m, k, n, t, dtype, True)
    desc.save_for_backward = 1
    assert lib.al_uses_tcgen05(desc, ends)
    fa = _lib.AlForwardArgs()
    out = torch.empty(m, n, device="cuda")
    xq = torch.empty_like(x)
    ir_rows = torch.empty(t, m, device="cuda")
    w_amax = torch.empty(t, n, device="cuda")
    w_tile_max = torch.empty(2 * t, device="cuda")
    codes16 = torch.empty(m, k, device="cuda", dtype=torch.bfloat16)
    w_planes = torch.empty(lib.al_f32_planes(), n, k, device="cuda", dtype=torch.bfloat16)
    fa.x, fa.w, fa.out, fa.tile_ends = x.data_ptr(), w.data_ptr(), out.data_ptr(), ends
    fa.xq, fa.ir_rows, fa.w_amax, fa.w_tile_max, fa.w_mod = (xq.data_ptr(), ir_rows.data_ptr(), w_amax.data_ptr(),
                                                            w_tile_max.data_ptr(), w.data_ptr())
    fa.codes16, fa.w_planes = codes16.data_ptr(), w_planes.data_ptr()
    _lib.check(lib.al_forward(desc, fa, stream))

    need = lib.al_backward_scratch_floats(m, k, n, t)
    splits, rows = ctypes.c_int32(), ctypes.c_int32()
    _lib.check(lib.al_wgrad_split_plan(m, k, n, t, ctypes.byref(splits), ctypes.byref(rows)))
    assert splits.value > 1
    arena = torch.full((need + GUARD,), float("nan"), device="cuda", dtype=torch.float32)
    arena[need:] = 12345.0
    g_planes = torch.empty(lib.al_backward_plane_elems(desc, ends), device="cuda", dtype=torch.bfloat16)
    ba = _lib.AlBackwardArgs()
    grad_x = torch.empty(m, k, device="cuda")
    grad_w = torch.empty(n, k, device="cuda")
    ba.grad_out, ba.xq, ba.w_mod, ba.ir_rows, ba.tile_ends = g.data_ptr(), xq.data_ptr(), w.data_ptr(), ir_rows.data_ptr(), ends
    ba.codes16, ba.w_planes, ba.g_planes, ba.g_planes_elems = (codes16.data_ptr(), w_planes.data_ptr(), g_planes.data_ptr(),
                                                              g_planes.numel())
    ba.grad_x, ba.grad_w = grad_x.data_ptr(), grad_w.data_ptr()
    ba.reduce_scratch, ba.reduce_scratch_floats = arena.data_ptr(), need
    _lib.check(lib.al_backward(desc, ba, stream))
    torch.cuda.synchronize()

    assert bool((arena[need:] == 12345.0).all()), "the backward wrote behind its scratch buffer"
    # the codes the GEMMs multiplied are the quantised inputs divided by their steps
    want_w = g.t() @ xq
    want_x = g @ w
    assert ((grad_w - want_w).norm() / want_w.norm()).item() <= 1e-5
    assert ((grad_x - want_x).norm() / want_x.norm()).item() <= 1e-5
    assert ((out - xq @ w.t()).norm() / out.norm()).item() <= 1e-5

    # a scratch buffer that is too small for the copies is refused on the host
    ba.reduce_scratch_floats = need - 1
    assert lib.al_backward(desc, ba, stream) == _lib.AL_ERR_BAD_ARGUMENT


@pytest.mark.parametrize("cin,cout,size,batch", [(16, 32, 32, 64), (32, 32, 16, 64)],
                         ids=["one-tile-144", "two-tiles-288"])
def test_conv2d_on_the_tensor_cores_matches_the_cuda_core_route(cin, cout, size, batch):
    """An fp32 convolution with enough patches runs its forward and weight gradient on the tcgen05
    kernels (patch extraction writes bf16 codes); same results as the CUDA-core engine within 1e-5."""
    from aihwkit_lightning_b200.nn import AnalogConv2d
    from aihwkit_lightning_b200.nn import functional as F
    from aihwkit_lightning_b200.simulator.configs import TorchInferenceRPUConfig

    rpu = TorchInferenceRPUConfig()
    rpu.mapping.max_input_size = 256
    rpu.forward.inp_res = 254
    rpu.forward.out_noise = 0.0
    rpu.pre_post.input_range.enable = True
    rpu.pre_post.input_range.dynamic = True
    torch.manual_seed(0)
    conv = AnalogConv2d(cin, cout, 3, padding=1, bias=True, rpu_config=rpu).cuda().train()
    x = torch.randn(batch, cin, size, size, device="cuda")  # batch * size^2 patches of 9 cin
    g = torch.randn(batch, cout, size, size, device="cuda")
    results = {}
    for engine in ("auto", "simt"):
        xin = x.clone().requires_grad_(True)
        conv.zero_grad(set_to_none=True)
        with F.operator_settings(engine=engine):
            out = conv(xin)
            out.backward(g)
        results[engine] = (out.detach(), xin.grad, conv.weight.grad.clone(), conv.bias.grad.clone())
    from aihwkit_lightning_b200 import _lib
    desc = F.make_desc(rpu, batch * size * size, 9 * cin, cout, len(conv.in_sizes), torch.float32, True)
    assert _lib.load().al_uses_tcgen05(desc, _lib.tile_ends_array(conv.in_sizes))
    for got, want in zip(results["auto"], results["simt"]):
        assert ((got - want).norm() / want.norm()).item() <= 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("cin,size,stride,max_in,batch,pad", [
    (16, 32, 1, 256, 3, 1),    # 144-element patches, one tile, 1152 groups of 4 per output row (kept in registers)
    (32, 16, 1, 256, 3, 1),    # two tiles of 144
    (64, 8, 1, 256, 5, 1),     # three tiles of 192
    (32, 32, 2, 256, 2, 1),    # strided
    (16, 64, 1, 256, 2, 1),    # 2304 groups per output row: gathered twice
    (16, 32, 1, 100, 2, 1),    # tiles of 72: whole groups, but four neighbouring groups may straddle two tiles
    (16, 30, 1, 256, 2, 1),    # image rows that are no multiple of 16 bytes: element-wise staging
    (16, 32, 1, 256, 2, 0),    # no padding
    (16, 32, 1, 256, 2, 2),    # two padding columns on either side
    (12, 20, 1, 256, 2, 1),    # 108-element patches
    (5, 20, 1, 256, 2, 1),     # 45-element patches: not a multiple of 4, the element-wise kernel
], ids=["c16", "c32-two-tiles", "c64-three-tiles", "stride2", "wide", "tiles-of-72", "odd-row-length", "no-padding",
        "padding-2", "patches-of-108", "ragged"])
def test_patch_extraction_with_the_dac_fused_is_bit_exact(dtype, cin, size, stride, max_in, batch, pad):
    """``al_unfold2d_dac`` writes the quantised patches, their integer codes as bf16 and the per-(tile, patch) ranges;
    all three equal, bit for bit, what the patch-extraction kernel followed by the stand-alone DAC of the linear
    layer produces (which the parity tests pin against the oracle)."""
    from aihwkit_lightning_b200 import _lib
    from aihwkit_lightning_b200.nn import AnalogLinear
    from aihwkit_lightning_b200.nn import functional as F
    from aihwkit_lightning_b200.simulator.configs import TorchInferenceRPUConfig

    rpu = TorchInferenceRPUConfig()
    rpu.mapping.max_input_size = max_in
    rpu.forward.inp_res = 254
    rpu.forward.out_noise = 0.0
    rpu.pre_post.input_range.enable = True
    rpu.pre_post.input_range.dynamic = True
    torch.manual_seed(5)
    x = (torch.randn(batch, cin, size, size, device="cuda") * 1.7).to(dtype)
    x[0, :, :5, :9] = 0.0       # patches that are zero throughout: range 0, step clamped to tiny
    x[1, 3, 7, 2] = 40.0        # an outlier that sets the range of the patches around it
    k = cin * 9
    patches = F.unfold2d(x, (3, 3), (1, 1), (pad, pad), (stride, stride)).reshape(-1, k)
    layer = AnalogLinear(k, 8, bias=False, rpu_config=rpu).to(device="cuda", dtype=dtype).eval()
    cap = {}
    with torch.no_grad(), F.operator_settings(capture=cap, engine="simt"):
        layer(patches)
    rows, t = patches.shape[0], len(layer.in_sizes)
    xq = torch.empty(rows, k, device="cuda", dtype=dtype)
    codes16 = torch.empty(rows, k, device="cuda", dtype=torch.bfloat16)
    ir_rows = torch.empty(t, rows, device="cuda", dtype=dtype)
    lib = _lib.load()
    geom = (batch, cin, size, size, 3, 3, stride, stride, pad, pad, 1, 1)
    ends = _lib.tile_ends_array(layer.in_sizes)
    stream = torch.cuda.current_stream().cuda_stream
    code = 1 if dtype == torch.bfloat16 else 0
    _lib.check(lib.al_unfold2d_dac(code, x.data_ptr(), *geom, ends, t, 254.0, xq.data_ptr(), ir_rows.data_ptr(),
                                   codes16.data_ptr(), stream))
    torch.cuda.synchronize()
    assert torch.equal(ir_rows, cap["ir_rows"].reshape(t, rows))
    assert torch.equal(xq, cap["xq"].reshape(rows, k))
    assert torch.equal(codes16.float(), cap["codes"].reshape(rows, k).float())
    # one output at a time gives the same bytes (the tensor-core route asks for the codes alone)
    only_codes = torch.zeros_like(codes16)
    _lib.check(lib.al_unfold2d_dac(code, x.data_ptr(), *geom, ends, t, 254.0, None, ir_rows.data_ptr(),
                                   only_codes.data_ptr(), stream))
    only_xq = torch.zeros_like(xq)
    _lib.check(lib.al_unfold2d_dac(code, x.data_ptr(), *geom, ends, t, 254.0, only_xq.data_ptr(), ir_rows.data_ptr(),
                                   None, stream))
    torch.cuda.synchronize()
    assert torch.equal(only_codes, codes16) and torch.equal(only_xq, xq)


@pytest.mark.parametrize("cin,cout,size,batch,ksize,pad", [
    (16, 16, 32, 8, 3, 1),      # bands of 8 rows, 4 pixels x 8 channels per thread
    (16, 16, 32, 224, 3, 1),    # the ResNet-32 stage-1 shape
    (8, 8, 6, 2, 3, 1),         # fewer than 8 rows: bands of 4, 2 pixels per thread
    (32, 32, 16, 64, 3, 1),     # 16 columns: a warp spans two rows; weights beyond 48 KB of shared memory
    (16, 32, 32, 4, 3, 1),
    (8, 12, 20, 3, 3, 1),       # a row length that does not divide 32
    (4, 4, 9, 2, 3, 0),         # no padding, a last band with a single row, 4 channels per thread
    (8, 8, 12, 2, 5, 2),        # 5 x 5 taps
    (64, 32, 8, 16, 3, 1),      # 64 input channels
], ids=["c16", "c16-batch-224", "h6", "c32-w16", "n32", "w20", "h9-no-padding", "taps-5x5", "c64"])
def test_direct_input_gradient_of_a_convolution_matches_the_patch_route(cin, cout, size, batch, ksize, pad):
    """fp32 convolutions with fewer than 64 output channels and no ADC compute their input gradient straight from
    the output gradient (``al_conv2d_input_grad``): same values as patch gradient + fold, and as the autograd of a
    float64 convolution with the same weights."""
    from aihwkit_lightning_b200.nn import AnalogConv2d
    from aihwkit_lightning_b200.nn import functional as F
    from aihwkit_lightning_b200.simulator.configs import TorchInferenceRPUConfig

    rpu = TorchInferenceRPUConfig()
    rpu.mapping.max_input_size = 256
    rpu.forward.inp_res = 254
    rpu.forward.out_noise = 0.0
    rpu.pre_post.input_range.enable = True
    rpu.pre_post.input_range.dynamic = True
    torch.manual_seed(1)
    conv = AnalogConv2d(cin, cout, ksize, padding=pad, bias=False, rpu_config=rpu).cuda().train()
    x = torch.randn(batch, cin, size, size, device="cuda")
    out_size = size + 2 * pad - ksize + 1
    g = torch.randn(batch, cout, out_size, out_size, device="cuda")
    lib = __import__("aihwkit_lightning_b200._lib", fromlist=["load"]).load()
    assert lib.al_conv2d_input_grad_supported(0, cout, batch, cin, size, size, ksize, ksize, 1, 1, pad, pad, 1, 1)
    grads = {}
    for direct in (True, False):
        xin = x.clone().requires_grad_(True)
        conv.zero_grad(set_to_none=True)
        with F.operator_settings(conv_direct_input_grad=direct):
            conv(xin).backward(g)
        grads[direct] = (xin.grad.clone(), conv.weight.grad.clone())
    assert ((grads[True][0] - grads[False][0]).norm() / grads[False][0].norm()).item() <= 1e-5
    assert torch.equal(grads[True][1], grads[False][1])   # the weight gradient does not depend on the route
    x64 = x.double().requires_grad_(True)
    w64 = conv.weight.detach().double().reshape(cout, cin, ksize, ksize)
    torch.nn.functional.conv2d(x64, w64, padding=pad).backward(g.double())
    assert ((grads[True][0].double() - x64.grad).norm() / x64.grad.norm()).item() <= 1e-5


def test_direct_input_gradient_is_refused_for_what_it_does_not_cover():
    from aihwkit_lightning_b200 import _lib
    lib = _lib.load()
    geom = (4, 16, 32, 32, 3, 3, 1, 1, 1, 1, 1, 1)
    assert lib.al_conv2d_input_grad_supported(0, 16, *geom) == 1
    assert lib.al_conv2d_input_grad_supported(1, 16, *geom) == 0                                   # bf16
    assert lib.al_conv2d_input_grad_supported(0, 16, 4, 16, 32, 32, 3, 3, 2, 2, 1, 1, 1, 1) == 0    # strided
    assert lib.al_conv2d_input_grad_supported(0, 16, 4, 16, 32, 32, 3, 3, 1, 1, 1, 1, 2, 2) == 0    # dilated
    assert lib.al_conv2d_input_grad_supported(0, 10, *geom) == 0                                   # N not a multiple of 4
    assert lib.al_conv2d_input_grad_supported(0, 16, 4, 3, 32, 32, 3, 3, 1, 1, 1, 1, 1, 1) == 0     # 3 input channels
    g = torch.zeros(4 * 16 * 16, 16, device="cuda")
    w = torch.zeros(16, 144, device="cuda")
    gx = torch.zeros(4, 16, 32, 32, device="cuda")
    status = lib.al_conv2d_input_grad(0, g.data_ptr(), w.data_ptr(), 16, 4, 16, 32, 32, 3, 3, 2, 2, 1, 1, 1, 1,
                                      gx.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert status == _lib.AL_ERR_UNSUPPORTED
