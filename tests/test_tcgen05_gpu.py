"""The tcgen05/TMA engine against the CPU oracle and against the CUDA-core engine.

Shapes exercise full and partial 128-row / 128-column blocks, tile widths that are not a
multiple of the 64-element K step (zero-filled by TMA), several analog tiles, learned and
dynamic input ranges, replayed noise, ADC clamp masks in the backward GEMMs, and the plain
(no input range, no modifier) configuration.  After every run the device error word of the
kernels (a bounded wait that gave up) must be clear.
"""
import ctypes

import pytest
import torch

import cases as C
from util import frac_equal, oracle_run, rel_fro, run_product_layer

pytestmark = pytest.mark.gpu

BF16_REL = 1e-2

SHAPES = [
    # base case, overrides
    ("bf16_dynamic_adc_noise", dict(in_shape=(256, 1024), out_features=512, max_input_size=256)),
    ("bf16_dynamic_adc_noise", dict(in_shape=(200, 576), out_features=264, max_input_size=72)),
    ("bf16_dynamic_adc_noise", dict(in_shape=(3, 130, 512), out_features=128, max_input_size=-1,
                                    out_noise_per_channel=True, clip_type="LayerGaussianPerChannel", clip_sigma=2.5)),
    ("bf16_static_noise", dict(in_shape=(384, 768), out_features=256, max_input_size=256, ir_init_value=2.0)),
    ("bf16_static_adc", dict(in_shape=(130, 512), out_features=520, max_input_size=128, ir_init_value=2.0)),
    ("bf16_dynamic_eval", dict(in_shape=(512, 1024), out_features=384, max_input_size=512)),
    ("bf16_discretize", dict(in_shape=(128, 256), out_features=128, max_input_size=64)),
    ("bf16_static_noise", dict(in_shape=(64, 320), out_features=72, max_input_size=-1, ir_enable=False,
                               inp_res=-1.0, out_noise=0.0, noise_type="AddNormal", std_dev=0.02)),
    # a clamp that rarely fires and a long reduction on a single CTA: stages are reused by transform
    # warps that had nothing to zero on the previous use
    ("bf16_dynamic_adc_noise", dict(in_shape=(128, 256), out_features=768, max_input_size=128, out_bound=10.0)),
    ("bf16_dynamic_adc_noise", dict(in_shape=(128, 256), out_features=1024, max_input_size=128, out_bound=10.0,
                                    out_noise=0.0, noise_type="None")),
    # an all-zero input row: input range 0, DAC and ADC steps clamped to the smallest normal number
    ("bf16_dynamic_adc_noise", dict(in_shape=(256, 512), out_features=256, max_input_size=256, zero_row=3)),
    # heavy ADC clamping: most rows of the staged gradient blocks have many blocked entries
    ("bf16_dynamic_adc_noise", dict(in_shape=(384, 512), out_features=392, max_input_size=128, out_bound=0.3)),
    ("bf16_static_adc", dict(in_shape=(200, 512), out_features=264, max_input_size=256, ir_init_value=2.0,
                             out_bound=0.5)),
    # 80 blocks of 256 x 256 for both backward GEMMs: on 74 CTA pairs the last 6 blocks run as 12 half blocks
    # (masked operands)
    ("bf16_dynamic_adc_noise", dict(in_shape=(2560, 2048), out_features=2560, max_input_size=512)),
    # the same for the weight gradient without a clamp mask and with tiles that end inside a block (84 blocks)
    ("bf16_static_noise", dict(in_shape=(384, 2304), out_features=1792, max_input_size=384, ir_init_value=2.0)),
]


def device_error():
    from aihwkit_lightning_b200 import _lib

    lib = _lib.load()
    code = ctypes.c_uint32(0)
    status = lib.al_read_device_error(torch.cuda.current_stream().cuda_stream, ctypes.byref(code))
    return status, code.value


@pytest.mark.parametrize("base,over", SHAPES, ids=[f"{b}-{'x'.join(map(str, o['in_shape']))}x{o['out_features']}" for b, o in SHAPES])
@pytest.mark.parametrize("engine", ["tcgen05_single", "tcgen05_pair"])
def test_tcgen05_engine_matches_oracle_and_simt(base, over, engine):
    """``engine`` picks the backward GEMM kernel: single CTAs or CTA pairs (cta_group::2)."""
    case = dict(C.CASES_BY_NAME[base])
    case.update(over)
    case["weight_scale"] = 0.05
    data = C.make_inputs(case)
    rec, grads = oracle_run(case, data, w_noise=data["w_noise"][-1], out_noise=data["out_noise"][-1])
    cap = {}
    layer, x, out = run_product_layer(case, data, engine=engine, capture=cap)
    assert cap["uses_tcgen05"]
    assert device_error() == (0, 0)
    layer2, x2, out2 = run_product_layer(case, data, engine="simt")

    got = dict(out=out.detach(), grad_x=x.grad, grad_w=layer.weight.grad)
    simt = dict(out=out2.detach(), grad_x=x2.grad, grad_w=layer2.weight.grad)
    want = dict(out=rec.out, grad_x=grads["grad_x"], grad_w=grads["grad_w"])
    if case["bias"]:
        got["grad_bias"], simt["grad_bias"], want["grad_bias"] = layer.bias.grad, layer2.bias.grad, grads["grad_bias"]
    for key in got:
        assert torch.isfinite(got[key].float()).all(), key
        assert rel_fro(got[key], want[key]) <= BF16_REL, f"{key} vs oracle: {rel_fro(got[key], want[key]):.3e}"
        assert rel_fro(got[key], simt[key]) <= BF16_REL, f"{key} vs simt: {rel_fro(got[key], simt[key]):.3e}"
    # with the reference's rounding chain emulated the two engines and the oracle agree on
    # almost every bf16 value of the forward output
    assert frac_equal(got["out"], want["out"]) >= 0.95
    if over.get("out_bound", 10.0) < 1.0:
        blocked = sum(int(((tr.pre_clamp < -tr.bound) | (tr.pre_clamp > tr.bound)).sum()) for tr in rec.tiles)
        assert blocked > 0.05 * rec.out.numel() * len(rec.tiles), "this case is meant to clamp heavily"
    if grads["grad_ir"] is not None and case["ir_learn"]:
        a, b = layer.input_range.grad.float().cpu(), grads["grad_ir"].float()
        assert torch.allclose(a, b, rtol=3e-2, atol=1e-4)


def test_tcgen05_internal_noise_statistics():
    """Output noise drawn inside the tcgen05 epilogue: zero mean, std as configured."""
    import math

    from aihwkit_lightning_b200.nn import AnalogLinear
    from aihwkit_lightning_b200.nn import functional as F
    from util import NS

    case = dict(C.DEFAULTS)
    case.update(ir_dynamic=True, out_noise=0.1, max_input_size=128, inp_res=254.0)
    rpu = C.build_rpu_config(NS, case)
    torch.manual_seed(0)
    layer = AnalogLinear(256, 512, bias=False, rpu_config=rpu).to(device="cuda", dtype=torch.bfloat16)
    x = torch.randn(512, 256, device="cuda").bfloat16()
    with F.operator_settings(engine="tcgen05", reference_rounding=False):
        layer.eval()
        clean = layer(x).float()
        layer.train()
        noisy = layer(x).float()
    assert device_error() == (0, 0)
    delta = (noisy - clean).cpu()
    w, xs = layer.weight.detach().float().cpu(), x.float().cpu()
    var = torch.zeros(512)
    for t in range(2):
        wmax = w[:, 128 * t:128 * (t + 1)].abs().max()
        ir = xs[:, 128 * t:128 * (t + 1)].abs().amax(1)
        var += (wmax * 0.1 / math.sqrt(2) * ir) ** 2
    z = delta / var.sqrt()[:, None]
    assert abs(z.mean().item()) < 0.02
    assert abs(z.std().item() - 1.0) < 0.03


def _dyadic_problem(m, k, n, tile, seed=0):
    """Inputs for which every product and partial sum of the GEMM is exact in fp32, so that the
    result does not depend on the accumulation order: per (row, tile) the inputs are integers
    with abs-max exactly 127 (dynamic range -> DAC step exactly 1, codes = inputs), weights are
    multiples of 1/64 in [-1, 1]."""
    gen = torch.Generator().manual_seed(seed)
    x = torch.randint(-126, 127, (m, k), generator=gen).float()
    for t in range(k // tile):
        x[:, t * tile] = 127.0 * (1 - 2 * torch.randint(0, 2, (m,), generator=gen)).float()
    w = torch.randint(-64, 65, (n, k), generator=gen).float() / 64.0
    w[:, ::tile] = 1.0  # abs-max of every (channel, tile) exactly 1
    g = torch.randint(-8, 9, (m, n), generator=gen).float() / 8.0
    return x.bfloat16(), w.bfloat16(), g.bfloat16()


@pytest.mark.parametrize("variant", ["adc_noise", "noise_only", "adc_eval", "static_adc_noise"])
def test_order_independent_problem_is_bit_exact(variant):
    """With an order-independent GEMM the whole per-tile chain (bf16 rounding after every op,
    replayed noise, ADC division / rint / clamp, running sum) must equal the CPU oracle bit for
    bit on both engines, and the clamp masks must make the backward GEMMs agree exactly too."""
    from aihwkit_lightning_b200.nn import AnalogLinear
    from aihwkit_lightning_b200.nn import functional as F
    import analog_oracle as O
    from util import NS

    m, k, n, tile = 256, 512, 384, 128
    x, w, g = _dyadic_problem(m, k, n, tile)
    case = dict(C.DEFAULTS)
    case.update(dtype="bf16", max_input_size=tile, ir_dynamic=True, bias=False, inp_res=254.0)
    if variant in ("adc_noise", "static_adc_noise"):
        case.update(out_bound=12.0, out_res=254.0, out_noise=0.05)
    elif variant == "noise_only":
        case.update(out_noise=0.05)
    else:
        case.update(out_bound=12.0, out_res=254.0, training=False)
    if variant == "static_adc_noise":
        case.update(ir_dynamic=False, ir_init_value=127.0, ir_decay=0.0)
    rpu = C.build_rpu_config(NS, case)
    gen = torch.Generator().manual_seed(5)
    t_count = k // tile
    out_noise = torch.randn(t_count, m, n, generator=gen).bfloat16()
    in_sizes = [tile] * t_count
    ir = idx = None
    if not case["ir_dynamic"]:
        ir = torch.full((t_count,), 127.0, dtype=torch.bfloat16)
        idx = torch.zeros(t_count, dtype=torch.bfloat16)
    rec = O.forward(x, w, None, ir, idx, None, None, in_sizes, case["training"], rpu,
                    O.NoiseReplay(None, out_noise))
    grads = O.backward(rec, g, w, False, ir, rpu)
    clipped = sum(int(((tr.pre_clamp < -tr.bound) | (tr.pre_clamp > tr.bound)).sum()) for tr in rec.tiles
                  if tr.pre_clamp is not None)
    if case["out_bound"] > 0:
        assert clipped > 0, "the test problem should exercise the ADC clamp"
    for engine in ("tcgen05", "simt"):
        layer = AnalogLinear(k, n, bias=False, rpu_config=rpu).to(device="cuda", dtype=torch.bfloat16)
        layer.set_weights(w.cuda())
        layer.train(case["training"])
        xin = x.cuda().requires_grad_(True)
        with F.operator_settings(engine=engine, out_noise=out_noise):
            out = layer(xin)
        out.backward(g.cuda())
        assert device_error() == (0, 0)
        assert torch.equal(out.detach().cpu(), rec.out), f"{engine}: forward differs"
        assert torch.equal(xin.grad.cpu(), grads["grad_x"]), f"{engine}: grad_x differs"
        assert torch.equal(layer.weight.grad.cpu(), grads["grad_w"]), f"{engine}: grad_w differs"


@pytest.mark.parametrize("k,tile", [(512, 128), (3072, 512), (8192, 512)], ids=["T4", "T6", "T16"])
@pytest.mark.parametrize("engine", ["tcgen05_single", "tcgen05_pair"])
def test_output_noise_without_adc_is_one_gaussian_per_output(engine, k, tile):
    """No ADC and no clamp: the tile terms s_t * xi_t of an output are drawn as one Gaussian of the
    summed variance.  Mean, variance (per row: it depends on the row's input ranges), Gaussian shape
    and independence across neighbouring outputs and across calls."""
    import math

    from aihwkit_lightning_b200.nn import AnalogLinear
    from aihwkit_lightning_b200.nn import functional as F
    from util import NS

    case = dict(C.DEFAULTS)
    # T4: a small layer; T6 / T16: the tilings of the decoder configuration (K = 3072 and 8192 in tiles of 512).
    # The wide layers have small weights (1 / sqrt(K)): their noise level is raised so that the noise stays
    # well above the bf16 rounding step of the outputs, which would otherwise show up in the statistics.
    out_noise = 0.1 if k == 512 else 1.0
    case.update(ir_dynamic=True, out_noise=out_noise, max_input_size=tile, inp_res=254.0)
    rpu = C.build_rpu_config(NS, case)
    torch.manual_seed(0)
    n, m, t_count = 512, 512, k // tile
    layer = AnalogLinear(k, n, bias=False, rpu_config=rpu).to(device="cuda", dtype=torch.bfloat16)
    x = (torch.randn(m, k, device="cuda") * torch.linspace(0.5, 2.0, m, device="cuda")[:, None]).bfloat16()
    with F.operator_settings(engine=engine):
        layer.eval()
        clean = layer(x).float()
        layer.train()
        noisy1 = layer(x).float()
        noisy2 = layer(x).float()
    assert device_error() == (0, 0)
    w, xs = layer.weight.detach().float().cpu(), x.float().cpu()
    var = torch.zeros(m)
    for t in range(t_count):
        wmax = w[:, tile * t:tile * (t + 1)].abs().max()
        ir = xs[:, tile * t:tile * (t + 1)].abs().amax(1)
        var += (wmax * out_noise / math.sqrt(t_count) * ir) ** 2
    z1 = (noisy1 - clean).cpu() / var.sqrt()[:, None]
    z2 = (noisy2 - clean).cpu() / var.sqrt()[:, None]
    assert abs(z1.mean().item()) < 0.02
    assert abs(z1.std().item() - 1.0) < 0.03
    assert (z1.std(dim=1) - 1.0).abs().max().item() < 0.2          # every row has its own scale
    kurt = (z1 ** 4).mean().item() / (z1 ** 2).mean().item() ** 2
    assert abs(kurt - 3.0) < 0.15
    assert abs((z1[:, 1:] * z1[:, :-1]).mean().item()) < 0.02       # neighbours
    assert abs((z1 * z2).mean().item()) < 0.02                      # calls


def test_weight_gradients_first_when_a_hook_asks_for_them():
    """Data-parallel overlap: with an ``after_wgrad`` hook the backward enqueues the weight-side
    kernels first, calls the hook with the weight gradient, then computes the input gradient
    (optionally leaving SMs free for the exchange).  Results are those of the plain backward."""
    from aihwkit_lightning_b200.nn import AnalogLinear
    from aihwkit_lightning_b200.nn import functional as F
    from aihwkit_lightning_b200.simulator.configs import TorchInferenceRPUConfig

    rpu = TorchInferenceRPUConfig()
    rpu.mapping.max_input_size = 512
    rpu.forward.inp_res = 254
    rpu.forward.out_res = 254
    rpu.forward.out_bound = 10.0
    rpu.pre_post.input_range.enable = True
    rpu.pre_post.input_range.dynamic = True
    torch.manual_seed(0)
    layer = AnalogLinear(1024, 1280, bias=True, rpu_config=rpu).to(device="cuda", dtype=torch.bfloat16).train()
    x = torch.randn(2048, 1024, device="cuda").bfloat16().requires_grad_(True)
    g = torch.randn(2048, 1280, device="cuda").bfloat16()
    for engine in ("tcgen05_pair", "tcgen05_single", "simt"):
        with F.operator_settings(engine=engine):
            layer.zero_grad(set_to_none=True)
            x.grad = None
            layer(x).backward(g)
            want = [t.detach().clone() for t in (x.grad, layer.weight.grad, layer.bias.grad)]
            seen = []
            layer.zero_grad(set_to_none=True)
            x.grad = None
            with F.operator_settings(after_wgrad=lambda grad: seen.append(tuple(grad.shape)), comm_sms=16):
                layer(x).backward(g)
        for got, ref in zip((x.grad, layer.weight.grad, layer.bias.grad), want):
            assert torch.equal(got, ref), engine
        assert seen == [(1280, 1024)]


@pytest.mark.parametrize("engine", ["tcgen05_single", "tcgen05_pair"])
def test_a_wait_that_runs_out_raises_the_error_word_and_the_context_stays_usable(engine):
    """Failure path of the bounded device-side waits.  With the wait limit at 2 ms and the forward
    kernel told to withhold the signal its output-stage warps wait for, that wait runs out: the
    warps raise the error word, every other role of the kernel sees the abort flag (or runs out
    itself), copies in flight are drained, tensor memory is freed and the kernel returns.  The host
    reads ``AL_ERR_DEVICE_TIMEOUT``; afterwards the same call works again and gives the same result
    as before.  Nothing traps, faults or waits without bound in this test."""
    from aihwkit_lightning_b200 import _lib
    from aihwkit_lightning_b200.nn import AnalogLinear
    from aihwkit_lightning_b200.nn import functional as F
    from aihwkit_lightning_b200.simulator.configs import TorchInferenceRPUConfig

    lib = _lib.load()
    rpu = TorchInferenceRPUConfig()
    rpu.mapping.max_input_size = 256
    rpu.forward.inp_res = 254
    rpu.forward.out_res = 254
    rpu.forward.out_bound = 10.0
    rpu.pre_post.input_range.enable = True
    rpu.pre_post.input_range.dynamic = True
    torch.manual_seed(0)
    layer = AnalogLinear(512, 512, bias=False, rpu_config=rpu).to(device="cuda", dtype=torch.bfloat16).eval()
    x = torch.randn(512, 512, device="cuda").bfloat16()
    with F.operator_settings(engine=engine), torch.no_grad():
        before = layer(x).clone()
        assert device_error() == (0, 0)
        torch.cuda.synchronize()
        _lib.check(lib.al_set_device_wait_limit_ns(2_000_000))
        _lib.check(lib.al_debug_withhold_forward_signal(1))
        try:
            layer(x)
            status, code = device_error()
        finally:
            _lib.check(lib.al_debug_withhold_forward_signal(0))
            _lib.check(lib.al_set_device_wait_limit_ns(0))
        assert status == _lib.AL_ERR_DEVICE_TIMEOUT
        assert code & 4, f"the output-stage warps must have given up (role mask {code:#x})"
        after = layer(x)
        torch.cuda.synchronize()
        assert device_error() == (0, 0)
        assert torch.equal(after, before)
