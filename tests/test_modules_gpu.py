"""Module-level behaviour on the GPU: API surface, conv path, optimizer hook, checkpoints,
internal noise generator statistics."""
import math

import pytest
import torch

import analog_oracle as O
import cases as C
from util import NS

pytestmark = pytest.mark.gpu


def make_cfg(**kw):
    case = dict(C.DEFAULTS)
    case.update(kw)
    return C.build_rpu_config(NS, case), case


def test_cpu_tensor_is_rejected():
    from aihwkit_lightning_b200.nn import AnalogLinear

    rpu, _ = make_cfg()
    layer = AnalogLinear(8, 4, rpu_config=rpu)
    with pytest.raises(ValueError):
        layer(torch.randn(2, 8))


def test_missing_rpu_config():
    from aihwkit_lightning_b200.nn import AnalogLinear

    with pytest.raises(ValueError):
        AnalogLinear(8, 4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_conv2d_matches_oracle_on_unfolded_patches(dtype):
    from aihwkit_lightning_b200.nn import AnalogConv2d

    rpu, case = make_cfg(ir_dynamic=True, max_input_size=10, out_bound=4.0, out_res=254.0, training=False)
    torch.manual_seed(0)
    conv = AnalogConv2d(4, 6, 3, padding=1, rpu_config=rpu).to(device="cuda", dtype=dtype).eval()
    x = torch.randn(2, 4, 9, 9).to(dtype)
    got = conv(x.cuda())
    patches = torch.nn.functional.unfold(x.float(), 3, padding=1).transpose(1, 2).to(dtype)
    rec = O.forward(patches, conv.weight.detach().cpu().view(6, -1), conv.bias.detach().cpu(), None, None,
                    None, None, conv.in_sizes, False, rpu)
    want = rec.out.transpose(1, 2).reshape(2, 6, 9, 9)
    if dtype == torch.float32:
        assert torch.allclose(got.cpu(), want, rtol=1e-5, atol=1e-5)
    else:
        assert (got.cpu().float() - want.float()).norm() <= 1e-2 * want.float().norm()


def test_conv2d_backward_runs_and_matches_fp32():
    from aihwkit_lightning_b200.nn import AnalogConv2d

    rpu, _ = make_cfg(ir_enable=False, inp_res=-1.0, max_input_size=-1)
    torch.manual_seed(0)
    conv = AnalogConv2d(3, 5, 3, stride=2, padding=1, rpu_config=rpu).cuda()
    ref = AnalogConv2d.to_digital(conv)
    x = torch.randn(4, 3, 8, 8, device="cuda", requires_grad=True)
    x2 = x.detach().clone().requires_grad_(True)
    conv(x).square().sum().backward()
    ref(x2).square().sum().backward()
    assert torch.allclose(x.grad, x2.grad, rtol=1e-4, atol=1e-4)
    assert torch.allclose(conv.weight.grad, ref.weight.grad, rtol=1e-4, atol=1e-4)


def test_optimizer_hook_clips_weights():
    from aihwkit_lightning_b200.nn import AnalogLinear
    from aihwkit_lightning_b200.optim import AnalogOptimizer

    rpu, _ = make_cfg(clip_type="LayerGaussian", clip_sigma=1.0, ir_dynamic=True)
    layer = AnalogLinear(64, 32, rpu_config=rpu).cuda()
    opt = AnalogOptimizer(torch.optim.SGD, layer.analog_layers, layer.parameters(), lr=0.0)
    before = layer.weight.detach().clone()
    layer(torch.randn(4, 64, device="cuda")).sum().backward()
    opt.step()
    lim = before.std().item()
    assert layer.weight.abs().max().item() <= lim * (1 + 1e-5)
    assert torch.equal(layer.weight.detach().cpu(), O.clip_weights(before.cpu(), "LayerGaussian", 1.0))


def test_state_dict_round_trip_and_reference_key_names(tmp_path):
    from aihwkit_lightning_b200.nn import AnalogLinear

    rpu, _ = make_cfg()
    layer = AnalogLinear(40, 24, rpu_config=rpu).cuda()
    assert list(layer.state_dict().keys()) == [
        "weight", "bias", "input_range", "input_range_update_idx", "x_min", "x_max"]
    path = tmp_path / "ckpt.pt"
    torch.save(layer.state_dict(), path)
    other = AnalogLinear(40, 24, rpu_config=make_cfg()[0]).cuda()
    other.load_state_dict(torch.load(path, weights_only=False))
    x = torch.randn(3, 40, device="cuda")
    layer.eval(), other.eval()
    assert torch.equal(layer(x), other(x))


def test_internal_generator_noise_moments():
    """Noise from the library's own counter-based generator: statistics as in the reference's
    test of its Triton noise (`tests/test_correctness_triton_mode.py:192-218`)."""
    from aihwkit_lightning_b200.nn import AnalogLinear

    rpu, _ = make_cfg(ir_dynamic=True, out_noise=0.1, max_input_size=128, inp_res=254.0)
    torch.manual_seed(0)
    layer = AnalogLinear(256, 512, bias=False, rpu_config=rpu).cuda()
    x = torch.randn(512, 256, device="cuda")
    layer.eval()
    clean = layer(x)
    layer.train()
    noisy1, noisy2 = layer(x), layer(x)
    delta = (noisy1 - clean).cpu()
    assert not torch.equal(noisy1, noisy2)
    # expected per-element std: sqrt(sum_t (wmax_t * out_noise/sqrt(T) * ir_t[m])^2)
    w, xs = layer.weight.detach().cpu(), x.cpu()
    var = torch.zeros(512)
    for t in range(2):
        wmax = w[:, 128 * t:128 * (t + 1)].abs().max()
        ir = xs[:, 128 * t:128 * (t + 1)].abs().amax(1)
        var += (wmax * 0.1 / math.sqrt(2) * ir) ** 2
    z = delta / var.sqrt()[:, None]
    assert abs(z.mean().item()) < 0.01
    assert abs(z.std().item() - 1.0) < 0.01

    rpu2, _ = make_cfg(ir_dynamic=True, noise_type="AddNormalPerChannel", std_dev=0.1, max_input_size=128)
    layer2 = AnalogLinear(256, 512, bias=False, rpu_config=rpu2).cuda().train()
    from aihwkit_lightning_b200.nn import functional as F
    cap = {}
    with F.operator_settings(capture=cap):
        layer2(x)
    dw = (cap["w_mod"] - layer2.weight.detach()).cpu()
    w2 = layer2.weight.detach().cpu()
    scale = torch.cat([w2[:, :128].abs().amax(1, keepdim=True).expand(-1, 128),
                       w2[:, 128:].abs().amax(1, keepdim=True).expand(-1, 128)], 1) * 0.1
    z = dw / scale
    assert abs(z.mean().item()) < 0.01
    assert abs(z.std().item() - 1.0) < 0.01


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("geom", [
    dict(c=3, h=32, w=32, k=(3, 3), s=(1, 1), p=(1, 1), d=(1, 1)),
    dict(c=16, h=9, w=11, k=(3, 2), s=(2, 1), p=(0, 2), d=(1, 2)),
    dict(c=5, h=7, w=7, k=(1, 1), s=(2, 2), p=(0, 0), d=(1, 1)),
    # channels split over several CTAs (the staged rows of all 96 do not fit), ragged last band
    dict(c=96, h=30, w=34, k=(3, 3), s=(1, 1), p=(1, 1), d=(1, 1)),
    dict(c=40, h=21, w=50, k=(5, 3), s=(2, 3), p=(2, 0), d=(2, 1)),
    # unit stride with dilation and more padding than the kernel reaches over; even kernel area
    dict(c=8, h=12, w=20, k=(3, 3), s=(1, 1), p=(2, 2), d=(2, 2)),
    dict(c=12, h=10, w=9, k=(2, 2), s=(1, 1), p=(3, 2), d=(1, 1)),
    # wide rows: the staged band needs the opt-in shared-memory size
    dict(c=4, h=9, w=100, k=(3, 3), s=(1, 1), p=(1, 1), d=(1, 1)),
    # a stride larger than the kernel: input rows no patch reads get a zero gradient
    dict(c=2, h=13, w=12, k=(2, 2), s=(5, 4), p=(0, 1), d=(1, 1)),
    # rows too long to stage: the unstaged kernels
    dict(c=1, h=3, w=12000, k=(3, 3), s=(1, 1), p=(1, 1), d=(1, 1)),
])
def test_unfold2d_and_its_adjoint_match_torch(dtype, geom):
    """The patch-extraction kernel is a pure copy (bit-equal to F.unfold + transpose); its
    backward is the gather form of col2im."""
    from aihwkit_lightning_b200.nn import functional as F

    torch.manual_seed(0)
    x = torch.randn(4, geom["c"], geom["h"], geom["w"], device="cuda").to(dtype).requires_grad_(True)
    x2 = x.detach().clone().requires_grad_(True)
    got = F.unfold2d(x, geom["k"], geom["d"], geom["p"], geom["s"])
    want = torch.nn.functional.unfold(x2.float(), geom["k"], dilation=geom["d"], padding=geom["p"],
                                      stride=geom["s"]).transpose(-1, -2)
    assert torch.equal(got.float(), want)
    g = torch.randn_like(got)
    got.backward(g)
    want.backward(g.float())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(x.grad.float(), x2.grad.float(), rtol=tol, atol=tol)
    # 3-D input (single image), as the reference accepts
    one = F.unfold2d(x.detach()[0], geom["k"], geom["d"], geom["p"], geom["s"])
    assert torch.equal(one, got.detach()[0])


@pytest.mark.parametrize("dims", [1, 3])
def test_conv1d_and_conv3d_match_their_digital_twins(dims):
    """With input range, DAC and modifier off the analog layer is the plain convolution: forward
    and all gradients against ``to_digital`` of the same layer."""
    from aihwkit_lightning_b200.nn import AnalogConv1d, AnalogConv3d

    rpu, _ = make_cfg(ir_enable=False, inp_res=-1.0, max_input_size=16)
    torch.manual_seed(0)
    torch.backends.cudnn.allow_tf32 = False  # the digital twin must compute in fp32 to be a yardstick
    if dims == 1:
        conv = AnalogConv1d(3, 5, 4, stride=2, padding=1, rpu_config=rpu).cuda()
        x = torch.randn(4, 3, 19, device="cuda", requires_grad=True)
        assert conv.weight.shape == (5, 3, 1, 4)
    else:
        conv = AnalogConv3d(2, 4, (2, 3, 2), stride=(1, 2, 1), padding=(1, 0, 1), rpu_config=rpu).cuda()
        x = torch.randn(2, 2, 5, 6, 7, device="cuda", requires_grad=True)
    ref = type(conv).to_digital(conv)
    x2 = x.detach().clone().requires_grad_(True)
    out, want = conv(x), ref(x2)
    assert out.shape == want.shape
    assert torch.allclose(out, want, rtol=1e-4, atol=1e-4)
    out.square().sum().backward()
    want.square().sum().backward()
    assert torch.allclose(x.grad, x2.grad, rtol=1e-4, atol=1e-4)
    assert torch.allclose(conv.weight.grad.reshape(ref.weight.shape), ref.weight.grad, rtol=1e-4, atol=1e-4)
    assert torch.allclose(conv.bias.grad, ref.bias.grad, rtol=1e-4, atol=1e-4)
    # unbatched input
    assert torch.allclose(conv(x.detach()[0]), ref(x2.detach()[0]), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("dims", [1, 3])
def test_conv1d_and_conv3d_match_oracle_on_patches(dims):
    from aihwkit_lightning_b200.nn import AnalogConv1d, AnalogConv3d
    from aihwkit_lightning_b200.nn.modules.conv import unfold3d

    rpu, _ = make_cfg(ir_dynamic=True, max_input_size=10, out_bound=4.0, out_res=254.0, training=False)
    torch.manual_seed(0)
    if dims == 1:
        conv = AnalogConv1d(4, 6, 5, padding=2, rpu_config=rpu).cuda().eval()
        x = torch.randn(3, 4, 21)
        patches = torch.nn.functional.unfold(x.unsqueeze(-2), (1, 5), padding=(0, 2)).transpose(1, 2)
    else:
        conv = AnalogConv3d(2, 5, 2, padding=1, rpu_config=rpu).cuda().eval()
        x = torch.randn(2, 2, 4, 5, 6)
        patches = unfold3d(x, (2, 2, 2), (1, 1, 1), (1, 1, 1))
    got = conv(x.cuda())
    rec = O.forward(patches, conv.weight.detach().cpu().view(conv.out_channels, -1), conv.bias.detach().cpu(),
                    None, None, None, None, conv.in_sizes, False, rpu)
    want = rec.out.transpose(1, 2).reshape(got.shape)
    assert torch.allclose(got.cpu(), want, rtol=1e-5, atol=1e-5)


def test_conv1d_conversion_and_checkpoint_use_pytorch_weight_shape():
    from aihwkit_lightning_b200.nn import AnalogConv1d, AnalogConv3d, convert_to_analog, convert_to_digital

    rpu, _ = make_cfg(ir_dynamic=True)
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Conv1d(3, 4, 3), torch.nn.Flatten(), torch.nn.Linear(4 * 6, 2))
    analog = convert_to_analog(model, rpu).cuda()
    assert isinstance(analog[0], AnalogConv1d)
    state = analog.state_dict()
    assert state["0.weight"].shape == (4, 3, 3)            # squeezed like torch.nn.Conv1d
    twin = convert_to_analog(model, rpu).cuda()
    twin.load_state_dict(state)
    assert twin[0].weight.shape == (4, 3, 1, 3)
    x = torch.randn(5, 3, 8, device="cuda")
    assert torch.equal(analog.eval()(x), twin.eval()(x))
    digital = convert_to_digital(analog)
    assert isinstance(digital[0], torch.nn.Conv1d) and digital[0].weight.shape == (4, 3, 3)
    assert isinstance(convert_to_analog(torch.nn.Conv3d(1, 2, 3), rpu), AnalogConv3d)
    with pytest.raises(ValueError):
        AnalogConv1d(3, 4, 3, dilation=2, rpu_config=rpu)



def test_after_wgrad_hook_gets_the_weight_gradient_before_the_input_gradient_is_enqueued():
    """Data-parallel training starts its gradient exchange from this hook: it must see the final
    weight gradient tensor, and splitting backward around it must not change any result."""
    from aihwkit_lightning_b200.nn import AnalogLinear
    from aihwkit_lightning_b200.nn import functional as F
    from aihwkit_lightning_b200.simulator.configs import TorchInferenceRPUConfig

    rpu = TorchInferenceRPUConfig()
    rpu.mapping.max_input_size = 64
    rpu.forward.inp_res = 254
    rpu.forward.out_res = 254
    rpu.forward.out_bound = 10.0
    rpu.pre_post.input_range.enable = True
    rpu.pre_post.input_range.dynamic = False
    rpu.pre_post.input_range.init_from_data = 0
    rpu.pre_post.input_range.init_value = 2.0
    torch.manual_seed(0)
    layer = AnalogLinear(128, 96, bias=True, rpu_config=rpu).cuda().train()
    x = torch.randn(40, 128, device="cuda", requires_grad=True)
    g = torch.randn(40, 96, device="cuda")
    layer(x).backward(g)
    want = [t.detach().clone() for t in (x.grad, layer.weight.grad, layer.bias.grad, layer.input_range.grad)]
    layer.zero_grad(set_to_none=True)
    x.grad = None
    seen = []  # addresses only: holding the tensor would make autograd store a copy instead of it
    with F.operator_settings(after_wgrad=lambda grad: seen.append((grad.data_ptr(), tuple(grad.shape)))):
        layer(x).backward(g)
    assert seen == [(layer.weight.grad.data_ptr(), (96, 128))]
    for got, ref in zip((x.grad, layer.weight.grad, layer.bias.grad, layer.input_range.grad), want):
        assert torch.equal(got, ref)



def test_shared_tile_statistics_override_the_local_ones():
    """Data-parallel init-from-data: with ``settings.sync_tile_std`` installed the range update uses
    the statistics that callable returns (the replica mean in training) instead of the local ones."""
    from aihwkit_lightning_b200.nn import AnalogLinear
    from aihwkit_lightning_b200.nn import functional as F
    from aihwkit_lightning_b200.simulator.configs import TorchInferenceRPUConfig

    rpu = TorchInferenceRPUConfig()
    rpu.mapping.max_input_size = 32
    rpu.forward.inp_res = 254
    rpu.pre_post.input_range.enable = True
    rpu.pre_post.input_range.init_from_data = 10
    rpu.pre_post.input_range.init_value = 3.0
    torch.manual_seed(0)
    layer = AnalogLinear(64, 16, rpu_config=rpu).cuda().train()
    x = torch.randn(128, 64, device="cuda")
    seen = []

    def doubled(std):
        seen.append(std.clone())
        return std * 2.0

    with F.operator_settings(sync_tile_std=doubled):
        layer(x)
    local = torch.stack([x[:, :32].std(), x[:, 32:].std()])
    assert torch.allclose(seen[0], local, rtol=1e-5)
    alpha = rpu.pre_post.input_range.init_std_alpha
    assert torch.allclose(layer.input_range.detach(), alpha * 2.0 * local, rtol=1e-5)  # idx 0: ir <- alpha * std
    assert layer.input_range_update_idx.tolist() == [1.0, 1.0]
