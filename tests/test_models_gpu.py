"""Whole-model parity at reduced size for the two model families of the benchmark
configurations: a Phi-3-shaped decoder in bf16 (config 3) and a CIFAR-shaped ResNet in fp32
(config 4).  The same randomly initialised model is evaluated (loss and gradients) once with
its layers converted by ``convert_to_analog`` on the GPU and once on the CPU with every
Linear / Conv2d routed through the oracle.  Noise is off (it cannot be replayed through a whole
model); DAC, dynamic input ranges, tiling and -- for the decoder -- the ADC are on."""
import copy

import pytest
import torch
from torch.nn import functional as TF

import cases as C
import model_zoo as Z
from util import NS, rel_fro

pytestmark = pytest.mark.gpu


def rpu_for(**kw):
    case = dict(C.DEFAULTS)
    case.update(ir_dynamic=True, inp_res=254.0, **kw)
    return C.build_rpu_config(NS, case)


def test_phi3_shaped_decoder_step_matches_oracle_model():
    from aihwkit_lightning_b200.nn import AnalogLinear, convert_to_analog

    torch.manual_seed(0)
    base = Z.TinyPhi3().bfloat16()
    ids = torch.randint(0, 512, (2, 64))
    labels = torch.randint(0, 512, (2, 64))
    rpu = rpu_for(max_input_size=128, out_bound=10.0, out_res=254.0)

    ref = Z.to_oracle(copy.deepcopy(base), rpu).train()
    loss_ref = TF.cross_entropy(ref(ids).float().view(-1, 512), labels.view(-1))
    loss_ref.backward()

    gpu = convert_to_analog(copy.deepcopy(base), rpu).cuda().train()
    assert sum(isinstance(m, AnalogLinear) for m in gpu.modules()) == 2 * 4 + 1
    loss = TF.cross_entropy(gpu(ids.cuda()).float().view(-1, 512), labels.cuda().view(-1))
    loss.backward()

    assert abs(loss.item() - loss_ref.item()) <= 1e-3 * abs(loss_ref.item())
    pairs = [(gpu.lm_head.weight.grad, ref.lm_head.weight.grad),
             (gpu.layers[1].down_proj.weight.grad, ref.layers[1].down_proj.weight.grad),
             (gpu.layers[0].qkv_proj.weight.grad, ref.layers[0].qkv_proj.weight.grad),
             (gpu.embed.weight.grad, ref.embed.weight.grad)]
    for got, want in pairs:
        # bf16 end to end through two decoder layers: measured 1.6e-3 .. 3.4e-3, while the oracle model moves by
        # 6e-3 .. 3e-2 when one per cent of its embedding entries change by one bf16 ulp
        assert rel_fro(got, want) <= 1e-2


@pytest.mark.parametrize("quantised", [False, True])
def test_resnet_shaped_step_matches_oracle_model(quantised):
    from aihwkit_lightning_b200.nn import AnalogConv2d, AnalogLinear, convert_to_analog
    from aihwkit_lightning_b200.optim import AnalogOptimizer

    torch.manual_seed(0)
    base = Z.TinyResNet(blocks=1)
    x = torch.randn(8, 3, 32, 32)
    y = torch.randint(0, 10, (8,))
    if quantised:
        rpu = rpu_for(max_input_size=256)
    else:  # tiling only: the model is then a smooth function and gradients must agree tightly
        rpu = rpu_for(max_input_size=256)
        rpu.pre_post.input_range.enable = False
        rpu.forward.inp_res = -1

    ref = Z.to_oracle(copy.deepcopy(base), rpu).train()
    loss_ref = TF.cross_entropy(ref(x), y)
    loss_ref.backward()

    gpu = convert_to_analog(copy.deepcopy(base), rpu).cuda().train()
    assert any(isinstance(m, AnalogConv2d) for m in gpu.modules())
    assert isinstance(gpu.fc, AnalogLinear)
    loss = TF.cross_entropy(gpu(x.cuda()), y.cuda())
    loss.backward()

    pairs = [(gpu.fc.weight.grad, ref.fc.weight.grad), (gpu.conv.weight.grad, ref.conv.conv.weight.grad),
             (gpu.blocks[2].conv2.weight.grad, ref.blocks[2].conv2.conv.weight.grad)]
    if not quantised:
        assert abs(loss.item() - loss_ref.item()) <= 1e-5 * abs(loss_ref.item())
        for got, want in pairs:
            assert rel_fro(got, want) <= 1e-3
    else:
        # Layer by layer the fp32 kernels agree with the oracle to 1e-5, but through a stack of
        # quantising layers, batch norm and ReLUs a last-ulp difference of an activation now and
        # then lands on the other side of a DAC rounding boundary downstream: the loss still
        # agrees closely, gradients only to within the quantisation noise they carry.
        assert abs(loss.item() - loss_ref.item()) <= 1e-3 * abs(loss_ref.item())
        # The yardstick is the oracle model itself: its gradients for an input that differs by 1e-6 relative
        # (far below anything the two implementations disagree on layer by layer).  The GPU model must stay
        # within 1.5 times that distance of the oracle (measured: 0.8 times), and within the fixed caps.
        torch.manual_seed(1)
        nudged = Z.to_oracle(copy.deepcopy(base), rpu).train()
        TF.cross_entropy(nudged(x * (1 + 1e-6 * torch.randn_like(x))), y).backward()
        yard = [rel_fro(nudged.fc.weight.grad, ref.fc.weight.grad),
                rel_fro(nudged.conv.conv.weight.grad, ref.conv.conv.weight.grad),
                rel_fro(nudged.blocks[2].conv2.conv.weight.grad, ref.blocks[2].conv2.conv.weight.grad)]
        caps = [2e-2, 0.25, 0.25]
        for (got, want), own, cap in zip(pairs, yard, caps):
            assert rel_fro(got, want) <= min(cap, 1.5 * max(own, 1e-3))

    # one optimizer step with the clipping hook runs and changes the weights
    layers = lambda: (m for m in gpu.modules() if isinstance(m, (AnalogConv2d, AnalogLinear)))  # noqa: E731
    opt = AnalogOptimizer(torch.optim.SGD, layers, gpu.parameters(), lr=0.1)
    before = gpu.fc.weight.detach().clone()
    opt.step()
    assert not torch.equal(before, gpu.fc.weight.detach())
