"""A training step captured in a CUDA graph draws fresh analog noise on every replay.

The call counter of the noise generator is an argument by value, which a captured call replays
unchanged; ``F.GraphNoise`` adds a counter in device memory that the kernels read when they
start (``AlForwardArgs.offset_base``).
"""
import pytest
import torch

import cases as C
from util import NS

pytestmark = pytest.mark.gpu


def build(dtype, k, n, max_in, adc):
    from aihwkit_lightning_b200.nn import AnalogLinear

    case = dict(C.DEFAULTS)
    case.update(dtype="bf16" if dtype == torch.bfloat16 else "fp32", max_input_size=max_in, ir_dynamic=True,
                inp_res=254.0, out_noise=0.1, noise_type="AddNormalPerChannel", std_dev=0.05, bias=False)
    if adc:
        case.update(out_res=254.0, out_bound=10.0)
    rpu = C.build_rpu_config(NS, case)
    torch.manual_seed(0)
    layer = AnalogLinear(k, n, bias=False, rpu_config=rpu).to(device="cuda", dtype=dtype)
    return layer.train()


@pytest.mark.parametrize("dtype,m,k,n,max_in,adc", [
    (torch.bfloat16, 256, 512, 256, 256, True),    # tcgen05 forward with noise + ADC, fused weight pre-pass
    (torch.bfloat16, 512, 1024, 512, 512, False),  # merged output noise
    (torch.float32, 128, 200, 48, 100, False),     # CUDA-core kernels, ragged tiles
    (torch.float32, 256, 512, 256, 256, False),    # fp32 on the tensor cores
], ids=["bf16-adc", "bf16-merged-noise", "f32-simt", "f32-tensor-core"])
def test_replays_draw_fresh_noise(dtype, m, k, n, max_in, adc):
    from aihwkit_lightning_b200.nn import functional as F

    layer = build(dtype, k, n, max_in, adc)
    x = torch.randn(m, k, device="cuda").to(dtype).requires_grad_(True)
    g = torch.randn(m, n, device="cuda").to(dtype)
    noise = F.GraphNoise(x.device)
    out_static = torch.empty(m, n, device="cuda", dtype=dtype)

    def step():
        noise.advance()
        layer.weight.grad = None
        x.grad = None
        out = layer(x)
        out.backward(g)
        out_static.copy_(out.detach())

    with F.operator_settings(graph_noise=noise):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):  # warm-up outside the capture (lazy initialisations)
                step()
        torch.cuda.current_stream().wait_stream(side)
        calls_per_step = noise.calls // 3
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
    assert noise.calls == 4 * calls_per_step  # the capture consumed host-side offsets like a step

    outs, grads = [], []
    for _ in range(3):
        graph.replay()
        torch.cuda.synchronize()
        outs.append(out_static.float().clone())
        grads.append(layer.weight.grad.float().clone())
    # fresh output noise and fresh weight noise on every replay
    assert not torch.equal(outs[0], outs[1]) and not torch.equal(outs[1], outs[2])
    diff = outs[0] - outs[1]
    assert diff.abs().mean() > 0
    # the same counter value reproduces the same step bit for bit
    value = noise.counter.clone()
    graph.replay()
    torch.cuda.synchronize()
    first = out_static.clone()
    noise.counter.copy_(value)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(first, out_static)
    # and the replays scatter around the noise-free result like eager calls do
    layer.eval()
    with torch.no_grad():
        clean = layer(x.detach()).float()
    layer.train()
    eager = []
    for _ in range(3):
        eager.append((layer(x.detach()).float() - clean).std().item())
    replayed = [(o - clean).std().item() for o in outs]
    assert abs(sum(replayed) / 3 - sum(eager) / 3) <= 0.1 * (sum(eager) / 3)
