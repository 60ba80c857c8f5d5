"""``al_peer_allreduce``: the library's gradient exchange over peer memory.

On one GPU the kernel runs with a world of one (it signals and waits for itself): slice
arithmetic, scaling, offsets and both element types are checked that way.  With two or more GPUs
(skipped otherwise) two processes map one another's buffers through PyTorch's symmetric memory
and exchange gradients with ``PeerGradientSync``: the result is the mean of the replicas'
gradients and every replica holds the same bits."""
import ctypes
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_world_of_one_scales_its_own_buffer_in_place(dtype):
    from aihwkit_lightning_b200 import _lib

    lib = _lib.load()
    n = 8 * 1000 + 8 * 37
    buf = torch.randn(n + 64, device="cuda").to(dtype)
    want = buf.clone()
    pad = torch.zeros(512, dtype=torch.int32, device="cuda")
    bufs = (ctypes.c_uint64 * 1)(buf.data_ptr())
    pads = (ctypes.c_uint64 * 1)(pad.data_ptr())
    code = _lib.AL_BF16 if dtype == torch.bfloat16 else _lib.AL_F32
    stream = torch.cuda.current_stream().cuda_stream
    offset = 64  # elements: the part in front must stay untouched
    for call in range(3):  # the signal counters only grow: several calls on the same pads
        _lib.check(lib.al_peer_allreduce(code, 1, 0, bufs, pads, 0, offset * buf.element_size(), n, call, 0.5, 4, stream))
        want[offset:] = (want[offset:].float() * 0.5).to(dtype)
    torch.cuda.synchronize()
    err = ctypes.c_uint32(0)
    assert lib.al_peer_read_error(ctypes.byref(err)) == 0 and err.value == 0
    assert torch.equal(buf, want)
    slots = pad[_lib.AL_PEER_SIGNAL_SLOT:_lib.AL_PEER_SIGNAL_SLOT + 9].tolist()
    assert slots[0] == 6 and slots[8] == 0  # 2 signals per call; the CTA counter is back at zero


def test_bad_arguments_are_refused():
    from aihwkit_lightning_b200 import _lib

    lib = _lib.load()
    one = (ctypes.c_uint64 * 1)(256)
    assert lib.al_peer_allreduce(_lib.AL_BF16, 9, 0, one, one, 0, 0, 8, 0, 1.0, 4, None) == _lib.AL_ERR_BAD_ARGUMENT
    assert lib.al_peer_allreduce(_lib.AL_BF16, 1, 0, one, one, 0, 0, 12, 0, 1.0, 4, None) == _lib.AL_ERR_BAD_ARGUMENT
    assert lib.al_peer_allreduce(_lib.AL_BF16, 1, 0, one, one, 0, 8, 16, 0, 1.0, 4, None) == _lib.AL_ERR_BAD_ARGUMENT
    assert lib.al_peer_allreduce(7, 1, 0, one, one, 0, 0, 16, 0, 1.0, 4, None) == _lib.AL_ERR_BAD_ARGUMENT


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir, multicast):
    import torch.distributed as dist

    from aihwkit_lightning_b200.distributed import PeerGradientSync
    from aihwkit_lightning_b200.nn import AnalogLinear
    from aihwkit_lightning_b200.nn import functional as F
    from aihwkit_lightning_b200.simulator.configs import TorchInferenceRPUConfig

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        rpu = TorchInferenceRPUConfig()
        rpu.mapping.max_input_size = 256
        rpu.forward.inp_res = 254
        rpu.pre_post.input_range.enable = True
        rpu.pre_post.input_range.dynamic = True
        torch.manual_seed(0)  # identical replicas
        model = torch.nn.Sequential(AnalogLinear(512, 384, rpu_config=rpu), torch.nn.Tanh(),
                                    AnalogLinear(384, 256, rpu_config=rpu)).to(device="cuda", dtype=torch.bfloat16)
        x = torch.randn(256, 512, device="cuda", generator=torch.Generator("cuda").manual_seed(10 + rank)).bfloat16()
        # reference: local gradients, averaged by a plain all-reduce in fp32
        model(x).float().square().sum().backward()
        want = []
        for p in model.parameters():
            g = p.grad.float().clone()
            dist.all_reduce(g)
            want.append(g / world)
        model.zero_grad(set_to_none=True)
        sync = PeerGradientSync(model.parameters(), n_ctas=8, use_multicast=multicast)
        with F.operator_settings(after_wgrad=sync, grad_w_alloc=sync.grad_buffer, comm_sms=8):
            for _ in range(2):  # two steps: the buffers and the signal counters are reused
                model.zero_grad(set_to_none=True)
                model(x).float().square().sum().backward()
                sync.finish()
        torch.cuda.synchronize()
        exchanged = sum(pool["calls"] for pool in sync._pools.values())  # pylint: disable=protected-access
        assert exchanged == 4, exchanged  # both weight matrices, both steps, went through the library's kernel
        for p, w in zip(model.parameters(), want):
            assert torch.allclose(p.grad.float(), w, rtol=2e-2, atol=2e-2 * w.abs().max().item())
        torch.save([p.grad.cpu() for p in model.parameters()], os.path.join(out_dir, f"peer{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("multicast", [False, True], ids=["peer_loads", "multimem"])
def test_two_replicas_exchange_gradients_over_peer_memory(tmp_path, multicast):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), multicast), nprocs=2, join=True)
    a, b = torch.load(tmp_path / "peer0.pt"), torch.load(tmp_path / "peer1.pt")
    for x, y in zip(a, b):
        assert torch.equal(x, y)  # bit-identical replicas
