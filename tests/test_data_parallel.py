"""Host logic of the data-parallel path with two gloo ranks on the CPU: row sharding covers the
batch exactly once, bucketed gradient all-reduce equals the mean of the per-rank gradients and
leaves every replica with identical values, per-rank noise seeds differ."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from aihwkit_lightning_b200.distributed import (
    EagerGradientSync, GradientBuckets, all_reduce_gradients, mean_over_replicas, rank_seed, shard_rows)


def test_shard_rows_partition():
    for total, world in ((8192, 8), (10, 4), (3, 8), (0, 2), (17, 1)):
        seen = []
        for rank in range(world):
            lo, hi = shard_rows(total, rank, world)
            assert 0 <= lo <= hi <= total
            seen.extend(range(lo, hi))
        assert seen == list(range(total))
        sizes = [shard_rows(total, r, world)[1] - shard_rows(total, r, world)[0] for r in range(world)]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_rows(10, 4, 4)


def test_rank_seeds_are_distinct():
    assert len({rank_seed(0, r) for r in range(8)}) == 8
    assert rank_seed(1, 0) != rank_seed(0, 0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)  # identical parameters on every replica
        shapes = [(24, 40), (24,), (3,), (9, 40), (9,), (5, 5)]
        params = [torch.nn.Parameter(torch.randn(s)) for s in shapes]
        params[3].requires_grad_(False)  # a frozen parameter must be skipped
        gen = torch.Generator().manual_seed(100 + rank)  # per-rank gradients
        for p in params:
            if p.requires_grad:
                p.grad = torch.randn(p.shape, generator=gen)
        params[5].grad = None  # a parameter that received no gradient on this rank counts as zero
        local = [None if p.grad is None else p.grad.clone() for p in params]

        buckets = GradientBuckets(params, bucket_bytes=24 * 40 * 4 + 100)  # forces several buckets
        assert len(buckets.buckets) >= 2
        assert sum(buckets.bucket_sizes()) == sum(p.numel() for p in params if p.requires_grad)
        buckets.reduce_all_async()
        buckets.finish()

        gathered = [None] * world
        dist.all_gather_object(gathered, local)
        for i, p in enumerate(params):
            if not p.requires_grad:
                assert p.grad is None
                continue
            want = sum((g[i] if g[i] is not None else torch.zeros(p.shape)) for g in gathered) / world
            assert torch.allclose(p.grad, want, rtol=1e-6, atol=1e-7), i

        # one-shot helper gives the same result
        for p, g in zip(params, local):
            if p.requires_grad:
                p.grad = None if g is None else g.clone()
        all_reduce_gradients(params)
        torch.save([None if p.grad is None else p.grad for p in params], os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_bucketed_all_reduce_two_gloo_ranks(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    a = torch.load(tmp_path / "r0.pt")
    b = torch.load(tmp_path / "r1.pt")
    for x, y in zip(a, b):
        if x is None:
            assert y is None
        else:
            assert torch.equal(x, y)  # replicas hold bit-identical averaged gradients


def _eager_worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)  # identical replicas
        model = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Tanh(), torch.nn.Linear(5, 3))
        model[2].bias.requires_grad_(False)
        sync = EagerGradientSync(small_numel=8).attach(model.parameters())  # the biases go the flat way
        x = torch.randn(4, 6, generator=torch.Generator().manual_seed(10 + rank))  # per-rank batch
        # the hook fires from inside backward, once per parameter that received a gradient
        model(x).square().sum().backward()
        assert len(sync._pending) == 2 and len(sync._small) == 1  # pylint: disable=protected-access
        local = model(x).square().sum()
        want = torch.autograd.grad(local, [p for p in model.parameters() if p.requires_grad])
        sync.finish()
        gathered = [None] * world
        dist.all_gather_object(gathered, [g.clone() for g in want])
        trainable = [p for p in model.parameters() if p.requires_grad]
        for i, p in enumerate(trainable):
            mean = sum(g[i] for g in gathered) / world
            assert torch.allclose(p.grad, mean, rtol=1e-6, atol=1e-7), i
        assert model[2].bias.grad is None
        torch.save([p.grad for p in trainable], os.path.join(out_dir, f"e{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_eager_gradient_sync_two_gloo_ranks(tmp_path):
    world = 2
    mp.spawn(_eager_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for x, y in zip(torch.load(tmp_path / "e0.pt"), torch.load(tmp_path / "e1.pt")):
        assert torch.equal(x, y)



def _ir_worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # the init-from-data update of a learned input range (`torch_linear.py:338-352`) with the per-tile
        # standard deviation shared between the replicas: ir <- (ir * idx + alpha * std) / (idx + 1)
        gen = torch.Generator().manual_seed(50 + rank)  # every replica sees its own batch
        ir, idx, alpha = torch.full((3,), 3.0), torch.zeros(3), 3.0
        local_ir = ir.clone()
        for _ in range(4):
            x = torch.randn(64, 48, generator=gen) * (1.0 + rank)
            std = torch.stack([x[:, 16 * t:16 * (t + 1)].std() for t in range(3)])
            local_ir = (local_ir * idx + alpha * std) / (idx + 1)
            shared = mean_over_replicas(std.clone())
            ir = (ir * idx + alpha * shared) / (idx + 1)
            idx = idx + 1
        torch.save((ir, local_ir), os.path.join(out_dir, f"ir{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_shared_tile_statistics_keep_input_ranges_identical(tmp_path):
    world = 2
    mp.spawn(_ir_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    (a, a_local), (b, b_local) = torch.load(tmp_path / "ir0.pt"), torch.load(tmp_path / "ir1.pt")
    assert torch.equal(a, b)                    # replicas agree bit for bit
    assert not torch.allclose(a_local, b_local)  # the purely local updates would have diverged


def test_mean_over_replicas_is_the_identity_without_a_group():
    v = torch.tensor([1.0, 2.0])
    assert mean_over_replicas(v) is v and v.tolist() == [1.0, 2.0]
