"""Data-parallel plumbing of the analog layers: one process per GPU, rows (tokens) sharded
across ranks, gradients summed with one collective per bucket.

Every per-row quantity of the analog linear path (dynamic input range, DAC codes, ADC bound,
output noise) is row-local, so a batch splits across ranks without any exchange inside the
forward or backward kernels; the only exchange step of a training step is the all-reduce of
the parameter gradients (weights, biases, learned input ranges).  The reference has no
distributed code of its own -- its examples delegate to DeepSpeed / Accelerate
(`examples/deepspeed_cifar10/cifar10_deepspeed.py:210-268`) -- so this module mirrors what
those do for this path: flat gradient buckets, asynchronous all-reduce on the process group's
stream while the rest of backward runs, averaging by the world size.

Works with any ``torch.distributed`` backend (NCCL on GPUs, gloo in the CPU tests).
"""
from typing import Iterable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_rows(total_rows: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Half-open row range of ``rank`` when ``total_rows`` rows are split as evenly as possible
    (the first ``total_rows % world_size`` ranks get one row more)."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of size {world_size}")
    base, extra = divmod(total_rows, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def rank_seed(seed: int, rank: int) -> int:
    """Per-rank generator seed: replicas must draw independent analog noise."""
    return (seed * 1_000_003 + 7919 * (rank + 1)) & 0x7FFFFFFFFFFFFFFF


def mean_over_replicas(values: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Mean of a small statistics tensor over all replicas (in place, returned for chaining).

    Installed as ``nn.functional.settings.sync_tile_std`` it makes the init-from-data phase of a
    learned input range use the per-tile standard deviation averaged over the replicas, so that
    every replica applies the same update.  The reference updates from the local batch
    (`nn/modules/torch_utils/torch_linear.py:338-352`) and its DeepSpeed example patches around the
    resulting divergence (`examples/deepspeed_and_huggingface/README.md:60-106`)."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(values, op=dist.ReduceOp.SUM, group=group)
        values.div_(dist.get_world_size(group))
    return values


class GradientBuckets:
    """Flat-bucket gradient all-reduce for a fixed list of parameters.

    ``reduce_async`` copies the gradients of one bucket into a flat buffer and launches one
    all-reduce for it; ``finish`` waits for all launched buckets, divides by the world size
    and copies the results back into ``param.grad``.  Buckets follow the reverse parameter
    order (the order backward produces gradients in), capped at ``bucket_bytes``.
    """

    def __init__(self, params: Iterable[torch.nn.Parameter], bucket_bytes: int = 64 << 20,
                 group: Optional[dist.ProcessGroup] = None, average: bool = True):
        self.params: List[torch.nn.Parameter] = [p for p in params if p.requires_grad]
        self.group = group
        self.average = average
        self.buckets: List[List[torch.nn.Parameter]] = []
        current: List[torch.nn.Parameter] = []
        size = 0
        for p in reversed(self.params):
            nbytes = p.numel() * p.element_size()
            if current and (size + nbytes > bucket_bytes or p.dtype != current[0].dtype
                            or p.device != current[0].device):
                self.buckets.append(current)
                current, size = [], 0
            current.append(p)
            size += nbytes
        if current:
            self.buckets.append(current)
        self._flat: List[Optional[torch.Tensor]] = [None] * len(self.buckets)
        self._pending: List[Tuple[int, "dist.Work"]] = []

    def bucket_sizes(self) -> List[int]:
        return [sum(p.numel() for p in b) for b in self.buckets]

    def reduce_async(self, index: int) -> None:
        bucket = self.buckets[index]
        total = sum(p.numel() for p in bucket)
        flat = self._flat[index]
        if flat is None or flat.numel() != total:
            flat = torch.empty(total, dtype=bucket[0].dtype, device=bucket[0].device)
            self._flat[index] = flat
        offset = 0
        for p in bucket:
            n = p.numel()
            if p.grad is None:
                flat[offset:offset + n].zero_()
            else:
                flat[offset:offset + n].copy_(p.grad.reshape(-1))
            offset += n
        work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        self._pending.append((index, work))

    def reduce_all_async(self) -> None:
        for i in range(len(self.buckets)):
            self.reduce_async(i)

    def finish(self) -> None:
        world = dist.get_world_size(self.group)
        for index, work in self._pending:
            work.wait()
            flat = self._flat[index]
            if self.average:
                flat.div_(world)
            offset = 0
            for p in self.buckets[index]:
                n = p.numel()
                if p.grad is None:
                    p.grad = flat[offset:offset + n].reshape(p.shape).clone()
                else:
                    p.grad.copy_(flat[offset:offset + n].reshape(p.shape))
                offset += n
        self._pending.clear()


def all_reduce_gradients(params: Sequence[torch.nn.Parameter], group: Optional[dist.ProcessGroup] = None,
                         bucket_bytes: int = 64 << 20) -> None:
    """One-shot helper: average the gradients of ``params`` over the group."""
    buckets = GradientBuckets(params, bucket_bytes=bucket_bytes, group=group)
    buckets.reduce_all_async()
    buckets.finish()


class EagerGradientSync:
    """Sums gradients over the replicas while the backward pass is still running.

    ``attach(params)`` registers a post-accumulate hook on every parameter.  A large gradient
    (at least ``small_numel`` elements: the weight matrices) is all-reduced in place on a side
    stream the moment autograd has stored it, so the exchange of layer L runs beside the backward
    kernels of layers L-1 .. 0.  Small gradients (norm weights, biases, learned input ranges) are
    copied into one flat buffer and exchanged by a single call in ``finish()``: a collective per
    tiny tensor costs more in launch latency than its bytes.  Installed as
    ``nn.functional.settings.after_wgrad`` the instance is also told the moment an analog layer's
    weight-gradient kernels are enqueued -- before its input-gradient kernels -- and the exchange
    of that gradient then waits only for that point.  ``finish()`` makes the compute stream wait
    for all exchanges and averages; call it before the optimizer step.
    """

    def __init__(self, group: Optional[dist.ProcessGroup] = None, average: bool = True,
                 small_numel: int = 1 << 16):
        self.group = group
        self.average = average
        self.small_numel = small_numel
        self.side: Optional[torch.cuda.Stream] = None
        # (address, shape) of a weight gradient -> event recorded when its kernels were enqueued;
        # entries live for one backward pass only (``finish`` drops what autograd never claimed)
        self._ready: dict = {}
        self._pending: List[Tuple[torch.Tensor, "dist.Work"]] = []
        self._small: List[torch.Tensor] = []
        self._flat: Optional[torch.Tensor] = None

    def attach(self, params: Iterable[torch.nn.Parameter]) -> "EagerGradientSync":
        for p in params:
            if p.requires_grad:
                p.register_post_accumulate_grad_hook(self._reduce)
        return self

    def __call__(self, grad: torch.Tensor) -> None:
        """``after_wgrad`` hook: remember when this gradient was complete on the compute stream (only
        the gradient's address and shape are kept: a second reference would make autograd copy the
        tensor)."""
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(grad.device))
        self._ready[(grad.data_ptr(), tuple(grad.shape))] = ready

    def _reduce(self, param: torch.nn.Parameter) -> None:
        grad = param.grad
        if grad is None:
            return
        if grad.numel() < self.small_numel:
            self._small.append(grad)
            return
        if not grad.is_cuda:  # host tensors (gloo): no streams to order, the exchange itself is asynchronous
            self._pending.append((grad, dist.all_reduce(grad, op=dist.ReduceOp.SUM, group=self.group, async_op=True)))
            return
        if self.side is None:
            self.side = torch.cuda.Stream(grad.device)
        # The early event is valid only if autograd kept the very tensor the layer produced (same
        # address and shape).  When it accumulated into an older ``.grad`` or copied the gradient,
        # the exchange waits for the compute stream as it stands now.
        ready = self._ready.pop((grad.data_ptr(), tuple(grad.shape)), None)
        if ready is None:
            ready = torch.cuda.Event()
            ready.record(torch.cuda.current_stream(grad.device))
        with torch.cuda.stream(self.side):
            self.side.wait_event(ready)
            work = dist.all_reduce(grad, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        self._pending.append((grad, work))

    def _reduce_small(self) -> None:
        if not self._small:
            return
        groups: dict = {}
        for g in self._small:
            groups.setdefault((g.dtype, g.device), []).append(g)
        for grads in groups.values():
            flat = torch.cat([g.reshape(-1) for g in grads])
            dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group)
            if self.average:
                flat.div_(dist.get_world_size(self.group))
            offset = 0
            for g in grads:
                n = g.numel()
                g.copy_(flat[offset:offset + n].reshape(g.shape))
                offset += n
        self._small.clear()

    def finish(self) -> None:
        world = dist.get_world_size(self.group)
        self._reduce_small()
        for grad, work in self._pending:
            work.wait()  # the current (compute) stream waits for the exchange
            if self.average:
                grad.div_(world)
        self._pending.clear()
        # an event autograd never claimed belongs to a tensor that is gone; its address may come back
        self._ready.clear()
