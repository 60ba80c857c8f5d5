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

    ``attach(params)`` registers a post-accumulate hook on every parameter: as soon as autograd
    has stored a gradient, its all-reduce (in place, on ``param.grad``) is issued on a side stream.
    Installed as ``nn.functional.settings.after_wgrad`` the instance is also told the moment an
    analog layer's weight-gradient kernels are enqueued -- before its input-gradient kernels --
    and the exchange of that gradient then waits only for that point, so it runs beside the
    input-gradient kernels.  ``finish()`` makes the compute stream wait for all exchanges and
    averages; call it before the optimizer step.
    """

    def __init__(self, group: Optional[dist.ProcessGroup] = None, average: bool = True):
        self.group = group
        self.average = average
        self.side: Optional[torch.cuda.Stream] = None
        self._ready: dict = {}  # data_ptr of a weight gradient -> event recorded when it was enqueued
        self._pending: List[Tuple[torch.Tensor, "dist.Work"]] = []
        self._keep: list = []

    def attach(self, params: Iterable[torch.nn.Parameter]) -> "EagerGradientSync":
        for p in params:
            if p.requires_grad:
                p.register_post_accumulate_grad_hook(self._reduce)
        return self

    def __call__(self, grad: torch.Tensor, progress=None) -> None:
        """``after_wgrad`` hook: remember when this gradient was complete on the compute stream, or,
        in chunked mode, the flags that say which of its rows are (only the gradient's address is
        kept: a second reference would make autograd copy the tensor)."""
        if len(self._ready) > 64:
            self._ready.clear()
        if progress is not None:
            self._ready[grad.data_ptr()] = progress
            return
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(grad.device))
        self._ready[grad.data_ptr()] = ready

    def _reduce(self, param: torch.nn.Parameter) -> None:
        grad = param.grad
        if grad is None:
            return
        if not grad.is_cuda:  # host tensors (gloo): no streams to order, the exchange itself is asynchronous
            self._pending.append((grad, dist.all_reduce(grad, op=dist.ReduceOp.SUM, group=self.group, async_op=True)))
            return
        if self.side is None:
            self.side = torch.cuda.Stream(grad.device)
        # the early event is only valid if autograd kept the very tensor the layer produced
        ready = self._ready.pop(grad.data_ptr(), None)
        if ready is not None and hasattr(ready, "flags"):
            self._reduce_chunks(grad, ready)
            return
        if ready is None:
            ready = torch.cuda.Event()
            ready.record(torch.cuda.current_stream(grad.device))
        with torch.cuda.stream(self.side):
            self.side.wait_event(ready)
            work = dist.all_reduce(grad, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        self._pending.append((grad, work))

    def _reduce_chunks(self, grad: torch.Tensor, progress) -> None:
        """One all-reduce per chunk of rows, each held back on the side stream until the
        weight-gradient kernel has raised the chunk's flag."""
        from . import _lib  # pylint: disable=import-outside-toplevel

        lib = _lib.load()
        rows, total = progress.rows, grad.shape[0]
        self.side.wait_event(progress.zeroed)  # never look at flags of an earlier use of that memory
        base = progress.flags.data_ptr()
        for c in range(progress.flags.numel()):
            lo, hi = c * rows, min(total, (c + 1) * rows)
            if lo >= hi:
                break
            _lib.check(lib.al_stream_wait_value32(self.side.cuda_stream, base + 4 * c, 1))
            part = grad[lo:hi]
            with torch.cuda.stream(self.side):
                work = dist.all_reduce(part, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
            self._pending.append((part, work))
        self._keep.append(progress)  # the flags must outlive the waits

    def finish(self) -> None:
        world = dist.get_world_size(self.group)
        for grad, work in self._pending:
            work.wait()  # the current (compute) stream waits for the exchange
            if self.average:
                grad.div_(world)
        self._pending.clear()
        self._keep.clear()
