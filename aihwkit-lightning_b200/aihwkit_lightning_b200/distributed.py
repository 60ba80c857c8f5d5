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


class PeerGradientSync(EagerGradientSync):
    """``EagerGradientSync`` whose large gradients are summed by the library's own peer-memory kernel
    (``al_peer_allreduce``) instead of a library collective.

    The weight gradients of the analog layers live in one buffer per dtype that every replica has
    mapped (PyTorch symmetric memory: NVLink peer mappings and, where the switch offers it, a
    multicast address).  Installed as ``settings.grad_w_alloc`` the instance makes the backward write
    each weight gradient straight into its place in that buffer; the moment the layer's
    weight-gradient kernels are enqueued, a kernel of ``n_ctas`` CTAs on the side stream signals the
    peers, reduces this rank's slice of the gradient over all replicas (through the switch with
    ``multimem`` when ``use_multicast``), writes it to every replica and waits for the peers' slices --
    beside the input-gradient GEMM, which leaves ``comm_sms`` SMs free for it.  Everything else (small
    gradients, gradients autograd did not leave in the buffer) goes the way of the base class.
    """

    def __init__(self, params: Iterable[torch.nn.Parameter], group: Optional[dist.ProcessGroup] = None,
                 average: bool = True, small_numel: int = 1 << 16, n_ctas: int = 16, use_multicast: bool = True):
        super().__init__(group=group, average=average, small_numel=small_numel)
        import torch.distributed._symmetric_memory as symm_mem  # pylint: disable=import-outside-toplevel

        from . import _lib  # pylint: disable=import-outside-toplevel

        self._lib = _lib
        self._peer_pending: list = []
        self.n_ctas = n_ctas
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._params = [p for p in params if p.requires_grad]
        self._slot: dict = {}    # weight address -> (parameter, pool, element offset)
        self._pools: dict = {}   # dtype -> pool
        group_obj = group if group is not None else dist.group.WORLD
        by_dtype: dict = {}
        for p in self._params:
            if p.is_cuda and p.numel() >= small_numel and p.dtype in (torch.bfloat16, torch.float32) \
                    and p.numel() % 8 == 0 and p.dim() == 2:
                by_dtype.setdefault(p.dtype, []).append(p)
        for dtype, plist in by_dtype.items():
            total = sum((p.numel() + 127) // 128 * 128 for p in plist)
            flat = symm_mem.empty(total, dtype=dtype, device=plist[0].device)
            handle = symm_mem.rendezvous(flat, group_obj)
            need = 4 * (_lib.AL_PEER_SIGNAL_SLOT + 9)
            if handle.signal_pad_size < need:
                raise RuntimeError(f"signal pads of {handle.signal_pad_size} bytes, {need} needed")
            import ctypes  # pylint: disable=import-outside-toplevel
            pool = dict(
                flat=flat, handle=handle, calls=0,
                bufs=(ctypes.c_uint64 * self.world)(*[int(a) for a in handle.buffer_ptrs]),
                pads=(ctypes.c_uint64 * self.world)(*[int(a) for a in handle.signal_pad_ptrs]),
                mc=int(handle.multicast_ptr) if (use_multicast and handle.has_multicast_support) else 0)
            self._pools[dtype] = pool
            offset = 0
            for p in plist:
                self._slot[p.data_ptr()] = (p, pool, offset)
                offset += (p.numel() + 127) // 128 * 128
        self.attach(self._params)

    def grad_buffer(self, weight_address: int, shape, dtype):
        """``settings.grad_w_alloc``: the place of this weight's gradient in the shared buffer, as a fresh
        view (autograd keeps a gradient it alone refers to, and copies one that is referred to twice)."""
        slot = self._slot.get(weight_address)
        if slot is None:
            return None
        param, pool, offset = slot
        if param.grad is not None or pool["flat"].dtype != dtype or tuple(param.shape) != tuple(shape):
            return None  # accumulation into an older gradient: let autograd handle it
        return pool["flat"][offset:offset + param.numel()].view(param.shape)

    def _reduce(self, param: torch.nn.Parameter) -> None:
        grad = param.grad
        slot = self._slot.get(param.data_ptr()) if grad is not None else None
        if slot is not None:
            _, pool, offset = slot
            flat = pool["flat"]
            if grad.data_ptr() == flat.data_ptr() + offset * flat.element_size() and grad.is_contiguous():
                self._peer_reduce(grad, pool, offset)
                return
        super()._reduce(param)

    def _peer_reduce(self, grad: torch.Tensor, pool: dict, offset: int) -> None:
        lib = self._lib.load()
        if self.side is None:
            self.side = torch.cuda.Stream(grad.device)
        ready = self._ready.pop((grad.data_ptr(), tuple(grad.shape)), None)
        if ready is None:
            ready = torch.cuda.Event()
            ready.record(torch.cuda.current_stream(grad.device))
        self.side.wait_event(ready)
        flat = pool["flat"]
        dtype_code = self._lib.AL_BF16 if flat.dtype == torch.bfloat16 else self._lib.AL_F32
        scale = 1.0 / self.world if self.average else 1.0
        self._lib.check(lib.al_peer_allreduce(dtype_code, self.world, self.rank, pool["bufs"], pool["pads"], pool["mc"],
                                              offset * flat.element_size(), grad.numel(), pool["calls"], scale,
                                              self.n_ctas, self.side.cuda_stream))
        pool["calls"] += 1
        done = torch.cuda.Event()
        done.record(self.side)
        self._peer_pending.append(done)

    def finish(self) -> None:
        for done in self._peer_pending:
            torch.cuda.current_stream().wait_event(done)
        self._peer_pending = []
        super().finish()
