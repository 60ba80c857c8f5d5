"""Benchmark of the analog linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--config c2|c1|c3|c4|c5]

Default workload (``--config c2``, N=1): the configuration the headline metric is quoted on --
``AnalogLinear`` 4096 -> 4096 in bf16, 8192 tokens ~N(0,1), ``max_input_size=512`` (8 analog
tiles), dynamic per-token input ranges with an 8-bit DAC, 8-bit ADC with ``out_bound=10``,
``out_noise=0.04``, weight noise 0.02 relative to the per-channel abs-max, training mode,
forward + backward.  A "step" is one forward + backward over one batch of synthetic tokens; the
metric is algorithmic TFLOP/s = 6*M*K*N / time.

* ``value``: inputs resident in HBM, CUDA-event timing over exactly K steps (max over ranks).
* ``e2e``: the same step through the public ``AnalogLinear`` call with the batch in pinned
  host memory: every step uploads its batch (double-buffered on a copy stream, so the upload
  of the next batch overlaps the current step) and copies its loss back to pinned host memory,
  where the host reads it one step later; all inside the timed region.  The upload is 67 MB per
  0.8 ms step, so this number is bound by the host link, not by the kernels.
* ``roofline``: the dominant kernel, timed live with CUDA events by the library's launch
  accounting, against the measured burst bf16 tensor peak (the timed region lasts milliseconds).
* ``cpu_baseline`` / ``--impl reference``: the CPU restatement of the reference's torch path
  (``oracle/analog_oracle.py::linear_autograd``) timed on the host cores on a bounded sample
  of the workload (fewer rows, same K, N and tiling).
* ``gpu_torch_baseline`` (N=1): the same restatement of the reference's torch path run on CUDA
  tensors of the full workload (cuBLAS per-tile GEMMs + eager element-wise kernels), timed after
  the library's own measurement: what the reference's torch backend costs on the same GPU.
* ``c3``: one full data-parallel training step of the Phi-3-mini-shaped decoder (32 layers,
  d=3072, MLP 8192, vocab 32064, every Linear analog, sequence 2048 x micro-batch 4 per GPU, AdamW),
  timed after the headline: tokens/s, analog TFLOP/s and the exposed part of the gradient exchange.
* N > 1 (torchrun): every rank runs on its own batch (weak scaling) and the weight gradients are
  summed over the replicas as in data-parallel training, by the library's own exchange kernel over
  peer memory (``BENCH_EXCHANGE=nccl``: by NCCL all-reduce calls instead).

``--config c1 | c4 | c5`` measure the other benchmark configurations with the same line format
(c1: the fp32 1024 x 1024 layer; c4: a ResNet-32 training step; c5: the inference shape sweep);
``--config c3`` prints the decoder step as a line of its own.
"""
import argparse
import json
import os
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "aihwkit-lightning_b200"))

M, K, N, MAX_IN = 8192, 4096, 4096, 512
CPU_SAMPLE_ROWS = 1024
FLOP_PER_STEP = 6.0 * M * K * N
L2_FLUSH_BYTES = 256 << 20
# DRAM bytes (read + write) of one forward-GEMM launch on the headline workload, from the ncu
# capture summarised in profiles/fwd_tc_kernel_c2.md
FWD_KERNEL_DRAM_BYTES = 119.6e6 + 77.4e6


def make_rpu_config(ns, max_in=MAX_IN, adc=True, out_noise=0.04, dynamic=True):
    rpu = ns.TorchInferenceRPUConfig()
    rpu.mapping.max_input_size = max_in
    rpu.forward.inp_res = 254.0
    if adc:
        rpu.forward.out_res = 254.0
        rpu.forward.out_bound = 10.0
    rpu.forward.out_noise = out_noise
    rpu.pre_post.input_range.enable = True
    rpu.pre_post.input_range.dynamic = dynamic
    rpu.modifier.noise_type = ns.WeightNoiseInjectionType.ADD_NORMAL_PER_CHANNEL
    rpu.modifier.std_dev = 0.02
    return rpu


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return dict(source="measured", hbm_gbs=p["hbm_gbs"], bf16=p["bf16_tflops"],
                    bf16_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]))
    return dict(source="fallback", hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                sm_max.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return dict(sm_mhz=sm[len(sm) // 2] if sm else None, sm_max_mhz=max(sm_max) if sm_max else None,
                    samples=len(sm), reasons=sorted(reasons))


# ---------------------------------------------------------------------------------------------
# reference arm / baselines (the only places that execute oracle/)
# ---------------------------------------------------------------------------------------------
def cpu_reference_run(steps: int, warmup: int, rows: int):
    """Time the CPU restatement of the reference's torch path (autograd flavour) on ``rows``
    rows of the workload with all host threads."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import analog_oracle as O
    from aihwkit_lightning_b200.simulator import configs as cfg

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    rpu = make_rpu_config(cfg)
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(rows, K, generator=gen).bfloat16()
    lin = torch.nn.Linear(K, N, bias=False)
    w = lin.weight.detach().bfloat16().requires_grad_(True)
    g = torch.randn(rows, N, generator=gen).bfloat16()
    in_sizes = O.split_sizes(K, MAX_IN)
    # bound the whole run to a few minutes: time one step, then shrink the row sample if needed
    t0 = time.perf_counter()
    O.linear_autograd(x.clone().requires_grad_(True), w, None, None, None, in_sizes, True, rpu).backward(g)
    first = time.perf_counter() - t0
    limit_s = 150.0
    if first * (warmup + steps) > limit_s:
        rows = max(128, int(rows * limit_s / (first * (warmup + steps))) // 128 * 128)
        x, g = x[:rows].contiguous(), g[:rows].contiguous()
    times = []
    for it in range(warmup + steps):
        xin = x.clone().requires_grad_(True)
        w.grad = None
        t0 = time.perf_counter()
        out = O.linear_autograd(xin, w, None, None, None, in_sizes, True, rpu)
        out.backward(g)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    sec = sum(times) / len(times)
    flop = 6.0 * rows * K * N
    return dict(value=flop / sec / 1e12, unit="TFLOP/s", cores=threads, kind="port",
                sample=f"{rows} of {M} rows, same K={K}, N={N}, 8 tiles; {len(times)} timed steps, "
                       f"{sec * 1e3:.0f} ms/step", ms_per_step=sec * 1e3)


def gpu_torch_baseline(dev, steps=5, warmup=2):
    """The reference's torch path (its op sequence under autograd, restated in
    ``oracle/analog_oracle.py::linear_autograd``) on CUDA tensors of the full headline workload:
    per-tile cuBLAS GEMMs and eager element-wise kernels on the same GPU."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import analog_oracle as O
    from aihwkit_lightning_b200.simulator import configs as cfg

    rpu = make_rpu_config(cfg)
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(M, K, generator=gen).bfloat16().to(dev).requires_grad_(True)
    torch.manual_seed(0)
    w = torch.nn.Linear(K, N, bias=False).weight.detach().bfloat16().to(dev).requires_grad_(True)
    g = torch.randn(M, N, generator=gen).bfloat16().to(dev)
    in_sizes = O.split_sizes(K, MAX_IN)
    stream = torch.cuda.current_stream(dev)
    events = []
    for it in range(warmup + steps):
        x.grad = None
        w.grad = None
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(stream)
        O.linear_autograd(x, w, None, None, None, in_sizes, True, rpu).backward(g)
        e.record(stream)
        if it >= warmup:
            events.append((s, e))
    torch.cuda.synchronize(dev)
    ms = sum(s.elapsed_time(e) for s, e in events) / len(events)
    del x, w, g
    torch.cuda.empty_cache()
    return dict(ms_per_step=ms, value=FLOP_PER_STEP / (ms * 1e-3) / 1e12, unit="TFLOP/s",
                what="reference torch op sequence (oracle restatement) on CUDA tensors, bf16, same workload, "
                     f"{len(events)} timed steps")


def base_record(args, n_gpus):
    return {
        "metric": "analog-layer fwd+bwd TFLOP/s",
        "unit": "TFLOP/s",
        "n_gpus": n_gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "config": {
            "workload": f"AnalogLinear {K}->{N} bf16, {M} tokens/GPU ~N(0,1), max_input_size={MAX_IN} (8 tiles), "
                        "dynamic input range, 8-bit DAC, 8-bit ADC out_bound=10, out_noise=0.04, "
                        "weight noise 0.02 per-channel, training fwd+bwd",
            "l2": "inputs larger than L2 (x 67 MB + w 34 MB + g 67 MB per step) and a 256 MB flush write between steps",
            "e2e": "bound by the host link: every step uploads its 67 MB batch from pinned host memory "
                   "(double-buffered) and reads its loss back",
            "parallelism": f"dp{n_gpus}",
        },
    }


def run_reference(args, rank, world):
    if rank != 0:
        return
    res = cpu_reference_run(args.steps, args.warmup, CPU_SAMPLE_ROWS)
    rec = base_record(args, world)
    rec.update({
        "impl": "reference",
        "value": res["value"],
        "ms_per_step": res["ms_per_step"],
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": res["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    })
    print(json.dumps(rec), flush=True)


# ---------------------------------------------------------------------------------------------
# shared helpers of the GPU arms
# ---------------------------------------------------------------------------------------------
class Ctx:
    """Rank, device and process group of one bench process."""

    def __init__(self):
        import torch.distributed as dist

        self.dist = dist
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.stream = torch.cuda.current_stream(self.dev)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier(device_ids=[self.local_rank])
        torch.cuda.synchronize(self.dev)

    def max_over_ranks(self, value: float) -> float:
        t = torch.tensor([value], device=self.dev, dtype=torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def make_gradient_sync(ctx, params, n_ctas=None, multicast_from=None):
    """Gradient exchange of the data-parallel arms: the library's peer-memory kernel
    (``PeerGradientSync``) when the replicas can map one another's memory, NCCL all-reduce otherwise or
    when BENCH_EXCHANGE=nccl.  Returns (sync, description)."""
    from aihwkit_lightning_b200.distributed import EagerGradientSync, PeerGradientSync
    from aihwkit_lightning_b200.nn import functional as F

    params = list(params)
    sync, how = None, None
    n_ctas = int(os.environ.get("BENCH_COMM_CTAS", "16")) if n_ctas is None else n_ctas
    if os.environ.get("BENCH_EXCHANGE", "peer") == "peer":
        try:
            # multicast_from: replica count from which the reduction runs in the switch (multimem): a rank then
            # moves 2/N of the buffer through its SMs instead of all of it
            multicast_env = os.environ.get("BENCH_MULTICAST", "auto")
            auto = multicast_from is not None and ctx.world >= multicast_from
            sync = PeerGradientSync(params, n_ctas=n_ctas,
                                    use_multicast=multicast_env == "1" or (multicast_env == "auto" and auto))
            F.settings.grad_w_alloc = sync.grad_buffer
            multicast = any(pool["mc"] for pool in sync._pools.values())  # pylint: disable=protected-access
            how = (f"library kernel over peer memory ({n_ctas} CTAs beside the input-gradient GEMM, "
                   f"{'switch reduction (multimem)' if multicast else 'peer loads and stores'}); "
                   "small gradients in one NCCL call")
        except Exception as exc:  # pylint: disable=broad-except
            if ctx.rank == 0:
                print(f"peer-memory exchange unavailable ({type(exc).__name__}: {exc}); using NCCL", file=sys.stderr)
            sync = None
    if sync is None:
        sync = EagerGradientSync().attach(params)
        how = "NCCL all-reduce per weight matrix on a side stream, small gradients in one flat call"
    # every rank must have taken the same route
    flag = torch.tensor([1.0 if isinstance(sync, PeerGradientSync) else 0.0], device=ctx.dev)
    lo = flag.clone()
    ctx.dist.all_reduce(lo, op=ctx.dist.ReduceOp.MIN)
    if lo.item() != flag.item():
        F.settings.grad_w_alloc = None
        sync = EagerGradientSync().attach(params)
        how = "NCCL all-reduce per weight matrix on a side stream (peer mapping failed on a rank)"
    F.settings.after_wgrad = sync
    return sync, how


def release_gradient_sync():
    from aihwkit_lightning_b200.nn import functional as F

    F.settings.after_wgrad = None
    F.settings.grad_w_alloc = None
    F.settings.comm_sms = 0
    F.settings.comm_sms_wgrad = 0


def timed_steps(ctx, fn, steps, between=None):
    """CUDA-event time (ms) of exactly `steps` calls of fn on the current stream; what `between`
    does before each call (the L2 flush) is not timed."""
    events = []
    for _ in range(steps):
        if between is not None:
            between()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(ctx.stream)
        fn()
        e.record(ctx.stream)
        events.append((s, e))
    torch.cuda.synchronize(ctx.dev)
    return sum(s.elapsed_time(e) for s, e in events)


def capture_step(step, dev):
    """One call of `step` as a CUDA graph.  The analog noise counters come from a ``GraphNoise``, whose
    device-side counter the graph advances as its first node, so every replay draws fresh noise."""
    from aihwkit_lightning_b200.nn import functional as F

    noise = F.GraphNoise(dev)
    F.settings.graph_noise = noise

    def body():
        noise.advance()
        return step()

    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        for _ in range(3):
            body()
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize(dev)
    torch.cuda.empty_cache()  # the capture allocates from a pool of its own
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        body()
    F.settings.graph_noise = None
    return graph


# In the forward of a large layer the weight pre-pass (class weight_modify) runs on a second stream beside the DAC
# pass (class dac): their two durations overlap in time, so the sum over classes exceeds the time the stream was busy.
KERNELS_NOTE = ("per class: CUDA events around every library launch; dac and weight_modify of a large layer run "
                "concurrently on two streams, so their times overlap and a sum over classes counts that span twice")


def kernel_table(prof):
    out = {}
    for name, (launches, timed_scopes, total) in prof.items():
        if launches:
            out[name] = dict(launches=launches, ms_total=round(total, 4), ms_avg=round(total / max(timed_scopes, 1), 5))
    return out


# ---------------------------------------------------------------------------------------------
# config 3: Phi-3-mini-shaped decoder, one data-parallel training step
# ---------------------------------------------------------------------------------------------
def build_decoder(dev, layers=32, d=3072, heads=32, mlp=8192, vocab=32064):
    from torch import nn
    from torch.nn import functional as TF
    from torch.nn.attention import SDPBackend, sdpa_kernel

    from aihwkit_lightning_b200.nn.decoder_ops import rotary_qkv, swiglu

    # cuDNN's attention first (1.1 ms per layer forward + backward at these shapes against 2.0 ms)
    ATTENTION_BACKENDS = [SDPBackend.CUDNN_ATTENTION, SDPBackend.FLASH_ATTENTION, SDPBackend.EFFICIENT_ATTENTION]

    class RMSNorm(nn.Module):
        def __init__(self, dim, eps=1e-5):
            super().__init__()
            self.weight = nn.Parameter(torch.ones(dim))
            self.eps = eps

        def forward(self, x):
            return TF.rms_norm(x, (x.shape[-1],), self.weight, self.eps)

    class Layer(nn.Module):
        def __init__(self):
            super().__init__()
            self.norm1, self.norm2 = RMSNorm(d), RMSNorm(d)
            self.qkv_proj = nn.Linear(d, 3 * d, bias=False)
            self.o_proj = nn.Linear(d, d, bias=False)
            self.gate_up_proj = nn.Linear(d, 2 * mlp, bias=False)
            self.down_proj = nn.Linear(mlp, d, bias=False)

        def forward(self, x, cos, sin):
            b, s, _ = x.shape
            hd = d // heads
            # rotary embedding of q and k and the split of the fused projection in one pass of the library
            q, k, v = (t.transpose(1, 2) for t in rotary_qkv(self.qkv_proj(self.norm1(x)).view(b, s, 3, heads, hd), cos, sin))
            with sdpa_kernel(ATTENTION_BACKENDS, set_priority=True):
                att = TF.scaled_dot_product_attention(q, k, v, is_causal=True)
            x = x + self.o_proj(att.transpose(1, 2).reshape(b, s, d))
            return x + self.down_proj(swiglu(self.gate_up_proj(self.norm2(x))))

    class Decoder(nn.Module):
        def __init__(self):
            super().__init__()
            self.embed = nn.Embedding(vocab, d)
            self.layers = nn.ModuleList([Layer() for _ in range(layers)])
            self.norm = RMSNorm(d)
            self.lm_head = nn.Linear(d, vocab, bias=False)
            self.hd = d // heads

        def forward(self, ids):
            s = ids.shape[1]
            pos = torch.arange(s, device=ids.device, dtype=torch.float32)
            inv = 1.0 / (10000 ** (torch.arange(0, self.hd, 2, device=ids.device, dtype=torch.float32) / self.hd))
            ang = pos[:, None] * inv[None, :]
            cos, sin = ang.cos(), ang.sin()  # [s, hd / 2] float32 tables of the rotary embedding
            x = self.embed(ids)
            for layer in self.layers:
                x = layer(x, cos, sin)
            return self.lm_head(self.norm(x))

    with torch.device(dev):
        model = Decoder().to(torch.bfloat16)
    return model


def run_c3(args, ctx, layers=32, steps=3, warmup=2, seq=2048, micro_batch=4):
    """One full data-parallel training step of the decoder: forward, loss, backward with the
    gradient exchange started from inside it, AdamW step.  Returns the fields of the ``c3`` block."""
    from torch.nn import functional as TF

    from aihwkit_lightning_b200 import _lib
    from aihwkit_lightning_b200.distributed import PeerGradientSync, rank_seed
    from aihwkit_lightning_b200.nn import AnalogLinear, convert_to_analog
    from aihwkit_lightning_b200.nn import functional as F
    from aihwkit_lightning_b200.optim import AnalogOptimizer
    from aihwkit_lightning_b200.simulator import configs as cfg

    dev, rank, world = ctx.dev, ctx.rank, ctx.world
    lib = _lib.load()
    vocab = 32064
    torch.manual_seed(0)  # identical replicas
    model = build_decoder(dev, layers=layers, vocab=vocab)
    rpu = make_rpu_config(cfg, adc=False)  # 8-bit DAC, out_noise 0.04, weight noise 0.02, no ADC
    model = convert_to_analog(model, rpu).train()
    analog = [m for m in model.modules() if isinstance(m, AnalogLinear)]
    tokens = seq * micro_batch
    flop = sum(6.0 * tokens * m.in_features * m.out_features for m in analog)
    torch.cuda.manual_seed(rank_seed(0, rank))  # independent analog noise per replica
    opt = AnalogOptimizer(torch.optim.AdamW, model.analog_layers, model.parameters(), lr=1e-5, fused=True,
                          capturable=world == 1)
    sync, how = None, None
    if world > 1:
        # Measured with the 225 ms step.  2 GPUs: plain peer loads on 16 CTAs with 16 SMs left free by the
        # input-gradient GEMMs 232.5 ms, on 8 CTAs / 8 SMs 245.2, switch reduction on 8 CTAs 243.3.  8 GPUs: switch
        # reduction on 8 CTAs / 8 SMs 241.6 ms, plain loads on 16 CTAs 244.1, on 8 CTAs 257.2 (15.7 ms exposed).
        # So: plain loads on 16 CTAs below 4 replicas, the reduction in the switch on 8 CTAs from 4 on.
        few = world < 4
        sync, how = make_gradient_sync(ctx, model.parameters(),
                                       n_ctas=int(os.environ.get("BENCH_C3_COMM_CTAS", "16" if few else "8")),
                                       multicast_from=4)
        if isinstance(sync, PeerGradientSync):
            F.settings.comm_sms = int(os.environ.get("BENCH_C3_COMM_SMS", "16" if few else "8"))
            F.settings.comm_sms_wgrad = int(os.environ.get("BENCH_C3_COMM_SMS_WGRAD", "0"))
            how += f"; backward GEMMs leave {F.settings.comm_sms} (input gradient) / {F.settings.comm_sms_wgrad} (weight gradient) SMs free"
    gen = torch.Generator().manual_seed(1000 + rank)
    ids_host = torch.randint(0, vocab, (micro_batch, seq), generator=gen).pin_memory()
    labels_host = torch.randint(0, vocab, (micro_batch, seq), generator=gen).pin_memory()
    exposed = []
    losses = []

    def step():
        ids = ids_host.to(dev, non_blocking=True)
        labels = labels_host.to(dev, non_blocking=True)
        opt.zero_grad(set_to_none=True)
        logits = model(ids)
        loss = TF.cross_entropy(logits.float().view(-1, vocab), labels.view(-1))
        loss.backward()
        if sync is not None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(ctx.stream)
            sync.finish()  # the compute stream waits here for what is left of the exchange
            e1.record(ctx.stream)
            exposed.append((e0, e1))
        opt.step()
        losses.append(loss.detach())

    for _ in range(warmup):
        step()
    ctx.barrier()
    exposed.clear()
    losses.clear()
    _lib.profile_read(reset=True)
    host_t0 = time.perf_counter()
    ms_total = timed_steps(ctx, step, steps)
    host_ms = (time.perf_counter() - host_t0) * 1e3 / steps  # includes the wait for the last step's kernels
    ctx.barrier()
    ms_step = ctx.max_over_ranks(ms_total) / steps
    exposed_ms = sum(a.elapsed_time(b) for a, b in exposed) / max(len(exposed), 1) if exposed else 0.0
    exposed_ms = ctx.max_over_ranks(exposed_ms)
    launches = sum(v[0] for v in _lib.profile_read(reset=True).values()) // steps
    # once more with every library kernel bracketed by events: the analog share of the step
    lib.al_profile_enable(1)
    timed_steps(ctx, step, steps)
    ctx.barrier()
    lib.al_profile_enable(0)
    prof = _lib.profile_read(reset=True)
    graph_ms = None
    if world == 1 and os.environ.get("BENCH_C3_GRAPH", "1") == "1":
        # the whole step as one CUDA graph (single GPU: the exchange kernels take their call counters by value)
        losses.clear()
        graph = capture_step(step, dev)
        for _ in range(2):
            graph.replay()
        graph_ms = timed_steps(ctx, graph.replay, steps) / steps
        del graph
    # replicas must hold the same parameters after the steps: compare a checksum over all ranks
    checksum = torch.stack([p.detach().double().sum() for p in list(model.parameters())[:16]]).sum().reshape(1)
    lo, hi = checksum.clone(), checksum.clone()
    if world > 1:
        ctx.dist.all_reduce(lo, op=ctx.dist.ReduceOp.MIN)
        ctx.dist.all_reduce(hi, op=ctx.dist.ReduceOp.MAX)
    grad_bytes = sum(p.numel() * p.element_size() for p in model.parameters())
    analog_ms = sum(v[2] for v in prof.values()) / steps
    out = {
        "workload": f"Phi-3-mini-shaped decoder, {layers} layers, d=3072, 32 heads, MLP 8192, vocab {vocab}, "
                    f"{len(analog)} analog linears (max_input_size=512, dynamic input range, 8-bit DAC, out_noise 0.04, "
                    f"weight noise 0.02), seq {seq} x micro-batch {micro_batch} per GPU, bf16, AdamW, random init, "
                    "uniform synthetic token ids",
        "n_gpus": world,
        "steps": steps,
        "warmup": warmup,
        "ms_per_step": ms_step,
        "host_ms_per_step": host_ms,
        "graph_ms_per_step": graph_ms,
        "tokens_per_s": tokens * world / (ms_step * 1e-3),
        "analog_tflops": flop * world / (ms_step * 1e-3) / 1e12,
        "analog_flop_per_gpu_step": flop,
        "analog_kernel_ms_per_step": analog_ms,
        "exposed_exchange_ms": exposed_ms,
        "exchange": None if world == 1 else
        f"{grad_bytes / 1e9:.2f} GB of gradients per step, each weight matrix exchanged from inside backward: {how}",
        "loss": float(losses[-1].item()),
        "replicas_identical": bool((lo == hi).all().item()),
        "gpu_launches": launches,
        "kernels": kernel_table(prof), "kernels_note": KERNELS_NOTE,
    }
    release_gradient_sync()
    del model, opt, analog, sync
    torch.cuda.empty_cache()
    return out


# ---------------------------------------------------------------------------------------------
# config 2 (headline): one analog layer, forward + backward
# ---------------------------------------------------------------------------------------------
def run_c2(args, ctx):
    from aihwkit_lightning_b200 import _lib
    from aihwkit_lightning_b200.distributed import PeerGradientSync, rank_seed
    from aihwkit_lightning_b200.nn import AnalogLinear
    from aihwkit_lightning_b200.nn import functional as F
    from aihwkit_lightning_b200.simulator import configs as cfg

    dev, rank, world, stream = ctx.dev, ctx.rank, ctx.world, ctx.stream
    lib = _lib.load()
    F.settings.engine = args.engine

    # synthetic data, seeded on the CPU so that the CPU baseline sees the same distribution
    gen = torch.Generator().manual_seed(rank)
    x_host = torch.randn(M, K, generator=gen).bfloat16().pin_memory()
    g = torch.randn(M, N, generator=gen).bfloat16().to(dev)
    torch.manual_seed(0)  # identical weights on every replica
    layer = AnalogLinear(K, N, bias=False, rpu_config=make_rpu_config(cfg)).to(device=dev, dtype=torch.bfloat16)
    layer.train()
    torch.cuda.manual_seed(rank_seed(0, rank))  # independent analog noise per replica
    # The only exchange step of data-parallel training: the weight gradient is summed over ranks.
    # Its all-reduce is issued from a hook inside backward, right after the weight-gradient kernel
    # and before the input-gradient kernel, and is complete when the step ends, as an optimizer
    # step would need it.
    sync, how = None, None
    if world > 1:
        sync, how = make_gradient_sync(ctx, layer.parameters())
        # SMs the input-gradient GEMM leaves to the exchange kernel that runs beside it
        default_sms = "16" if isinstance(sync, PeerGradientSync) else "0"
        F.settings.comm_sms = int(os.environ.get("BENCH_COMM_SMS", default_sms))
    x_dev = x_host.to(dev).requires_grad_(True)
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)

    def step_resident():
        layer.weight.grad = None
        x_dev.grad = None
        out = layer(x_dev)
        out.backward(g)
        if sync is not None:
            sync.finish()

    # end to end: the batch lives in pinned host memory; the upload of batch i+1 is enqueued on
    # a copy stream before step i runs (double buffering), every step reads its loss back.
    copy_stream = torch.cuda.Stream(dev)
    slots = [torch.empty(M, K, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    loss_host = [torch.empty(1, dtype=torch.float32).pin_memory() for _ in range(2)]
    loss_done = [torch.cuda.Event() for _ in range(2)]
    state = {"i": 0, "losses": []}

    def upload(slot):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[slot])
            slots[slot].copy_(x_host, non_blocking=True)
            ready[slot].record(copy_stream)

    def step_e2e():
        i = state["i"]
        slot = i & 1
        if i == 0:
            upload(0)
        upload(slot ^ 1)  # next batch, overlaps this step's kernels
        stream.wait_event(ready[slot])
        layer.weight.grad = None
        x = slots[slot].detach().requires_grad_(True)
        out = layer(x)
        loss = (out * g).sum(dtype=torch.float32)
        loss.backward()
        consumed[slot].record(stream)
        if sync is not None:
            sync.finish()
        # device -> host read of this step's loss: copied to pinned memory on the compute stream
        # and picked up by the host one step later, so the host can already enqueue the next step
        loss_host[slot].copy_(loss.detach().reshape(1), non_blocking=True)
        loss_done[slot].record(stream)
        if i > 0:
            loss_done[slot ^ 1].synchronize()
            state["losses"].append(float(loss_host[slot ^ 1][0]))
        state["i"] = i + 1

    # ---- device-resident timing ----------------------------------------------------------
    for _ in range(args.warmup):
        step_resident()
    ctx.barrier()
    # Inside the timed region only the dominant kernel (the forward GEMM) is bracketed by events:
    # every bracket costs about a microsecond of stream time, ten of them per step 1 % of the step.
    names = [lib.al_kernel_class_name(i).decode() for i in range(_lib.AL_K_COUNT)]
    _lib.profile_read(reset=True)
    lib.al_profile_select(1 << names.index("fwd_gemm"))
    lib.al_profile_enable(1)
    sampler = ClockSampler(ctx.local_rank)
    if rank == 0:
        sampler.start()
    ms_total = timed_steps(ctx, step_resident, args.steps, between=lambda: flush.fill_(1))
    ctx.barrier()
    lib.al_profile_enable(0)
    prof_timed = _lib.profile_read(reset=True)
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = ctx.max_over_ranks(ms_total) / args.steps
    value = FLOP_PER_STEP * world / (ms_per_step * 1e-3) / 1e12
    # the same steps once more with every kernel bracketed: the per-kernel table
    lib.al_profile_select(0xFFFFFFFF)
    lib.al_profile_enable(1)
    ms_all = timed_steps(ctx, step_resident, args.steps, between=lambda: flush.fill_(1))
    ctx.barrier()
    lib.al_profile_enable(0)
    prof = _lib.profile_read(reset=True)

    # ---- end to end through the public API, batch in pinned host memory -------------------
    for slot in range(2):
        consumed[slot].record(stream)
    for _ in range(3):
        step_e2e()
    ctx.barrier()
    e2e_ms = timed_steps(ctx, step_e2e, args.steps)
    ctx.barrier()
    e2e_ms_per_step = ctx.max_over_ranks(e2e_ms) / args.steps
    e2e_value = FLOP_PER_STEP * world / (e2e_ms_per_step * 1e-3) / 1e12

    uses_tc = bool(lib.al_uses_tcgen05(
        F.make_desc(layer.rpu_config, M, K, N, len(layer.in_sizes), torch.bfloat16, True),
        _lib.tile_ends_array(layer.in_sizes)))
    comm_sms = F.settings.comm_sms
    release_gradient_sync()
    h2d_bytes = x_host.numel() * x_host.element_size()
    del layer, slots, x_dev, flush, x_host, sync
    torch.cuda.empty_cache()

    peaks = load_peaks()
    gemm_flop = {"fwd_gemm": 2.0 * M * K * N, "dgrad_gemm": 2.0 * M * K * N, "wgrad_gemm": 2.0 * M * K * N}
    dominant = max(gemm_flop, key=lambda k: prof[k][2])
    # the dominant kernel's duration comes from the timed region itself when it is the bracketed one
    _, d_timed, d_ms = prof_timed[dominant] if prof_timed[dominant][1] else prof[dominant]
    achieved = gemm_flop[dominant] / (d_ms / max(d_timed, 1) * 1e-3) / 1e12 if d_ms > 0 else 0.0
    rec = base_record(args, world)
    if world > 1:
        rec["config"]["grad_sync"] = (f"weight gradient (34 MB) summed over the replicas inside backward, after the "
                                      f"weight-gradient kernel and beside the input-gradient GEMM ({comm_sms} SMs left to "
                                      f"it), complete at step end: {how}")
    rec.update({
        "value": value,
        "ms_per_step": ms_per_step,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms_per_step,
                "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4},
        "gpu_launches": sum(v[0] for v in prof_timed.values()),
        "pct_of_bf16_peak": {"burst": 100 * value / world / peaks["bf16"],
                             "sustained": 100 * value / world / peaks["bf16_sustained"]},
        "roofline": {"kernel": dominant, "bound": "tensor", "achieved": achieved,
                     "peak": peaks["bf16"], "unit": "TFLOP/s",
                     "frac": achieved / peaks["bf16"],
                     "frac_sustained": achieved / peaks["bf16_sustained"],
                     "peak_source": f"{peaks['source']} (burst; sustained {peaks['bf16_sustained']})",
                     "traffic": FWD_KERNEL_DRAM_BYTES if dominant == "fwd_gemm" else None},
        "kernels": kernel_table(prof), "kernels_note": KERNELS_NOTE,
        "kernels_from": f"a second pass of the same {args.steps} steps with every kernel bracketed by events "
                        f"({ms_all / args.steps:.4f} ms per step on this rank)",
        "engine": {"requested": args.engine, "tcgen05": uses_tc},
        "clocks": clocks,
    })
    return rec


# ---------------------------------------------------------------------------------------------
# the other configurations (lines of their own; kept under profiles/)
# ---------------------------------------------------------------------------------------------
def run_c1(args, ctx):
    """Config 1: AnalogLinear 1024 -> 1024 fp32, 512 rows, 2 tiles, learned static input range 3.0,
    inp_res 254, out_noise 0.04, weight noise 0.02 (per channel), no ADC; forward + backward."""
    from aihwkit_lightning_b200 import _lib
    from aihwkit_lightning_b200.nn import AnalogLinear
    from aihwkit_lightning_b200.simulator import configs as cfg

    dev = ctx.dev
    lib = _lib.load()
    m, k, n = args.c1_rows, args.c1_size, args.c1_size  # other sizes: the same layer where the GEMMs bound the step
    rpu = make_rpu_config(cfg, max_in=512, adc=False, dynamic=False)
    rpu.pre_post.input_range.learn_input_range = True
    rpu.pre_post.input_range.init_value = 3.0
    rpu.pre_post.input_range.init_from_data = 0
    torch.manual_seed(0)
    layer = AnalogLinear(k, n, bias=True, rpu_config=rpu).to(dev).train()
    with torch.no_grad():
        layer.weight.uniform_(-1 / 32, 1 / 32)
    x = torch.randn(m, k, device=dev, requires_grad=True)
    g = torch.randn(m, n, device=dev)
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)

    def step():
        layer.zero_grad(set_to_none=True)
        x.grad = None
        layer(x).backward(g)

    for _ in range(max(args.warmup, 3)):
        step()
    ctx.barrier()
    _lib.profile_read(reset=True)
    lib.al_profile_enable(1)
    sampler = ClockSampler(ctx.local_rank)
    sampler.start()
    ms = timed_steps(ctx, step, args.steps, between=lambda: flush.fill_(1)) / args.steps
    lib.al_profile_enable(0)
    prof = _lib.profile_read(reset=True)
    clocks = sampler.stop()
    eager_ms = ms
    # the same step as one CUDA graph: the layer's eight launches cost the host more than the GPU
    graph = capture_step(step, dev)
    for _ in range(3):
        graph.replay()
    ms = timed_steps(ctx, graph.replay, args.steps, between=lambda: flush.fill_(1)) / args.steps
    flop = 6.0 * m * k * n
    peaks = load_peaks()
    gemm_ms = sum(prof[c][2] for c in ("fwd_gemm", "dgrad_gemm", "wgrad_gemm")) / args.steps
    rec = base_record(args, 1)
    rec.update({
        "dtype": "f32",
        "config": {"workload": f"config 1: AnalogLinear {k}->{n} fp32, {m} rows ~N(0,1), weights ~U(-1/32,1/32), "
                               f"max_input_size=512 ({k // 512} tiles), inp_res=254, learned static input range 3.0, out_noise 0.04, "
                               "weight noise 0.02 per-channel, no ADC, training fwd+bwd",
                   "l2": "256 MB flush write between steps", "parallelism": "dp1"},
        "value": flop / (ms * 1e-3) / 1e12, "ms_per_step": ms, "eager_ms_per_step": eager_ms,
        "launch": "the step replayed as one CUDA graph (noise counters advanced on the device); "
                  "eager_ms_per_step: the same step launched call by call, with the per-kernel events of the table",
        "gpu_launches": sum(v[0] for v in prof.values()),
        "roofline": {"kernel": "fwd+dgrad+wgrad GEMMs", "bound": "tensor", "achieved": flop / (gemm_ms * 1e-3) / 1e12,
                     "peak": peaks["bf16"], "unit": "TFLOP/s", "frac": flop / (gemm_ms * 1e-3) / 1e12 / peaks["bf16"],
                     "note": f"{flop / 1e9:.1f} GFLOP per step; at the configuration's own size the step is bound by launch "
                             "latency, not by a pipe", "traffic": None},
        "kernels": kernel_table(prof), "kernels_note": KERNELS_NOTE, "clocks": clocks,
    })
    return rec


def run_c4(args, ctx):
    """Config 4: ResNet-32 (CIFAR shape) with AnalogConv2d / AnalogLinear, batch 256 per GPU, fp32,
    max_input_size=256, 8-bit DAC, out_noise 0.02; one SGD training step."""
    from torch import nn
    from torch.nn import functional as TF

    from aihwkit_lightning_b200 import _lib
    from aihwkit_lightning_b200.nn import AnalogConv2d, AnalogLinear, convert_to_analog
    from aihwkit_lightning_b200.optim import AnalogOptimizer
    from aihwkit_lightning_b200.simulator import configs as cfg

    dev = ctx.dev
    lib = _lib.load()

    class Block(nn.Module):
        def __init__(self, cin, cout, stride):
            super().__init__()
            self.conv1 = nn.Conv2d(cin, cout, 3, stride=stride, padding=1, bias=False)
            self.bn1 = nn.BatchNorm2d(cout)
            self.conv2 = nn.Conv2d(cout, cout, 3, padding=1, bias=False)
            self.bn2 = nn.BatchNorm2d(cout)
            self.short = nn.Conv2d(cin, cout, 1, stride=stride, bias=False) if (stride != 1 or cin != cout) else None

        def forward(self, x):
            y = TF.relu(self.bn1(self.conv1(x)))
            y = self.bn2(self.conv2(y))
            return TF.relu(y + (x if self.short is None else self.short(x)))

    class ResNet32(nn.Module):
        def __init__(self):
            super().__init__()
            self.conv = nn.Conv2d(3, 16, 3, padding=1, bias=False)
            self.bn = nn.BatchNorm2d(16)
            blocks, cin = [], 16
            for cout, stride in ((16, 1), (32, 2), (64, 2)):
                for i in range(5):
                    blocks.append(Block(cin, cout, stride if i == 0 else 1))
                    cin = cout
            self.blocks = nn.Sequential(*blocks)
            self.fc = nn.Linear(64, 10)

        def forward(self, x):
            return self.fc(self.blocks(TF.relu(self.bn(self.conv(x)))).mean((2, 3)))

    batch = 256
    rpu = make_rpu_config(cfg, max_in=256, adc=False, out_noise=0.02)
    torch.manual_seed(0)
    model = convert_to_analog(ResNet32(), rpu).to(dev).train()
    layers = [m for m in model.modules() if isinstance(m, (AnalogConv2d, AnalogLinear))]
    opt = AnalogOptimizer(torch.optim.SGD, model.analog_layers, model.parameters(), lr=0.05, momentum=0.9)
    gen = torch.Generator().manual_seed(ctx.rank)
    x_host = torch.randn(batch, 3, 32, 32, generator=gen).pin_memory()
    y_host = torch.randint(0, 10, (batch,), generator=gen).pin_memory()
    # algorithmic bytes of the analog layers: input activation, output activation and weights of every
    # layer, each once per pass (forward, input gradient, weight gradient); shapes from a forward hook
    act_bytes = [0.0]

    def count(mod, inp, out):
        act_bytes[0] += 4.0 * (inp[0].numel() + out.numel() + mod.weight.numel())

    hooks = [m.register_forward_hook(count) for m in layers]
    with torch.no_grad():
        model(x_host.to(dev))
    for h in hooks:
        h.remove()
    alg_bytes = 3.0 * act_bytes[0]

    def step():
        x = x_host.to(dev, non_blocking=True)
        y = y_host.to(dev, non_blocking=True)
        opt.zero_grad(set_to_none=True)
        loss = TF.cross_entropy(model(x), y)
        loss.backward()
        opt.step()
        return loss

    for _ in range(max(args.warmup, 3)):
        step()
    ctx.barrier()
    _lib.profile_read(reset=True)
    lib.al_profile_enable(1)
    sampler = ClockSampler(ctx.local_rank)
    sampler.start()
    t0 = time.perf_counter()
    ms = timed_steps(ctx, step, args.steps) / args.steps
    wall_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    lib.al_profile_enable(0)
    prof = _lib.profile_read(reset=True)
    clocks = sampler.stop()
    lib_ms = sum(v[2] for v in prof.values()) / args.steps
    eager_ms = ms
    # the same step (upload, forward, loss, backward, SGD) as one CUDA graph
    graph = capture_step(step, dev)
    for _ in range(3):
        graph.replay()
    ms = timed_steps(ctx, graph.replay, args.steps) / args.steps
    peaks = load_peaks()
    rec = base_record(args, 1)
    rec.update({
        "eager_ms_per_step": eager_ms,
        "launch": "the step replayed as one CUDA graph (noise counters advanced on the device); eager_ms_per_step, "
                  "host_ms_per_step and the kernel table: the same step launched call by call",
        "metric": "ResNet-32 training images/s", "unit": "images/s", "dtype": "f32",
        "config": {"workload": f"config 4: ResNet-32 (CIFAR shape), AnalogConv2d/AnalogLinear ({len(layers)} analog layers), "
                               "batch 256 of 32x32x3 ~N(0,1), uniform labels, max_input_size=256, 8-bit DAC, out_noise 0.02, "
                               "weight noise 0.02, fp32, SGD step", "parallelism": "dp1"},
        "value": batch / (ms * 1e-3), "ms_per_step": ms, "host_ms_per_step": wall_ms,
        "library_kernel_ms_per_step": lib_ms,
        "gpu_launches": sum(v[0] for v in prof.values()),
        "e2e": {"value": batch / (ms * 1e-3), "unit": "images/s",
                "h2d_bytes_per_step": x_host.numel() * 4 + y_host.numel() * 8, "d2h_bytes_per_step": 0},
        "roofline": {"kernel": "all library kernels of a step", "bound": "hbm",
                     "achieved": alg_bytes / (lib_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": alg_bytes / (lib_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "traffic": None,
                     "note": "algorithmic bytes = activations in + out + weights of every analog layer, three passes"},
        "kernels": kernel_table(prof), "kernels_note": KERNELS_NOTE, "clocks": clocks,
    })
    return rec


def run_c5(args, ctx):
    """Config 5: inference sweep, noise off: M in {1,16,256,4096,16384} x K=N in {2048,4096,8192,16384},
    max_input_size in {256,512,1024}, 8-bit DAC/ADC, bf16, forward only."""
    from aihwkit_lightning_b200 import _lib
    from aihwkit_lightning_b200.nn import AnalogLinear
    from aihwkit_lightning_b200.simulator import configs as cfg

    dev = ctx.dev
    peaks = load_peaks()
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
    points = []
    total_flop = total_ms = 0.0
    _lib.profile_read(reset=True)
    for kn in (2048, 4096, 8192, 16384):
        for max_in in (256, 512, 1024):
            rpu = make_rpu_config(cfg, max_in=max_in, out_noise=0.0)
            rpu.modifier.noise_type = cfg.WeightNoiseInjectionType.NONE
            torch.manual_seed(0)
            layer = AnalogLinear(kn, kn, bias=False, rpu_config=rpu).to(device=dev, dtype=torch.bfloat16).eval()
            with torch.no_grad():
                layer.weight.normal_(0, 0.02)
            for m in (1, 16, 256, 4096, 16384):
                x = torch.randn(m, kn, device=dev).bfloat16()
                reps = 3 if m * kn * kn > 1e12 else 10
                with torch.no_grad():
                    for _ in range(3):
                        layer(x)
                    ms = timed_steps(ctx, lambda: layer(x), reps, between=lambda: flush.fill_(1)) / reps  # noqa: B023
                flop = 2.0 * m * kn * kn
                nbytes = 2.0 * (kn * kn + m * kn + m * kn)
                tensor_bound = m >= 256
                ach = flop / (ms * 1e-3) / 1e12 if tensor_bound else nbytes / (ms * 1e-3) / 1e9
                peak = peaks["bf16"] if tensor_bound else peaks["hbm_gbs"]
                points.append(dict(M=m, K=kn, N=kn, max_input_size=max_in, ms=round(ms, 5),
                                   tflops=round(flop / (ms * 1e-3) / 1e12, 3), bound="tensor" if tensor_bound else "hbm",
                                   achieved=round(ach, 2), frac=round(ach / peak, 4)))
                total_flop += flop
                total_ms += ms
                del x
            del layer
            torch.cuda.empty_cache()
    prof = _lib.profile_read(reset=True)
    rec = base_record(args, 1)
    best = max((p for p in points if p["bound"] == "tensor"), key=lambda p: p["frac"])
    rec.update({
        "metric": "analog-layer forward TFLOP/s (inference sweep)",
        "config": {"workload": "config 5: eval forward, noise off, M in {1,16,256,4096,16384} x K=N in {2048,4096,8192,16384} x "
                               "max_input_size in {256,512,1024}, 8-bit DAC + ADC out_bound=10, dynamic input range, bf16, "
                               "weights ~N(0,0.02); value = total FLOP / total time over the 60 points",
                   "l2": "256 MB flush write between calls", "parallelism": "dp1"},
        "value": total_flop / (total_ms * 1e-3) / 1e12, "ms_per_step": total_ms,
        "gpu_launches": sum(v[0] for v in prof.values()),
        "roofline": {"kernel": f"best tensor-bound point M={best['M']} K=N={best['K']} max_input_size={best['max_input_size']}",
                     "bound": "tensor", "achieved": best["achieved"], "peak": peaks["bf16"], "unit": "TFLOP/s",
                     "frac": best["frac"], "traffic": None},
        "points": points,
    })
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--engine", default="auto", choices=["auto", "simt", "tcgen05"])
    ap.add_argument("--config", default="c2", choices=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gpu-baseline", action="store_true")
    ap.add_argument("--no-c3", action="store_true", help="headline line only, without the decoder step")
    ap.add_argument("--c1-size", type=int, default=1024, help="in = out features of the fp32 layer of --config c1")
    ap.add_argument("--c1-rows", type=int, default=512, help="input rows of the fp32 layer of --config c1")
    ap.add_argument("--c3-layers", type=int, default=32)
    ap.add_argument("--c3-steps", type=int, default=3)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    if args.impl == "reference":
        run_reference(args, int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")))
        return

    ctx = Ctx()
    try:
        if args.config == "c2":
            rec = run_c2(args, ctx)
            if not args.no_c3:
                rec["c3"] = run_c3(args, ctx, layers=args.c3_layers, steps=args.c3_steps)
            if ctx.rank == 0 and ctx.world == 1:
                if not args.no_gpu_baseline:
                    base = gpu_torch_baseline(ctx.dev)
                    base["ratio_to_value"] = rec["value"] / base["value"]
                    rec["gpu_torch_baseline"] = base
                if not args.no_cpu_baseline:
                    res = cpu_reference_run(steps=3, warmup=1, rows=CPU_SAMPLE_ROWS)
                    rec["cpu_baseline"] = {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")}
        elif args.config == "c3":
            c3 = run_c3(args, ctx, layers=args.c3_layers, steps=args.c3_steps)
            rec = base_record(args, ctx.world)
            rec.update({"metric": "decoder training tokens/s", "unit": "tokens/s", "value": c3["tokens_per_s"],
                        "ms_per_step": c3["ms_per_step"], "steps": c3["steps"], "warmup": c3["warmup"],
                        "gpu_launches": c3["gpu_launches"],
                        "config": {"workload": c3["workload"], "parallelism": f"dp{ctx.world}"}, "c3": c3})
        else:
            assert ctx.world == 1, "configs 1, 4 and 5 are single-GPU lines"
            rec = {"c1": run_c1, "c4": run_c4, "c5": run_c5}[args.config](args, ctx)
        if ctx.rank == 0:
            print(json.dumps(rec), flush=True)
    finally:
        ctx.close()


if __name__ == "__main__":
    main()
