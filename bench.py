"""Benchmark of the analog linear hot path (forward + backward of one analog layer).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N=1): the configuration the headline metric is quoted on -- ``AnalogLinear``
4096 -> 4096 in bf16, 8192 tokens ~N(0,1), ``max_input_size=512`` (8 analog tiles), dynamic
per-token input ranges with an 8-bit DAC, 8-bit ADC with ``out_bound=10``, ``out_noise=0.04``,
weight noise 0.02 relative to the per-channel abs-max, training mode, forward + backward.
A "step" is one forward + backward over one batch of synthetic tokens; the metric is
algorithmic TFLOP/s = 6*M*K*N / time.

* ``value``: inputs resident in HBM, CUDA-event timing over exactly K steps (max over ranks).
* ``e2e``: the same step through the public ``AnalogLinear`` call with the batch in pinned
  host memory: every step uploads its batch (double-buffered on a copy stream, so the upload
  of the next batch overlaps the current step) and copies its loss back to pinned host memory,
  where the host reads it one step later; all inside the timed region.
* ``roofline``: the dominant kernel, timed live with CUDA events by the library's launch
  accounting, against the measured bf16 tensor peak.
* ``cpu_baseline`` / ``--impl reference``: the CPU restatement of the reference's torch path
  (``oracle/analog_oracle.py::linear_autograd``) timed on the host cores on a bounded sample
  of the workload (fewer rows, same K, N and tiling).
* N > 1 (torchrun): every rank runs the layer on its own batch (weak scaling) and the weight
  gradient is all-reduced over NCCL, as in data-parallel training.
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
FWD_KERNEL_DRAM_BYTES = 120.1e6 + 76.4e6


def make_rpu_config(ns):
    rpu = ns.TorchInferenceRPUConfig()
    rpu.mapping.max_input_size = MAX_IN
    rpu.forward.inp_res = 254.0
    rpu.forward.out_res = 254.0
    rpu.forward.out_bound = 10.0
    rpu.forward.out_noise = 0.04
    rpu.pre_post.input_range.enable = True
    rpu.pre_post.input_range.dynamic = True
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--engine", default="auto", choices=["auto", "simt", "tcgen05"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch.distributed as dist

    from aihwkit_lightning_b200 import _lib
    from aihwkit_lightning_b200.distributed import EagerGradientSync, GradientBuckets, rank_seed
    from aihwkit_lightning_b200.nn import AnalogLinear
    from aihwkit_lightning_b200.nn import functional as F
    from aihwkit_lightning_b200.simulator import configs as cfg

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
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
    # "eager" (default): the all-reduce of the weight gradient is issued from a hook inside backward and
    # is complete when the step ends, as an optimizer step would need it.
    # "deferred" (BENCH_GRAD_SYNC=deferred): the all-reduce of step i runs beside step i+1 (a step then
    # ends with a gradient that is one step old; measured 4 % faster on 2 GPUs, not the default).
    eager = os.environ.get("BENCH_GRAD_SYNC", "eager") != "deferred"
    buckets = GradientBuckets(layer.parameters()) if world > 1 and not eager else None
    sync = EagerGradientSync().attach(layer.parameters()) if world > 1 and eager else None
    if sync is not None:
        from aihwkit_lightning_b200.nn import functional as analog_functional
        analog_functional.settings.after_wgrad = sync
        # SMs the input-gradient GEMM leaves to the all-reduce kernel beside it.  Measured on 2 GPUs:
        # with 20 SMs free (64 CTA pairs = 8 full rounds of the 512 output blocks) the GEMM takes 39 us
        # longer and the exposed all-reduce 45 us less -- no net gain, so the default is 0.
        analog_functional.settings.comm_sms = int(os.environ.get("BENCH_COMM_SMS", "0"))
    x_dev = x_host.to(dev).requires_grad_(True)
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev)

    def step_resident():
        layer.weight.grad = None
        x_dev.grad = None
        out = layer(x_dev)
        out.backward(g)
        if sync is not None:
            sync.finish()
        if buckets is not None:
            buckets.finish()  # previous step's all-reduce (overlapped with this step's kernels)
            buckets.reduce_all_async()

    def drain():
        if buckets is not None:
            buckets.finish()

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
        if buckets is not None:
            buckets.reduce_all_async()
            buckets.finish()
        # device -> host read of this step's loss: copied to pinned memory on the compute stream
        # and picked up by the host one step later, so the host can already enqueue the next step
        loss_host[slot].copy_(loss.detach().reshape(1), non_blocking=True)
        loss_done[slot].record(stream)
        if i > 0:
            loss_done[slot ^ 1].synchronize()
            state["losses"].append(float(loss_host[slot ^ 1][0]))
        state["i"] = i + 1

    def timed(fn, steps, between=None):
        """CUDA-event time of exactly `steps` calls; the L2 flush between steps is excluded."""
        total = 0.0
        events = []
        for _ in range(steps):
            if between is not None:
                between()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(stream)
            fn()
            e.record(stream)
            events.append((s, e))
        drain()
        torch.cuda.synchronize(dev)
        for s, e in events:
            total += s.elapsed_time(e)
        return total

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize(dev)

    # ---- device-resident timing ----------------------------------------------------------
    for _ in range(args.warmup):
        step_resident()
    drain()
    barrier()
    _lib.profile_read(reset=True)
    lib.al_profile_enable(1)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms_total = timed(step_resident, args.steps, between=lambda: flush.fill_(1))
    barrier()
    lib.al_profile_enable(0)
    prof = _lib.profile_read(reset=True)
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    ms_per_step = ms_total / args.steps
    value = FLOP_PER_STEP * world / (ms_per_step * 1e-3) / 1e12

    # ---- end to end through the public API, batch in pinned host memory -------------------
    for slot in range(2):
        consumed[slot].record(stream)
    for _ in range(3):
        step_e2e()
    barrier()
    e2e_ms = timed(step_e2e, args.steps)
    barrier()
    t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms_per_step = float(t.item()) / args.steps
    e2e_value = FLOP_PER_STEP * world / (e2e_ms_per_step * 1e-3) / 1e12

    if rank == 0:
        peaks = load_peaks()
        gemm_flop = {"fwd_gemm": 2.0 * M * K * N, "dgrad_gemm": 2.0 * M * K * N, "wgrad_gemm": 2.0 * M * K * N}
        kernels = {}
        for name, (launches, timed_scopes, total) in prof.items():
            if launches:
                kernels[name] = dict(launches=launches, ms_total=round(total, 4),
                                     ms_avg=round(total / max(timed_scopes, 1), 5))
        dominant = max(gemm_flop, key=lambda k: prof[k][2])
        d_launches, d_timed, d_ms = prof[dominant]
        achieved = gemm_flop[dominant] / (d_ms / max(d_timed, 1) * 1e-3) / 1e12 if d_ms > 0 else 0.0
        rec = base_record(args, world)
        if world > 1:
            rec["config"]["grad_sync"] = (
                "NCCL all-reduce of the weight gradient, started inside backward after the weight-gradient kernels, "
                "complete at step end" if eager else
                "NCCL all-reduce of the weight gradient of step i overlapped with step i+1")
        rec.update({
            "value": value,
            "ms_per_step": ms_per_step,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms_per_step,
                    "h2d_bytes_per_step": x_host.numel() * x_host.element_size(),
                    "d2h_bytes_per_step": 4},
            "gpu_launches": sum(v[0] for v in prof.values()),
            "pct_of_bf16_peak": {"burst": 100 * value / world / peaks["bf16"],
                                 "sustained": 100 * value / world / peaks["bf16_sustained"]},
            "roofline": {"kernel": dominant, "bound": "tensor", "achieved": achieved,
                         "peak": peaks["bf16_sustained"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["bf16_sustained"],
                         "peak_source": f"{peaks['source']} (sustained; burst {peaks['bf16']})",
                         # DRAM bytes (read + write) of one fwd_tc_kernel launch on this workload,
                         # from the ncu capture summarised in profiles/fwd_tc_kernel_c2.md
                         "traffic": FWD_KERNEL_DRAM_BYTES if dominant == "fwd_gemm" else None},
            "kernels": kernels,
            "engine": {"requested": args.engine,
                       "tcgen05": bool(lib.al_uses_tcgen05(
                           F.make_desc(layer.rpu_config, M, K, N, len(layer.in_sizes), torch.bfloat16, True),
                           _lib.tile_ends_array(layer.in_sizes)))},
            "clocks": clocks,
        })
        if not args.no_cpu_baseline and world == 1:
            res = cpu_reference_run(steps=3, warmup=1, rows=CPU_SAMPLE_ROWS)
            rec["cpu_baseline"] = {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(rec), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
