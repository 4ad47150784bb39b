#!/usr/bin/env python
"""Benchmark of the ConvRot quantized-linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): BASELINE config 1 -- one INT4 ConvRot linear at the DiT MLP
shape, activations f32 [4608][3072], weight int4 [12288][3072] packed two per
byte, per-row f32 scales, output f32 [4608][12288].  One step = one pass of the
hot path over one batch of activations: rotate + per-token quantise (prep), then
the tcgen05 int8 GEMM with the dequant fused in.  Seeded synthetic data stands
in for a checkpoint.

Metric: int8 tera-ops per second, 2*M*N*K operations per step, whole job.
  value  inputs resident in HBM when the timed region starts
  e2e    the same step through the host-buffer entry (pinned host x -> device,
         compute, y -> pinned host) inside the timed region
With N > 1 GPUs (one process per GPU, torchrun) every rank runs the same step on
its own batch -- independent requests, no data-path collective (weak scaling).

The default line also carries, under `secondary`, the other parts of the metric
measured in the same run: the Q8_0 decode GEMV (config 2, six cases, fraction of
HBM bandwidth), the INT8 DiT step (config 3, s/step), the weight-streamed INT4 DiT
step over a batch of 8 latents sharded 8/N per GPU (config 4) and, with N > 1, the
one GEMM split along N with the all-gather fused into its epilogue.

`--impl reference` times the reference's CPU semantics for this path (the C
restatement of its `--backend cpu` float path; Zig is not installed, so the
reference binary itself cannot run) on the host cores, on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M, N, K, BITS = 4608, 12288, 3072, 4
OPS_PER_STEP = 2.0 * M * N * K
METRIC = "convrot_qgemm_int8_tops"
UNIT = "TOPS"
N_SETS = 4  # distinct input sets rotated through, so each step's inputs come from HBM, not L2
WORKLOAD = ("config1: INT4 ConvRot linear (activation prep + int4 weights on the int8 tcgen05 GEMM + fused dequant), "
            "M=4608 K=3072 N=12288, one batch of 4608 tokens per GPU")
TOTAL_LATENTS = 8     # config 4: a batch of 8 independent latents, sharded 8/N per GPU
MIN_REGION_MS = 200.0  # the timed regions are repeated back to back for at least this long


def bind_to_gpu_numa_node(local: int):
    """Restrict this process to the CPUs NVML reports as local to GPU `local`, so that its
    pinned host buffers (first-touch placement) sit on the NUMA node the GPU's PCIe root
    hangs off.  Matters when several ranks drive host<->device copies at once; best effort."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(local)
        n_words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, n_words)
        cpus = {64 * i + b for i, w in enumerate(mask) for b in range(64) if (w >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
        return sorted(cpus)
    except Exception:
        return None


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def stop(self):
        self._halt.set()
        self.join(timeout=1.0)
        return {"sm_mhz": float(np.median(self.samples)) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except Exception:
            return local
    return local


# ---------------------------------------------------------------------------------------
# CPU arms (the only place outside tests/ that runs the CPU checker)
# ---------------------------------------------------------------------------------------

def host_threads() -> int:
    """The host threads this process may use.  Asked from the scheduler, not from OpenMP: a launcher
    such as torch.distributed.run exports OMP_NUM_THREADS=1, which would leave the CPU arm on one core."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_float_path_sample(target_seconds: float = 12.0):
    """Times the CPU restatement of the reference's `--backend cpu` path on a slice
    of the workload's weight rows (all M activation rows, full K), sized for about
    `target_seconds`.  Returns (TOPS, cores, sample description, seconds)."""
    from oracle import oracle
    from tensorpencil_b200 import synth
    cores = host_threads()
    x = synth.activations(M, K, seed=1001)
    probe_rows = 16 * cores if 16 * cores <= N else N
    w = synth.convrot_weights(probe_rows, K, BITS, seed=1001)
    t0 = time.perf_counter()
    oracle.linear_cpu_backend(x, w["w_packed"], BITS, w["w_scale"], probe_rows, K, nthreads=cores)
    dt = time.perf_counter() - t0
    rate = 2.0 * M * probe_rows * K / dt
    rows = int(min(N, max(probe_rows, (rate * target_seconds) / (2.0 * M * K))))
    rows = max(16, rows // 16 * 16)
    w = synth.convrot_weights(rows, K, BITS, seed=1002)
    reps, dt = 0, 0.0
    t0 = time.perf_counter()
    while dt < target_seconds * 0.8 or reps == 0:
        oracle.linear_cpu_backend(x, w["w_packed"], BITS, w["w_scale"], rows, K, nthreads=cores)
        reps += 1
        dt = time.perf_counter() - t0
    tops = 2.0 * M * rows * K * reps / dt / 1e12
    return tops, cores, (f"{reps} x ({rows} of {N} weight rows x all {M} tokens x K={K}), float path "
                         f"(dequantise, un-rotate, f32 FMA GEMM), {dt:.1f} s"), dt


def run_reference_arm(args, rank: int, world: int):
    if rank != 0:
        return
    from oracle import oracle
    from tensorpencil_b200 import synth
    cores = host_threads()
    x = synth.activations(M, K, seed=1001)
    # size one step at ~2 s of CPU work, bounded so the whole run stays within minutes
    probe_rows = min(N, 16 * cores)
    w = synth.convrot_weights(probe_rows, K, BITS, seed=1001)
    t0 = time.perf_counter()
    oracle.linear_cpu_backend(x, w["w_packed"], BITS, w["w_scale"], probe_rows, K, nthreads=cores)
    rate = 2.0 * M * probe_rows * K / (time.perf_counter() - t0)
    rows = int(min(N, max(16, rate * 2.0 / (2.0 * M * K)))) // 16 * 16 or 16
    w = synth.convrot_weights(rows, K, BITS, seed=1002)
    for _ in range(args.warmup):
        oracle.linear_cpu_backend(x, w["w_packed"], BITS, w["w_scale"], rows, K, nthreads=cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.linear_cpu_backend(x, w["w_packed"], BITS, w["w_scale"], rows, K, nthreads=cores)
    dt = time.perf_counter() - t0
    tops = 2.0 * M * rows * K * args.steps / dt / 1e12
    sample = f"{rows} of {N} weight rows x all {M} tokens per step (float path: dequantise, un-rotate, f32 FMA GEMM)"
    line = {
        "impl": "reference", "metric": METRIC, "value": tops, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "m": M, "n": N, "k": K, "bits": BITS,
                   "note": "CPU restatement of the reference's --backend cpu path (Zig absent: the reference binary "
                           "cannot run), on a bounded sample of the workload's weight rows"},
        "cpu_baseline": {"value": tops, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------

# DRAM bytes of one full-size launch of the int8 GEMM (dram__bytes_read.sum + dram__bytes_write.sum
# of one ncu capture of that launch, per output type).  A profiler figure: this program cannot
# measure it, so the line says where it comes from.
GEMM_DRAM_TRAFFIC_BYTES = {"f32": 225.1e6, "bf16": 118.9e6}


def timed_regions(fn, steps: int, stream, min_total_ms: float = MIN_REGION_MS, max_regions: int = 400):
    """Runs regions of exactly `steps` calls of fn(i) back to back, each bracketed by two CUDA
    events on `stream`, until their estimated total reaches `min_total_ms` (at least 3 regions).
    The caller synchronises before and after.  Returns the events; read them with
    region_stats() once the device is idle.  One region of a 0.16 ms step lasts only a few
    milliseconds, too short for the clocks to settle or to be sampled: the median over a
    fifth of a second of continuous work is the figure that holds under load."""
    import torch
    probe0, probe1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    probe0.record(stream)
    for i in range(steps):
        fn(i)
    probe1.record(stream)
    probe1.synchronize()
    est = max(probe0.elapsed_time(probe1), 1e-3)
    regions = int(min(max_regions, max(3, np.ceil(min_total_ms / est))))
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(regions + 1)]
    evs[0].record(stream)
    for r in range(regions):
        for i in range(steps):
            fn(r * steps + i)
        evs[r + 1].record(stream)
    return evs


def region_stats(evs):
    ms = [evs[i].elapsed_time(evs[i + 1]) for i in range(len(evs) - 1)]
    return {"count": len(ms), "median_ms": float(np.median(ms)), "min_ms": float(min(ms)), "max_ms": float(max(ms)),
            "total_ms": float(sum(ms))}


def run_ours(args, rank: int, local: int, world: int):
    import torch
    import torch.distributed as dist

    from tensorpencil_b200 import synth
    from tensorpencil_b200.backend import Backend

    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    be = Backend(local)
    out_dtype = torch.float32 if args.out_dtype == "f32" else torch.bfloat16
    out_bytes = 4 if args.out_dtype == "f32" else 2
    peaks = measured_peaks()

    # N_SETS distinct (x, W) pairs on the device; rank-specific seeds = independent requests.
    xs, ws, wss = [], [], []
    for s in range(N_SETS):
        c = synth.convrot_linear(M, N, K, BITS, seed=1001 + 17 * s + 1000 * rank)
        xs.append(torch.from_numpy(c["x"]).cuda())
        ws.append(torch.from_numpy(c["w_packed"]).cuda())
        wss.append(torch.from_numpy(c["w_scale"]).cuda())
        x_host_src = c["x"] if s == 0 else x_host_src
    y = torch.empty((M, N), dtype=out_dtype, device="cuda")
    stream = torch.cuda.current_stream()

    def step(i: int):
        # one library call per linear: int4 weights -> int8 tensor-core operand, activation prep, GEMM
        s = i % N_SETS
        be.convrot_linear(xs[s], ws[s], wss[s], N, BITS, y=y)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def reduce_max(vals):
        if world == 1:
            return [float(v) for v in vals]
        t = torch.tensor(list(vals), device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t]

    warm = max(args.warmup, 3)
    for i in range(warm):
        step(i)
    sync_all()
    be.status_poll()

    # ---- timed region 1: inputs resident in HBM.  Regions of exactly args.steps steps, back to
    # back for >= MIN_REGION_MS, the clocks sampled throughout; the line reports the median region.
    sampler = ClockSampler(physical_gpu_index(local))
    launches0 = be.launches
    sync_all()
    sampler.start()
    evs = timed_regions(step, args.steps, stream)
    sync_all()
    clocks = sampler.stop()
    reg = region_stats(evs)
    gpu_launches = (be.launches - launches0) // (reg["count"] + 1)   # per region of args.steps steps
    be.status_poll()
    ms_total = reg["median_ms"]

    # ---- the dominant kernel alone, for the roofline: the int8 GEMM on the widened weights of
    # the same sets (rotating, so operands come from HBM) ----
    w8s = []
    for s_ in range(N_SETS):
        w8 = torch.empty((N, K), dtype=torch.int8, device="cuda")
        be._check(be.lib.tpb_convrot_w4_expand(be.h, be._stream(), ws[s_].data_ptr(), N, K, w8.data_ptr()))
        w8s.append(w8)
    be.i8_bits = 8   # the prepped activations of the last step stay; the weights are int8 now

    def gemm_only(i):
        be._gemm(y, w8s[i % N_SETS], wss[i % N_SETS], N, 8)

    for i in range(3):
        gemm_only(i)
    sync_all()
    gevs = timed_regions(gemm_only, args.steps, stream)
    sync_all()
    greg = region_stats(gevs)
    gemm_ms = greg["median_ms"] / args.steps
    be.status_poll()

    # the same kernel looped for >= 2 s with the clocks sampled: what it sustains once the part
    # sits at its power limit (rank 0's GPU; every rank runs the loop so the node is loaded alike)
    sustained = None
    if not args.no_sustained:
        n_loop = int(max(100, 2000.0 / max(gemm_ms, 1e-3)))
        s2 = ClockSampler(physical_gpu_index(local))
        s0_, s1_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync_all()
        s2.start()
        s0_.record(stream)
        for i in range(n_loop):
            gemm_only(i)
        s1_.record(stream)
        sync_all()
        c2 = s2.stop()
        sus_ms = s0_.elapsed_time(s1_) / n_loop
        sus_tops = OPS_PER_STEP / (sus_ms * 1e-3) / 1e12
        sustained = {"launches": n_loop, "seconds": sus_ms * n_loop / 1e3, "gemm_ms": sus_ms, "tops": sus_tops,
                     "frac_of_dense_int8_spec_4500": sus_tops / 4500.0,
                     "frac_of_2x_measured_bf16_sustained": (sus_tops / (2.0 * peaks["bf16_tflops_sustained"])
                                                            if peaks.get("bf16_tflops_sustained") else None),
                     "clocks": c2,
                     "ms_x_mhz": (sus_ms * c2["sm_mhz"]) if c2.get("sm_mhz") else None}
        be.status_poll()

    # every GEMM shape of the DiT block (dit_cuda.zig:464-517), f32 and bf16 outputs, int8 weights
    shapes = None
    if not args.no_secondary:
        shapes = []
        for (n_, k_) in ((3072, 3072), (12288, 3072), (3072, 12288)):
            qq = torch.randint(-127, 128, (M, k_), dtype=torch.int8, device="cuda")
            wsets = [torch.randint(-127, 128, (n_, k_), dtype=torch.int8, device="cuda") for _ in range(N_SETS)]
            wsc = torch.rand(n_, device="cuda") * 9e-3 + 1e-3
            saved = (be.i8_x, be.i8_scale, be.i8_m, be.i8_cols)
            be.i8_x, be.i8_scale = qq.reshape(-1), torch.rand(M, device="cuda")
            be.i8_m, be.i8_cols = M, k_
            for dt_name, dt_ in (("f32", torch.float32), ("bf16", torch.bfloat16)):
                yy = torch.empty((M, n_), dtype=dt_, device="cuda")
                fn = lambda i: be._gemm(yy, wsets[i % N_SETS], wsc, n_, 8)
                for i in range(3):
                    fn(i)
                torch.cuda.synchronize()
                e = timed_regions(fn, 20, stream, min_total_ms=60.0)
                torch.cuda.synchronize()
                ms = region_stats(e)["median_ms"] / 20
                tops = 2.0 * M * n_ * k_ / (ms * 1e-3) / 1e12
                shapes.append({"m": M, "n": n_, "k": k_, "out": dt_name, "us": ms * 1e3, "tops": tops,
                               "frac_of_dense_int8_spec_4500": tops / 4500.0,
                               "frac_of_2x_measured_bf16": tops / (2.0 * peaks["bf16_tflops"])})
                del yy
            # context only: the library's int8 GEMM (cuBLASLt through torch._int_mm) on the same operands,
            # raw int32 output (4 bytes per element like the f32 case), no dequantisation
            try:
                fn = lambda i: torch._int_mm(qq, wsets[i % N_SETS].t())
                for i in range(3):
                    fn(i)
                torch.cuda.synchronize()
                e = timed_regions(fn, 20, stream, min_total_ms=60.0)
                torch.cuda.synchronize()
                ms = region_stats(e)["median_ms"] / 20
                tops = 2.0 * M * n_ * k_ / (ms * 1e-3) / 1e12
                shapes.append({"m": M, "n": n_, "k": k_, "out": "s32, library torch._int_mm (comparison only, not a product path)",
                               "us": ms * 1e3, "tops": tops, "frac_of_dense_int8_spec_4500": tops / 4500.0})
            except Exception as ex:      # the library has no int8 GEMM for this device / shape
                shapes.append({"m": M, "n": n_, "k": k_, "out": "s32, library torch._int_mm", "unavailable": f"{type(ex).__name__}: {ex}"[:200]})
            be.i8_x, be.i8_scale, be.i8_m, be.i8_cols = saved
            del qq, wsets
        be.status_poll()
    del w8s

    # ---- timed region 2: end to end through the host-buffer entry ----
    x_pin = torch.from_numpy(x_host_src).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))

    def host_loop(y_pin, copy_only):
        for _ in range(2):
            be.convrot_linear_host(x_pin, ws[0], wss[0], N, BITS, y_pin, copy_only=copy_only)
        sync_all()
        h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        h0.record(stream)
        for i in range(e2e_steps):
            be.convrot_linear_host(x_pin, ws[i % N_SETS], wss[i % N_SETS], N, BITS, y_pin, copy_only=copy_only)
        h1.record(stream)
        sync_all()
        return h0.elapsed_time(h1)

    y_pin = torch.empty((M, N), dtype=out_dtype).pin_memory()
    e2e_ms = host_loop(y_pin, False)
    checksum = float(y_pin[0, :8].float().sum())  # the result really arrived on the host
    copy_ms = host_loop(y_pin, True)               # the same bytes over the same buffers and streams, no kernels
    other = torch.bfloat16 if out_dtype == torch.float32 else torch.float32
    y_pin2 = torch.empty((M, N), dtype=other).pin_memory()
    e2e2_ms = host_loop(y_pin2, False)
    copy2_ms = host_loop(y_pin2, True)
    del y_pin2

    # max over ranks, on the device clock
    ms_total, e2e_ms, copy_ms, e2e2_ms, copy2_ms = reduce_max([ms_total, e2e_ms, copy_ms, e2e2_ms, copy2_ms])

    line = None
    if rank == 0:
        value = OPS_PER_STEP * args.steps * world / (ms_total * 1e-3) / 1e12
        e2e_value = OPS_PER_STEP * e2e_steps * world / (e2e_ms * 1e-3) / 1e12
        gemm_tops = OPS_PER_STEP / (gemm_ms * 1e-3) / 1e12
        # The GEMM loop above runs for a fifth of a second and more without a pause, i.e. at the power-capped
        # clock: its median region is compared with the SUSTAINED library figure; the first (fastest) region
        # ran at the full clock and is compared with the burst figure.
        long_loop = greg["total_ms"] >= 100.0 and bool(peaks.get("bf16_tflops_sustained"))
        int8_peak = 2.0 * (peaks["bf16_tflops_sustained"] if long_loop else peaks["bf16_tflops"])
        burst_ms = greg["min_ms"] / args.steps
        burst_tops = OPS_PER_STEP / (burst_ms * 1e-3) / 1e12
        ob2 = 2 if out_bytes == 4 else 4
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms_total / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s8",
            "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "m": M, "n": N, "k": K, "bits": BITS, "out_dtype": args.out_dtype,
                       "l2": f"rotating {N_SETS} distinct input sets ({N_SETS * (M * K * 4 + N * K // 2) >> 20} MiB) > 126 MB L2, "
                             f"plus a {M * N * out_bytes >> 20} MiB output written every step",
                       "timing": f"{reg['count']} regions of exactly {args.steps} steps, back to back "
                                 f"({reg['total_ms']:.0f} ms of continuous work), CUDA events around each; value and "
                                 "ms_per_step are the median region, max over ranks",
                       "parallelism": f"replicas x{world} (independent batches, no collective)"},
            "regions": {"count": reg["count"], "steps_each": args.steps, "ms_per_step_median": reg["median_ms"] / args.steps,
                        "ms_per_step_min": reg["min_ms"] / args.steps, "ms_per_step_max": reg["max_ms"] / args.steps},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": M * K * 4,
                    "d2h_bytes_per_step": M * N * out_bytes, "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                    "checksum": checksum,
                    "copy_only_ms_per_step": copy_ms / e2e_steps,
                    "fraction_of_copy_only": (copy_ms / e2e_ms) if e2e_ms > 0 else None,
                    "host_gbs_aggregate": world * (M * K * 4 + M * N * out_bytes) / (e2e_ms / e2e_steps * 1e-3) / 1e9,
                    "other_out_dtype": {"out_dtype": "bf16" if out_bytes == 4 else "f32",
                                        "value": OPS_PER_STEP * e2e_steps * world / (e2e2_ms * 1e-3) / 1e12,
                                        "d2h_bytes_per_step": M * N * ob2, "ms_per_step": e2e2_ms / e2e_steps,
                                        "copy_only_ms_per_step": copy2_ms / e2e_steps}},
            "gpu_launches": gpu_launches,
            "roofline": {"bound": "tensor", "kernel": "convrot_gemm2_kernel (tcgen05 kind::i8, cta_group::2), timed alone over the same operands",
                         "achieved": gemm_tops, "peak": int8_peak, "unit": "TOP/s", "frac": gemm_tops / int8_peak,
                         "peak_note": f"2 x the {'sustained' if long_loop else 'burst'} cuBLAS bf16 figure of {peaks['source']} peaks "
                                      f"(the int8 tensor rate is twice bf16); achieved is the median of "
                                      f"{greg['total_ms']:.0f} ms of back-to-back launches",
                         "frac_of_dense_int8_spec_4500": gemm_tops / 4500.0,
                         "gemm_ms": gemm_ms,
                         "burst": {"gemm_ms": burst_ms, "tops": burst_tops,
                                   "frac_of_2x_measured_bf16_burst": burst_tops / (2.0 * peaks["bf16_tflops"]),
                                   "frac_of_dense_int8_spec_4500": burst_tops / 4500.0,
                                   "what": "fastest region of the same loop (full clock, before the power cap engages)"},
                         "regions": {"count": greg["count"], "launches_each": args.steps,
                                     "ms_min": greg["min_ms"] / args.steps, "ms_max": greg["max_ms"] / args.steps},
                         "traffic": GEMM_DRAM_TRAFFIC_BYTES[args.out_dtype],
                         "traffic_source": "one ncu capture of this launch (dram__bytes_read.sum + dram__bytes_write.sum); "
                                           "not measured by this run",
                         "sustained": sustained, "shapes": shapes},
        }

    # ---- the other parts of the metric, measured in the same run.  The headline above is
    # complete before they start: if one of them fails it says so in its own entry, and if
    # they overrun their time limit the line is printed without the rest. ----
    secondary = {}
    done = threading.Event()

    def emit():
        if rank == 0:
            if not args.no_secondary:
                line["secondary"] = secondary
            print(json.dumps(line), flush=True)

    def watchdog():
        if not done.wait(args.secondary_limit):
            secondary["timeout"] = f"stopped after {args.secondary_limit} s"
            emit()
            sys.stdout.flush()
            os._exit(0)

    if not args.no_secondary:
        threading.Thread(target=watchdog, daemon=True).start()
        del xs, ws, wss, y
        torch.cuda.empty_cache()

        def agree(ok: bool) -> bool:
            """True when every rank got through its set-up (allocations can fail on one rank only;
            the ranks must then skip the part together, or the others wait in a collective)."""
            if world == 1:
                return ok
            t = torch.tensor([1 if ok else 0], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            return bool(t[0])

        parts = [("gemv", lambda: measure_gemv(be, peaks, 50, all_formats=True)),
                 ("dit", lambda: measure_dit(be, sync_all, reduce_max, rank, steps=8, agree=agree,
                                             names=("unfused_f32", "fused_f32", "fused_bf16_whole_batch",
                                                    "fused_bf16_paired_mlp", "fused_bf16_grouped",
                                                    "fused_bf16_with_attention"))),
                 ("dit_stream", lambda: measure_dit_stream(be, sync_all, reduce_max, rank, world, steps=3, agree=agree))]
        if world > 1:
            parts.append(("nsplit", lambda: measure_nsplit(be, args, rank, world, steps=20, agree=agree)))
        for name, fn in parts:
            t0 = time.perf_counter()
            try:
                secondary[name] = fn()
            except Exception as e:
                secondary[name] = {"error": f"{type(e).__name__}: {e}"}
            if isinstance(secondary[name], dict):
                secondary[name]["wall_s"] = time.perf_counter() - t0
            torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        tops, cores, sample, _ = cpu_float_path_sample()
        line["cpu_baseline"] = {"value": tops, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
    done.set()
    emit()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    be.close()


# ---------------------------------------------------------------------------------------
# The other BASELINE configurations: measured by the default line (under `secondary`) and by
# the --mode switches, which print the same dictionaries on their own
# ---------------------------------------------------------------------------------------

def _events_ms(fn, steps, sync):
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    sync()
    return e0.elapsed_time(e1)


DIT_VARIANTS = {
    "unfused_f32": ("reference sequence: rmsMod/sigmoidMul/siluMul/gatedAdd as separate kernels, f32, 2048-row MLP tiles",
                    dict(mode="unfused")),
    "fused_f32": ("producers fused into the prep kernels, gated residuals into the GEMM epilogues, f32, 2048-row MLP tiles",
                  dict(mode="fused")),
    "fused_bf16_whole_batch": ("fused, bf16 activation chain, one MLP pass over all rows",
                               dict(mode="fused", bf16=True, whole=True)),
    "fused_bf16_paired_mlp": ("fused_bf16_whole_batch with the MLP's gate and up projections in one launch and the SiLU "
                              "gate in its epilogue", dict(mode="fused", bf16=True, whole=True, pair=True)),
    "fused_bf16_grouped": ("fused_bf16_paired_mlp with the q, k, v and gate projections of a block in one launch",
                           dict(mode="fused", bf16=True, whole=True, pair=True, group=True)),
    "linears_only": ("prep + GEMM launches only, one MLP pass over all rows", dict(mode="linears", whole=True)),
    "fused_bf16_with_attention": ("fused_bf16_grouped plus qk-norm, RoPE and softmax attention (24 heads x 128) in "
                                  "every block: the whole block stack of a step",
                                  dict(mode="fused", bf16=True, whole=True, attn=True, pair=True, group=True)),
}


def _dit_runner(be, harness, w, x_list, mod, attn, spec, latents=1):
    import torch
    rows = x_list[0].shape[0]
    kw = dict(mode=spec["mode"], mod=mod if spec["mode"] != "linears" else None, latents=latents)
    if spec.get("bf16"):
        kw["out_dtype"] = torch.bfloat16
    if spec.get("whole"):
        kw["mlp_tile"] = rows
    if spec.get("attn"):
        kw["attn"] = attn
    if spec.get("pair"):
        kw["mlp_pair"] = True
    if spec.get("group"):
        kw["qkvg_group"] = True
    return lambda i: harness.dit_step_linears(be, w, x_list[i % len(x_list)], **kw)


def _same(ok):
    return ok


def measure_dit(be, sync, reduce_max, rank, steps, names, agree=_same):
    """Config 3: one synthetic INT8 ConvRot DiT step (28 blocks, hidden 3072, MLP 12288, 4608
    tokens, one latent per GPU), weights resident."""
    import torch
    from tensorpencil_b200 import harness, synth
    T = synth.DIT_TOKENS
    w, err = None, None
    try:
        w = harness.DitWeights(be, 8, distinct_blocks=4)
        x_list = [torch.from_numpy(synth.activations(T, synth.DIT_HIDDEN, seed=1003 + 10 * rank + i)).cuda() for i in range(2)]
        mod = harness.dit_modulation(be, synth.DIT_BLOCKS, synth.DIT_HIDDEN)
        _, _, _, qn, kn, cos, sin = harness.attention_inputs(T, 1, 1, be.device)
        attn = {"q_norm": qn, "k_norm": kn, "cos": cos, "sin": sin, "heads": synth.DIT_HIDDEN // 128}
    except Exception as e:
        err = f"{type(e).__name__}: {e}"
    if not agree(err is None):
        if w is not None:
            w.close()
        return {"skipped": err or "set-up failed on another rank"}
    ms_of = {}
    for n in names:
        fn = _dit_runner(be, harness, w, x_list, mod, attn, DIT_VARIANTS[n][1])
        for i in range(2):
            fn(i)
        ms_of[n] = _events_ms(fn, steps, sync) / steps
    be.status_poll()
    # What launching from Python costs: the host time to enqueue one step, and the same step
    # captured once into a CUDA graph and replayed (no host work per launch at all).
    host_side = {}
    for n in names:
        if n not in ("fused_bf16_grouped", "fused_bf16_with_attention"):
            continue
        fn = _dit_runner(be, harness, w, x_list, mod, attn, DIT_VARIANTS[n][1])
        entry = {}
        try:
            enq = []
            for i in range(3):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                fn(i)
                enq.append((time.perf_counter() - t0) * 1e3)
            entry["host_enqueue_ms_per_step"] = min(enq)
            torch.cuda.synchronize()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fn(0)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                fn(0)
            graph.replay()
            entry["graph_replay_s_per_step"] = _events_ms(lambda i: graph.replay(), steps, torch.cuda.synchronize) / steps / 1e3   # local sync: a rank whose capture failed must not leave the others in a barrier
            be.status_poll()
            del graph
        except Exception as e:
            entry["graph"] = f"{type(e).__name__}: {e}"[:200]
        host_side[n] = entry
    vals = reduce_max([ms_of[n] for n in names])
    ops = harness.dit_linear_ops(T, synth.DIT_BLOCKS, synth.DIT_HIDDEN, synth.DIT_MLP)
    out = {"workload": "config3: INT8 ConvRot DiT step, 28 blocks, hidden 3072, MLP 12288, 4608 tokens, one latent per GPU, "
                       "weights resident", "steps": steps, "unit": "s/step",
           "scope": "the eight quantised linears per block with their elementwise neighbours (RMS norm + modulation, "
                    "sigmoid and SiLU gates, gated residual); attention runs in the variant that names it (elsewhere v "
                    "stands in for its output); tops counts the linears' 2*M*N*K only",
           "variants": {n: {"s_per_step": v / 1e3, "linear_tops": ops / (v * 1e-3) / 1e12, "what": DIT_VARIANTS[n][0]}
                        for n, v in zip(names, vals)}}
    for n, entry in host_side.items():
        out["variants"][n].update(entry)
        if "graph_replay_s_per_step" in entry:
            g = entry["graph_replay_s_per_step"]
            out["variants"][n + "_cuda_graph"] = {
                "s_per_step": g, "linear_tops": ops / g / 1e12,
                "what": DIT_VARIANTS[n][0] + "; the step captured once into a CUDA graph and replayed (rank-local figure)"}
    w.close()
    return out


def measure_dit_stream(be, sync, reduce_max, rank, world, steps, latents_per_gpu=None, agree=_same):
    """Config 4: the same model in INT4 with every block's weights streamed from pinned host
    memory under a 2 GiB device budget; a batch of TOTAL_LATENTS independent latents sharded
    TOTAL_LATENTS / world per GPU.  A block is acquired once per step and used by every local
    latent before it is released, so its image crosses PCIe once per step per GPU.  The same
    step with the weights resident runs beside it: the difference is what streaming costs."""
    import torch
    from tensorpencil_b200 import harness, synth
    L = latents_per_gpu if latents_per_gpu else max(1, TOTAL_LATENTS // world)
    T = synth.DIT_TOKENS
    names = ("fused_bf16_grouped", "fused_bf16_with_attention")
    res = {}
    x = mod = attn = None
    # On several GPUs the default route shares the host link: every rank pulls 1/world of each block
    # through PCIe and the pieces are exchanged over NVLink (all-gather on the transfer stream), so the
    # node reads each block from host memory once.  "own_copies" = every GPU pulling every byte itself.
    group = None
    routes = [("own_copies", 2 << 30, None)]
    share = world >= 4      # the default route: shared host link from four GPUs on (measured: a tie at two)
    if world > 1:
        import torch.distributed as dist
        group = dist.group.WORLD
        routes = [("shared_link", 2 << 30, group), ("own_copies", 2 << 30, None)]
    default_route = "shared_link" if share else "own_copies"
    routes.append(("resident", None, None))
    for label, budget, grp in routes:
        w, err = None, None
        try:
            if x is None:
                x = torch.cat([torch.from_numpy(synth.activations(T, synth.DIT_HIDDEN, seed=1003 + 100 * rank + i)).cuda()
                               for i in range(L)], dim=0)
                mod = harness.dit_modulation(be, synth.DIT_BLOCKS, synth.DIT_HIDDEN)
                _, _, _, qn, kn, cos, sin = harness.attention_inputs(T, 1, 1, be.device)
                attn = {"q_norm": qn, "k_norm": kn, "cos": cos, "sin": sin, "heads": synth.DIT_HIDDEN // 128}
            w = harness.DitWeights(be, 4, stream_budget=budget, distinct_blocks=4, stream_group=grp)
        except Exception as e:
            err = f"{type(e).__name__}: {e}"
        if not agree(err is None):
            if w is not None:
                w.close()
            return {"skipped": f"{label}: " + (err or "set-up failed on another rank")}
        for n in names:
            fn = _dit_runner(be, harness, w, [x], mod, attn, DIT_VARIANTS[n][1], latents=L)
            fn(0)
            c0 = w.streamer.bytes_copied() if w.streamer else 0
            ms = _events_ms(fn, steps, sync) / steps
            copied = ((w.streamer.bytes_copied() - c0) / steps) if w.streamer else 0
            res[(label, n)] = (ms, copied)
        be.status_poll()
        if w.streamer and label == default_route:
            res["slots"] = {"slot_bytes": w.block_bytes, "budget_bytes": budget}
        w.close()
        del w
        torch.cuda.empty_cache()
    labels = [r[0] for r in routes]
    keys = [(l, n) for l in labels for n in names]
    vals = reduce_max([res[k][0] for k in keys])
    ms = dict(zip(keys, vals))
    out = {"workload": f"config4: INT4 ConvRot DiT step, weights streamed from pinned host memory under a 2 GiB budget, "
                       f"batch of {TOTAL_LATENTS} latents, {L} per GPU on {world} GPU(s); max over ranks",
           "latents_per_gpu": L, "latents_total": L * world, "steps": steps, "unit": "s/step (whole batch)",
           "route": (("each block crosses the host link once per node: every GPU copies 1/%d of it, the pieces are "
                      "all-gathered over NVLink on the transfer stream (default from four GPUs on)" % world) if share else
                     ("every GPU copies every block through its own link" + (" (default at two GPUs, where the host keeps "
                      "up and the exchange kernel would only take SMs from the step)" if world > 1 else ""))),
           "slots": res.get("slots"), "variants": {}}
    for n in names:
        s_ms, r_ms = ms[(default_route, n)], ms[("resident", n)]
        copied = res[(default_route, n)][1]
        out["variants"][n] = {"s_per_step": s_ms / 1e3, "s_per_step_weights_resident": r_ms / 1e3,
                              "streaming_overhead": s_ms / r_ms - 1.0,
                              "streamed_bytes_per_step_per_gpu": copied,
                              "h2d_gbs_per_gpu": copied / (s_ms * 1e-3) / 1e9,
                              "s_per_latent": s_ms / 1e3 / L, "what": DIT_VARIANTS[n][0]}
        if world > 1:
            out["variants"][n].update({"s_per_step_shared_host_link": ms[("shared_link", n)] / 1e3,
                                       "s_per_step_every_gpu_copies_everything": ms[("own_copies", n)] / 1e3,
                                       "h2d_bytes_per_step_per_gpu_shared_host_link": res[("shared_link", n)][1],
                                       "h2d_bytes_per_step_per_gpu_every_gpu_copies_everything": res[("own_copies", n)][1]})
    return out


def run_mode_dit(args, rank, local, world, streamed: bool):
    """--mode dit / dit-stream: configs 3 / 4 on their own (every variant)."""
    import torch
    import torch.distributed as dist
    from tensorpencil_b200.backend import Backend
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    be = Backend(local)

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def reduce_max(vals):
        if world == 1:
            return [float(v) for v in vals]
        t = torch.tensor(list(vals), device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t]

    steps = max(1, min(args.steps, 20))
    if streamed:
        out = measure_dit_stream(be, sync, reduce_max, rank, world, steps, latents_per_gpu=args.latents or None)
        if "skipped" in out:
            raise SystemExit(out["skipped"])
        head = out["variants"]["fused_bf16_grouped"]["s_per_step"]
        metric = "dit_int4_streamed_s_per_step"
    else:
        out = measure_dit(be, sync, reduce_max, rank, steps, tuple(DIT_VARIANTS))
        head = out["variants"]["fused_f32"]["s_per_step"]
        metric = "dit_linears_s_per_step"
    if rank == 0:
        line = {"metric": metric, "value": head, "unit": "s/step", "n_gpus": world, "steps": steps,
                "higher_is_better": False, "scaling": "strong" if streamed else "weak", "dtype": "s8", "data": "synthetic",
                "config": {"workload": out["workload"]}}
        line.update(out)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    be.close()


def measure_nsplit(be, args, rank, world, steps, agree=_same):
    """Config 4, second half: one [4608x3072]x[3072x12288] INT8 GEMM split along N over the
    ranks, every rank ending with the whole output.  Three exchanges are timed: the GEMM whose
    epilogue performs the all-gather itself (peer stores over NVLink, row-major or column-blocked
    destination; one NVSwitch multicast store per element where available), and the plain GEMM
    followed by NCCL's all-gather (compute and collective also timed separately)."""
    import torch
    import torch.distributed as dist
    from tensorpencil_b200 import nsplit, synth
    c = synth.convrot_linear(M, N, K, 8, seed=1004)   # same inputs on every rank
    lo, hi = nsplit.shard_bounds(N, world, rank)
    x = torch.from_numpy(c["x"]).cuda()
    w_shard = torch.from_numpy(c["w_i8"][lo:hi]).cuda()
    ws_shard = torch.from_numpy(c["w_scale"][lo:hi]).cuda()
    w_full, ws_full = torch.from_numpy(c["w_i8"]).cuda(), torch.from_numpy(c["w_scale"]).cuda()
    chunks = 4 if (N // world) % 64 == 0 else 1

    def sync():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    be.opI8Prep(x, M, K)
    out = {"workload": "config4: INT8 GEMM 4608x12288x3072 split along N across the GPUs, every rank ends with the "
                       "whole output (all-gather fused into the GEMM epilogue; NCCL version beside it)",
           "steps": steps, "ops_per_step": OPS_PER_STEP}
    from tensorpencil_b200.peer import MulticastBuffers, PeerBuffers
    # one pair of exchange buffers, sized for the f32 output, serves both output types
    pb = PeerBuffers(be, M * N * 4)
    mb, mb_err = None, None
    try:
        mb = MulticastBuffers(be, M * N * 4)
    except Exception as e:      # no symmetric-memory / multicast support: the unicast forms still run
        mb_err = f"{type(e).__name__}: {e}"
    have_mc = agree(mb is not None and mb.available)
    if not have_mc:
        out["multicast"] = mb_err or "not available on every rank"
    for dt_name, out_dtype, esz in (("f32", torch.float32, 4), ("bf16", torch.bfloat16, 2)):
        def compute(a, b):
            yy = torch.empty((M, b - a), dtype=out_dtype, device="cuda")
            be.opI8Gemm(yy, w_shard[a - lo:b - lo], ws_shard[a - lo:b - lo], b - a)
            return yy

        y_full = torch.empty((M, N), dtype=out_dtype, device="cuda")
        be.opI8Gemm(y_full, w_full, ws_full, N)
        gathered = torch.empty((chunks, world, M, (hi - lo) // chunks), dtype=out_dtype, device="cuda")
        for _ in range(3):
            nsplit.nsplit_gemm_allgather(compute, M, N, chunks=chunks, out=gathered)
        same_nccl = bool(torch.equal(nsplit.assemble(gathered), y_full))
        ms_total = _events_ms(lambda i: nsplit.nsplit_gemm_allgather(compute, M, N, chunks=chunks, out=gathered), steps, sync)
        ms_compute = _events_ms(lambda i: compute(lo, hi), steps, sync)
        ms_single = _events_ms(lambda i: be.opI8Gemm(y_full, w_full, ws_full, N), steps, sync)
        shard = torch.empty((M, hi - lo), dtype=out_dtype, device="cuda")
        flat = torch.empty((world * M, hi - lo), dtype=out_dtype, device="cuda")
        ms_gather = _events_ms(lambda i: dist.all_gather_into_tensor(flat, shard), steps, sync)
        del gathered, flat, shard

        def fused(i):
            pb.gemm_allgather(w_shard, ws_shard, hi - lo, 8, y_dtype=out_dtype)
            pb.barrier()

        def fused_blocked(i):
            pb.gemm_allgather_blocked(w_shard, ws_shard, hi - lo, 8, y_dtype=out_dtype)
            pb.barrier()

        variants = {}
        # Row-major unicast: every 128-byte row segment of a tile goes to world-1 peers at a pitch of
        # N*esz bytes; at 8 GPUs x f32 that pattern collapses (milliseconds), so beyond 4 ranks only the
        # blocked and multicast forms are offered.
        if world <= 4:
            pb.barrier()
            for i in range(3):
                fused(i)
            sync()
            same = bool(torch.equal(pb.tensor((M, N), out_dtype), y_full))
            variants["fused_rowmajor_unicast"] = [_events_ms(fused, steps, sync), same]
        pb.barrier()
        for i in range(3):
            fused_blocked(i)
        sync()
        same = bool(torch.equal(nsplit.assemble(pb.tensor((1, world, M, hi - lo), out_dtype)), y_full))
        variants["fused_blocked_unicast"] = [_events_ms(fused_blocked, steps, sync), same]
        be.status_poll()
        if have_mc:
            def fused_mc(i):
                mb.gemm_allgather(w_shard, ws_shard, hi - lo, 8, y_dtype=out_dtype)
                mb.barrier()

            mb.barrier()
            for i in range(3):
                fused_mc(i)
            sync()
            same = bool(torch.equal(mb.tensor((M, N), out_dtype), y_full))
            variants["fused_rowmajor_multicast"] = [_events_ms(fused_mc, steps, sync), same]
            be.status_poll()
        del y_full
        names = sorted(variants)
        t = torch.tensor([ms_total, ms_compute, ms_gather, ms_single] + [variants[n][0] for n in names],
                         device="cuda", dtype=torch.float64)
        flags = torch.tensor([int(same_nccl)] + [int(variants[n][1]) for n in names], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        recv = (world - 1) / world * M * N * esz
        nvlink_floor_ms = recv / 770e9 * 1e3
        d = {"single_gpu_gemm_ms": float(t[3]) / steps,
             "nvlink_receive_floor_ms": nvlink_floor_ms,
             "nvlink_floor_note": "each GPU must receive (g-1)/g of the output: bytes / 770 GB/s measured peer bandwidth",
             "nccl": {"ms_total": float(t[0]) / steps, "ms_compute_only": float(t[1]) / steps,
                      "ms_allgather_only": float(t[2]) / steps, "chunks": chunks,
                      "tops": OPS_PER_STEP / (float(t[0]) / steps * 1e-3) / 1e12,
                      "allgather_recv_gbs_per_gpu": recv / (float(t[2]) / steps * 1e-3) / 1e9,
                      "bit_identical_to_single_gpu": bool(flags[0]),
                      "layout": "gathered[chunk][rank][M][N/world/chunks] (column-blocked)"}}
        for i, n in enumerate(names):
            ms = float(t[4 + i]) / steps
            d[n] = {"ms": ms, "tops": OPS_PER_STEP / (ms * 1e-3) / 1e12, "recv_gbs_per_gpu": recv / (ms * 1e-3) / 1e9,
                    "frac_of_nvlink_floor": nvlink_floor_ms / ms, "bit_identical_to_single_gpu": bool(flags[1 + i])}
        rowmajor = [n for n in names if "rowmajor" in n]
        best_rm = min(rowmajor, key=lambda n: d[n]["ms"]) if rowmajor else None
        best = min(names, key=lambda n: d[n]["ms"])
        d["best_rowmajor"] = best_rm
        d["best"] = best
        d["limiter"] = ("NVLink receive" if d[best]["ms"] < 1.6 * nvlink_floor_ms else "not the link: see the variants")
        out[dt_name] = d
    if mb is not None:
        mb.close()
    pb.close()
    return out


def run_mode_nsplit(args, rank, local, world):
    import torch
    import torch.distributed as dist
    from tensorpencil_b200.backend import Backend
    if world < 2:
        raise SystemExit("--mode nsplit needs at least 2 ranks (torchrun)")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    be = Backend(local)
    steps = max(3, min(args.steps, 50))
    out = measure_nsplit(be, args, rank, world, steps)
    if rank == 0:
        d = out[args.out_dtype]
        best = d["best"]
        line = {"metric": "nsplit_gemm_allgather_tops", "value": d[best]["tops"], "unit": "TOPS", "n_gpus": world,
                "steps": steps, "higher_is_better": True, "scaling": "strong", "dtype": "s8", "data": "synthetic",
                "ms_per_step": d[best]["ms"], "config": {"workload": out["workload"], "out_dtype": args.out_dtype}}
        line.update(out)
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    be.close()


def measure_gemv(be, peaks, steps, all_formats=True):
    """Config 2: Q8_0 decode GEMV, K=5120 -> N=17408 and the down projection, M in {1,4,8},
    four rotating weight buffers (379 MB > L2) so every launch streams from HBM; then the other
    GGUF formats at the up-projection shape and three of them at the down-projection shape.  Algorithmic
    bytes = the weight matrix."""
    import torch
    from tensorpencil_b200 import harness, synth
    rows_out = []
    for (n, k) in ((17408, 5120), (5120, 17408)):
        ws = harness.rotating_q8_weights(n, k, 4, be.device)
        for m in (1, 4, 8):
            x = torch.randn(m, k, device="cuda")
            y = torch.empty(m, n, device="cuda")
            be.opGemvQuantizeX(x, m * k)
            fn = lambda i: be.opGemvQuantQ8N("q8_0", y, ws[i % 4], 1.0, n, k, m, 0, m)
            for i in range(5):
                fn(i)
            ms = _events_ms(fn, steps, torch.cuda.synchronize) / steps
            gbs = n * (k // 32) * 34 / (ms * 1e-3) / 1e9
            rows_out.append({"fmt": "q8_0", "n": n, "k": k, "m": m, "us": ms * 1e3, "gbs": gbs,
                             "frac_of_hbm": gbs / peaks["hbm_gbs"]})
        del ws
    if all_formats:
        # the up projection for every format; the down projection (long rows: the k-quants' second kernel) for three
        shapes = [(fmt, 17408, 5120, (1, 4, 8)) for fmt in ("q4_k", "q5_k", "q6_k", "q4_0", "iq4_nl")]
        shapes += [(fmt, 5120, 17408, (1, 2)) for fmt in ("q4_k", "q5_k", "q4_0")]
        for fmt, n, k, ms_ in shapes:
            base = torch.from_numpy(synth.gguf_weights(fmt, n, k, seed=11)).cuda()
            copies = 8
            ws = [base] + [base.clone() for _ in range(copies - 1)]       # 8 x 50..61 MB > 126 MB of L2
            wbytes = base.numel()
            for m in ms_:
                x = torch.randn(m, k, device="cuda")
                y = torch.empty(m, n, device="cuda")
                be.opGemvQuantizeX(x, m * k)
                fn = lambda i: be.opGemvQuantQ8N(fmt, y, ws[i % copies], 1.0, n, k, m, 0, m)
                for i in range(5):
                    fn(i)
                ms = _events_ms(fn, steps, torch.cuda.synchronize) / steps
                gbs = wbytes / (ms * 1e-3) / 1e9
                rows_out.append({"fmt": fmt, "n": n, "k": k, "m": m, "us": ms * 1e3, "gbs": gbs,
                                 "frac_of_hbm": gbs / peaks["hbm_gbs"]})
            del ws, base
    be.status_poll()
    q8 = [r for r in rows_out if r["fmt"] == "q8_0"]
    return {"workload": "config2: GGUF decode GEMV, K=5120 -> N=17408 and K=17408 -> N=5120, M in {1,4,8}; "
                        f"{steps} back-to-back launches over rotating weight copies larger than L2",
            "peak_hbm_gbs": peaks["hbm_gbs"], "peak_note": f"{peaks['source']} copy bandwidth",
            "bar": 0.75, "q8_0_cases_at_or_above_bar": sum(1 for r in q8 if r["frac_of_hbm"] >= 0.75),
            "q8_0_min_frac": min(r["frac_of_hbm"] for r in q8), "cases": rows_out}


def run_mode_gemv(args, rank, local, world):
    import torch
    from tensorpencil_b200.backend import Backend
    torch.cuda.set_device(local)
    be = Backend(local)
    peaks = measured_peaks()
    out = measure_gemv(be, peaks, max(20, args.steps))
    head = out["cases"][0]
    line = {"metric": "qgemv_hbm_gbs", "value": head["gbs"], "unit": "GB/s", "n_gpus": 1,
            "higher_is_better": True, "dtype": "s8", "data": "synthetic",
            "roofline": {"bound": "hbm", "achieved": head["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": head["frac_of_hbm"], "peak_note": f"{peaks['source']} copy bandwidth"},
            "config": {"workload": "config2: Q8_0 GEMV, headline = M=1, K=5120 -> N=17408"}}
    line.update(out)
    print(json.dumps(line), flush=True)
    be.close()


def run_mode_gemv_shapes(args, local):
    """The Q8_0 decode GEMV on ten weight shapes at M = 1 .. 8, as the library dispatches it and with each of its
    two kernels forced (TPB_GEMV_KERNEL): the table the dispatch rule of tpb_q8_0_gemv_q8n was written from.
    Also the other GGUF formats' two kernels (TPB_GEMVK_KERNEL) at M = 1, 2."""
    import torch
    from tensorpencil_b200 import harness, synth
    from tensorpencil_b200.backend import Backend
    torch.cuda.set_device(local)
    be = Backend(local)
    peaks = measured_peaks()

    def best_of_3(fn, n=50):
        for i in range(5):
            fn(i)
        return min(_events_ms(fn, n, torch.cuda.synchronize) / n for _ in range(3))

    rows_out = []
    shapes = ((17408, 5120), (5120, 17408), (32000, 4096), (4096, 14336), (14336, 4096), (8192, 8192), (28672, 8192),
              (8192, 28672), (6144, 4096), (4096, 11008))
    for (n, k) in shapes:
        wbytes = n * (k // 32) * 34
        copies = max(2, min(8, int(400e6 // wbytes) + 1))
        ws = harness.rotating_q8_weights(n, k, copies, be.device)
        for m in (1, 2, 3, 4, 5, 6, 8):
            x = torch.randn(m, k, device="cuda")
            y = torch.empty(m, n, device="cuda")
            be.opGemvQuantizeX(x, m * k)
            fn = lambda i: be.opGemvQuantQ8N("q8_0", y, ws[i % copies], 1.0, n, k, m, 0, m)
            row = {"fmt": "q8_0", "n": n, "k": k, "m": m}
            for name, env in (("auto", None), ("dp4a", "dp4a"), ("mma", "mma")):
                if env is None:
                    os.environ.pop("TPB_GEMV_KERNEL", None)
                else:
                    os.environ["TPB_GEMV_KERNEL"] = env
                row[name + "_us"] = best_of_3(fn) * 1e3
            os.environ.pop("TPB_GEMV_KERNEL", None)
            row["auto_over_best"] = row["auto_us"] / min(row["dp4a_us"], row["mma_us"])
            row["auto_frac_of_hbm"] = wbytes / (row["auto_us"] * 1e-6) / 1e9 / peaks["hbm_gbs"]
            rows_out.append(row)
        del ws
    kq = []
    for fmt in ("q4_k", "q4_0", "q5_k"):
        for (n, k) in ((17408, 5120), (5120, 17408), (32000, 4096), (4096, 14336), (8192, 8192), (14336, 4096)):
            base = torch.from_numpy(synth.gguf_weights(fmt, n, k, seed=11)).cuda()
            ws = [base] + [base.clone() for _ in range(7)]
            for m in (1, 2):
                x = torch.randn(m, k, device="cuda")
                y = torch.empty(m, n, device="cuda")
                be.opGemvQuantizeX(x, m * k)
                fn = lambda i: be.opGemvQuantQ8N(fmt, y, ws[i % 8], 1.0, n, k, m, 0, m)
                row = {"fmt": fmt, "n": n, "k": k, "m": m}
                for name, env in (("auto", None), ("warp", "warp"), ("ring", "ring")):
                    if env is None:
                        os.environ.pop("TPB_GEMVK_KERNEL", None)
                    else:
                        os.environ["TPB_GEMVK_KERNEL"] = env
                    row[name + "_us"] = best_of_3(fn) * 1e3
                os.environ.pop("TPB_GEMVK_KERNEL", None)
                row["auto_frac_of_hbm"] = base.numel() / (row["auto_us"] * 1e-6) / 1e9 / peaks["hbm_gbs"]
                kq.append(row)
            del ws, base
    be.status_poll()
    q = [r["auto_over_best"] for r in rows_out]
    print(json.dumps({"mode": "gemv-shapes", "what": "best of three 50-launch regions per entry, rotating weight copies larger than L2",
                      "q8_0_auto_over_best_mean": float(np.mean(q)), "q8_0_auto_over_best_max": float(np.max(q)),
                      "q8_0": rows_out, "other_formats": kq}), flush=True)
    be.close()


def run_mode_attn(args, local):
    """The attention of one DiT block at config 3's shape (seq 4608, 24 heads x 128, non-causal):
    the prepare pass (qk-norm + RoPE + per-head bf16 layout) and the tcgen05 softmax(q k^T) v
    kernel timed separately, with torch's scaled_dot_product_attention on the same operands
    beside it as the library figure.  FLOPs = 4 * seq^2 * head_dim * heads."""
    import torch
    from tensorpencil_b200 import harness
    from tensorpencil_b200.backend import Backend
    torch.cuda.set_device(local)
    be = Backend(local)
    peaks = measured_peaks()
    cases = []
    for (seq, heads, kv_heads) in ((4608, 24, 24), (4608, 24, 8), (1024, 24, 24), (16384, 24, 24)):
        q, k, v, qn, kn, cos, sin = harness.attention_inputs(seq, heads, kv_heads, be.device, torch.bfloat16)
        out = torch.empty(seq, heads * 128, dtype=torch.bfloat16, device="cuda")
        be.attention(q, k, v, qn, kn, cos, sin, heads, kv_heads, out=out)
        lib = be.lib
        qb, kb, vt = be._attn_qb, be._attn_kb, be._attn_vt
        TPB_BF16 = 1
        prep = lambda i: be._check(lib.tpb_attn_prepare(be.h, be._stream(), q.data_ptr(), k.data_ptr(), v.data_ptr(), TPB_BF16,
                                                        qn.data_ptr(), kn.data_ptr(), 1e-5, cos.data_ptr(), sin.data_ptr(),
                                                        seq, heads, kv_heads, 128, qb.data_ptr(), kb.data_ptr(), vt.data_ptr()))
        att = lambda i: be._check(lib.tpb_attention(be.h, be._stream(), out.data_ptr(), TPB_BF16, qb.data_ptr(), kb.data_ptr(),
                                                    vt.data_ptr(), seq, seq, heads, kv_heads, 128, 128 ** -0.5))
        steps = max(10, min(args.steps, 50))
        for i in range(3):
            prep(i), att(i)
        ms_prep = _events_ms(prep, steps, torch.cuda.synchronize) / steps
        ms_att = _events_ms(att, steps, torch.cuda.synchronize) / steps
        # library figure: torch SDPA on [1][heads][seq][128] bf16 views of the same prepared operands
        qt = qb.unsqueeze(0)
        kt = kb.repeat_interleave(heads // kv_heads, dim=0).unsqueeze(0)
        vv = v.reshape(seq, kv_heads, 128).permute(1, 0, 2).repeat_interleave(heads // kv_heads, dim=0).unsqueeze(0).contiguous()
        sd = lambda i: torch.nn.functional.scaled_dot_product_attention(qt, kt, vv)
        for i in range(3):
            sd(i)
        ms_sdpa = _events_ms(sd, steps, torch.cuda.synchronize) / steps
        ref = sd(0)[0].permute(1, 0, 2).reshape(seq, heads * 128).float()
        diff = (out.float() - ref).abs().max().item()
        flops = 4.0 * seq * seq * 128 * heads
        cases.append({"seq": seq, "heads": heads, "kv_heads": kv_heads, "prepare_us": ms_prep * 1e3,
                      "attention_us": ms_att * 1e3, "tflops": flops / (ms_att * 1e-3) / 1e12,
                      "frac_of_bf16_peak": flops / (ms_att * 1e-3) / 1e12 / peaks["bf16_tflops"],
                      "torch_sdpa_us": ms_sdpa * 1e3, "max_abs_diff_vs_sdpa": diff})
        del q, k, v, out, qt, kt, vv, ref
    be.status_poll()
    head = cases[0]
    print(json.dumps({"metric": "attention_tflops", "value": head["tflops"], "unit": "TFLOP/s", "n_gpus": 1,
                      "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
                      "roofline": {"bound": "tensor", "achieved": head["tflops"], "peak": peaks["bf16_tflops"],
                                   "unit": "TFLOP/s", "frac": head["frac_of_bf16_peak"],
                                   "peak_note": f"{peaks['source']} cuBLAS bf16 burst"},
                      "config": {"workload": "config3's attention: seq 4608, 24 heads x 128, non-causal, bf16 operands"},
                      "cases": cases}), flush=True)
    be.close()


def run_mode_one_kernel(args, local):
    """Launches one kernel of the path a few times through the C ABI -- a small,
    self-ending command to run under a profiler."""
    import torch
    from tensorpencil_b200 import harness
    from tensorpencil_b200.backend import Backend
    torch.cuda.set_device(local)
    case = args.case
    if case in ("gemm-w4-fused", "gemm-w4-fused-small"):
        os.environ["TPB_W4_FUSED"] = "1"       # read when the handle is created
    if case == "gemm-ablation":
        # What each part of the two-CTA GEMM's pipeline costs the tensor pipe: the same launch with
        # loads of q, loads of w and / or the epilogue switched off (TPB_GEMM_ABLATE, read when a
        # handle is created; results are meaningless, timings are not).  Variants are interleaved
        # and repeated so that clock drift under the power cap hits them alike; time x sampled SM
        # MHz is printed beside the time for the same reason.
        variants = (("full", 0), ("no q loads", 1), ("no w loads", 2), ("no loads", 3), ("no epilogue", 4),
                    ("no loads, no epilogue", 7), ("epilogue reads tensor memory only", 8),
                    ("epilogue without its stores", 16), ("no loads, epilogue reads tensor memory only", 11),
                    ("no loads, epilogue without its stores", 19))
        dt = torch.bfloat16 if args.out_dtype == "bf16" else torch.float32
        rows = {name: [] for name, _ in variants}
        q = torch.randint(-127, 128, (M, K), dtype=torch.int8, device="cuda")
        ws_ = [torch.randint(-127, 128, (N, K), dtype=torch.int8, device="cuda") for _ in range(N_SETS)]
        sc, y = torch.rand(N, device="cuda"), torch.empty(M, N, dtype=dt, device="cuda")
        asc = torch.rand(M, device="cuda")
        for rep in range(3):
            for name, bits in variants:
                os.environ["TPB_GEMM_ABLATE"] = str(bits)
                be = Backend(local)
                be.i8_x, be.i8_scale = q.reshape(-1), asc
                be.i8_m, be.i8_cols, be.i8_bits = M, K, 8
                fn = lambda i: be._gemm(y, ws_[i % N_SETS], sc, N, 8)
                for i in range(3):
                    fn(i)
                sampler = ClockSampler(physical_gpu_index(local))
                torch.cuda.synchronize()
                sampler.start()
                ms = _events_ms(fn, 100, torch.cuda.synchronize) / 100
                clk = sampler.stop()
                try:
                    be.status_poll()
                except Exception as e:
                    print(json.dumps({"variant": name, "error": str(e)}), flush=True)
                rows[name].append((ms, clk.get("sm_mhz")))
                be.close()
        os.environ.pop("TPB_GEMM_ABLATE", None)
        out = []
        for name, _ in variants:
            ms = float(np.median([r[0] for r in rows[name]]))
            mhz = [r[1] for r in rows[name] if r[1]]
            mhz = float(np.median(mhz)) if mhz else None
            tops = OPS_PER_STEP / (ms * 1e-3) / 1e12
            out.append({"variant": name, "us": ms * 1e3, "tops": tops, "sm_mhz": mhz,
                        "us_x_ghz": ms * 1e3 * mhz / 1e3 if mhz else None,
                        "tensor_util_at_sampled_clock": (tops / (148 * 8192 * 2 * mhz * 1e6 / 1e12)) if mhz else None})
        print(json.dumps({"mode": "one-kernel", "case": case, "out_dtype": args.out_dtype, "m": M, "n": N, "k": K,
                          "variants": out}), flush=True)
        return
    be = Backend(local)
    reps = max(1, min(args.steps, 5))
    if case in ("prep", "prep-mlp"):
        m, k = (M, K) if case == "prep" else (2048, N)
        x = torch.randn(m, k, device="cuda")
        for _ in range(reps):
            be._prep(x, m, k, 8)
    elif case in ("gemm", "gemm-bf16", "gemm-small", "gemm-w4", "gemm-w4-fused", "gemm-w4-small", "gemm-w4-fused-small"):
        # the -small cases (2048 x 6144 x 3072) are the ones the multi-pass ncu captures run on
        m, n, k = (2048, 6144, 3072) if case.endswith("-small") else (M, N, K)
        dt = torch.bfloat16 if case == "gemm-bf16" else torch.float32
        w4 = case.startswith("gemm-w4")
        q = torch.randint(-7 if w4 else -127, 8 if w4 else 128, (m, k), dtype=torch.int8, device="cuda")
        w = (torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda") if w4
             else torch.randint(-127, 128, (n, k), dtype=torch.int8, device="cuda"))
        be.i8_x, be.i8_scale = q.reshape(-1), torch.rand(m, device="cuda")
        be.i8_sum = q.to(torch.int32).sum(dim=1).to(torch.int32)
        be.i8_m, be.i8_cols, be.i8_bits = m, k, 4 if w4 else 8
        ws, y = torch.rand(n, device="cuda"), torch.empty(m, n, dtype=dt, device="cuda")
        for _ in range(reps):
            be._gemm(y, w, ws, n, 4 if w4 else 8)
    elif case in ("gemv1-q4k", "gemv1-q6k", "gemv8-q4k"):
        from tensorpencil_b200 import synth
        m = int(case[4])
        fmt = "q4_k" if case.endswith("q4k") else "q6_k"
        n, k = 17408, 5120
        w = torch.from_numpy(synth.gguf_weights(fmt, n, k, seed=11)).cuda()
        x = torch.randn(m, k, device="cuda")
        y = torch.empty(m, n, device="cuda")
        be.opGemvQuantizeX(x, m * k)
        for _ in range(reps):
            be.opGemvQuantQ8N(fmt, y, w, 1.0, n, k, m, 0, m)
    elif case == "copy-sweep":
        # What a plain device-to-device copy reaches at the byte counts of this path's HBM-bound
        # kernels (the measured HBM peak is for buffers of gigabytes): rotating buffers, 50
        # back-to-back copies between two events, traffic = read + write.
        out = []
        for mb in (14, 28, 35, 47, 56, 113, 452):
            nbytes = mb * 1024 * 1024
            xs = [torch.empty(nbytes, dtype=torch.uint8, device="cuda") for _ in range(4)]
            ys = [torch.empty(nbytes, dtype=torch.uint8, device="cuda") for _ in range(4)]
            ms = _events_ms(lambda i: ys[i % 4].copy_(xs[i % 4]), 50, torch.cuda.synchronize) / 50
            out.append({"traffic_mb": 2 * nbytes / 1e6, "us": ms * 1e3, "gbs": 2 * nbytes / (ms * 1e-3) / 1e9})
            del xs, ys
        print(json.dumps({"mode": "one-kernel", "case": case, "copies": out}), flush=True)
        be.close()
        return
    elif case == "dit-blocks":
        # two blocks of the fused bf16 DiT step with attention, run twice: the launch list of one block
        from tensorpencil_b200 import synth
        T = synth.DIT_TOKENS
        w = harness.DitWeights(be, 8, blocks=2)
        x = torch.from_numpy(synth.activations(T, synth.DIT_HIDDEN, seed=1003)).cuda()
        mod = harness.dit_modulation(be, 2, synth.DIT_HIDDEN)
        _, _, _, qn, kn, cos, sin = harness.attention_inputs(T, 1, 1, be.device)
        attn = {"q_norm": qn, "k_norm": kn, "cos": cos, "sin": sin, "heads": synth.DIT_HIDDEN // 128}
        for _ in range(2):
            harness.dit_step_linears(be, w, x, out_dtype=torch.bfloat16, mode="fused", mod=mod, mlp_tile=T, attn=attn,
                                     mlp_pair=True, qkvg_group=True)
        reps = 2
    elif case == "attn":
        seq, heads = 4608, 24
        q, k, v, qn, kn, cos, sin = harness.attention_inputs(seq, heads, heads, be.device, torch.bfloat16)
        for _ in range(reps):
            be.attention(q, k, v, qn, kn, cos, sin, heads, heads)
    elif case == "prep-silu":
        m, k = 2048, N
        g, u = torch.randn(m, k, device="cuda"), torch.randn(m, k, device="cuda")
        for _ in range(reps):
            be.prepSiluMul(g, u, m, k, 8)
    elif case in ("gemv1", "gemv4", "gemv8", "gemv1-down", "gemv4-down", "gemv8-down"):
        m = int(case[4]) if case[4].isdigit() else 1
        n, k = (5120, 17408) if case.endswith("down") else (17408, 5120)
        w = harness.rotating_q8_weights(n, k, 1, be.device)[0]
        x = torch.randn(m, k, device="cuda")
        y = torch.empty(m, n, device="cuda")
        be.opGemvQuantizeX(x, m * k)
        for _ in range(reps):
            be.opGemvQuantQ8N("q8_0", y, w, 1.0, n, k, m, 0, m)
    else:
        raise SystemExit(f"unknown --case {case}")
    torch.cuda.synchronize()
    be.status_poll()
    print(json.dumps({"mode": "one-kernel", "case": case, "launches": reps}), flush=True)
    be.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--out-dtype", choices=["f32", "bf16"], default="f32")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="headline only: skip configs 2-4 and the per-shape table")
    ap.add_argument("--no-sustained", action="store_true", help="skip the 2 s sustained loop of the GEMM")
    ap.add_argument("--secondary-limit", type=float, default=420.0,
                    help="seconds after which the line is printed without the unfinished secondary parts")
    ap.add_argument("--latents", type=int, default=0, help="--mode dit-stream: latents per GPU (default 8 / GPUs)")
    ap.add_argument("--mode", choices=["linear", "dit", "dit-stream", "nsplit", "gemv", "gemv-shapes", "attn", "one-kernel"], default="linear",
                    help="linear = the driver's default line (config 1); the others cover configs 2-4")
    ap.add_argument("--case", default="gemm", help="kernel for --mode one-kernel: prep, prep-mlp, gemm, gemm-bf16, "
                    "gemm-small, gemm-w4, gemm-w4-fused, gemm-w4-small, gemm-w4-fused-small, gemm-ablation, gemv1, gemv4, gemv8, gemv1-down, gemv4-down, gemv8-down, gemv1-q4k, gemv1-q6k, gemv8-q4k, prep-silu, attn, dit-blocks")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch multi-GPU runs with torch.distributed.run (one process per GPU)")
    if world > 1:
        bind_to_gpu_numa_node(local)
    if args.mode == "dit":
        return run_mode_dit(args, rank, local, world, streamed=False)
    if args.mode == "dit-stream":
        return run_mode_dit(args, rank, local, world, streamed=True)
    if args.mode == "nsplit":
        return run_mode_nsplit(args, rank, local, world)
    if args.mode == "gemv":
        return run_mode_gemv(args, rank, local, world)
    if args.mode == "gemv-shapes":
        return run_mode_gemv_shapes(args, local)
    if args.mode == "attn":
        return run_mode_attn(args, local)
    if args.mode == "one-kernel":
        return run_mode_one_kernel(args, local)
    run_ours(args, rank, local, world)


if __name__ == "__main__":
    main()
