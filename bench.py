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

# DRAM bytes of one full-size GEMM launch (dram__bytes_read.sum + dram__bytes_write.sum)
# from the ncu capture summarised in profiles/convrot_gemm2_config1.md, per output type.
GEMM_DRAM_TRAFFIC_BYTES = {"f32": 227.4e6, "bf16": 118.9e6}


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
        "config": {"workload": "config1: INT4 ConvRot linear M=4608 K=3072 N=12288", "m": M, "n": N, "k": K,
                   "bits": BITS, "note": "CPU restatement of the reference's --backend cpu path (Zig absent: the reference binary cannot run)"},
        "cpu_baseline": {"value": tops, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------

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
        # one library call per linear: int4 -> int8 weight expansion, activation prep, GEMM
        s = i % N_SETS
        be.convrot_linear(xs[s], ws[s], wss[s], N, BITS, y=y)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(i)
    sync_all()
    be.status_poll()

    # ---- timed region 1: inputs resident in HBM ----
    sampler = ClockSampler(physical_gpu_index(local))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = be.launches
    sync_all()
    sampler.start()
    e0.record(stream)
    for i in range(args.steps):
        step(i)
    e1.record(stream)
    sync_all()
    clocks = sampler.stop()
    ms_total = e0.elapsed_time(e1)
    gpu_launches = be.launches - launches0
    be.status_poll()

    # ---- the dominant kernel alone, for the roofline: the int8 GEMM on the expanded weights of
    # the same sets (rotating, so operands come from HBM), args.steps back-to-back launches ----
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
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    g0.record(stream)
    for i in range(args.steps):
        gemm_only(i)
    g1.record(stream)
    sync_all()
    gemm_ms = g0.elapsed_time(g1) / args.steps
    be.status_poll()
    del w8s

    # ---- timed region 2: end to end through the host-buffer entry ----
    x_pin = torch.from_numpy(x_host_src).pin_memory()
    y_pin = torch.empty((M, N), dtype=out_dtype).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        be.convrot_linear_host(x_pin, ws[0], wss[0], N, BITS, y_pin)
    sync_all()
    h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    h0.record(stream)
    for i in range(e2e_steps):
        be.convrot_linear_host(x_pin, ws[i % N_SETS], wss[i % N_SETS], N, BITS, y_pin)
    h1.record(stream)
    sync_all()
    e2e_ms = h0.elapsed_time(h1)
    checksum = float(y_pin[0, :8].float().sum())  # the result really arrived on the host

    # max over ranks, on the device clock
    if world > 1:
        t = torch.tensor([ms_total, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, e2e_ms = float(t[0]), float(t[1])

    if rank == 0:
        peaks = measured_peaks()
        value = OPS_PER_STEP * args.steps * world / (ms_total * 1e-3) / 1e12
        e2e_value = OPS_PER_STEP * e2e_steps * world / (e2e_ms * 1e-3) / 1e12
        gemm_tops = OPS_PER_STEP / (gemm_ms * 1e-3) / 1e12
        int8_peak = 2.0 * peaks["bf16_tflops"]
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s8",
            "data": "synthetic",
            "config": {"workload": "config1: INT4 ConvRot linear (prep + int4->int8 tcgen05 GEMM + fused dequant), "
                                   "M=4608 K=3072 N=12288, batch of 4608 tokens per GPU",
                       "m": M, "n": N, "k": K, "bits": BITS, "out_dtype": args.out_dtype,
                       "l2": f"rotating {N_SETS} distinct input sets ({N_SETS * (M * K * 4 + N * K // 2) >> 20} MiB) > 126 MB L2, "
                             f"plus a {M * N * out_bytes >> 20} MiB output written every step",
                       "parallelism": f"replicas x{world} (independent batches, no collective)"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": M * K * 4,
                    "d2h_bytes_per_step": M * N * out_bytes, "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                    "checksum": checksum},
            "gpu_launches": gpu_launches,
            "roofline": {"bound": "tensor", "kernel": "convrot_gemm2_kernel (tcgen05 kind::i8, cta_group::2), timed alone over the same operands",
                         "achieved": gemm_tops, "peak": int8_peak, "unit": "TOP/s", "frac": gemm_tops / int8_peak,
                         "peak_note": f"2 x bf16 cuBLAS burst of {peaks['source']} peaks (the int8 tensor rate is twice bf16)",
                         "frac_of_dense_int8_spec_4500": gemm_tops / 4500.0,
                         "gemm_ms": gemm_ms, "traffic": GEMM_DRAM_TRAFFIC_BYTES[args.out_dtype]},
        }
        if world == 1 and not args.no_cpu_baseline:
            tops, cores, sample, _ = cpu_float_path_sample()
            line["cpu_baseline"] = {"value": tops, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    be.close()


# ---------------------------------------------------------------------------------------
# Secondary modes (not the driver's default line): the other BASELINE configurations
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


def run_mode_dit(args, rank, local, world, streamed: bool):
    """Configs 3/4: one synthetic ConvRot DiT step (28 blocks, hidden 3072, MLP 12288,
    4608 tokens), linears only; INT8 resident, or INT4 streamed from pinned host
    memory under a 2 GiB budget.  Independent latents: one per rank."""
    import torch
    import torch.distributed as dist
    from tensorpencil_b200 import harness, synth
    from tensorpencil_b200.backend import Backend
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    be = Backend(local)
    bits = 4 if streamed else 8
    budget = 2 << 30 if streamed else None
    w = harness.DitWeights(be, bits, stream_budget=budget, distinct_blocks=4)
    latents = [torch.from_numpy(synth.activations(synth.DIT_TOKENS, synth.DIT_HIDDEN, seed=1003 + 10 * rank + i)).cuda()
               for i in range(2)]

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    mod = harness.dit_modulation(be, synth.DIT_BLOCKS, synth.DIT_HIDDEN)
    T = synth.DIT_TOKENS
    _, _, _, qn, kn, cos, sin = harness.attention_inputs(T, 1, 1, be.device)
    attn = {"q_norm": qn, "k_norm": kn, "cos": cos, "sin": sin, "heads": synth.DIT_HIDDEN // 128}
    # name -> (what it runs, call).  "headline" = the reference's op sequence with every
    # elementwise op fused into the prep kernels, f32 activations, reference MLP tiling.
    variants = {
        "unfused_f32": ("reference sequence: rmsMod/sigmoidMul/siluMul/gatedAdd as separate kernels, f32, 2048-row MLP tiles",
                        lambda i: harness.dit_step_linears(be, w, latents[i % 2], mode="unfused", mod=mod)),
        "fused_f32": ("producers fused into the prep kernels, gated residuals into the GEMM epilogues, f32, 2048-row MLP tiles",
                      lambda i: harness.dit_step_linears(be, w, latents[i % 2], mode="fused", mod=mod)),
        "fused_bf16_whole_batch": ("fused, bf16 activation chain, one MLP pass over all 4608 tokens",
                                   lambda i: harness.dit_step_linears(be, w, latents[i % 2], out_dtype=torch.bfloat16,
                                                                      mode="fused", mod=mod, mlp_tile=T)),
        "linears_only": ("prep + GEMM launches only, one MLP pass over all tokens",
                         lambda i: harness.dit_step_linears(be, w, latents[i % 2], mode="linears", mlp_tile=T)),
        "fused_bf16_with_attention": ("fused_bf16_whole_batch plus qk-norm, RoPE and softmax attention (24 heads x 128) in "
                                      "every block: the whole block stack of a step",
                                      lambda i: harness.dit_step_linears(be, w, latents[i % 2], out_dtype=torch.bfloat16,
                                                                         mode="fused", mod=mod, mlp_tile=T, attn=attn)),
    }
    steps = max(1, min(args.steps, 20))
    ms_of = {}
    copied = {}
    for name, (_, fn) in variants.items():
        for i in range(max(args.warmup, 3) if name == "unfused_f32" else 2):
            fn(i)
        c0 = w.streamer.bytes_copied() if w.streamer else 0
        ms_of[name] = _events_ms(fn, steps, sync)
        copied[name] = (w.streamer.bytes_copied() - c0) if w.streamer else 0
    be.status_poll()
    names = list(variants)
    if world > 1:
        t = torch.tensor([ms_of[n] for n in names], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_of = {n: float(t[i]) for i, n in enumerate(names)}
    if rank == 0:
        ops = harness.dit_linear_ops(synth.DIT_TOKENS, synth.DIT_BLOCKS, synth.DIT_HIDDEN, synth.DIT_MLP)
        head = "fused_f32"
        s_per_step = ms_of[head] / steps / 1e3
        line = {"metric": "dit_linears_s_per_step", "value": s_per_step, "unit": "s/step", "n_gpus": world,
                "steps": steps, "higher_is_better": False, "scaling": "weak", "dtype": "s8", "data": "synthetic",
                "tops": ops / s_per_step / 1e12,
                "variants": {n: {"s_per_step": ms_of[n] / steps / 1e3, "tops": ops / (ms_of[n] / steps / 1e3) / 1e12,
                                 "what": variants[n][0]} for n in names},
                "config": {"workload": ("config4: INT4 DiT step, weights streamed from pinned host memory, 2 GiB budget"
                                        if streamed else "config3: INT8 DiT step, weights resident"),
                           "blocks": synth.DIT_BLOCKS, "hidden": synth.DIT_HIDDEN, "mlp": synth.DIT_MLP,
                           "tokens": synth.DIT_TOKENS, "latents_per_gpu": 1,
                           "scope": "the eight quantised linears per block and their elementwise neighbours (RMS norm + "
                                    "modulation, sigmoid and SiLU gates, gated residual); attention proper runs only in the "
                                    "variant that names it (elsewhere v stands in for its output); tops counts the "
                                    "linears' 2*M*N*K only"}}
        if w.streamer:
            line["h2d_gbs"] = copied[head] / (ms_of[head] * 1e-3) / 1e9
            line["streamed_bytes_per_step"] = copied[head] / steps
        print(json.dumps(line), flush=True)
    w.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    be.close()


def run_mode_nsplit(args, rank, local, world):
    """Config 4, second half: one [4608x3072]x[3072x12288] INT8 GEMM split along N over
    the ranks, output shards all-gathered (NCCL).  Compute and collective are timed
    separately and together (the chunked version overlaps them)."""
    import torch
    import torch.distributed as dist
    from tensorpencil_b200 import nsplit, synth
    from tensorpencil_b200.backend import Backend
    if world < 2:
        raise SystemExit("--mode nsplit needs at least 2 ranks (torchrun)")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    be = Backend(local)
    c = synth.convrot_linear(M, N, K, 8, seed=1004)   # same inputs on every rank
    lo, hi = nsplit.shard_bounds(N, world, rank)
    x = torch.from_numpy(c["x"]).cuda()
    w_shard = torch.from_numpy(c["w_i8"][lo:hi]).cuda()
    ws_shard = torch.from_numpy(c["w_scale"][lo:hi]).cuda()
    out_dtype = torch.float32 if args.out_dtype == "f32" else torch.bfloat16
    chunks = 4 if (N // world) % 64 == 0 else 1

    def compute(a, b):
        y = torch.empty((M, b - a), dtype=out_dtype, device="cuda")
        be.opI8Gemm(y, w_shard[a - lo:b - lo], ws_shard[a - lo:b - lo], b - a)
        return y

    def sync():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    be.opI8Prep(x, M, K)
    gathered = torch.empty((chunks, world, M, (hi - lo) // chunks), dtype=out_dtype, device="cuda")
    for _ in range(3):
        nsplit.nsplit_gemm_allgather(compute, M, N, chunks=chunks, out=gathered)
    # parity with the single-GPU result on sampled columns of every shard
    full_cols = torch.arange(0, N, 97, device="cuda")
    y_full = torch.empty((M, N), dtype=out_dtype, device="cuda")
    be.opI8Gemm(y_full, torch.from_numpy(c["w_i8"]).cuda(), torch.from_numpy(c["w_scale"]).cuda(), N)
    same = bool(torch.equal(nsplit.assemble(gathered)[:, full_cols], y_full[:, full_cols]))
    steps = max(3, min(args.steps, 50))
    ms_total = _events_ms(lambda i: nsplit.nsplit_gemm_allgather(compute, M, N, chunks=chunks, out=gathered), steps, sync)
    ms_compute = _events_ms(lambda i: [compute(lo + j * (hi - lo) // chunks, lo + (j + 1) * (hi - lo) // chunks)
                                       for j in range(chunks)], steps, sync)
    shard = torch.empty((M, hi - lo), dtype=out_dtype, device="cuda")
    flat = gathered.view(world * M, hi - lo) if chunks == 1 else torch.empty((world * M, hi - lo), dtype=out_dtype, device="cuda")
    ms_gather = _events_ms(lambda i: dist.all_gather_into_tensor(flat, shard), steps, sync)
    # the same split with the exchange done by the GEMM epilogue itself (peer stores over
    # NVLink, row-major result on every rank); one device-side barrier per step
    from tensorpencil_b200.peer import PeerBuffers
    esz = 4 if args.out_dtype == "f32" else 2
    pb = PeerBuffers(be, M * N * esz)

    def fused(i):
        pb.gemm_allgather(w_shard, ws_shard, hi - lo, 8, y_dtype=out_dtype)
        pb.barrier()

    pb.barrier()
    for i in range(3):
        fused(i)
    sync()
    same_fused = bool(torch.equal(pb.tensor((M, N), out_dtype), y_full))
    ms_fused = _events_ms(fused, steps, sync)
    be.status_poll()
    # unicast stores again, column-blocked destination (one contiguous block per sender)
    def fused_blocked(i):
        pb.gemm_allgather_blocked(w_shard, ws_shard, hi - lo, 8, y_dtype=out_dtype)
        pb.barrier()

    pb.barrier()
    for i in range(3):
        fused_blocked(i)
    sync()
    same_blk = bool(torch.equal(nsplit.assemble(pb.tensor((1, world, M, hi - lo), out_dtype)), y_full))
    ms_blk = _events_ms(fused_blocked, steps, sync)
    be.status_poll()
    # the same with one NVSwitch multicast store per element (each GPU sends its shard once)
    from tensorpencil_b200.peer import MulticastBuffers
    mb = MulticastBuffers(be, M * N * esz)
    ms_mc, same_mc = 0.0, True
    if mb.available:
        def fused_mc(i):
            mb.gemm_allgather(w_shard, ws_shard, hi - lo, 8, y_dtype=out_dtype)
            mb.barrier()

        mb.barrier()
        for i in range(3):
            fused_mc(i)
        sync()
        same_mc = bool(torch.equal(mb.tensor((M, N), out_dtype), y_full))
        ms_mc = _events_ms(fused_mc, steps, sync)
        be.status_poll()
    t = torch.tensor([ms_total, ms_compute, ms_gather, ms_fused, ms_mc, ms_blk], device="cuda", dtype=torch.float64)
    flags = torch.tensor([int(same), int(same_fused and same_blk), int(same_mc)], device="cuda")
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    same, same_fused, same_mc = bool(flags[0]), bool(flags[1]), bool(flags[2])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        recv = (world - 1) / world * M * N * esz
        have_mc = float(t[4]) > 0
        best = min(float(t[3]), float(t[4])) if have_mc else float(t[3])
        line = {"metric": "nsplit_gemm_allgather_tops", "value": OPS_PER_STEP * steps / (best * 1e-3) / 1e12,
                "unit": "TOPS", "n_gpus": world, "steps": steps, "higher_is_better": True, "scaling": "strong",
                "dtype": "s8", "data": "synthetic", "bit_identical_to_single_gpu": same_fused and same_mc,
                "ms_per_step": best / steps,
                "fused_multicast": ({"ms": float(t[4]) / steps, "what": "one GEMM launch whose epilogue writes each tile once "
                                     "with multimem.st to the NVSwitch multicast address of y (replicated into every rank's "
                                     "row-major y by the switch), then one device-side barrier",
                                     "nvlink_send_gbs_per_gpu": (M * N * esz / world) / (float(t[4]) / steps * 1e-3) / 1e9,
                                     "bit_identical_to_single_gpu": same_mc} if have_mc else "no multicast support"),
                "fused": {"ms": float(t[3]) / steps, "what": "one GEMM launch whose epilogue stores each tile into "
                          "every rank's row-major y over NVLink, then one device-side barrier",
                          "nvlink_send_gbs_per_gpu": recv / (float(t[3]) / steps * 1e-3) / 1e9,
                          "bit_identical_to_single_gpu": same_fused},
                "fused_blocked": {"ms": float(t[5]) / steps, "what": "as fused, but each sender's shard lands as one "
                                  "contiguous [M][N/world] block (column-blocked result, like NCCL's)"},
                "nccl": {"ms_total": float(t[0]) / steps, "ms_compute_only": float(t[1]) / steps,
                         "ms_allgather_only": float(t[2]) / steps, "chunks": chunks,
                         "tops": OPS_PER_STEP * steps / (float(t[0]) * 1e-3) / 1e12,
                         "allgather_recv_gbs_per_gpu": recv / (float(t[2]) / steps * 1e-3) / 1e9,
                         "bit_identical_to_single_gpu": same,
                         "layout": "gathered[chunk][rank][M][N/world/chunks] (column-blocked)"},
                "config": {"workload": "config4: INT8 GEMM 4608x12288x3072 split along N across the GPUs, output "
                                       "all-gathered (fused into the epilogue; NCCL version beside it)",
                           "out_dtype": args.out_dtype}}
        print(json.dumps(line), flush=True)
    mb.close()
    pb.close()
    dist.barrier()
    dist.destroy_process_group()
    be.close()


def run_mode_gemv(args, rank, local, world):
    """Config 2: Q8_0 decode GEMV, K=5120 -> N=17408 and the down projection, M in {1,4,8},
    four rotating weight buffers (379 MB > L2) so every launch streams from HBM."""
    import torch
    from tensorpencil_b200 import harness
    from tensorpencil_b200.backend import Backend
    torch.cuda.set_device(local)
    be = Backend(local)
    peaks = measured_peaks()
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
            steps = max(20, args.steps)
            ms = _events_ms(fn, steps, torch.cuda.synchronize) / steps
            gbs = n * (k // 32) * 34 / (ms * 1e-3) / 1e9
            rows_out.append({"fmt": "q8_0", "n": n, "k": k, "m": m, "us": ms * 1e3, "gbs": gbs,
                             "frac_of_hbm": gbs / peaks["hbm_gbs"]})
        del ws
    # the other GGUF formats at the up-projection shape; enough rotating copies to exceed L2
    from tensorpencil_b200 import synth
    n, k = 17408, 5120
    for fmt in ("q4_k", "q5_k", "q6_k", "q4_0", "iq4_nl"):
        base = torch.from_numpy(synth.gguf_weights(fmt, n, k, seed=11)).cuda()
        copies = 8
        ws = [base] + [base.clone() for _ in range(copies - 1)]       # 8 x 50..61 MB > 126 MB of L2
        wbytes = base.numel()
        for m in (1, 4, 8):
            x = torch.randn(m, k, device="cuda")
            y = torch.empty(m, n, device="cuda")
            be.opGemvQuantizeX(x, m * k)
            fn = lambda i: be.opGemvQuantQ8N(fmt, y, ws[i % copies], 1.0, n, k, m, 0, m)
            for i in range(5):
                fn(i)
            steps = max(24, args.steps)
            ms = _events_ms(fn, steps, torch.cuda.synchronize) / steps
            gbs = wbytes / (ms * 1e-3) / 1e9
            rows_out.append({"fmt": fmt, "n": n, "k": k, "m": m, "us": ms * 1e3, "gbs": gbs,
                             "frac_of_hbm": gbs / peaks["hbm_gbs"]})
        del ws, base
    be.status_poll()
    head = rows_out[0]
    print(json.dumps({"metric": "qgemv_hbm_gbs", "value": head["gbs"], "unit": "GB/s", "n_gpus": 1,
                      "higher_is_better": True, "dtype": "s8", "data": "synthetic",
                      "roofline": {"bound": "hbm", "achieved": head["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                   "frac": head["frac_of_hbm"], "peak_note": f"{peaks['source']} copy bandwidth"},
                      "config": {"workload": "config2: Q8_0 GEMV, headline = M=1, K=5120 -> N=17408"},
                      "cases": rows_out}), flush=True)
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
    """Launches one kernel of the path a few times through the C ABI -- the small,
    self-ending command the ncu captures under profiles/ are taken from."""
    import torch
    from tensorpencil_b200 import harness
    from tensorpencil_b200.backend import Backend
    torch.cuda.set_device(local)
    case = args.case
    if case == "gemm-w4-fused":
        os.environ["TPB_W4_FUSED"] = "1"       # read when the handle is created
    be = Backend(local)
    reps = max(1, min(args.steps, 5))
    if case in ("prep", "prep-mlp"):
        m, k = (M, K) if case == "prep" else (2048, N)
        x = torch.randn(m, k, device="cuda")
        for _ in range(reps):
            be._prep(x, m, k, 8)
    elif case in ("gemm", "gemm-bf16", "gemm-small", "gemm-w4", "gemm-w4-fused"):
        m, n, k = (2048, 6144, 3072) if case == "gemm-small" else (M, N, K)
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
            harness.dit_step_linears(be, w, x, out_dtype=torch.bfloat16, mode="fused", mod=mod, mlp_tile=T, attn=attn)
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
    elif case in ("gemv1", "gemv4", "gemv8", "gemv1-down"):
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
    ap.add_argument("--mode", choices=["linear", "dit", "dit-stream", "nsplit", "gemv", "attn", "one-kernel"], default="linear",
                    help="linear = the driver's default line (config 1); the others cover configs 2-4")
    ap.add_argument("--case", default="gemm", help="kernel for --mode one-kernel: prep, prep-mlp, gemm, gemm-bf16, "
                    "gemm-small, gemm-w4, gemm-w4-fused, gemv1, gemv4, gemv8, gemv1-down, gemv1-q4k, gemv1-q6k, gemv8-q4k, prep-silu, attn, dit-blocks")
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
    if args.mode == "attn":
        return run_mode_attn(args, local)
    if args.mode == "one-kernel":
        return run_mode_one_kernel(args, local)
    run_ours(args, rank, local, world)


if __name__ == "__main__":
    main()
