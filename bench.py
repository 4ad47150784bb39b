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

# DRAM bytes of one GEMM launch (dram__bytes_read.sum + dram__bytes_write.sum)
# from the ncu capture summarised in profiles/; None until a capture exists.
GEMM_DRAM_TRAFFIC_BYTES = None


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

def cpu_float_path_sample(target_seconds: float = 12.0):
    """Times the CPU restatement of the reference's `--backend cpu` path on a slice
    of the workload's weight rows (all M activation rows, full K), sized for about
    `target_seconds`.  Returns (TOPS, cores, sample description, seconds)."""
    from oracle import oracle
    from tensorpencil_b200 import synth
    cores = oracle.num_threads()
    x = synth.activations(M, K, seed=1001)
    probe_rows = 16 * cores if 16 * cores <= N else N
    w = synth.convrot_weights(probe_rows, K, BITS, seed=1001)
    t0 = time.perf_counter()
    oracle.linear_cpu_backend(x, w["w_packed"], BITS, w["w_scale"], probe_rows, K)
    dt = time.perf_counter() - t0
    rate = 2.0 * M * probe_rows * K / dt
    rows = int(min(N, max(probe_rows, (rate * target_seconds) / (2.0 * M * K))))
    rows = max(16, rows // 16 * 16)
    w = synth.convrot_weights(rows, K, BITS, seed=1002)
    t0 = time.perf_counter()
    oracle.linear_cpu_backend(x, w["w_packed"], BITS, w["w_scale"], rows, K)
    dt = time.perf_counter() - t0
    tops = 2.0 * M * rows * K / dt / 1e12
    return tops, cores, f"{rows} of {N} weight rows x all {M} tokens x K={K}, float path, {dt:.1f} s", dt


def run_reference_arm(args, rank: int, world: int):
    if rank != 0:
        return
    from oracle import oracle
    from tensorpencil_b200 import synth
    cores = oracle.num_threads()
    x = synth.activations(M, K, seed=1001)
    # size one step at ~2 s of CPU work, bounded so the whole run stays within minutes
    probe_rows = min(N, 16 * cores)
    w = synth.convrot_weights(probe_rows, K, BITS, seed=1001)
    t0 = time.perf_counter()
    oracle.linear_cpu_backend(x, w["w_packed"], BITS, w["w_scale"], probe_rows, K)
    rate = 2.0 * M * probe_rows * K / (time.perf_counter() - t0)
    rows = int(min(N, max(16, rate * 2.0 / (2.0 * M * K)))) // 16 * 16 or 16
    w = synth.convrot_weights(rows, K, BITS, seed=1002)
    for _ in range(args.warmup):
        oracle.linear_cpu_backend(x, w["w_packed"], BITS, w["w_scale"], rows, K)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.linear_cpu_backend(x, w["w_packed"], BITS, w["w_scale"], rows, K)
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

    def step(i: int, gemm_events=None):
        s = i % N_SETS
        be.opI4Prep(xs[s], M, K)
        if gemm_events is not None:
            gemm_events[0].record(stream)
        be.opI4Gemm(y, ws[s], wss[s], N)
        if gemm_events is not None:
            gemm_events[1].record(stream)

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
    gemm_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
               for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = be.launches
    sync_all()
    sampler.start()
    e0.record(stream)
    for i in range(args.steps):
        step(i, gemm_ev[i])
    e1.record(stream)
    sync_all()
    clocks = sampler.stop()
    ms_total = e0.elapsed_time(e1)
    gpu_launches = be.launches - launches0
    gemm_ms = float(np.mean([a.elapsed_time(b) for a, b in gemm_ev]))
    be.status_poll()

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
            "roofline": {"bound": "tensor", "kernel": "convrot_gemm_kernel (tcgen05 kind::i8)",
                         "achieved": gemm_tops, "peak": int8_peak, "unit": "TOP/s", "frac": gemm_tops / int8_peak,
                         "peak_note": f"2 x bf16 cuBLAS burst of {peaks['source']} peaks (the int8 tensor rate is twice bf16)",
                         "frac_of_dense_int8_spec_4500": gemm_tops / 4500.0,
                         "gemm_ms": gemm_ms, "traffic": GEMM_DRAM_TRAFFIC_BYTES},
        }
        if world == 1 and not args.no_cpu_baseline:
            tops, cores, sample, _ = cpu_float_path_sample()
            line["cpu_baseline"] = {"value": tops, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    be.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--out-dtype", choices=["f32", "bf16"], default="f32")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch multi-GPU runs with torch.distributed.run (one process per GPU)")
    run_ours(args, rank, local, world)


if __name__ == "__main__":
    main()
