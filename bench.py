#!/usr/bin/env python
"""Benchmark of the ragged-dot hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--only fwd|dlhs|drhs] [--no-e2e] [--no-cpu-baseline]

One JSON line on stdout (rank 0).  N = 1: one step is ragged_dot forward + its full backward
(dlhs through the transposed grouped GEMM, drhs through tgmm) on the Mixtral-8x7B-shaped
workload, m=8192, k=4096, n=14336, g=8, bf16 with fp32 accumulation; `value` counts useful
flops, 2*m*k*n per GEMM.  N > 1 (torchrun): the expert-parallel workload -- per GPU 8192
tokens x top-4 routing over 64 experts sharded 64/N per GPU, NCCL all-to-all of the rows, then
the local ragged_dot.

`--impl reference` times the CPU oracle (oracle/ragged_dot_oracle.py, the restatement of the
reference semantics; jax is not installed, so jax.lax.ragged_dot on XLA-CPU cannot run) on a
bounded sample of the same workload with all host threads.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of each kernel on this workload, from
# the ncu captures summarised in profiles/ragged_gemm_mixtral_m8192_k4096_n14336_g8.md.
DRAM_TRAFFIC_BYTES_PER_LAUNCH = {"fwd": 1.140598e9 + 229.923328e6, "dlhs": 1.588072e9 + 60.262912e6,
                                 "drhs": 332.787968e6 + 884.06144e6}

METRIC = "ragged_dot fwd+bwd TFLOP/s (2*m*k*n useful flops per GEMM)"
UNIT = "TFLOP/s"


# ---------------------------------------------------------------------------- helpers
def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {
            "bf16_tflops": float(p["bf16_tflops"]),
            "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
            "hbm_gbs": float(p["hbm_gbs"]),
            "source": "measured",
        }
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.02):
        self.index = index
        self.period = period_s
        self.samples = []
        self.power_w = []
        self.power_limit_w = None
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
            try:
                self.power_limit_w = pynvml.nvmlDeviceGetEnforcedPowerLimit(self._h) / 1000.0
            except Exception:
                self.power_limit_w = None
        except Exception:
            self._nvml = None
            return self
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def _run(self):
        nv = self._nvml
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
                self.power_w.append(nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
            # board power beside the clock: these kernels pull the board to its power limit within
            # milliseconds, and the clock drops with it before NVML's reason bits show the cap
            "power_w": statistics.median(self.power_w) if self.power_w else None,
            "power_max_w": max(self.power_w) if self.power_w else None,
            "power_limit_w": self.power_limit_w,
        }


def physical_gpu_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except Exception:
            return local_index
    return local_index


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ---------------------------------------------------------------------------- reference arm (CPU)
def cpu_oracle_sample(shape, rows, threads, seed=0):
    """Inputs for a CPU run on the first `rows` rows of the workload (group sizes scaled)."""
    from gpu_ragged_dot_b200 import workloads

    gs_full = workloads.group_sizes_mixtral_ragged(seed).astype(np.int64)
    gs = (gs_full * rows) // shape.m
    gs[-1] += rows - gs.sum()
    x = workloads.normal_tensor((rows, shape.k), 1.0, 11, "cpu")
    A = workloads.normal_tensor((shape.g, shape.k, shape.n), shape.k ** -0.5, 12, "cpu")
    dout = workloads.normal_tensor((rows, shape.n), 1.0, 13, "cpu")
    return x, A, dout, torch.from_numpy(gs.astype(np.int32))


def cpu_oracle_step(x, A, dout, gs, only=None):
    from oracle import ragged_dot_oracle as oracle

    if only in (None, "fwd"):
        oracle.ragged_dot(x, A, gs, native_16bit=True)
    if only in (None, "dlhs"):
        oracle.ragged_dot(dout, A, gs, trans_rhs=True, native_16bit=True)
    if only in (None, "drhs"):
        oracle.trans_ragged_dot(x, dout, gs, native_16bit=True)


def run_reference(args):
    from gpu_ragged_dot_b200 import workloads

    rank, world, _ = dist_env()
    if rank != 0:
        return
    # All the host threads this process may use (torchrun presets OMP_NUM_THREADS=1 for its ranks).
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(threads)
    if max(world, args.gpus) > 1:
        return run_reference_expert_parallel(args, max(world, args.gpus), threads)
    shape = workloads.MIXTRAL
    gemms = 3 if args.only is None else 1
    # Calibrate on 128 rows, then size the per-step sample so warmup+steps stay near 2 minutes.
    x, A, dout, gs = cpu_oracle_sample(shape, 128, threads)
    t0 = time.perf_counter()
    cpu_oracle_step(x, A, dout, gs, args.only)
    t_probe = time.perf_counter() - t0
    budget = 120.0 / max(args.steps + args.warmup, 1)
    rows = int(min(shape.m, max(128, 128 * budget / max(t_probe, 1e-3))))
    rows = max(128, (rows // 128) * 128)
    x, A, dout, gs = cpu_oracle_sample(shape, rows, threads)
    for _ in range(args.warmup):
        cpu_oracle_step(x, A, dout, gs, args.only)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_oracle_step(x, A, dout, gs, args.only)
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    flops = 2.0 * rows * shape.k * shape.n * gemms
    value = flops / dt / 1e12
    sample = (f"rows 0..{rows - 1} of {shape.m} (group sizes scaled), all {shape.g} experts' weights, "
              f"{'fwd+dlhs+drhs' if args.only is None else args.only} per step; torch CPU bf16 matmul (oneDNN, fp32 accumulate) per group")
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": dt * 1e3,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": shape.name + "_fwd_bwd", "m": shape.m, "k": shape.k, "n": shape.n,
                   "g": shape.g, "reference": "CPU restatement of jax.lax.ragged_dot semantics (jax not installed)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample,
                         "host_cpus": os.cpu_count()},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_reference_expert_parallel(args, world, threads):
    """Reference arm of the N > 1 workload (expert-parallel forward): the same routing, permutation
    by expert and ragged_dot over all 64 experts, on the host cores of rank 0.  There is no
    exchange on one host; each step is a bounded sample of the job's tokens."""
    from gpu_ragged_dot_b200 import workloads
    from oracle import ragged_dot_oracle as oracle

    shape = workloads.EP_PREFILL
    tokens_job, top_k, experts = 8192 * world, 4, shape.g
    A = workloads.normal_tensor((experts, shape.k, shape.n), shape.k ** -0.5, 12, "cpu")

    def make(tokens):
        x = workloads.normal_tensor((tokens, shape.k), 1.0, 11, "cpu")
        routing = torch.from_numpy(workloads.topk_routing(tokens, experts, top_k, seed=3000)).to(torch.int64)
        return x, routing

    def step(x, routing):
        flat = routing.reshape(-1)
        order = torch.argsort(flat, stable=True)
        gs = torch.bincount(flat, minlength=experts).to(torch.int32)
        rows = x.index_select(0, order // top_k)
        return oracle.ragged_dot(rows, A, gs, native_16bit=True)

    x, routing = make(256)
    step(x, routing)
    t0 = time.perf_counter()
    step(x, routing)
    t_probe = time.perf_counter() - t0
    budget = 120.0 / max(args.steps + args.warmup, 1)
    tokens = int(min(tokens_job, max(256, 256 * budget / max(t_probe, 1e-3))))
    tokens = max(256, (tokens // 256) * 256)
    x, routing = make(tokens)
    for _ in range(args.warmup):
        step(x, routing)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step(x, routing)
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    value = 2.0 * tokens * top_k * shape.k * shape.n / dt / 1e12
    sample = (f"{tokens} of the job's {tokens_job} tokens x top-{top_k} per step: sort by expert, gather rows, "
              f"ragged_dot over all {experts} experts' weights; torch CPU bf16 matmul (oneDNN, fp32 accumulate) per group")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"expert_parallel_fwd_{shape.name}_w{world}", "tokens_per_gpu": 8192,
                   "top_k": top_k, "experts": experts, "k": shape.k, "n": shape.n,
                   "reference": "CPU restatement of jax.lax.ragged_dot semantics (jax not installed), one host"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample,
                         "host_cpus": os.cpu_count()},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------- our arm, N = 1
def run_single(args):
    from gpu_ragged_dot_b200 import _lib, ops, workloads
    import gpu_ragged_dot_b200 as rd

    _lib.load()  # fail loudly if the CUDA library is missing
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    shape = {"mixtral": workloads.MIXTRAL, "decode": workloads.EP_DECODE,
             "deepseek": workloads.DEEPSEEK_V3}[args.workload]
    peaks = measured_peaks()
    kernels = ["fwd", "dlhs", "drhs"] if args.only is None else [args.only]
    # Allocate only what the selected kernels touch (keeps profiler captures small).
    x, A, dout = workloads.make_inputs(shape, dev, seed=0, with_dout=kernels != ["fwd"])
    if kernels == ["dlhs"]:
        x = None
    if kernels == ["drhs"]:
        A = None
    if args.workload == "mixtral":
        gs_fwd_np, gs_bwd_np = workloads.group_sizes_mixtral(0), workloads.group_sizes_mixtral_ragged(0)
    elif args.workload == "decode":
        gs_fwd_np = gs_bwd_np = workloads.group_sizes_from_routing(workloads.topk_routing(64, 64, 4, seed=5), 64)
    else:
        gs_fwd_np = gs_bwd_np = workloads.group_sizes_deepseek(0)
    gs_fwd = torch.from_numpy(gs_fwd_np).to(dev)
    gs_bwd = torch.from_numpy(gs_bwd_np).to(dev)
    y = torch.empty((shape.m, shape.n), dtype=torch.bfloat16, device=dev) if "fwd" in kernels else None
    dx = torch.empty((shape.m, shape.k), dtype=torch.bfloat16, device=dev) if "dlhs" in kernels else None
    dA = (torch.empty((shape.g, shape.k, shape.n), dtype=torch.bfloat16, device=dev)
          if "drhs" in kernels else None)
    ws = ops._workspace(shape.m, shape.g, dev)

    def launch(name):
        if name == "fwd":
            ops.gmm_forward(x, A, gs_fwd, out=y, workspace=ws)
        elif name == "dlhs":
            ops.gmm_forward(dout, A, gs_bwd, trans_rhs=True, out=dx, workspace=ws)
        else:
            ops.tgmm_forward(x, dout, gs_bwd, out=dA, workspace=ws)

    for _ in range(max(args.warmup, 3)):
        for name in kernels:
            launch(name)
    torch.cuda.synchronize()

    stream = torch.cuda.current_stream(dev)
    marks = [[torch.cuda.Event(enable_timing=True) for _ in range(len(kernels) + 1)] for _ in range(args.steps)]
    sampler = ClockSampler(physical_gpu_index(0)).start()
    torch.cuda.synchronize()
    for s in range(args.steps):
        marks[s][0].record(stream)
        for i, name in enumerate(kernels):
            launch(name)
            marks[s][i + 1].record(stream)
    torch.cuda.synchronize()
    clocks = sampler.stop()
    status = ops.device_status(ws)
    if status != 0:
        raise RuntimeError(f"device status {status} after the timed region")

    total_ms = marks[0][0].elapsed_time(marks[-1][-1])
    ms_per_step = total_ms / args.steps
    per_kernel_ms = {
        name: sum(marks[s][i].elapsed_time(marks[s][i + 1]) for s in range(args.steps)) / args.steps
        for i, name in enumerate(kernels)
    }
    gemm_flops = 2.0 * shape.m * shape.k * shape.n
    value = gemm_flops * len(kernels) / (ms_per_step * 1e-3) / 1e12

    # roofline of the dominant (slowest) kernel; every GEMM here is tensor-bound (AI ~ 775 flop/B)
    dom = max(per_kernel_ms, key=per_kernel_ms.get)
    per_kernel = {}
    for name, ms in per_kernel_ms.items():
        tf = gemm_flops / (ms * 1e-3) / 1e12
        per_kernel[name] = {"ms": ms, "tflops": tf, "frac_of_measured_burst": tf / peaks["bf16_tflops"],
                            "frac_of_measured_sustained": tf / peaks["bf16_tflops_sustained"]}
    traffic = DRAM_TRAFFIC_BYTES_PER_LAUNCH if args.workload == "mixtral" else {}
    gplus_f, gplus_b = int((gs_fwd_np > 0).sum()), int((gs_bwd_np > 0).sum())
    alg_bytes = {
        "fwd": 2.0 * (shape.m * shape.k + gplus_f * shape.k * shape.n + shape.m * shape.n),
        "dlhs": 2.0 * (shape.m * shape.n + gplus_b * shape.k * shape.n + shape.m * shape.k),
        "drhs": 2.0 * (shape.m * shape.k + shape.m * shape.n + shape.g * shape.k * shape.n),
    }
    for name, ms in per_kernel_ms.items():
        gbs = alg_bytes[name] / (ms * 1e-3) / 1e9
        per_kernel[name]["algorithmic_GBps"] = gbs
        per_kernel[name]["frac_of_measured_hbm"] = gbs / peaks["hbm_gbs"]
    hbm_bound = alg_bytes[dom] / (peaks["hbm_gbs"] * 1e9) > gemm_flops / (peaks["bf16_tflops"] * 1e12)
    if hbm_bound:
        roofline = {
            "bound": "hbm",
            "kernel": {"fwd": "ragged_gemm(2)_kernel<gmm>", "dlhs": "ragged_gemm(2)_kernel<gmm, trans_rhs>",
                       "drhs": "ragged_gemm2_kernel<tgmm>"}[dom],
            "achieved": per_kernel[dom]["algorithmic_GBps"], "peak": peaks["hbm_gbs"],
            "peak_source": f"{peaks['source']} (copy bandwidth)", "unit": "GB/s",
            "frac": per_kernel[dom]["frac_of_measured_hbm"], "traffic": None,
            "algorithmic_bytes_per_launch": alg_bytes[dom], "algorithmic_flops_per_launch": gemm_flops,
            "per_kernel": per_kernel,
        }
    else:
        roofline = {
            "bound": "tensor",
            "kernel": {"fwd": "ragged_gemm2_kernel<gmm>", "dlhs": "ragged_gemm2_kernel<gmm, trans_rhs>",
                       "drhs": "ragged_gemm2_kernel<tgmm>"}[dom],
            "achieved": per_kernel[dom]["tflops"],
            "peak": peaks["bf16_tflops"],
            "peak_source": f"{peaks['source']} (burst cuBLAS bf16); sustained {peaks['bf16_tflops_sustained']}",
            "unit": "TFLOP/s",
            "frac": per_kernel[dom]["tflops"] / peaks["bf16_tflops"],
            "frac_of_sustained": per_kernel[dom]["tflops"] / peaks["bf16_tflops_sustained"],
            "traffic": traffic.get(dom),
            "algorithmic_flops_per_launch": gemm_flops,
            "algorithmic_bytes_per_launch": alg_bytes[dom],
            "per_kernel": per_kernel,
        }

    line = {
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "config": {
            "workload": shape.name + ("_fwd_bwd" if args.only is None else "_" + args.only),
            "m": shape.m, "k": shape.k, "n": shape.n, "g": shape.g,
            "group_sizes": {"mixtral": "fwd: multinomial(Dirichlet(2)); bwd: same, each group at a random offset mod 128",
                            "decode": "64 tokens x uniform top-4 of 64 experts",
                            "deepseek": "multinomial(Dirichlet(0.3)), ~20% empty"}[args.workload],
            "l2": "inputs larger than L2 (weights %d MB per GEMM)" % (shape.g * shape.k * shape.n * 2 // 1000000),
            "timing": "CUDA events on the launch stream; per-kernel events inside the timed region",
        },
        "clocks": clocks,
        "gpu_launches": 2 * len(kernels) * args.steps,
        "roofline": roofline,
    }

    if not args.no_e2e and args.only is None and args.workload == "mixtral":
        line["e2e"] = run_e2e(args, shape, dev, rd, x, A, dout, gs_fwd, kernels)
    if args.only is None and not args.no_other_workloads and args.workload == "mixtral":
        del x, A, dout, y, dx, dA
        torch.cuda.empty_cache()
        line["other_workloads"] = run_other_workloads(dev, peaks)
    if not args.no_cpu_baseline and args.workload == "mixtral":
        line["cpu_baseline"] = run_cpu_baseline(shape, kernels)
    print(json.dumps(line), flush=True)


def run_permute(args):
    """`--workload permute`: the MoE-layer use of the path on the Mixtral shape (4096 tokens, top-2
    routing over 8 experts -> 8192 sorted rows): y[out_rows[r]] = x[in_rows[r]] @ A[expert of r].
    Times the permutation-fused kernels (rd_gmm_permuted / rd_tgmm_permuted) against
    rd_gather_rows + rd_gmm / rd_tgmm + rd_gather_rows, variants interleaved in one process."""
    import random
    import statistics

    from gpu_ragged_dot_b200 import _lib, ops, workloads

    _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    shape = workloads.MIXTRAL
    top_k = 2
    tokens = shape.m // top_k
    routing = workloads.topk_routing(tokens, shape.g, top_k, seed=0)  # [tokens, top_k]
    flat = routing.reshape(-1)
    order = np.argsort(flat, kind="stable")
    gs = torch.from_numpy(np.bincount(flat, minlength=shape.g).astype(np.int32)).to(dev)
    in_rows = torch.from_numpy((order // top_k).astype(np.int32)).to(dev)
    out_rows = torch.from_numpy(order.astype(np.int32)).to(dev)
    inv_rows = torch.empty_like(out_rows)
    inv_rows[out_rows.long()] = torch.arange(shape.m, dtype=torch.int32, device=dev)
    x = workloads.normal_tensor((tokens, shape.k), 1.0, 1, dev)
    A = workloads.normal_tensor((shape.g, shape.k, shape.n), shape.k ** -0.5, 2, dev)
    dy = workloads.normal_tensor((shape.m, shape.n), 1.0, 3, dev)
    ws = ops._workspace(shape.m, shape.g, dev)
    xs = torch.empty((shape.m, shape.k), dtype=torch.bfloat16, device=dev)
    ys = torch.empty((shape.m, shape.n), dtype=torch.bfloat16, device=dev)
    y = torch.empty((shape.m, shape.n), dtype=torch.bfloat16, device=dev)
    dys = torch.empty((shape.m, shape.n), dtype=torch.bfloat16, device=dev)
    dA = torch.empty_like(A)

    def fwd_fused():
        ops.gmm_permuted_forward(x, A, gs, in_rows=in_rows, out_rows=out_rows, out=y, y_rows=shape.m, workspace=ws)

    def fwd_fused_gather_only():
        ops.gmm_permuted_forward(x, A, gs, in_rows=in_rows, out=ys, workspace=ws)

    def fwd_two_pass():
        ops.gather_rows(x, in_rows, out=xs)
        ops.gmm_forward(xs, A, gs, out=ys, workspace=ws)
        ops.gather_rows(ys, inv_rows, out=y)

    def fwd_two_pass_gather_only():
        ops.gather_rows(x, in_rows, out=xs)
        ops.gmm_forward(xs, A, gs, out=ys, workspace=ws)

    def drhs_fused():
        ops.tgmm_permuted_forward(x, dy, gs, x_rows_index=in_rows, y_rows_index=out_rows, out=dA, workspace=ws)

    def drhs_two_pass():
        ops.gather_rows(x, in_rows, out=xs)
        ops.gather_rows(dy, out_rows, out=dys)
        ops.tgmm_forward(xs, dys, gs, out=dA, workspace=ws)

    variants = {"fwd_fused": fwd_fused, "fwd_two_pass": fwd_two_pass,
                "fwd_fused_gather_only": fwd_fused_gather_only,
                "fwd_two_pass_gather_only": fwd_two_pass_gather_only,
                "drhs_fused": drhs_fused, "drhs_two_pass": drhs_two_pass}
    for fn in variants.values():
        for _ in range(max(args.warmup, 3)):
            fn()
    torch.cuda.synchronize()
    sampler = ClockSampler(physical_gpu_index(0))
    sampler.start()
    times = {name: [] for name in variants}
    rng = random.Random(0)
    for _ in range(5):
        names = list(variants)
        rng.shuffle(names)
        for name in names:
            times[name].append(_time_ms(variants[name], args.steps))
    clocks = sampler.stop()
    assert ops.device_status(ws) == 0, "device reported an expired wait"
    flops = 2.0 * shape.m * shape.k * shape.n
    res = {name: {"ms": round(statistics.median(v), 4),
                  "tflops": round(flops / statistics.median(v) / 1e9, 1)} for name, v in times.items()}
    ms = res["fwd_fused"]["ms"]
    print(json.dumps({
        "metric": "ragged_dot_permuted_fwd_tflops", "value": res["fwd_fused"]["tflops"], "unit": UNIT,
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "permute: mixtral shape, 4096 tokens x top-2 of 8 experts, gather + scatter "
                               "fused into the GEMM", "m": shape.m, "k": shape.k, "n": shape.n, "g": shape.g,
                   "l2": "operands larger than L2"},
        "variants": res, "clocks": clocks, "gpu_launches": 2 * args.steps,
    }), flush=True)


def _time_ms(fn, reps):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def run_other_workloads(dev, peaks):
    """Short device-resident measurements of the bandwidth-bound configurations (not part of the
    headline `value`): the decode shape (m=256 over 64 experts) and the DeepSeek-V3 shape."""
    from gpu_ragged_dot_b200 import ops, workloads

    out = {}
    hbm = peaks["hbm_gbs"]

    def entry(ms, flops, nbytes):
        gbs = nbytes / (ms * 1e-3) / 1e9
        return {"ms": ms, "tflops": flops / (ms * 1e-3) / 1e12, "algorithmic_GBps": gbs,
                "frac_of_measured_hbm": gbs / hbm}

    # decode: 64 tokens x top-4 over 64 experts -> m = 256, weights 805 MB (larger than L2)
    s = workloads.EP_DECODE
    gs_np = workloads.group_sizes_from_routing(workloads.topk_routing(64, 64, 4, seed=5), 64)
    gplus = int((gs_np > 0).sum())
    x, A, _ = workloads.make_inputs(s, dev, with_dout=False)
    gs = torch.from_numpy(gs_np).to(dev)
    ws = ops._workspace(s.m, s.g, dev)
    y = torch.empty((s.m, s.n), dtype=torch.bfloat16, device=dev)
    ms = _time_ms(lambda: ops.gmm_forward(x, A, gs, out=y, workspace=ws), 30)
    out[s.name + "_fwd"] = entry(ms, 2.0 * s.m * s.k * s.n, 2.0 * (s.m * s.k + gplus * s.k * s.n + s.m * s.n))
    out[s.name + "_fwd"]["nonempty_groups"] = gplus
    del x, A, y
    torch.cuda.empty_cache()

    # DeepSeek-V3 shaped: heavy-tailed groups, ~20 % empty
    s = workloads.DEEPSEEK_V3
    gs_np = workloads.group_sizes_deepseek(0)
    gplus = int((gs_np > 0).sum())
    x, A, dout = workloads.make_inputs(s, dev)
    gs = torch.from_numpy(gs_np).to(dev)
    ws = ops._workspace(s.m, s.g, dev)
    y = torch.empty((s.m, s.n), dtype=torch.bfloat16, device=dev)
    dx = torch.empty((s.m, s.k), dtype=torch.bfloat16, device=dev)
    dA = torch.empty_like(A)
    fl = 2.0 * s.m * s.k * s.n
    b_gmm = 2.0 * (s.m * s.k + gplus * s.k * s.n + s.m * s.n)
    b_tgmm = 2.0 * (s.m * s.k + s.m * s.n + s.g * s.k * s.n)
    out[s.name + "_fwd"] = entry(_time_ms(lambda: ops.gmm_forward(x, A, gs, out=y, workspace=ws), 8), fl, b_gmm)
    out[s.name + "_dlhs"] = entry(
        _time_ms(lambda: ops.gmm_forward(dout, A, gs, trans_rhs=True, out=dx, workspace=ws), 8), fl, b_gmm)
    out[s.name + "_drhs"] = entry(_time_ms(lambda: ops.tgmm_forward(x, dout, gs, out=dA, workspace=ws), 8), fl, b_tgmm)
    out[s.name + "_fwd"]["nonempty_groups"] = gplus
    # drhs writes 7.5 GB and reads 0.6 GB: it is bound by the WRITE bandwidth, which on these parts
    # is well below the read+write copy figure.  A memset of the same output measured here is its ceiling.
    ms_set = _time_ms(lambda: dA.zero_(), 5)
    out[s.name + "_drhs"]["memset_of_the_output_ms"] = ms_set
    out[s.name + "_drhs"]["write_GBps_of_memset"] = dA.numel() * 2 / (ms_set * 1e-3) / 1e9
    out[s.name + "_drhs"]["time_vs_memset_of_the_output"] = out[s.name + "_drhs"]["ms"] / ms_set
    return out


def run_e2e(args, shape, dev, rd, x, A, dout, gs, kernels):
    """Same step with HOST buffers, everything inside the timed region: pinned H2D of x, A,
    group_sizes and dout, ragged_dot + backward on the device, D2H of y, dlhs and drhs.

    `value` goes through `HostRaggedDot` (the host-buffer entry of the package: expert chunks are
    copied in, multiplied and copied out on three streams, so both directions of the PCIe link and
    the GPU work at once).  `one_stream_ms` is the plain way beside it: `ragged_dot` + autograd
    on device tensors with the copies around it on one stream."""
    full = len(kernels) == 3
    hx, hA, hd = (t.cpu().pin_memory() for t in (x, A, dout))
    hgs = gs.cpu().pin_memory()
    hy = torch.empty((shape.m, shape.n), dtype=torch.bfloat16).pin_memory()
    hdx = torch.empty_like(hx).pin_memory()
    hdA = torch.empty_like(hA).pin_memory()
    steps = max(2, min(args.steps, 5))

    def step_one_stream():
        dx_ = hx.to(dev, non_blocking=True)
        dA_ = hA.to(dev, non_blocking=True)
        dg_ = hgs.to(dev, non_blocking=True)
        if full:
            dd_ = hd.to(dev, non_blocking=True)
            dx_.requires_grad_(True)
            dA_.requires_grad_(True)
        yv = rd.ragged_dot(dx_, dA_, dg_)
        if full:
            yv.backward(dd_)
            hdx.copy_(dx_.grad, non_blocking=True)
            hdA.copy_(dA_.grad, non_blocking=True)
        hy.copy_(yv.detach(), non_blocking=True)

    pipe = rd.HostRaggedDot(shape.m, shape.k, shape.n, shape.g, device=dev, backward=full)

    def step_pipelined():
        if full:
            pipe(hx, hA, hgs, hd, y=hy, dlhs=hdx, drhs=hdA)
        else:
            pipe(hx, hA, hgs, y=hy)

    def timed(step, reps):
        for _ in range(2):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            step()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    ms_serial = timed(step_one_stream, steps)
    torch.cuda.empty_cache()
    ms = timed(step_pipelined, steps)
    nbytes = lambda t: t.numel() * t.element_size()
    h2d = nbytes(hx) + nbytes(hA) + nbytes(hgs) + (nbytes(hd) if full else 0)
    d2h = nbytes(hy) + ((nbytes(hdx) + nbytes(hdA)) if full else 0)
    flops = 2.0 * shape.m * shape.k * shape.n * (3 if full else 1)
    return {"value": flops / (ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms, "steps": steps,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "h2d_GBps": h2d / (ms * 1e-3) / 1e9, "d2h_GBps": d2h / (ms * 1e-3) / 1e9,
            "api": "gpu_ragged_dot_b200.HostRaggedDot (pinned host buffers; chunks of experts copied in, "
                   "multiplied by rd_gmm/rd_tgmm and copied out on three streams)",
            "one_stream_ms": ms_serial, "one_stream_value": flops / (ms_serial * 1e-3) / 1e12,
            "one_stream_api": "gpu_ragged_dot_b200.ragged_dot + autograd backward, copies on the same stream"}


def run_cpu_baseline(shape, kernels):
    threads = torch.get_num_threads()
    rows = 4096
    x, A, dout, gs = cpu_oracle_sample(shape, rows, threads)
    only = None if len(kernels) == 3 else kernels[0]
    cpu_oracle_step(x[:128], A, dout[:128], torch.tensor([16] * shape.g, dtype=torch.int32), only)  # warm-up
    t0 = time.perf_counter()
    reps = 0
    while reps < 3 and time.perf_counter() - t0 < 20.0:
        cpu_oracle_step(x, A, dout, gs, only)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    flops = 2.0 * rows * shape.k * shape.n * len(kernels)
    return {"value": flops / dt / 1e12, "unit": UNIT, "cores": threads, "kind": "port",
            "host_cpus": os.cpu_count(),
            "sample": f"rows 0..{rows - 1} of {shape.m} (group sizes scaled 1/{shape.m // rows}), all {shape.g} "
                      f"experts' weights, {'+'.join(kernels)} x{reps}; oracle = torch CPU bf16 matmul (oneDNN, fp32 accumulate) per group"}


# ---------------------------------------------------------------------------- our arm, N > 1
def run_expert_parallel(args):
    """N > 1: expert parallel forward.  Three dispatch modes are timed on the same inputs ("overlap":
    ring-phased peer stores running under the flag-gated local GEMM), among them:
    "nccl" (sort + gather + NCCL all-to-all with host-known split sizes) and "p2p" (device-side
    plan + rows stored straight into the owners' receive buffers through peer memory, no host
    round trip).  `value` is the faster one; both are reported."""
    import torch.distributed as dist
    from gpu_ragged_dot_b200 import _lib, ep, workloads

    _lib.load()
    rank, world, local = dist_env()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    shape = workloads.EP_PREFILL
    tokens, top_k, experts = 8192, 4, shape.g
    x_tokens = workloads.normal_tensor((tokens, shape.k), 1.0, 1000 + rank, dev)
    routing = torch.from_numpy(workloads.topk_routing(tokens, experts, top_k, seed=3000 + rank)).to(dev)
    peaks = measured_peaks()
    results = {}
    clocks = None
    for mode in ("nccl", "p2p", "overlap", "fused"):
        try:
            layer = ep.ExpertParallelRaggedDot(experts, shape.k, shape.n, dev, seed=2000 + rank, dispatch=mode)
            for _ in range(max(args.warmup, 3)):
                layer.forward(x_tokens, routing)
            torch.cuda.synchronize()
            ok = torch.ones(1, device=dev)
        except Exception as e:  # e.g. no peer access for symmetric memory
            if rank == 0:
                sys.stderr.write(f"bench: dispatch mode {mode} unavailable: {e!r}\n")
            ok = torch.zeros(1, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok) == 0:
            continue
        dist.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(physical_gpu_index(local)).start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        layer.reset_timers()
        e0.record()
        for _ in range(args.steps):
            layer.forward(x_tokens, routing, timed=True)
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        clocks = sampler.stop()
        ms = e0.elapsed_time(e1) / args.steps
        parts = layer.timers_ms(args.steps)
        if mode in ("overlap", "fused"):
            # a bounded wait that expired inside a kernel (status word != 0) makes the timing meaningless
            from gpu_ragged_dot_b200 import ops as _ops
            bad = torch.tensor([float(_ops.device_status(layer._ov["ws"]) != 0)], device=dev)
            dist.all_reduce(bad, op=dist.ReduceOp.MAX)
            if float(bad) != 0:
                if rank == 0:
                    sys.stderr.write(f"bench: dispatch mode {mode} dropped: a device-side wait expired\n")
                del layer
                torch.cuda.empty_cache()
                continue
        t = torch.tensor([ms, parts["gemm"], parts["a2a"], parts["permute"], parts.get("own_rows", 0.0)],
                         dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        results[mode] = t.tolist()
        del layer
        torch.cuda.empty_cache()
    # Decode-shaped case of the same expert layout: 64 tokens x top-4 per GPU (m = 256 rows per rank),
    # weight-bandwidth bound on every rank.  Timed with the two host-sync-free modes.
    decode = {}
    d_tokens = 64
    xd = workloads.normal_tensor((d_tokens, shape.k), 1.0, 5000 + rank, dev)
    rd_ = torch.from_numpy(workloads.topk_routing(d_tokens, experts, top_k, seed=6000 + rank)).to(dev)
    for mode in ("p2p", "fused"):
        try:
            layer = ep.ExpertParallelRaggedDot(experts, shape.k, shape.n, dev, seed=2000 + rank, dispatch=mode,
                                               capacity_rows=d_tokens * top_k * world)
            for _ in range(max(args.warmup, 3)):
                out = layer.forward(xd, rd_)
            torch.cuda.synchronize()
            ok = torch.ones(1, device=dev)
        except Exception as e:
            if rank == 0:
                sys.stderr.write(f"bench: decode case, mode {mode} unavailable: {e!r}\n")
            ok = torch.zeros(1, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok) == 0:
            continue
        seg = out[1]
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            layer.forward(xd, rd_)
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        local = experts // world
        touched = int((seg.view(world, local).sum(0) > 0).sum())  # local experts with at least one row
        t = torch.tensor([e0.elapsed_time(e1) / args.steps, float(touched)], dtype=torch.float64, device=dev)
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        decode[mode] = {"ms_per_step": float(tmax[0]),
                        "weight_GBps_all_gpus": float(t[1]) * shape.k * shape.n * 2 / (float(tmax[0]) * 1e-3) / 1e9,
                        "experts_touched": int(t[1])}
        del layer
        torch.cuda.empty_cache()
    # End to end at N GPUs: every step copies this rank's tokens and routing from pinned host memory,
    # runs the fastest mode's public forward() and reads the local result rows back to the host.
    e2e = None
    if results:
        best_t = torch.tensor([results.get(m, [1e30])[0] for m in ("nccl", "p2p", "overlap", "fused")],
                              dtype=torch.float64, device=dev)
        dist.broadcast(best_t, src=0)
        mode = ("nccl", "p2p", "overlap", "fused")[int(torch.argmin(best_t))]
        layer = ep.ExpertParallelRaggedDot(experts, shape.k, shape.n, dev, seed=2000 + rank, dispatch=mode)
        hx = x_tokens.cpu().pin_memory()
        hr = routing.to(torch.int32).cpu().pin_memory()
        rows_back = tokens * top_k
        hy = torch.empty((rows_back, shape.n), dtype=torch.bfloat16).pin_memory()

        def step():  # copy-in of the next step runs under this step's exchange, GEMM and copy-out
            layer.forward_host(hx, hr, hy)

        for _ in range(2):
            step()
        torch.cuda.synchronize()
        dist.barrier()
        e2e_steps = max(3, min(args.steps, 10))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            step()
        layer.wait_host_outputs()
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1) / e2e_steps], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t[0])
        e2e = {"value": 2.0 * tokens * top_k * world * shape.k * shape.n / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
               "ms_per_step": e2e_ms, "steps": e2e_steps, "dispatch": mode,
               "h2d_bytes_per_step": world * (hx.numel() * 2 + hr.numel() * 4),
               "d2h_bytes_per_step": world * hy.numel() * 2,
               "api": "ExpertParallelRaggedDot.forward_host per rank, pinned host buffers (copy-in of step i+1 under step i)"}
        del layer
        torch.cuda.empty_cache()
    if rank == 0 and results:
        best = min(results, key=lambda m: results[m][0])
        ms, gemm_ms, a2a_ms, first_ms, _ = results[best]
        rows_global = tokens * top_k * world
        flops = 2.0 * rows_global * shape.k * shape.n
        gemm_tf = 2.0 * tokens * top_k * shape.k * shape.n / (gemm_ms * 1e-3) / 1e12
        row_bytes_out = tokens * top_k * shape.k * 2 * (world - 1) / world
        modes = {}
        for m_, (t_ms, g_ms, x_ms, p_ms, own_ms) in results.items():
            modes[m_] = {
                "ms_per_step": t_ms, "tflops": flops / (t_ms * 1e-3) / 1e12,
                "breakdown_ms": ({"sort_plan_gather": p_ms, "all_to_all": x_ms, "local_ragged_dot": g_ms}
                                 if m_ == "nccl" else
                                 {"count_allgather_plan": p_ms, "peer_store_dispatch_and_barrier": x_ms,
                                  "local_ragged_dot": g_ms} if m_ == "p2p" else
                                 {"count_allgather_plan": p_ms, "peer_store_phases_from_plan_end": x_ms,
                                  "own_rows_copied_from_plan_end": own_ms,
                                  "flag_gated_ragged_dot_from_plan_end": g_ms} if m_ == "overlap" else
                                 {"count_allgather_plan_assign": p_ms, "own_rows_copied_from_plan_end": own_ms,
                                  "fused_send_and_ragged_dot_from_plan_end": g_ms}),
                # fused: the exchange has no span of its own; rate over the whole send + GEMM kernel
                ("exchange_GBps_per_gpu_over_the_fused_kernel" if m_ == "fused" else "exchange_GBps_per_gpu"):
                    row_bytes_out / ((g_ms if m_ == "fused" else x_ms) * 1e-3) / 1e9,
            }
        line = {
            "metric": METRIC, "value": flops / (ms * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"expert_parallel_fwd_{shape.name}_w{world}", "tokens_per_gpu": tokens,
                       "top_k": top_k, "experts": experts, "experts_per_gpu": experts // world,
                       "k": shape.k, "n": shape.n, "dispatch": best,
                       "collective": {"nccl": "NCCL all-to-all (rows) + all-to-all (counts)",
                                      "p2p": "NCCL all-gather (counts) + peer stores over NVLink + symmetric-memory barrier",
                                      "overlap": "NCCL all-gather (counts) + ring-phased peer stores over NVLink overlapped "
                                                 "with the local GEMM, which waits per source on ready flags",
                                      "fused": "NCCL all-gather (counts) + ONE kernel whose sender CTAs store rows to the "
                                               "peers over NVLink (ring phases) while its other CTAs multiply the rows "
                                               "that have arrived (ready flags)"}[best],
                       "l2": "inputs larger than L2 (268 MB of rows per GPU)"},
            "clocks": clocks,
            "gpu_launches": {"nccl": 3, "p2p": 5, "overlap": 4 + world, "fused": 6}[best] * args.steps,
            "roofline": ({"bound": "tensor", "kernel": "ragged_gemm2_kernel<gmm> (local experts)",
                          "achieved": gemm_tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                          "frac": gemm_tf / peaks["bf16_tflops"], "traffic": None,
                          "peak_source": peaks["source"]} if best not in ("overlap", "fused") else
                         # fused exchange + GEMM: target = slower of flops / GEMM peak and NVLink bytes / 770 GB/s
                         # (measured peer-copy bandwidth per direction per GPU); achieved is over the span from
                         # the end of the plan to the end of the GEMM, waits on remote rows included.
                         {"bound": "tensor", "kernel": "ragged_gemm2_kernel<gmm> gated by ready flags, " +
                                                      ("sender CTAs in the same launch" if best == "fused"
                                                       else "ep_dispatch_phase_kernel on a side stream"),
                          "achieved": gemm_tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                          "target_ms": max(2.0 * tokens * top_k * shape.k * shape.n / (peaks["bf16_tflops"] * 1e9),
                                           row_bytes_out / 770e9 * 1e3),
                          "frac": max(2.0 * tokens * top_k * shape.k * shape.n / (peaks["bf16_tflops"] * 1e9),
                                      row_bytes_out / 770e9 * 1e3) / gemm_ms,
                          "traffic": None, "peak_source": peaks["source"] + "; NVLink 770 GB/s per direction"}),
            "dispatch_modes": modes,
            "decode_case": {"tokens_per_gpu": d_tokens, "top_k": top_k, "rows_per_gpu": d_tokens * top_k,
                            "note": "exchange + local ragged_dot per step; latency-bound (a few small kernels and "
                                    "one all-gather), weights read once per touched expert", "modes": decode},
            "e2e": e2e,
        }
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default=None, choices=["fwd", "dlhs", "drhs"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-workloads", action="store_true")
    ap.add_argument("--workload", default="mixtral", choices=["mixtral", "decode", "deepseek", "permute"],
                    help="N=1 only; the headline line is the default (mixtral); the others are for profiling")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product has no CPU path (use --impl reference for the CPU oracle)")
    _, world, _ = dist_env()
    if world > 1 or args.gpus > 1:
        run_expert_parallel(args)
    elif args.workload == "permute":
        run_permute(args)
    else:
        run_single(args)


if __name__ == "__main__":
    main()
