"""Benchmark of the hot path on B200: one JSON line per run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Default workload (N = 1): the bf16 tile product C = A @ B^T with M = N = K = 8192, f32 accumulation, bf16
output — the configuration the headline metric is quoted on. A "step" is one pass of the hot path over one
batch of synthetic operands (seeded N(0,1) rounded to bf16). Other workloads (`gemm_fp8`, `attn_fwd`,
`attn_decode`) measure the other configurations with the same harness.

Keys of the line:
  value       whole-job TFLOP/s with operands resident in HBM (CUDA events on the launching stream, max over ranks)
  e2e         the same metric through the C-ABI call with HOST buffers: every step copies the operands from pinned
              host memory, runs the kernel and reads the result back, all inside the timed region
  roofline    achieved vs measured peak for the dominant kernel (algorithmic FLOPs / event time)
  cpu_baseline  the CPU restatement of the reference's C backend timed on this machine's cores on a bounded sample
  clocks      SM clock and throttle reasons sampled by nvidia-smi during the timed region

With N > 1 (launched by torch.distributed.run, one rank per GPU) the product is sharded by output column blocks:
rank r multiplies A by its rows of B, the column blocks are all-gathered over NCCL and laid out as one row-major
C on every rank; total work is fixed, so scaling is "strong".

`--impl reference` times the reference's CPU implementation of the path (its C backend restated in oracle/, since
the reference itself needs Python 3.14 + clang) on the host cores, rank 0 only.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "bf16_tile_gemm_tflops"

# DRAM bytes per launch of the dominant kernel from the committed ncu capture (profiles/), or None when no
# capture of that workload exists yet.
NCU_TRAFFIC_BYTES = {"gemm_bf16": None, "gemm_fp8": None, "attn_fwd": None, "attn_decode": None}


def measured_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU every 100 ms while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index, self.samples, self.process = index, [], None

    def __enter__(self) -> "ClockSampler":
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.process = None
        return self

    def _read(self) -> None:
        for line in self.process.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6 and parts[0].isdigit():
                self.samples.append(parts)

    def __exit__(self, *exc) -> None:
        if self.process is not None:
            self.process.terminate()
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        clocks = sorted(int(s[0]) for s in self.samples)
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [name for i, name in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": clocks[len(clocks) // 2], "sm_max_mhz": int(self.samples[0][1]), "reasons": reasons,
                "samples": len(self.samples)}


# ---- workloads --------------------------------------------------------------------------------------------------


class GemmBf16:
    """C = A @ B^T, bf16, M = N = K = 8192 (seed 1). Sharded by output column blocks across ranks."""

    name, dtype, unit, bound = "gemm_bf16", "bf16", "TFLOP/s", "tensor"
    description = "bf16 tile GEMM C=A@B^T M=N=K=8192, f32 accumulate, bf16 out (seed 1, N(0,1))"
    m = n = k = 8192

    def __init__(self, torch, rank: int, world: int, size: list[int] | None = None) -> None:
        self.torch, self.rank, self.world = torch, rank, world
        if size:
            self.m, self.n, self.k = size
            self.description = f"bf16 tile GEMM C=A@B^T M={self.m} N={self.n} K={self.k} (profiling case)"
        self.n_local = self.n // world
        gen = torch.Generator(device="cuda").manual_seed(1)
        self.a = torch.randn((self.m, self.k), device="cuda", generator=gen).to(torch.bfloat16)
        b = torch.randn((self.n, self.k), device="cuda", generator=gen).to(torch.bfloat16)
        self.b = b[rank * self.n_local:(rank + 1) * self.n_local].contiguous()
        del b
        self.c_local = torch.empty((self.m, self.n_local), device="cuda", dtype=torch.bfloat16)
        if world > 1:
            self.slabs = torch.empty((world, self.m, self.n_local), device="cuda", dtype=torch.bfloat16)
            self.c = torch.empty((self.m, self.n), device="cuda", dtype=torch.bfloat16)
        self.launches_per_step = 1 if world == 1 else 2

    config = property(lambda self: {
        "workload": self.description,
        "m": self.m, "n": self.n, "k": self.k, "sharding": f"N-column blocks x{self.world}",
        "l2": "operands and output (384 MiB) exceed the 126 MB L2; no flush between steps"})

    def flops(self) -> float:
        return 2.0 * self.m * self.n * self.k

    def kernel_flops(self) -> float:
        return 2.0 * self.m * self.n_local * self.k

    def step(self, calls) -> None:
        stream = self.torch.cuda.current_stream()
        calls.gemm_tn(self.a, self.b, self.c_local, stream)
        if self.world > 1:
            self.torch.distributed.all_gather_into_tensor(self.slabs, self.c_local)
            calls.scatter_columns(self.slabs, self.c, self.world, stream)

    def kernel_only(self, calls) -> None:
        calls.gemm_tn(self.a, self.b, self.c_local, self.torch.cuda.current_stream())

    def host_buffers(self):
        torch = self.torch
        self.host_in = [t.cpu().pin_memory() for t in (self.a, self.b)]
        self.host_out = torch.empty(self.c_local.shape, dtype=self.c_local.dtype).pin_memory()
        return sum(t.numel() * t.element_size() for t in self.host_in), self.host_out.numel() * self.host_out.element_size()

    def e2e_step(self, calls) -> None:
        self.a.copy_(self.host_in[0], non_blocking=True)
        self.b.copy_(self.host_in[1], non_blocking=True)
        calls.gemm_tn(self.a, self.b, self.c_local, self.torch.cuda.current_stream())
        self.host_out.copy_(self.c_local, non_blocking=True)

    def cpu_sample(self, oracle, cores: int, columns: int | None = None):
        """The faithful block loop (128x128x32 tiles) on the first `cores` block rows of the same problem, one
        block row per thread; `columns` restricts N to bound the time. Returns (flops, description, callable)."""
        n = columns or self.n
        rows = 128 * cores
        a, b = oracle.config_gemm_bf16(rows, n, self.k, seed=1)

        def run() -> None:
            oracle.gemm(a, b, ab_type=oracle.BF16, c_type=oracle.BF16, tile=(128, 128, 32), threads=cores)

        return 2.0 * rows * n * self.k, f"first {rows} rows x {n} columns of the 8192^3 product, K=8192, {cores} threads", run


WORKLOADS = {"gemm_bf16": GemmBf16}


def reference_arm(args, rank: int) -> int:
    """The reference's CPU implementation of the path (restated C backend) on the host cores; rank 0 only."""
    if rank != 0:
        return 0
    from oracle import oracle

    cores = min(os.cpu_count() or 1, 64)
    workload = WORKLOADS[args.workload].__new__(WORKLOADS[args.workload])
    workload.world = 1
    flops, sample, run = workload.cpu_sample(oracle, cores, columns=1024)
    for _ in range(min(args.warmup, 1)):
        run()
    start = time.perf_counter()
    for _ in range(args.steps):
        run()
    seconds = time.perf_counter() - start
    value = flops * args.steps / seconds / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": workload.unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": seconds / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": workload.dtype,
        "data": "synthetic", "config": {"workload": workload.description},
        "cpu_baseline": {"value": value, "unit": workload.unit, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": workload.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default="gemm_bf16", choices=sorted(WORKLOADS))
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--kernel-only", action="store_true", help="profiling: skip the e2e and CPU legs")
    parser.add_argument("--size", type=int, nargs="+", default=None, help="profiling: override the problem extents")
    args = parser.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return reference_arm(args, rank)

    import torch

    from krn_b200.runtime import calls, native

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the hot path")
    native.library()
    torch.cuda.set_device(local_rank)
    distributed = world > 1
    if distributed:
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    warmup = max(args.warmup, 3)
    workload = WORKLOADS[args.workload](torch, rank, world, args.size)
    peaks, peak_kind = measured_peaks()

    def barrier() -> None:
        if distributed:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps: int) -> float:
        """Milliseconds for `steps` calls of fn, on the device, max over ranks."""
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for _ in range(steps):
            fn()
        stop.record()
        barrier()
        ms = torch.tensor([start.elapsed_time(stop)], device="cuda", dtype=torch.float64)
        if distributed:
            torch.distributed.all_reduce(ms, op=torch.distributed.ReduceOp.MAX)
        return float(ms.item())

    # ---- resident-operand throughput ---------------------------------------------------------------------------------
    for _ in range(warmup):
        workload.step(calls)
    with ClockSampler(local_rank) as sampler:
        total_ms = timed(lambda: workload.step(calls), args.steps)
        # keep the GPU busy long enough for nvidia-smi to see it under load
        deadline = time.time() + 0.6
        while time.time() < deadline and len(sampler.samples) < 3:
            workload.step(calls)
            torch.cuda.synchronize()
    clocks = sampler.summary()
    native.raise_device_status()
    ms_per_step = total_ms / args.steps
    value = workload.flops() / (ms_per_step * 1e-3) / 1e12

    # ---- the dominant kernel alone (roofline) ---------------------------------------------------------------------
    kernel_ms = timed(lambda: workload.kernel_only(calls), args.steps) / args.steps
    achieved = workload.kernel_flops() / (kernel_ms * 1e-3) / 1e12
    peak = peaks["bf16_tflops"]
    roofline = {"bound": workload.bound, "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": NCU_TRAFFIC_BYTES[workload.name], "peak_kind": f"{peak_kind} burst (cuBLAS bf16 8192^3)",
                "kernel_ms": kernel_ms, "frac_of_nominal_dense_peak": achieved / 2250.0}

    # ---- end to end with host buffers ---------------------------------------------------------------------------------
    e2e = None
    if not args.kernel_only:
        h2d, d2h = workload.host_buffers()
        for _ in range(2):
            workload.e2e_step(calls)
        e2e_steps = max(3, min(args.steps, 10))
        e2e_ms = timed(lambda: workload.e2e_step(calls), e2e_steps) / e2e_steps
        e2e = {"value": workload.flops() / (e2e_ms * 1e-3) / 1e12, "unit": workload.unit,
               "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world, "ms_per_step": e2e_ms}
        native.raise_device_status()

    # ---- CPU baseline (rank 0, N = 1 only) ---------------------------------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and not args.kernel_only:
        from oracle import oracle

        cores = min(os.cpu_count() or 1, 64)
        flops, sample, run = workload.cpu_sample(oracle, cores)
        start = time.perf_counter()
        run()
        seconds = time.perf_counter() - start
        cpu = {"value": flops / seconds / 1e12, "unit": workload.unit, "cores": cores, "kind": "port", "sample": sample,
               "seconds": seconds}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": workload.unit, "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": workload.dtype, "data": "synthetic", "config": workload.config, "roofline": roofline,
            "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": workload.launches_per_step * args.steps, "clocks": clocks,
            "frac_of_nominal_dense_peak": value / (2250.0 * world),
        }
        print(json.dumps(line), flush=True)
    if distributed:
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
