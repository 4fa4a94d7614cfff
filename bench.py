"""Benchmark of the hot path on B200: one JSON line per run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Headline workload: the bf16 tile product C = A @ B^T with M = N = K = 8192, f32 accumulation, bf16 output — the
configuration the headline metric is quoted on. A "step" is one pass of the hot path over one batch of synthetic
operands (seeded N(0,1), generated on the device). With the default `--workload all` the line also carries
`workloads`: one sub-record with the same keys for each of the other configurations — `gemm_fp8` (block-scaled e4m3,
8192 x 28672 x 8192), `gemm_mxfp8` and `gemm_nvfp4` (the same extents in the MXFP8 and NVFP4 formats, scales applied by the tensor cores), `attn_fwd` (causal GQA flash attention, B=8, Hq=32, Hkv=8, S=4096, D=128), `attn_decode` (paged
FP8 decode, 64 sequences, contexts 1024..8192). `--workload NAME` measures that one alone as the headline.

Timing: W (at least 3) warm-up steps, then TRIALS of exactly K steps each, every trial bracketed by a barrier and a
synchronisation on both sides and timed with CUDA events on the launching stream, max over ranks; as many trials (at
least 5) as it takes for them to last about a second together, so that the nvidia-smi clock samples in `clocks` fall
INSIDE the timed region. `ms_per_step` is the median over trials of (trial time / K); min and max are in `timing`.

Keys of the line (and of each sub-record):
  value         whole-job throughput with operands resident in HBM
  e2e           the same metric through the public host-operand API (krn_b200.streaming) with HOST buffers: every step
                copies the operands from pinned host memory, runs the kernels and reads the result back, all inside the
                timed region (panels of the copies overlap the kernels)
  roofline      achieved vs measured peak for the dominant kernel (algorithmic FLOPs or bytes / event time); `frac` is
                against the burst cuBLAS figure, `frac_of_sustained_peak` against the seconds-long one
  rel_frobenius the kernel's output on a sample of the workload against the CPU oracle on the same operands
  cpu_baseline  the CPU restatement of the reference's C backend timed on this machine's cores on a bounded sample,
                on all cores and (`one_thread`) on one, which is how the reference itself runs a kernel call
  clocks        SM clock and throttle reasons sampled by nvidia-smi during the timed region

With N > 1 (launched by torch.distributed.run, one rank per GPU) total work is fixed ("strong" scaling): the tile
products are sharded by output column blocks and every rank ends with the whole row-major C — the all-gather of the
column blocks and the cross-rank completion are done by the product kernel itself (TMA stores into every rank's C over
NVLink; the last CTA exchanges flags with the peers; KRN_B200_GATHER=nccl selects an NCCL all-gather + re-layout kernel
instead); attention is sharded by (batch, kv head) and decode by sequence, with no collective. The end-to-end leg of
the products copies `a` once per node (each rank its share of the rows, all-gathered over NVLink).

`--impl reference` times the reference's CPU implementation of the path (its C backend restated in oracle/, since
the reference itself needs Python 3.14 + clang and holds no C sources) on the host cores, rank 0 only; each step is a
bounded sample whose extents are in `config.sample`.
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

# DRAM bytes per launch of the dominant kernel from the committed ncu captures (profiles/), None where no capture of
# that workload exists yet.
# gemm_bf16 / gemm_fp8 / attn_fwd: captured on a smaller case (see profiles/) and scaled to the full launch by the
# algorithmic bytes, which DRAM traffic follows for these streaming operand/output patterns; attn_decode: captured on
# the bench workload itself.
NCU_TRAFFIC_BYTES = {"gemm_mxfp8": int(223.0e6 * 781.2 / 195.3), "gemm_bf16": int(218.7e6 * 402.7 / 167.8), "gemm_fp8": int(220.3e6 * 773.9 / 193.5),
                     "attn_fwd": int(137.6e6 * 671.1 / 167.8), "attn_decode": int(690.2e6),
                     # NVFP4: the small capture ended with part of its output still in L2, so only its READ bytes are scaled
                     # (by the operand bytes, 169.9 / 42.4 MB); the output is counted once in full
                     "gemm_nvfp4": int(73.4e6 * 169.9 / 42.4 + 469.8e6)}


L2_BYTES = 126 * 10**6


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


class Workload:
    name = metric = dtype = description = ""
    unit, bound = "TFLOP/s", "tensor"
    launches_per_step = 1
    reference_columns = 1024     # extent that bounds the CPU sample of `--impl reference` (columns, or sequence length)
    single_thread_columns = 512  # the same for the faithful one-thread CPU sample

    def __init__(self, torch, rank: int, world: int, size: list[int] | None = None) -> None:
        self.torch, self.rank, self.world = torch, rank, world

    def scale(self, work: float, ms: float) -> float:
        return work / (ms * 1e-3) / 1e12  # flop -> TFLOP/s (bytes -> GB/s overridden below)

    @staticmethod
    def rotation(set_bytes: int) -> int:
        """How many copies of a step's tensors to rotate through so that consecutive steps never find their inputs in
        the 126 MB L2: one when a single set is already twice the L2, else enough for 384 MB in total."""
        return 1 if set_bytes >= 2 * L2_BYTES else -(-3 * L2_BYTES // max(1, set_bytes))

    @staticmethod
    def l2_note(what: str, set_bytes: int, copies: int) -> str:
        size = f"{what} ({set_bytes / 2**20:.0f} MiB per rank)"
        if copies == 1:
            return f"{size} exceed the 126 MB L2; no flush between steps"
        return f"{size} would fit the 126 MB L2: steps rotate through {copies} copies ({copies * set_bytes / 2**20:.0f} MiB)"

    def peak(self, peaks: dict) -> tuple[float, str]:
        return peaks["bf16_tflops_sustained"], "sustained cuBLAS bf16 8192^3 (seconds-long loop under the power cap)"


class GemmBf16(Workload):
    """C = A @ B^T, bf16, M = N = K = 8192 (seed 1). Sharded by output column blocks across ranks."""

    name, metric, dtype = "gemm_bf16", "bf16_tile_gemm_tflops", "bf16"
    description = "bf16 tile GEMM C=A@B^T M=N=K=8192, f32 accumulate, bf16 out (seed 1, N(0,1))"
    m = n = k = 8192

    def __init__(self, torch, rank, world, size=None) -> None:
        super().__init__(torch, rank, world)
        from krn_b200 import sharding

        if size:
            self.m, self.n, self.k = size
            self.description = f"bf16 tile GEMM C=A@B^T M={self.m} N={self.n} K={self.k} (profiling case)"
        begin, end = sharding.column_block(self.n, rank, world, 256) if world > 1 else (0, self.n)
        self.n_local = end - begin
        gen = torch.Generator(device="cuda").manual_seed(1)
        self.a = torch.randn((self.m, self.k), device="cuda", generator=gen).to(torch.bfloat16)
        b = torch.randn((self.n, self.k), device="cuda", generator=gen).to(torch.bfloat16)
        self.b = b[begin:end].contiguous()
        del b
        self.columns = slice(begin, end)
        self.c_local = torch.empty((self.m, self.n_local), device="cuda", dtype=torch.bfloat16)
        self.fused = None
        if world > 1:
            if os.environ.get("KRN_B200_GATHER", "fused") == "fused":
                self.fused = sharding.GatheredProduct(self.m, self.n, torch.bfloat16)
            else:
                self.slabs = torch.empty((world, self.m, self.n_local), device="cuda", dtype=torch.bfloat16)
                self.c = torch.empty((self.m, self.n), device="cuda", dtype=torch.bfloat16)
                self.launches_per_step = 2

    @property
    def config(self) -> dict:
        gather = ("all-gather of the output columns and the cross-rank completion fused into the product kernel (TMA "
                  "stores into every rank's C over NVLink, flags exchanged by the last CTA)" if self.fused
                  else "NCCL all-gather of the output columns + re-layout kernel")
        return {"workload": self.description, "m": self.m, "n": self.n, "k": self.k,
                "sharding": f"N-column blocks x{self.world}, {gather}" if self.world > 1 else "one GPU, no exchange",
                "l2": self.l2_note("operands and output", 2 * (self.m * self.k + self.n_local * self.k + self.m * (
                    self.n if self.world > 1 else self.n_local)), 1)}

    def work(self) -> float:
        return 2.0 * self.m * self.n * self.k

    def kernel_work(self) -> float:
        return 2.0 * self.m * self.n_local * self.k

    def step(self, calls) -> None:
        stream = self.torch.cuda.current_stream()
        if self.fused is not None:
            self.fused.run(self.a, self.b, stream)
            return
        calls.gemm_tn(self.a, self.b, self.c_local, stream)
        if self.world > 1:
            from krn_b200 import sharding

            sharding.gather_columns(self.c_local, self.slabs, self.c, self.world, stream=stream)

    def kernel_only(self, calls) -> None:
        calls.gemm_tn(self.a, self.b, self.c_local, self.torch.cuda.current_stream())

    def host_buffers(self):
        """End to end = `krn_b200.streaming.StreamedProduct`: pinned host A, this rank's rows of B and its column block
        of C, streamed through the device in panels (copies overlap the products of neighbouring panels)."""
        from krn_b200 import streaming

        self.host_in = [t.cpu().pin_memory() for t in (self.a, self.b)]
        self.host_out = self.torch.empty(self.c_local.shape, dtype=self.c_local.dtype).pin_memory()
        if self.world > 1 and self.m % self.world == 0:
            # a crosses PCIe once per node: each rank copies M / G of its rows, NVLink all-gathers them
            self.streamed = streaming.ShardedStreamedProduct(self.m, self.n_local, self.k, self.torch.bfloat16)
            h2d = (self.host_in[0].numel() // self.world + self.host_in[1].numel()) * 2
        else:
            self.streamed = streaming.StreamedProduct(self.m, self.n_local, self.k, self.torch.bfloat16)
            h2d = sum(t.numel() * t.element_size() for t in self.host_in)
        return h2d, self.host_out.numel() * self.host_out.element_size()

    def e2e_step(self, calls) -> None:
        self.streamed.run(self.host_in[0], self.host_in[1], self.host_out)

    def parity_sample(self, oracle, calls) -> dict:
        """Relative Frobenius error of sampled output rows against the CPU oracle on the same operands."""
        import numpy as np

        torch = self.torch
        self.kernel_only(calls)
        torch.cuda.synchronize()
        rows = [0, 1, 127, 128, self.m // 2 - 1, self.m // 2, self.m - 129, self.m - 1]
        words = lambda t: t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
        want = oracle.bf16_values(oracle.gemm(words(self.a[rows]), words(self.b), ab_type=oracle.BF16, c_type=oracle.BF16,
                                              threads=8))
        got = oracle.bf16_values(words(self.c_local[rows]))
        return {"value": oracle.rel_frobenius(got, want), "tolerance": 1e-2,
                "sample": f"{len(rows)} rows x all {self.n_local} columns against the oracle's k-ordered fma chain"}

    def cpu_sample(self, oracle, cores: int, columns: int | None = None):
        """The faithful block loop (128x128x32 tiles) on the first `cores` block rows of the same problem, one
        block row per thread; `columns` restricts N to bound the time. Returns (work, description, callable)."""
        n = columns or self.n
        rows = 128 * cores
        a, b = oracle.config_gemm_bf16(rows, n, self.k, seed=1)

        def run() -> None:
            oracle.gemm(a, b, ab_type=oracle.BF16, c_type=oracle.BF16, tile=(128, 128, 32), threads=cores)

        return 2.0 * rows * n * self.k, f"first {rows} rows x {n} columns of the product, K={self.k}, {cores} threads", run


class GemmFp8(Workload):
    """Block-scaled e4m3 product, M=8192 N=28672 K=8192 (seed 2), 1x128 A scales, 128x128 B scales, bf16 out."""

    name, metric, dtype = "gemm_fp8", "fp8_blockscaled_gemm_tflops", "fp8_e4m3"
    description = "FP8 e4m3 block-scaled GEMM M=8192 N=28672 K=8192, fp32 scales 1x128 (A) / 128x128 (B), bf16 out (seed 2)"
    m, n, k = 8192, 28672, 8192

    def __init__(self, torch, rank, world, size=None) -> None:
        super().__init__(torch, rank, world)
        from krn_b200 import sharding

        if size:
            self.m, self.n, self.k = size
            self.description = f"FP8 block-scaled GEMM M={self.m} N={self.n} K={self.k} (profiling case)"
        begin, end = sharding.column_block(self.n, rank, world, 256) if world > 1 else (0, self.n)
        self.n_local = end - begin
        gen = torch.Generator(device="cuda").manual_seed(2)
        self.a, self.sa = self._quantize(torch.randn((self.m, self.k), device="cuda", generator=gen), 1)
        b = torch.randn((self.n, self.k), device="cuda", generator=gen)[begin:end].contiguous()
        self.b, self.sb = self._quantize(b, 128)
        del b
        self.c_local = torch.empty((self.m, self.n_local), device="cuda", dtype=torch.bfloat16)
        self.fused = None
        if world > 1:
            if os.environ.get("KRN_B200_GATHER", "fused") == "fused":
                self.fused = sharding.GatheredProduct(self.m, self.n, torch.bfloat16, multiple=256)
            else:
                self.slabs = torch.empty((world, self.m, self.n_local), device="cuda", dtype=torch.bfloat16)
                self.c = torch.empty((self.m, self.n), device="cuda", dtype=torch.bfloat16)
                self.launches_per_step = 2

    def _quantize(self, x, block_rows: int):
        """Codes with each block's absmax mapped to 448 (scale = absmax / 448), blocks of block_rows x 128."""
        torch = self.torch
        rows, cols = x.shape
        blocks = x.view(rows // block_rows, block_rows, cols // 128, 128)
        absmax = blocks.abs().amax(dim=(1, 3))
        scale = torch.where(absmax > 0, absmax / 448.0, torch.ones_like(absmax))
        codes = (blocks / scale[:, None, :, None]).reshape(rows, cols).to(torch.float8_e4m3fn)
        return codes, scale.contiguous()

    @property
    def config(self) -> dict:
        return {"workload": self.description, "m": self.m, "n": self.n, "k": self.k,
                "sharding": (f"N-column blocks x{self.world}, " + (
                    "all-gather of the output columns and the cross-rank completion fused into the product kernel (TMA "
                    "stores into every rank's C over NVLink, flags exchanged by the last CTA)" if self.fused
                    else "NCCL all-gather of the output columns + re-layout kernel"))
                if self.world > 1 else "one GPU, no exchange",
                "l2": self.l2_note("operands and output", self.m * self.k + self.n_local * self.k + 2 * self.m * (
                    self.n if self.world > 1 else self.n_local), 1)}

    def work(self) -> float:
        return 2.0 * self.m * self.n * self.k

    def kernel_work(self) -> float:
        return 2.0 * self.m * self.n_local * self.k

    def peak(self, peaks: dict) -> tuple[float, str]:
        return 2.0 * peaks["bf16_tflops_sustained"], "2 x sustained cuBLAS bf16 (no FP8 peak was measured on this pool)"

    def step(self, calls) -> None:
        stream = self.torch.cuda.current_stream()
        if self.fused is not None:
            self.fused.run_fp8(self.a, self.sa, self.b, self.sb, stream)
            return
        calls.gemm_fp8_blockscaled_tn(self.a, self.sa, self.b, self.sb, self.c_local, stream)
        if self.world > 1:
            from krn_b200 import sharding

            sharding.gather_columns(self.c_local, self.slabs, self.c, self.world, stream=stream)

    def kernel_only(self, calls) -> None:
        calls.gemm_fp8_blockscaled_tn(self.a, self.sa, self.b, self.sb, self.c_local, self.torch.cuda.current_stream())

    def host_buffers(self):
        """End to end = `krn_b200.streaming.StreamedFp8Product` over pinned host codes, scales and output."""
        from krn_b200 import streaming

        torch = self.torch
        self.host_in = [t.view(torch.uint8).cpu().pin_memory() if t.dtype == torch.float8_e4m3fn else t.cpu().pin_memory()
                        for t in (self.a, self.sa, self.b, self.sb)]
        self.host_out = torch.empty(self.c_local.shape, dtype=self.c_local.dtype).pin_memory()
        h2d = sum(t.numel() * t.element_size() for t in self.host_in)
        if self.world > 1 and self.m % self.world == 0:
            # a and its scales cross PCIe once per node: each rank copies M / G of the rows, NVLink all-gathers them
            self.streamed = streaming.ShardedStreamedFp8Product(self.m, self.n_local, self.k, self.c_local.dtype)
            h2d -= sum(t.numel() * t.element_size() for t in self.host_in[:2]) * (self.world - 1) // self.world
        else:
            self.streamed = streaming.StreamedFp8Product(self.m, self.n_local, self.k, self.c_local.dtype)
        return h2d, self.host_out.numel() * self.host_out.element_size()

    def e2e_step(self, calls) -> None:
        self.streamed.run(*self.host_in, self.host_out)

    def parity_sample(self, oracle, calls) -> dict:
        import numpy as np

        torch = self.torch
        self.kernel_only(calls)
        torch.cuda.synchronize()
        rows = [0, 1, 127, 128, 255, 256, self.m // 2, self.m - 257, self.m - 256, self.m - 1]
        host = lambda t: t.contiguous().view(torch.uint8).cpu().numpy() if t.dtype == torch.float8_e4m3fn else t.cpu().numpy()
        errors = []
        for lo in (0, (self.n_local // 2) // 256 * 256, self.n_local - 256):  # first, a middle and the last 256-column tile
            want = oracle.bf16_values(oracle.gemm_fp8_blockscaled(
                host(self.a[rows]), host(self.sa[rows]), host(self.b[lo:lo + 256]), host(self.sb[lo // 128:lo // 128 + 2]),
                threads=8))
            got = oracle.bf16_values(self.c_local[rows, lo:lo + 256].contiguous().view(torch.int16).cpu().numpy().view(np.uint16))
            errors.append(oracle.rel_frobenius(got, want))
        return {"value": max(errors), "tolerance": 3e-2,
                "sample": f"{len(rows)} rows x the first, a middle and the last 256-column tile against the oracle"}

    def cpu_sample(self, oracle, cores: int, columns: int | None = None):
        n = columns or 2048
        rows = 64 * cores
        a_codes, sa, b_codes, sb = oracle.config_gemm_fp8(rows, n, self.k, seed=2)

        def run() -> None:
            oracle.gemm_fp8_blockscaled(a_codes, sa, b_codes, sb, threads=cores)

        return 2.0 * rows * n * self.k, f"first {rows} rows x {n} columns of the product, K={self.k}, {cores} threads", run


class GemmMxfp8(Workload):
    """MXFP8 product (e4m3 codes, one e8m0 scale per 1 x 32 block, scales applied by the tensor cores) at the C3 extents
    M=8192 N=28672 K=8192 (seed 2), bf16 out. One GPU only (no sharded entry point exists for it)."""

    name, metric, dtype = "gemm_mxfp8", "mxfp8_gemm_tflops", "fp8_e4m3"
    description = "MXFP8 GEMM M=8192 N=28672 K=8192, e8m0 scales per 1x32 block fed to the block-scaled MMA, bf16 out (seed 2)"
    m, n, k = 8192, 28672, 8192
    launches_per_step = 2  # the scale layout kernel and the product; both inside the timed call

    def __init__(self, torch, rank, world, size=None) -> None:
        super().__init__(torch, rank, world)
        if size:
            self.m, self.n, self.k = size
            self.description = f"MXFP8 GEMM M={self.m} N={self.n} K={self.k} (profiling case)"
        if world > 1:
            raise RuntimeError("the MXFP8 product has no sharded entry point: measured on one GPU only")
        gen = torch.Generator(device="cuda").manual_seed(2)
        self.a, self.sa = self._quantize(torch.randn((self.m, self.k), device="cuda", generator=gen))
        self.b, self.sb = self._quantize(torch.randn((self.n, self.k), device="cuda", generator=gen))
        self.c = torch.empty((self.m, self.n), device="cuda", dtype=torch.bfloat16)

    def _quantize(self, x):
        """The OCP MX floor rule on the device: scale 2^(floor(log2 absmax) - 8) per 1 x 32 block, codes e4m3(x / scale)."""
        torch = self.torch
        rows, cols = x.shape
        blocks = x.view(rows, cols // 32, 32)
        absmax = blocks.abs().amax(dim=2)
        exponent = torch.where(absmax > 0, torch.floor(torch.log2(torch.where(absmax > 0, absmax, torch.ones_like(absmax)))) - 8,
                               torch.zeros_like(absmax)).clamp_(-127, 127)
        codes = (blocks * torch.exp2(-exponent)[:, :, None]).clamp_(-448, 448).reshape(rows, cols).to(torch.float8_e4m3fn)
        return codes, (exponent + 127).to(torch.uint8).contiguous()

    @property
    def config(self) -> dict:
        return {"workload": self.description, "m": self.m, "n": self.n, "k": self.k, "sharding": "one GPU, no exchange",
                "l2": self.l2_note("operands and output", self.m * self.k + self.n * self.k + 2 * self.m * self.n, 1)}

    def work(self) -> float:
        return 2.0 * self.m * self.n * self.k

    kernel_work = work

    def peak(self, peaks: dict) -> tuple[float, str]:
        return 2.0 * peaks["bf16_tflops_sustained"], "2 x sustained cuBLAS bf16 (no FP8 peak was measured on this pool)"

    def step(self, calls) -> None:
        calls.gemm_mxfp8_tn(self.a, self.sa, self.b, self.sb, self.c, self.torch.cuda.current_stream())

    kernel_only = step

    form = "mxfp8"  # the block format's name for krn_b200.streaming.StreamedScaledProduct

    def host_buffers(self):
        """End to end = `krn_b200.streaming.StreamedScaledProduct` over pinned host codes, scale bytes and output."""
        from krn_b200 import streaming

        torch = self.torch
        self.host_in = [t.view(torch.uint8).cpu().pin_memory() for t in (self.a, self.sa, self.b, self.sb)]
        self.host_out = torch.empty(self.c.shape, dtype=self.c.dtype).pin_memory()
        self.streamed = streaming.StreamedScaledProduct(self.form, self.m, self.n, self.k, self.c.dtype)
        return (sum(t.numel() * t.element_size() for t in self.host_in), self.host_out.numel() * self.host_out.element_size())

    def e2e_step(self, calls) -> None:
        self.streamed.run(*self.host_in, self.host_out, getattr(self, "alpha", 1.0))

    def parity_sample(self, oracle, calls) -> dict:
        import numpy as np

        torch = self.torch
        self.step(calls)
        torch.cuda.synchronize()
        rows = [0, 1, 127, 128, self.m // 2, self.m - 129, self.m - 128, self.m - 1]
        host = lambda t: t.contiguous().view(torch.uint8).cpu().numpy()
        errors = []
        for lo in (0, (self.n // 2) // 256 * 256, self.n - 256):
            want = oracle.bf16_values(oracle.gemm_mxfp8(host(self.a[rows]), host(self.sa[rows]), host(self.b[lo:lo + 256]),
                                                        host(self.sb[lo:lo + 256]), threads=8))
            got = oracle.bf16_values(self.c[rows, lo:lo + 256].contiguous().view(torch.int16).cpu().numpy().view(np.uint16))
            errors.append(oracle.rel_frobenius(got, want))
        return {"value": max(errors), "tolerance": 3e-2,
                "sample": f"{len(rows)} rows x the first, a middle and the last 256-column tile against the oracle"}

    def cpu_sample(self, oracle, cores: int, columns: int | None = None):
        import numpy as np

        n = columns or 2048
        rows = 64 * cores
        rng = np.random.default_rng(2)
        a_codes, sa = oracle.quantize_mxfp8(rng.standard_normal((rows, self.k), np.float32))
        b_codes, sb = oracle.quantize_mxfp8(rng.standard_normal((n, self.k), np.float32))

        def run() -> None:
            oracle.gemm_mxfp8(a_codes, sa, b_codes, sb, threads=cores)

        return 2.0 * rows * n * self.k, f"first {rows} rows x {n} columns of the product, K={self.k}, {cores} threads", run


class GemmNvfp4(GemmMxfp8):
    """NVFP4 product (packed e2m1 codes, one e4m3 scale per 1 x 16 block applied by the tensor cores, one f32 tensor scale
    per matrix) at the C3 extents M=8192 N=28672 K=8192 (seed 2), bf16 out. One GPU only."""

    name, metric, dtype = "gemm_nvfp4", "nvfp4_gemm_tflops", "fp4_e2m1"
    form = "nvfp4"
    description = "NVFP4 GEMM M=8192 N=28672 K=8192, e4m3 scales per 1x16 block fed to the block-scaled MMA, bf16 out (seed 2)"

    def __init__(self, torch, rank, world, size=None) -> None:
        Workload.__init__(self, torch, rank, world)
        if size:
            self.m, self.n, self.k = size
            self.description = f"NVFP4 GEMM M={self.m} N={self.n} K={self.k} (profiling case)"
        if world > 1:
            raise RuntimeError("the NVFP4 product has no sharded entry point: measured on one GPU only")
        gen = torch.Generator(device="cuda").manual_seed(2)
        self.a, self.sa, ta = self._quantize(torch.randn((self.m, self.k), device="cuda", generator=gen))
        self.b, self.sb, tb = self._quantize(torch.randn((self.n, self.k), device="cuda", generator=gen))
        self.alpha = ta * tb
        self.c = torch.empty((self.m, self.n), device="cuda", dtype=torch.bfloat16)

    def _quantize(self, x):
        """The NVFP4 rule on the device: tensor scale = absmax / (6 * 448), block scale = e4m3(block absmax / 6 / tensor
        scale), codes = e2m1(x / (scale * tensor scale)) packed two per byte, low nibble first."""
        torch = self.torch
        rows, cols = x.shape
        tensor_scale = float(x.abs().max()) / (6.0 * 448.0)
        blocks = x.view(rows, cols // 16, 16)
        absmax = blocks.abs().amax(dim=2)
        scale_codes = (absmax / 6.0 / tensor_scale).clamp_(max=448.0).to(torch.float8_e4m3fn)
        scale = scale_codes.float() * tensor_scale
        mag = torch.where(scale[:, :, None] > 0, blocks.abs() / torch.where(scale > 0, scale, torch.ones_like(scale))[:, :, None],
                          torch.zeros_like(blocks))
        code = ((mag > 0.25).to(torch.uint8) + (mag >= 0.75) + (mag > 1.25) + (mag >= 1.75) + (mag > 2.5) + (mag >= 3.5) +
                (mag > 5.0)).to(torch.uint8)
        code |= (blocks < 0).to(torch.uint8) << 3
        code = code.view(rows, cols)
        packed = (code[:, 0::2] | (code[:, 1::2] << 4)).contiguous()
        return packed, scale_codes.view(torch.uint8).contiguous(), tensor_scale

    @property
    def config(self) -> dict:
        return {"workload": self.description, "m": self.m, "n": self.n, "k": self.k, "sharding": "one GPU, no exchange",
                "l2": self.l2_note("operands and output", (self.m * self.k + self.n * self.k) // 2 + 2 * self.m * self.n, 1)}

    def peak(self, peaks: dict) -> tuple[float, str]:
        return 4.0 * peaks["bf16_tflops_sustained"], "4 x sustained cuBLAS bf16 (no FP4 peak was measured on this pool)"

    def step(self, calls) -> None:
        calls.gemm_nvfp4_tn(self.a, self.sa, self.b, self.sb, self.c, self.alpha, self.torch.cuda.current_stream())

    kernel_only = step

    def parity_sample(self, oracle, calls) -> dict:
        import numpy as np

        torch = self.torch
        self.step(calls)
        torch.cuda.synchronize()
        rows = [0, 1, 127, 128, self.m // 2, self.m - 129, self.m - 128, self.m - 1]
        host = lambda t: t.contiguous().cpu().numpy()
        errors = []
        for lo in (0, (self.n // 2) // 256 * 256, self.n - 256):
            want = oracle.bf16_values(oracle.gemm_nvfp4(host(self.a[rows]), host(self.sa[rows]), host(self.b[lo:lo + 256]),
                                                        host(self.sb[lo:lo + 256]), self.alpha, threads=8))
            got = oracle.bf16_values(self.c[rows, lo:lo + 256].contiguous().view(torch.int16).cpu().numpy().view(np.uint16))
            errors.append(oracle.rel_frobenius(got, want))
        return {"value": max(errors), "tolerance": 3e-2,
                "sample": f"{len(rows)} rows x the first, a middle and the last 256-column tile against the oracle"}

    def cpu_sample(self, oracle, cores: int, columns: int | None = None):
        import numpy as np

        n = columns or 2048
        rows = 64 * cores
        rng = np.random.default_rng(2)
        a, sa, ta = oracle.quantize_nvfp4(rng.standard_normal((rows, self.k), np.float32))
        b, sb, tb = oracle.quantize_nvfp4(rng.standard_normal((n, self.k), np.float32))

        def run() -> None:
            oracle.gemm_nvfp4(a, sa, b, sb, ta * tb, threads=cores)

        return 2.0 * rows * n * self.k, f"first {rows} rows x {n} columns of the product, K={self.k}, {cores} threads", run


class AttnFwd(Workload):
    """Causal GQA flash attention forward, B=8 Hq=32 Hkv=8 S=4096 D=128, bf16 (seed 3). Sharded by batch."""

    name, metric, dtype = "attn_fwd", "flash_attn_fwd_tflops", "bf16"
    description = "bf16 causal flash-attention forward B=8 Hq=32 Hkv=8 S=4096 D=128 (seed 3, N(0,1))"
    batch, hq, hkv, seq, d = 8, 32, 8, 4096, 128

    def __init__(self, torch, rank, world, size=None) -> None:
        super().__init__(torch, rank, world)
        from krn_b200 import sharding

        if size:
            self.batch, self.hq, self.hkv, self.seq, self.d = size
            self.description = f"causal flash attention B={self.batch} Hq={self.hq} Hkv={self.hkv} S={self.seq} D={self.d}"
        units = sharding.contiguous_units(self.batch, rank, world)  # whole batches = contiguous (batch, kv head) units
        self.batch_local = len(units)
        gen = torch.Generator(device="cuda").manual_seed(3)
        shape_q, shape_kv = (self.batch, self.hq, self.seq, self.d), (self.batch, self.hkv, self.seq, self.d)
        q, k, v = (torch.randn(s, device="cuda", generator=gen).to(torch.bfloat16) for s in (shape_q, shape_kv, shape_kv))
        self.q, self.k, self.v = (t[units.start:units.stop].contiguous() for t in (q, k, v))
        del q, k, v
        self.o = torch.empty_like(self.q)
        self.scale_log2 = math.log2(math.e) / math.sqrt(self.d)
        self.set_bytes = sum(t.numel() * 2 for t in (self.q, self.k, self.v, self.o))
        self.sets = [(self.q, self.k, self.v, self.o)]
        for _ in range(self.rotation(self.set_bytes) - 1 if self.batch_local else 0):
            self.sets.append(tuple(t.clone() for t in self.sets[0]))
        self.turn = 0

    @property
    def config(self) -> dict:
        return {"workload": self.description, "sharding": f"(batch, kv head) units x{self.world}, no collective",
                "l2": self.l2_note("Q, K, V, O", self.set_bytes, len(self.sets))}

    def work(self) -> float:
        return 4.0 * self.batch * self.hq * self.d * self.seq * (self.seq + 1) / 2

    def kernel_work(self) -> float:
        return self.work() * self.batch_local / self.batch

    def run(self, calls, tensors) -> None:
        if self.batch_local:
            q, k, v, o = tensors
            calls.attention_forward(q, k, v, o, self.scale_log2, True, self.torch.cuda.current_stream())

    def step(self, calls) -> None:
        self.run(calls, self.sets[self.turn % len(self.sets)])
        self.turn += 1

    kernel_only = step

    def host_buffers(self):
        """End to end = `krn_b200.streaming.StreamedAttention` over pinned host q, k, v, o, one batch at a time."""
        from krn_b200 import streaming

        self.host_in = [t.cpu().pin_memory() for t in (self.q, self.k, self.v)]
        self.host_out = self.torch.empty(self.o.shape, dtype=self.o.dtype).pin_memory()
        if self.batch_local:
            self.streamed = streaming.StreamedAttention(self.batch_local, self.hq, self.hkv, self.seq, self.d,
                                                        self.torch.bfloat16, groups=self.batch_local)
        return sum(t.numel() * t.element_size() for t in self.host_in), self.host_out.numel() * self.host_out.element_size()

    def e2e_step(self, calls) -> None:
        if self.batch_local:
            self.streamed.run(*self.host_in, self.host_out, self.scale_log2, True)

    def parity_sample(self, oracle, calls) -> dict:
        """Causal attention of the first 1024 queries depends on the first 1024 keys only, so that prefix of four q heads
        (one kv head) is checked against the oracle's statement-by-statement attention on the same prefix."""
        import numpy as np

        torch = self.torch
        q, k, v, o = self.sets[0]
        self.run(calls, self.sets[0])
        torch.cuda.synchronize()
        rows = min(1024, self.seq)
        words = lambda t: t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
        group = self.hq // self.hkv
        want = oracle.bf16_values(oracle.flash_attention(words(q[:1, :group, :rows]), words(k[:1, :1, :rows]),
                                                         words(v[:1, :1, :rows]), dtype=oracle.BF16, scale=self.scale_log2,
                                                         causal=True, bq=64, bk=64, threads=group))
        got = oracle.bf16_values(words(o[:1, :group, :rows]))
        return {"value": oracle.rel_frobenius(got, want), "tolerance": 1e-2,
                "sample": f"the first {rows} query rows of {group} q heads (batch 0, kv head 0) against the oracle"}

    def cpu_sample(self, oracle, cores: int, columns: int | None = None):
        heads = cores
        seq = columns or 2048
        q, k, v = oracle.config_attention(1, heads, max(1, heads // 4), seq, self.d, seed=3)

        def run() -> None:
            oracle.flash_attention(q, k, v, dtype=oracle.BF16, scale=self.scale_log2, causal=True, bq=64, bk=64, threads=cores)

        return (4.0 * heads * self.d * seq * (seq + 1) / 2,
                f"{heads} q heads of one batch at S={seq} (causal, 64x64 tiles), {cores} threads", run)


class AttnDecode(Workload):
    """Paged FP8 decode attention, 64 sequences with contexts U[1024, 8192] (seed 4). HBM-bound: GB/s."""

    name, metric, dtype = "attn_decode", "paged_fp8_decode_gbs", "fp8_e4m3"
    unit, bound = "GB/s", "hbm"
    description = "FP8 e4m3 paged decode attention B=64 Hq=32 Hkv=8 D=128, contexts U[1024,8192], page 64 (seed 4)"
    batch, hq, hkv, d, page = 64, 32, 8, 128, 64
    launches_per_step = 2  # the split-KV kernel and its merge

    def __init__(self, torch, rank, world, size=None) -> None:
        super().__init__(torch, rank, world)
        import numpy as np

        from krn_b200 import sharding
        from krn_b200.runtime import calls

        rng = np.random.default_rng(4)
        lens = rng.integers(1024, 8193, self.batch).astype(np.int32)
        mine = sharding.balanced_by_length(lens, world)[rank]
        self.all_tokens = int(lens.sum())
        lens = lens[mine]
        self.local = len(mine)
        self.tokens = int(lens.sum())
        pages = -(-lens // self.page)
        self.max_pages = 8192 // self.page
        pool = int(pages.sum())
        order = rng.permutation(pool).astype(np.int32)
        table = np.zeros((self.local, self.max_pages), np.int32)
        cursor = 0
        for i, count in enumerate(pages):
            table[i, :count] = order[cursor:cursor + count]
            cursor += int(count)
        gen = torch.Generator(device="cuda").manual_seed(4 + rank)
        shape = (pool, self.page, self.hkv, self.d)
        # codes of N(0, 1) * 100 clamped into the finite e4m3 range (the conversion itself does not saturate)
        self.k_pages = (torch.randn(shape, device="cuda", generator=gen) * 100).clamp_(-448, 448).to(torch.float8_e4m3fn)
        self.v_pages = (torch.randn(shape, device="cuda", generator=gen) * 100).clamp_(-448, 448).to(torch.float8_e4m3fn)
        self.k_scale = torch.rand((self.local, self.hkv), device="cuda", generator=gen) * 0.01 + 0.005
        self.v_scale = torch.rand((self.local, self.hkv), device="cuda", generator=gen) * 0.01 + 0.005
        self.q = torch.randn((self.local, self.hq, self.d), device="cuda", generator=gen).to(torch.bfloat16)
        self.table, self.lens = torch.from_numpy(table).cuda(), torch.from_numpy(lens).cuda()
        self.o = torch.empty_like(self.q)
        self.scale_log2 = math.log2(math.e) / math.sqrt(self.d)
        self.workspace = torch.empty(calls.decode_workspace_bytes(self.local, self.hq, self.d, 8192), device="cuda",
                                     dtype=torch.uint8)
        self.set_bytes = int(self.kernel_work())
        self.pools = [(self.k_pages, self.v_pages)]
        for _ in range(self.rotation(self.set_bytes) - 1):
            self.pools.append((self.k_pages.clone(), self.v_pages.clone()))
        self.turn = 0

    @property
    def config(self) -> dict:
        return {"workload": self.description, "sharding": f"sequences balanced by length x{self.world}, no collective",
                "l2": self.l2_note("the cache pages read per step", self.set_bytes, len(self.pools))}

    def _bytes(self, tokens: int, sequences: int) -> float:
        return tokens * 2.0 * self.hkv * self.d + 2.0 * sequences * self.hq * self.d * 2 + 4.0 * tokens / self.page

    def work(self) -> float:
        return self._bytes(self.all_tokens, self.batch)

    def kernel_work(self) -> float:
        return self._bytes(self.tokens, self.local)

    def scale(self, work: float, ms: float) -> float:
        return work / (ms * 1e-3) / 1e9  # GB/s

    def peak(self, peaks: dict) -> tuple[float, str]:
        return peaks["hbm_gbs"], "STREAM-style copy bandwidth"

    def step(self, calls) -> None:
        k_pages, v_pages = self.pools[self.turn % len(self.pools)]
        self.turn += 1
        calls.attention_decode_fp8_paged(self.q, k_pages, v_pages, self.table, self.lens, self.k_scale,
                                         self.v_scale, self.o, self.scale_log2, 8192, self.workspace,
                                         self.torch.cuda.current_stream())

    kernel_only = step

    def host_buffers(self):
        # the cache lives on the device in a decode loop; per step the host sends the query and reads the output
        self.host_in = [self.q.cpu().pin_memory()]
        self.host_out = self.torch.empty(self.o.shape, dtype=self.o.dtype).pin_memory()
        return self.host_in[0].numel() * 2, self.host_out.numel() * 2

    def e2e_step(self, calls) -> None:
        self.q.copy_(self.host_in[0], non_blocking=True)
        self.step(calls)
        self.host_out.copy_(self.o, non_blocking=True)

    def parity_sample(self, oracle, calls) -> dict:
        import numpy as np

        torch = self.torch
        k_pages, v_pages = self.pools[0]
        calls.attention_decode_fp8_paged(self.q, k_pages, v_pages, self.table, self.lens, self.k_scale, self.v_scale, self.o,
                                         self.scale_log2, 8192, self.workspace, torch.cuda.current_stream())
        torch.cuda.synchronize()
        words = lambda t: t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
        codes = lambda t: t.view(torch.uint8).cpu().numpy()
        want = oracle.bf16_values(oracle.decode_fp8_paged(
            words(self.q), codes(k_pages), codes(v_pages), self.table.cpu().numpy(), self.lens.cpu().numpy(),
            self.k_scale.cpu().numpy(), self.v_scale.cpu().numpy(), scale_log2=self.scale_log2, threads=8))
        return {"value": oracle.rel_frobenius(oracle.bf16_values(words(self.o)), want), "tolerance": 3e-2,
                "sample": f"all {self.local} sequences against the oracle"}

    def cpu_sample(self, oracle, cores: int, columns: int | None = None):
        config = oracle.config_decode(batch=cores, q_heads=self.hq, kv_heads=self.hkv, d=self.d, low=1024, high=2048, seed=4)
        tokens = int(config[4].sum())

        def run() -> None:
            oracle.decode_fp8_paged(*config, scale_log2=self.scale_log2, threads=cores)

        return self._bytes(tokens, cores), f"{cores} sequences with contexts U[1024,2048], {cores} threads", run


WORKLOADS = {w.name: w for w in (GemmBf16, GemmFp8, GemmMxfp8, GemmNvfp4, AttnFwd, AttnDecode)}


def cpu_rates(workload, oracle, cores: int, columns: int | None, repeats: int = 1) -> dict:
    """The CPU restatement of the reference's C backend on a bounded sample of the workload: once on `cores` threads (the
    grid split over threads, the way the reference gets concurrency across streams) and once on ONE thread, which is
    how the reference runs a single kernel call (src/krn/runtime/cpu.py:137-140)."""
    work, sample, run = workload.cpu_sample(oracle, cores, columns)
    start = time.perf_counter()
    for _ in range(repeats):
        run()
    seconds = (time.perf_counter() - start) / repeats
    work1, sample1, run1 = workload.cpu_sample(oracle, 1, workload.single_thread_columns)
    start = time.perf_counter()
    run1()
    seconds1 = time.perf_counter() - start
    return {"value": workload.scale(work, seconds * 1e3), "unit": workload.unit, "cores": cores, "kind": "port",
            "sample": sample, "seconds": seconds,
            "one_thread": {"value": workload.scale(work1, seconds1 * 1e3), "unit": workload.unit, "cores": 1,
                           "sample": sample1, "seconds": seconds1}}


def reference_arm(args, rank: int) -> int:
    """The reference's CPU implementation of the path (restated C backend) on the host cores; rank 0 only. Each step is a
    bounded sample of the workload (its extents are in `config.sample`); the value is the sample's rate."""
    if rank != 0:
        return 0
    from oracle import oracle

    cores = min(os.cpu_count() or 1, 64)
    kind = WORKLOADS[args.workload if args.workload != "all" else "gemm_bf16"]
    workload = kind.__new__(kind)
    workload.world, workload.scale_log2 = 1, math.log2(math.e) / math.sqrt(128)
    work, sample, run = workload.cpu_sample(oracle, cores, columns=kind.reference_columns)
    for _ in range(args.warmup):
        run()
    start = time.perf_counter()
    for _ in range(args.steps):
        run()
    seconds = time.perf_counter() - start
    value = workload.scale(work * args.steps, seconds * 1e3)
    work1, sample1, run1 = workload.cpu_sample(oracle, 1, kind.single_thread_columns)
    start = time.perf_counter()
    run1()
    seconds1 = time.perf_counter() - start
    line = {
        "impl": "reference", "metric": workload.metric, "value": value, "unit": workload.unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": workload.dtype, "data": "synthetic",
        "config": {"workload": workload.description, "sample": sample,
                   "note": "each step runs the sample, not the full problem; value is the sample's rate"},
        "cpu_baseline": {"value": value, "unit": workload.unit, "cores": cores, "kind": "port", "sample": sample,
                         "one_thread": {"value": workload.scale(work1, seconds1 * 1e3), "unit": workload.unit, "cores": 1,
                                        "sample": sample1, "seconds": seconds1}},
        "e2e": {"value": value, "unit": workload.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


class Harness:
    """Timing of one workload: device events around `steps` calls, several trials, the median; max over ranks."""

    def __init__(self, torch, args, rank: int, world: int, local_rank: int) -> None:
        self.torch, self.args, self.rank, self.world, self.local_rank = torch, args, rank, world, local_rank
        self.distributed = world > 1
        self.peaks, self.peak_kind = measured_peaks()

    def barrier(self) -> None:
        if self.distributed:
            self.torch.distributed.barrier()
        self.torch.cuda.synchronize()

    def trial(self, fn, steps: int) -> float:
        """Milliseconds for `steps` calls of fn, on the device, max over ranks."""
        torch = self.torch
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        start.record()
        for _ in range(steps):
            fn()
        stop.record()
        self.barrier()
        ms = torch.tensor([start.elapsed_time(stop)], device="cuda", dtype=torch.float64)
        if self.distributed:
            torch.distributed.all_reduce(ms, op=torch.distributed.ReduceOp.MAX)
        return float(ms.item())

    def trials(self, fn, steps: int, budget_ms: float, least: int = 5, most: int = 400) -> list[float]:
        """Per-step milliseconds of each of several trials of `steps` calls: at least `least` trials and as many as it
        takes for the trials together to last `budget_ms` (every rank runs the same number: rank 0 decides)."""
        torch = self.torch
        first = self.trial(fn, steps)
        count = max(least - 1, min(most, int(math.ceil(budget_ms / max(first, 1e-3))) - 1))
        if self.distributed:
            agreed = torch.tensor([count], device="cuda")
            torch.distributed.broadcast(agreed, 0)
            count = int(agreed.item())
        return [first / steps] + [self.trial(fn, steps) / steps for _ in range(count)]

    def measure(self, workload, calls, native, *, e2e: bool, cpu: bool, check: bool) -> dict:
        args, torch = self.args, self.torch
        warmup = max(args.warmup, 3)
        for _ in range(warmup):
            workload.step(calls)
        torch.cuda.synchronize()
        # ---- resident-operand throughput: the clock sampler runs for the whole timed region (>= 1 s of launches)
        with ClockSampler(self.local_rank) as sampler:
            per_step = self.trials(lambda: workload.step(calls), args.steps, args.region_ms)
        clocks = sampler.summary()
        native.raise_device_status()
        per_step.sort()
        ms_per_step = per_step[len(per_step) // 2]
        value = workload.scale(workload.work(), ms_per_step)

        # ---- the dominant kernel alone (roofline)
        kernel = self.trials(lambda: workload.kernel_only(calls), args.steps, args.region_ms / 4)
        kernel.sort()
        kernel_ms = kernel[len(kernel) // 2]
        achieved = workload.scale(workload.kernel_work(), kernel_ms)
        best = workload.scale(workload.kernel_work(), kernel[0])
        peak, peak_note = workload.peak(self.peaks)
        roofline = {"bound": workload.bound, "achieved": achieved, "peak": peak, "unit": workload.unit,
                    "frac": achieved / peak,
                    "traffic": None if args.size or self.world > 1 else NCU_TRAFFIC_BYTES.get(workload.name),
                    "peak_kind": f"{self.peak_kind}: {peak_note}", "kernel_ms": kernel_ms}
        if workload.bound == "tensor":
            # `achieved` is the median of a run of back-to-back launches that lasts long enough for the power cap to
            # settle the clock, so its denominator is the cuBLAS figure measured the same way (sustained); the best trial
            # (launches on a cool part) is set against the cuBLAS best-of-10 burst figure
            factor = 4.0 if workload.dtype.startswith("fp4") else 2.0 if workload.dtype.startswith("fp8") else 1.0
            burst = factor * self.peaks["bf16_tflops"]
            roofline["burst"] = {"achieved": best, "peak": burst, "frac": best / burst,
                                 "note": "best trial over the burst (best-of-10) cuBLAS figure"}
            roofline["frac_of_nominal_dense_peak"] = achieved / (2250.0 * factor)
            roofline["best_frac_of_nominal_dense_peak"] = best / (4500.0 if factor == 2.0 else 2250.0)

        record = {"metric": workload.metric, "value": value, "unit": workload.unit, "ms_per_step": ms_per_step,
                  "trials": len(per_step), "ms_per_step_min": per_step[0], "ms_per_step_max": per_step[-1],
                  "dtype": workload.dtype, "config": workload.config, "roofline": roofline, "clocks": clocks,
                  "gpu_launches": workload.launches_per_step * args.steps * len(per_step)}

        # ---- end to end with host buffers
        if e2e:
            try:
                h2d, d2h = workload.host_buffers()
                for _ in range(2):
                    workload.e2e_step(calls)
                e2e_steps = max(3, min(args.steps, 10))
                e2e_ms = sorted(self.trial(lambda: workload.e2e_step(calls), e2e_steps) / e2e_steps for _ in range(3))[1]
                record["e2e"] = {"value": workload.scale(workload.work(), e2e_ms), "unit": workload.unit,
                                 "h2d_bytes_per_step": h2d * self.world, "d2h_bytes_per_step": d2h * self.world,
                                 "ms_per_step": e2e_ms}
                native.raise_device_status()
            except Exception as error:  # the device-resident numbers stand on their own; say why this leg is absent
                record["e2e"] = None
                record["e2e_error"] = f"{type(error).__name__}: {error}"
        else:
            record["e2e"] = None

        # ---- parity on a sample and the CPU baseline (rank 0, N = 1 only)
        if self.rank == 0 and self.world == 1 and (check or cpu):
            from oracle import oracle

            if check:
                record["rel_frobenius"] = workload.parity_sample(oracle, calls)
            if cpu:
                record["cpu_baseline"] = cpu_rates(workload, oracle, min(os.cpu_count() or 1, 64), None)
        record.setdefault("cpu_baseline", None)
        return record


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default="all", choices=["all", *sorted(WORKLOADS)],
                        help="all: the headline workload (gemm_bf16) plus a sub-record for each of the others")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--kernel-only", action="store_true", help="profiling: skip the e2e, parity and CPU legs")
    parser.add_argument("--size", type=int, nargs="+", default=None, help="profiling: override the problem extents")
    parser.add_argument("--region-ms", type=float, default=1000.0,
                        help="how long the timed trials of a workload last together (the clock sampler needs ~1 s)")
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
    if world > 1:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # the fused gather uses unicast peer stores only
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    harness = Harness(torch, args, rank, world, local_rank)
    extras = not args.kernel_only
    headline_name = "gemm_bf16" if args.workload == "all" else args.workload
    workload = WORKLOADS[headline_name](torch, rank, world, args.size)
    head = harness.measure(workload, calls, native, e2e=extras, cpu=extras and not args.no_cpu_baseline, check=extras)
    del workload
    torch.cuda.empty_cache()

    others = {}
    if args.workload == "all" and not args.size:
        for name in ("gemm_fp8", "gemm_mxfp8", "gemm_nvfp4", "attn_fwd", "attn_decode") if world == 1 else ("gemm_fp8", "attn_fwd", "attn_decode"):
            try:
                workload = WORKLOADS[name](torch, rank, world, None)
                # with N > 1 the sub-records carry the device-resident numbers only (the run stays within minutes)
                others[name] = harness.measure(workload, calls, native, e2e=extras and world == 1,
                                               cpu=extras and world == 1 and not args.no_cpu_baseline,
                                               check=extras and world == 1)
                del workload
            except Exception as error:  # one workload failing must not take the headline line with it
                others[name] = {"error": f"{type(error).__name__}: {error}"}
            torch.cuda.empty_cache()

    if rank == 0:
        line = {
            "metric": head["metric"], "value": head["value"], "unit": head["unit"], "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": head["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": head["dtype"], "data": "synthetic",
            "config": head["config"], "roofline": head["roofline"], "cpu_baseline": head["cpu_baseline"],
            "e2e": head["e2e"], "gpu_launches": head["gpu_launches"], "clocks": head["clocks"],
            "timing": {"trials": head["trials"], "statistic": "median over trials of (ms of `steps` launches) / steps",
                       "ms_per_step_min": head["ms_per_step_min"], "ms_per_step_max": head["ms_per_step_max"]},
        }
        for key in ("rel_frobenius", "e2e_error"):
            if key in head:
                line[key] = head[key]
        if others:
            line["workloads"] = others
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
