"""The MXFP8 and NVFP4 products at the benchmark extents (M = 8192, N = 28672, K = 8192): what the persistent tile
scheduler, the operand ring and the scale ring are built for and what the small parity cases never reach.

Operands are the bench workloads' own (seed 2, N(0,1), quantised on the device). Sampled rows of the first, a middle and
the last 256-column tile go against the CPU oracle; the whole matrix goes through linearity,
(A B^T) 1 = A (B^T 1), evaluated in float64 on the device from the dequantised operands."""

from __future__ import annotations

import numpy as np
import pytest

import bench
from krn_b200.runtime import calls
from oracle import oracle as o

pytestmark = pytest.mark.gpu

E2M1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]


def values_mxfp8(torch, codes, scales):
    return codes.double() * torch.exp2(scales.double() - 127).repeat_interleave(32, 1)


def values_nvfp4(torch, packed, scales, tensor_scale=1.0):
    table = torch.tensor(E2M1, device="cuda", dtype=torch.float64)
    rows, half = packed.shape
    out = torch.empty((rows, 2 * half), device="cuda", dtype=torch.float64)
    out[:, 0::2], out[:, 1::2] = table[(packed & 15).long()], table[(packed >> 4).long()]
    return out * scales.view(torch.float8_e4m3fn).double().repeat_interleave(16, 1) * tensor_scale


def column_sums(torch, b_values_of, rows: int) -> "torch.Tensor":
    total = None
    for lo in range(0, rows, 4096):  # slabs bound the float64 temporaries
        part = b_values_of(lo, min(rows, lo + 4096)).sum(0)
        total = part if total is None else total + part
    return total


def test_mxfp8_at_the_configured_extents(cuda) -> None:
    torch = cuda
    w = bench.GemmMxfp8(torch, 0, 1)
    sample = w.parity_sample(o, calls)
    assert sample["value"] < 1e-2, sample
    assert bool(torch.isfinite(w.c.float()).all())
    weights = column_sums(torch, lambda lo, hi: values_mxfp8(torch, w.b[lo:hi], w.sb[lo:hi]), w.n)
    rhs = values_mxfp8(torch, w.a, w.sa) @ weights[:, None]
    lhs = w.c.double() @ torch.ones((w.n, 1), device="cuda", dtype=torch.float64)
    assert float((lhs - rhs).norm() / rhs.norm()) < 5e-3


def test_nvfp4_at_the_configured_extents(cuda) -> None:
    torch = cuda
    w = bench.GemmNvfp4(torch, 0, 1)
    sample = w.parity_sample(o, calls)
    assert sample["value"] < 1e-2, sample
    assert bool(torch.isfinite(w.c.float()).all())
    weights = column_sums(torch, lambda lo, hi: values_nvfp4(torch, w.b[lo:hi], w.sb[lo:hi]), w.n)
    rhs = (values_nvfp4(torch, w.a, w.sa) @ weights[:, None]) * w.alpha
    lhs = w.c.double() @ torch.ones((w.n, 1), device="cuda", dtype=torch.float64)
    assert float((lhs - rhs).norm() / rhs.norm()) < 5e-3
