"""MXFP8 tile product on the GPU (scale factors applied by the tensor cores), through the C ABI, against the CPU oracle.

PARITY UNPINNED for the product: the reference declares the MXFP8 format (src/krn/data/formats.py:138-144) and the
`QTile @ QTile` product (src/krn/frontend/memory.py:173-193) but implements neither, so the oracle's definition
(oracle/krn_oracle.c) is ours; the FORMAT's value tables are pinned (tests/test_quantize_cpu.py). The acceptance
tolerance is the benchmark's 3e-2 relative Frobenius error for FP8."""

from __future__ import annotations

import numpy as np
import pytest

import krn_b200 as krn
from krn_b200 import ops
from krn_b200.runtime import calls
from oracle import oracle as o

pytestmark = pytest.mark.gpu


def run(torch, a_codes, sa, b_codes, sb, out="bf16"):
    m, n = a_codes.shape[0], b_codes.shape[0]
    dtype = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[out]
    c = torch.full((m, n), float("nan"), device="cuda", dtype=dtype)
    fp8 = torch.float8_e4m3fn
    calls.gemm_mxfp8_tn(torch.from_numpy(a_codes).cuda().view(fp8), torch.from_numpy(sa).cuda(),
                        torch.from_numpy(b_codes).cuda().view(fp8), torch.from_numpy(sb).cuda(), c)
    torch.cuda.synchronize()
    return c.float().cpu().numpy()


def draw(m, n, k, seed):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((m, k), np.float32) * np.exp2(rng.integers(-4, 5, (m, 1))).astype(np.float32)
    b = rng.standard_normal((n, k), np.float32) * np.exp2(rng.integers(-4, 5, (n, 1))).astype(np.float32)
    return (*o.quantize_mxfp8(a), *o.quantize_mxfp8(b))


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (128, 256, 512), (256, 512, 1024), (384, 768, 640), (1024, 1024, 2048),
                                   (100, 200, 384), (130, 264, 256), (16, 8, 128), (257, 136, 1152)])
@pytest.mark.parametrize("out", ["bf16", "f32"])
def test_mxfp8_product_against_oracle(cuda, m, n, k, out) -> None:
    a_codes, sa, b_codes, sb = draw(m, n, k, seed=m + n + k)
    got = run(cuda, a_codes, sa, b_codes, sb, out)
    want_words = o.gemm_mxfp8(a_codes, sa, b_codes, sb, c_type=o.BF16 if out == "bf16" else o.F32, threads=8)
    want = o.bf16_values(want_words) if out == "bf16" else want_words
    exact = o.mxfp8_values(a_codes, sa) @ o.mxfp8_values(b_codes, sb).T
    assert np.isfinite(got).all()
    assert o.rel_frobenius(got, exact) < 3e-2          # the benchmark's tolerance
    assert o.rel_frobenius(got, want) < (1e-2 if out == "bf16" else 1e-5)


def test_small_integer_codes_and_power_of_two_scales_are_exact(cuda) -> None:
    """Small-integer codes with scales that differ per 32-wide block: every term is exactly representable, so the result
    must equal the oracle bit for bit — and any mix-up of scale bytes (row, block, or which of the four bytes of a
    tensor-memory column an instruction reads) shows as a wrong power of two."""
    rng = np.random.default_rng(21)
    m, n, k = 300, 520, 640
    a_codes = o.e4m3_encode(rng.integers(-4, 5, (m, k)).astype(np.float32))
    b_codes = o.e4m3_encode(rng.integers(-4, 5, (n, k)).astype(np.float32))
    sa = (127 + rng.integers(-3, 4, (m, k // 32))).astype(np.uint8)
    sb = (127 + rng.integers(-3, 4, (n, k // 32))).astype(np.uint8)
    got = run(cuda, a_codes, sa, b_codes, sb, "f32")
    want = o.gemm_mxfp8(a_codes, sa, b_codes, sb, c_type=o.F32, threads=8)
    np.testing.assert_array_equal(got, want)
    np.testing.assert_array_equal(got, (o.mxfp8_values(a_codes, sa) @ o.mxfp8_values(b_codes, sb).T).astype(np.float32))


def test_ragged_edges_leave_neighbours_alone(cuda) -> None:
    torch = cuda
    a_codes, sa, b_codes, sb = draw(33, 24, 256, seed=5)
    c = torch.full((40, 48), 5.0, device="cuda", dtype=torch.bfloat16)
    fp8 = torch.float8_e4m3fn
    calls.gemm_mxfp8_tn(torch.from_numpy(a_codes).cuda().view(fp8), torch.from_numpy(sa).cuda(),
                        torch.from_numpy(b_codes).cuda().view(fp8), torch.from_numpy(sb).cuda(), c[:33, :24])
    torch.cuda.synchronize()
    assert bool((c[33:] == 5).all()) and bool((c[:, 24:] == 5).all())
    want = o.bf16_values(o.gemm_mxfp8(a_codes, sa, b_codes, sb))
    assert o.rel_frobenius(c[:33, :24].float().cpu().numpy(), want) < 1e-2


def test_quantised_containers_and_refusals(cuda) -> None:
    """`ops.quantize` + `ops.matmul_q`: the QMatrix struct end to end, for both pairings that have kernels."""
    torch = cuda
    device = krn.host.Device.current()
    rng = np.random.default_rng(9)
    x, w = rng.standard_normal((256, 512), np.float32), rng.standard_normal((384, 512), np.float32)
    exact = x.astype(np.float64) @ w.astype(np.float64).T
    qx, qw = ops.quantize(x, krn.formats.MXFP8()), ops.quantize(w, krn.formats.MXFP8())
    assert qx.shape == (256, 512) and qx.scales.shape == (256, 16) and qx.fmt.name == "mxfp8" and qx.tensor_scale is None
    out = device.empty(krn.bf16, 256, 384)
    ops.matmul_q(qx, qw, out)
    torch.cuda.synchronize()
    assert o.rel_frobenius(o.bf16_values(out.to_host().view(np.uint16)), exact) < 6e-2  # two quantisations of N(0,1) data
    qx, qw = ops.quantize(x, krn.formats.FP8FN()), ops.quantize(w, krn.formats.FP8FNWeights())
    ops.matmul_q(qx, qw, out)
    torch.cuda.synchronize()
    assert o.rel_frobenius(o.bf16_values(out.to_host().view(np.uint16)), exact) < 6e-2
    with pytest.raises(krn.TargetError, match="no prebuilt kernel multiplies this pair"):
        ops.matmul_q(qx, ops.quantize(w, krn.formats.MXFP8()), out)
    fp8 = torch.float8_e4m3fn
    a = torch.zeros((128, 96), device="cuda", dtype=torch.uint8).view(fp8)
    s = torch.zeros((128, 3), device="cuda", dtype=torch.uint8)
    with pytest.raises(Exception, match="K = 96 is not available on sm_100a"):
        calls.gemm_mxfp8_tn(a, s, a, s, torch.zeros((128, 128), device="cuda", dtype=torch.bfloat16))
