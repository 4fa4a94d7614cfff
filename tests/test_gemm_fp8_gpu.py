"""Block-scaled FP8 e4m3 tile product on the GPU, through the C ABI, against the CPU oracle.

PARITY UNPINNED: the reference has neither an implementation nor a test of this product; the oracle's
definition (oracle/krn_oracle.c) is ours, and the acceptance tolerance is the benchmark's: relative Frobenius
error at most 3e-2 against an fp32 evaluation of the same codes and scales."""

from __future__ import annotations

import numpy as np
import pytest

from oracle import oracle as o
from krn_b200.runtime import calls

pytestmark = pytest.mark.gpu


def device(torch, array: np.ndarray, dtype=None):
    tensor = torch.from_numpy(np.ascontiguousarray(array)).cuda()
    return tensor.view(dtype) if dtype is not None else tensor


def run(torch, a_codes, sa, b_codes, sb, out="bf16"):
    m, n = a_codes.shape[0], b_codes.shape[0]
    out_dtype = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[out]
    c = torch.full((m, n), float("nan"), device="cuda", dtype=out_dtype)
    calls.gemm_fp8_blockscaled_tn(device(torch, a_codes, torch.float8_e4m3fn), device(torch, sa),
                                  device(torch, b_codes, torch.float8_e4m3fn), device(torch, sb), c)
    torch.cuda.synchronize()
    return c.float().cpu().numpy()


def exact(a_codes, sa, b_codes, sb):
    m, k = a_codes.shape
    n = b_codes.shape[0]
    a = o.e4m3_decode(a_codes).astype(np.float64) * np.repeat(sa.astype(np.float64), 128, axis=1)[:, :k]
    b = o.e4m3_decode(b_codes).astype(np.float64) * np.repeat(np.repeat(sb.astype(np.float64), 128, axis=0), 128, axis=1)[:n, :k]
    return a @ b.T


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (256, 256, 256), (256, 512, 1024), (384, 768, 640), (1024, 1024, 2048),
                                   (100, 200, 384), (130, 264, 144), (16, 8, 16), (257, 136, 400)])
@pytest.mark.parametrize("out", ["bf16", "f32"])
def test_blockscaled_product_against_oracle(cuda, m, n, k, out) -> None:
    a_codes, sa, b_codes, sb = o.config_gemm_fp8(m, n, k, seed=2)
    got = run(cuda, a_codes, sa, b_codes, sb, out)
    want_words = o.gemm_fp8_blockscaled(a_codes, sa, b_codes, sb, c_type=o.BF16 if out == "bf16" else o.F32, threads=8)
    want = o.bf16_values(want_words) if out == "bf16" else want_words
    reference = exact(a_codes, sa, b_codes, sb)
    assert o.rel_frobenius(got, reference) < 3e-2          # the benchmark's tolerance
    assert o.rel_frobenius(got, want) < (1e-2 if out == "bf16" else 1e-5)
    if out == "f32":  # reordered f32 accumulation of exact products: the reference's bound applies
        a = o.e4m3_decode(a_codes).astype(np.float64) * np.repeat(sa, 128, axis=1)[:, :k]
        b = o.e4m3_decode(b_codes).astype(np.float64) * np.repeat(np.repeat(sb, 128, axis=0), 128, axis=1)[:n, :k]
        assert np.all(np.abs(got - reference) <= o.forward_error_bound(a, b.T, k) + 1e-30)


def test_unit_scales_and_small_codes_are_exact(cuda) -> None:
    """With scales of one and small-integer codes every partial sum is exact: bit-identical to the oracle."""
    rng = np.random.default_rng(12)
    m, n, k = 300, 520, 640
    a = o.e4m3_encode(rng.integers(-4, 5, (m, k)).astype(np.float32))
    b = o.e4m3_encode(rng.integers(-4, 5, (n, k)).astype(np.float32))
    sa, sb = np.ones((m, 5), np.float32), np.ones((5, 5), np.float32)
    got = run(cuda, a, sa, b, sb, "f32")
    want = o.gemm_fp8_blockscaled(a, sa, b, sb, c_type=o.F32, threads=8)
    np.testing.assert_array_equal(got, want)


def test_scales_select_their_blocks(cuda) -> None:
    """Power-of-two scales that differ per block keep the arithmetic exact and expose any block mix-up."""
    rng = np.random.default_rng(13)
    m, n, k = 256, 384, 512
    a = o.e4m3_encode(rng.integers(-3, 4, (m, k)).astype(np.float32))
    b = o.e4m3_encode(rng.integers(-3, 4, (n, k)).astype(np.float32))
    sa = (2.0 ** rng.integers(-3, 4, (m, 4))).astype(np.float32)
    sb = (2.0 ** rng.integers(-3, 4, (3, 4))).astype(np.float32)
    got = run(cuda, a, sa, b, sb, "f32")
    np.testing.assert_array_equal(got, exact(a, sa, b, sb).astype(np.float32))


def test_k_zero_and_ragged_edges_leave_neighbours_alone(cuda) -> None:
    torch = cuda
    c = torch.full((40, 48), 5.0, device="cuda", dtype=torch.bfloat16)
    a_codes, sa, b_codes, sb = o.config_gemm_fp8(33, 24, 144, seed=5)
    calls.gemm_fp8_blockscaled_tn(device(torch, a_codes, torch.float8_e4m3fn), device(torch, sa),
                                  device(torch, b_codes, torch.float8_e4m3fn), device(torch, sb), c[:33, :24])
    torch.cuda.synchronize()
    assert bool((c[33:] == 5).all()) and bool((c[:, 24:] == 5).all())
    want = o.bf16_values(o.gemm_fp8_blockscaled(a_codes, sa, b_codes, sb))
    assert o.rel_frobenius(c[:33, :24].float().cpu().numpy(), want) < 1e-2


def test_config_three_as_configured(cuda) -> None:
    """The benchmark configuration itself: M = 8192, N = 28672, K = 8192 drawn with `np.random.default_rng(2)` (A, then
    B), 1x128 / 128x128 absmax scales. 32 x 112 CTA-pair tiles over 64 K blocks is what the persistent scheduler and
    the scale ring are built for and what small cases never reach. Sampled rows (first and last row of the first, middle
    and last 256-row tiles, and tile-boundary neighbours) in the first, a middle and the last column tiles against the
    oracle; the whole matrix through linearity, (sum_kb sa sb A8 B8^T) 1 = sum_kb sa (A8 (sb B8)^T 1)."""
    torch = cuda
    m, n, k = 8192, 28672, 8192
    a_codes, sa, b_codes, sb = o.config_gemm_fp8(m, n, k, seed=2)
    fp8 = torch.float8_e4m3fn
    a, b = torch.from_numpy(a_codes).cuda().view(fp8), torch.from_numpy(b_codes).cuda().view(fp8)
    dsa, dsb = torch.from_numpy(sa).cuda(), torch.from_numpy(sb).cuda()
    c = torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16)
    calls.gemm_fp8_blockscaled_tn(a, dsa, b, dsb, c)
    torch.cuda.synchronize()
    rows = [0, 1, 127, 128, 255, 256, 257, 2047, 2048, 4095, 4096, 4351, 6143, 6144, 7935, 7936, 8063, 8191]
    bands = [(0, 256), (256, 512), (14208, 14464), (n - 512, n - 256), (n - 256, n)]  # whole 256-column tiles
    assert bool(torch.isfinite(c.float()).all())
    for lo, hi in bands:
        sub_b, sub_sb = b_codes[lo:hi], sb[lo // 128:hi // 128]
        want = o.bf16_values(o.gemm_fp8_blockscaled(a_codes[rows], sa[rows], sub_b, sub_sb, threads=6))
        got = c[rows, lo:hi].float().cpu().numpy()
        assert o.rel_frobenius(got, want) < 1e-2, (lo, hi)
        assert o.rel_frobenius(got, exact(a_codes[rows], sa[rows], sub_b, sub_sb)) < 3e-2, (lo, hi)  # the benchmark's tolerance
    # linearity over the whole matrix, in float64 on the device
    ones = torch.ones((n, 1), device="cuda", dtype=torch.float64)
    weights = torch.zeros((k,), device="cuda", dtype=torch.float64)
    for lo in range(0, n, 4096):  # sum_n sb[n // 128, k // 128] * B8[n, k], in slabs to bound the f64 temporaries
        hi = min(n, lo + 4096)
        scales = dsb[lo // 128:hi // 128].double().repeat_interleave(128, 0).repeat_interleave(128, 1)
        weights += (b[lo:hi].double() * scales).sum(0)
    rhs = (a.double() * dsa.double().repeat_interleave(128, 1)) @ weights[:, None]
    assert float((c.double() @ ones - rhs).norm() / rhs.norm()) < 5e-3
    del c
    c32 = torch.empty((m, n), device="cuda", dtype=torch.float32)
    calls.gemm_fp8_blockscaled_tn(a, dsa, b, dsb, c32)
    torch.cuda.synchronize()
    assert float((c32.double() @ ones - rhs).norm() / rhs.norm()) < 1e-5
    for lo, hi in bands:
        want32 = o.gemm_fp8_blockscaled(a_codes[rows], sa[rows], b_codes[lo:hi], sb[lo // 128:hi // 128], c_type=o.F32, threads=6)
        assert o.rel_frobenius(c32[rows, lo:hi].cpu().numpy(), want32) < 1e-5, (lo, hi)


def test_column_sharded_fp8_product_stores_into_every_destination(cuda) -> None:
    """The sharded entry point on one GPU: two "ranks" are two launches, each storing its column block into both
    destination buffers; both copies must equal the unsharded product bit for bit."""
    torch = cuda
    from krn_b200.runtime import native

    m, n, k, ranks = 384, 1024, 512, 2
    a_codes, sa, b_codes, sb = o.config_gemm_fp8(m, n, k, seed=41)
    fp8 = torch.float8_e4m3fn
    a, b = torch.from_numpy(a_codes).cuda().view(fp8), torch.from_numpy(b_codes).cuda().view(fp8)
    dsa, dsb = torch.from_numpy(sa).cuda(), torch.from_numpy(sb).cuda()
    whole = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
    calls.gemm_fp8_blockscaled_tn(a, dsa, b, dsb, whole)
    copies = [torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(ranks)]
    pointers = [int(c.data_ptr()) for c in copies]
    width = n // ranks
    for rank in range(ranks):
        rows = slice(rank * width, (rank + 1) * width)
        calls.gemm_fp8_blockscaled_tn_gather(a, dsa, b[rows], dsb[rank * width // 128:(rank + 1) * width // 128], pointers,
                                             rank, width, n, native.BF16)
        torch.cuda.synchronize()
        if rank == 0:
            assert all(bool(torch.isnan(c[:, width:].float()).all()) for c in copies)  # the other block is untouched
    for c in copies:
        assert torch.equal(c, whole)
    with pytest.raises(Exception, match="scale block"):
        calls.gemm_fp8_blockscaled_tn_gather(a, dsa, b[:192], dsb[:2], pointers, 0, 192, n, native.BF16)
