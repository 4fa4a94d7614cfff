"""Unscaled fp8 pair products on the GPU, through the C ABI and through `@kernel`, against the CPU oracle.

PINNED: this is the one FP8 product the reference itself tests — random codes in [0, 112) | sign from seed 81,
every e4m3 / e5m2 pairing, b stored (K, N), result under the bound 8 * 2^-24 * (k + 8) * |A| |B|
(tests/compiler/test_tensor_cores.py:219-239,395-401). The same draw and bound are used here; the oracle side is
`o.gemm(..., ab_type=, b_type=)`, itself pinned to that test in tests/test_oracle_pins.py."""

from __future__ import annotations

import numpy as np
import pytest

import krn_b200 as krn
from krn_b200 import formats
from krn_b200.runtime import calls
from oracle import oracle as o
from tests.kernels import tile_kernels as K

pytestmark = pytest.mark.gpu

TABLE = {o.E4M3: np.array(formats.E4M3FN.table), o.E5M2: np.array(formats.E5M2.table)}
PAIRS = [(o.E4M3, o.E4M3), (o.E4M3, o.E5M2), (o.E5M2, o.E4M3), (o.E5M2, o.E5M2)]


def draw(m: int, n: int, k: int, seed: int = 81) -> list[np.ndarray]:
    """The reference's code draw: a (m, k) then b (k, n), magnitude codes below 112 so no NaN / inf code occurs."""
    rng = np.random.default_rng(seed)
    return [rng.integers(0, 112, shape, dtype=np.uint8) | (rng.integers(0, 2, shape, dtype=np.uint8) << 7)
            for shape in ((m, k), (k, n))]


def on_device(torch, codes: np.ndarray, kind: int):
    return torch.from_numpy(np.ascontiguousarray(codes)).cuda().view(torch.float8_e4m3fn if kind == o.E4M3 else torch.float8_e5m2)


def within_bound(actual: np.ndarray, a: np.ndarray, b_kn: np.ndarray, k: int) -> bool:
    exact = a @ b_kn
    return bool(np.all(np.abs(actual.astype(np.float64) - exact) <= o.forward_error_bound(a, b_kn, k)))


@pytest.mark.parametrize("a_kind,b_kind", PAIRS)
@pytest.mark.parametrize("m,n,k", [(50, 38, 70), (19, 7, 33), (65, 19, 0)])
def test_reference_fp8_card(cuda, a_kind, b_kind, m, n, k) -> None:
    """The reference's three shapes: ragged and unaligned (they take the plain fma kernel, which follows the oracle's
    k-ordered chain exactly) and K = 0."""
    torch = cuda
    a_codes, b_codes = draw(m, n, k)
    c = torch.full((m, n), float("nan"), device="cuda", dtype=torch.float32)
    calls.gemm_fp8(on_device(torch, a_codes, a_kind), on_device(torch, b_codes, b_kind), c, b_kn=True)
    torch.cuda.synchronize()
    got = c.cpu().numpy()
    assert within_bound(got, TABLE[a_kind][a_codes], TABLE[b_kind][b_codes], k)
    want = o.gemm(a_codes, b_codes, ab_type=a_kind, b_type=b_kind, c_type=o.F32, b_kn=True)
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("a_kind,b_kind", PAIRS)
@pytest.mark.parametrize("m,n,k,b_kn", [(256, 512, 1024, True), (256, 512, 1024, False), (384, 272, 400, True),
                                        (130, 264, 144, False), (100, 128, 160, True), (1024, 1024, 2048, True)])
def test_tensor_core_path_on_the_reference_draw(cuda, a_kind, b_kind, m, n, k, b_kn) -> None:
    """The same kind of draw at shapes TMA can describe, so the tcgen05 kernel runs (CTA pairs and single CTAs, both
    layouts of b, ragged edges): the reference's bound, and agreement with the oracle's chain within it."""
    torch = cuda
    a_codes, b_codes = draw(m, n, k)
    b_stored = b_codes if b_kn else np.ascontiguousarray(b_codes.T)
    c = torch.full((m, n), float("nan"), device="cuda", dtype=torch.float32)
    calls.gemm_fp8(on_device(torch, a_codes, a_kind), on_device(torch, b_stored, b_kind), c, b_kn=b_kn)
    torch.cuda.synchronize()
    got = c.cpu().numpy()
    a, b = TABLE[a_kind][a_codes], TABLE[b_kind][b_codes]
    assert within_bound(got, a, b, k)
    want = o.gemm(a_codes, b_codes, ab_type=a_kind, b_type=b_kind, c_type=o.F32, b_kn=True, threads=8)
    assert o.rel_frobenius(got, want) < 1e-5


def test_small_integer_codes_are_bit_identical(cuda) -> None:
    """Codes of small integers make every partial sum exact, so the tensor-core result must equal the oracle bit for
    bit in every layout and output type."""
    torch = cuda
    rng = np.random.default_rng(7)
    m, n, k = 300, 520, 640
    a_codes = o.e4m3_encode(rng.integers(-4, 5, (m, k)).astype(np.float32))
    b_codes = o.e4m3_encode(rng.integers(-4, 5, (k, n)).astype(np.float32))
    want = o.gemm(a_codes, b_codes, ab_type=o.E4M3, c_type=o.F32, b_kn=True, threads=8)
    for b_kn in (True, False):
        b_stored = b_codes if b_kn else np.ascontiguousarray(b_codes.T)
        for dtype in (torch.float32, torch.bfloat16):
            c = torch.full((m, n), float("nan"), device="cuda", dtype=dtype)
            calls.gemm_fp8(on_device(torch, a_codes, o.E4M3), on_device(torch, b_stored, o.E4M3), c, b_kn=b_kn)
            torch.cuda.synchronize()
            expected = want if dtype == torch.float32 else o.bf16_values(o.bf16_words(want))
            np.testing.assert_array_equal(c.float().cpu().numpy(), expected)


def test_block_scaled_kernel_with_unit_scales_meets_the_reference_bound(cuda) -> None:
    """Ties the block-scaled tensor-core kernel to the reference's own FP8 pin: with scales of one it computes the
    unscaled product of the seed-81 draw, which must satisfy the reference's bound and agree with the oracle's
    unscaled e4m3 chain."""
    torch = cuda
    m, n, k = 256, 384, 512
    a_codes, b_codes = draw(m, n, k)
    b_nk = np.ascontiguousarray(b_codes.T)
    sa, sb = np.ones((m, k // 128), np.float32), np.ones((n // 128, k // 128), np.float32)
    c = torch.full((m, n), float("nan"), device="cuda", dtype=torch.float32)
    calls.gemm_fp8_blockscaled_tn(on_device(torch, a_codes, o.E4M3), torch.from_numpy(sa).cuda(),
                                  on_device(torch, b_nk, o.E4M3), torch.from_numpy(sb).cuda(), c)
    torch.cuda.synchronize()
    got = c.cpu().numpy()
    assert within_bound(got, TABLE[o.E4M3][a_codes], TABLE[o.E4M3][b_codes], k)
    want = o.gemm(a_codes, b_codes, ab_type=o.E4M3, c_type=o.F32, b_kn=True, threads=8)
    assert o.rel_frobenius(got, want) < 1e-5


def test_fp8_pairs_through_the_kernel_language(cuda) -> None:
    """`acc += a8[rows, ks] @ b8[ks, cols]` and `a8[rows, ks] @ b8[cols, ks].transpose()` as `@kernel` functions on the
    device (src/krn/compiler/capture.py:3185-3192): recognised, routed to the unscaled fp8 entry point, same results."""
    device = krn.host.Device.current()
    a_codes, b_codes = draw(50, 38, 70)
    a = device.to_device(a_codes, krn.f8e4m3fn)
    b = device.to_device(b_codes, krn.f8e5m2)
    c = device.empty(krn.f32, 50, 38)
    assert "krn_b200_gemm_fp8" in str(K.fp8_pair_kn.explain(a, b, c))
    K.fp8_pair_kn(a, b, c)
    device.default_stream.record().wait(60)
    want = o.gemm(a_codes, b_codes, ab_type=o.E4M3, b_type=o.E5M2, c_type=o.F32, b_kn=True)
    np.testing.assert_array_equal(c.to_host(), want)

    a_codes, b_codes = draw(256, 384, 512)
    a = device.to_device(a_codes, krn.f8e4m3fn)
    b = device.to_device(np.ascontiguousarray(b_codes.T), krn.f8e4m3fn)
    c = device.empty(krn.bf16, 256, 384)
    K.fp8_pair_nt(a, b, c)
    device.default_stream.record().wait(60)
    want = o.bf16_values(o.gemm(a_codes, b_codes, ab_type=o.E4M3, c_type=o.BF16, b_kn=True, threads=8))
    got = o.bf16_values(c.to_host().view(np.uint16))
    assert o.rel_frobenius(got, want) < 1e-2
