"""bf16 / f16 tile product on the GPU, called through the C ABI, against the CPU oracle."""

from __future__ import annotations

import numpy as np
import pytest

from oracle import oracle as o
from krn_b200.runtime import calls, native

pytestmark = pytest.mark.gpu

TORCH_OF = {"bf16": "bfloat16", "f16": "float16", "f32": "float32"}
ORACLE_OF = {"bf16": o.BF16, "f16": o.F16, "f32": o.F32}


def to_device(torch, words: np.ndarray, dtype: str):
    tensor = torch.from_numpy(words).cuda()
    return tensor if dtype == "f32" else tensor.view(getattr(torch, TORCH_OF[dtype]))


def to_words(torch, tensor, dtype: str) -> np.ndarray:
    return tensor.cpu().numpy() if dtype == "f32" else tensor.view(torch.uint16 if hasattr(torch, "uint16") else torch.int16).cpu().numpy().view(np.uint16)


def values(words: np.ndarray, dtype: str) -> np.ndarray:
    return words if dtype == "f32" else (words.view(np.float16).astype(np.float32) if dtype == "f16" else o.bf16_values(words))


def operands(m: int, n: int, k: int, dtype: str, seed: int, normal: bool = False):
    rng = np.random.default_rng(seed)
    draw = (lambda s: rng.standard_normal(s, np.float32)) if normal else (lambda s: rng.uniform(-1, 1, s).astype(np.float32))
    a, b = draw((m, k)), draw((n, k))
    if dtype == "f16":
        return a.astype(np.float16).view(np.uint16), b.astype(np.float16).view(np.uint16)
    return o.bf16_words(a), o.bf16_words(b)


def run(torch, aw, bw, dtype, output):
    m, n = aw.shape[0], bw.shape[0]
    a, b = to_device(torch, aw, dtype), to_device(torch, bw, dtype)
    c = torch.full((m, n), float("nan"), device="cuda", dtype=getattr(torch, TORCH_OF[output]))
    calls.gemm_tn(a, b, c)
    torch.cuda.synchronize()
    return to_words(torch, c, output)


def check(got_words, aw, bw, dtype, output, k):
    """Within the reference's reordered-accumulation bound of the exact product, and within one output rounding
    step of the oracle (the tensor cores add in a different order than the k-ordered fma chain)."""
    av, bv = values(aw, dtype), values(bw, dtype)
    exact = av.astype(np.float64) @ bv.astype(np.float64).T
    bound = o.forward_error_bound(av, np.ascontiguousarray(bv.T), k)
    got = values(got_words, output).astype(np.float64)
    want_words = o.gemm(aw, bw, ab_type=ORACLE_OF[dtype], c_type=ORACLE_OF[output], threads=8)
    want = values(want_words, output).astype(np.float64)
    if output != "f32":
        bound = bound + np.abs(want - exact) + np.spacing(np.abs(exact).astype(np.float16 if output == "f16" else np.float32)) * (1 if output == "f16" else 2**16)
    assert np.all(np.abs(got - exact) <= bound)
    assert o.rel_frobenius(got, want) < 1e-2
    return got, want


SHAPES = [(128, 256, 64), (256, 256, 128), (384, 512, 1024), (1024, 1024, 1024), (50, 40, 72), (130, 72, 104),
          (257, 136, 40), (64, 64, 64), (33, 24, 56), (130, 264, 40), (16, 8, 8), (1, 8, 8), (129, 8, 4096)]


@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("output", ["same", "f32"])
def test_product_against_oracle(cuda, m, n, k, dtype, output) -> None:
    """Uniform[-1,1) operands from seed 0 as the reference's card test draws them
    (tests/compiler/test_tensor_cores.py:314-392); ragged shapes keep K and N multiples of 8 (16-byte rows)."""
    output = dtype if output == "same" else output
    aw, bw = operands(m, n, k, dtype, seed=0)
    check(run(cuda, aw, bw, dtype, output), aw, bw, dtype, output, k)


def test_exactly_representable_products_are_bit_identical_to_the_oracle(cuda) -> None:
    """Small-integer operands make every partial sum exact, so any accumulation order gives the oracle's bits."""
    rng = np.random.default_rng(9)
    m, n, k = 300, 520, 328
    a = rng.integers(-4, 5, (m, k)).astype(np.float32)
    b = rng.integers(-4, 5, (n, k)).astype(np.float32)
    aw, bw = o.bf16_words(a), o.bf16_words(b)
    for output in ("bf16", "f32"):
        got = run(cuda, aw, bw, "bf16", output)
        want = o.gemm(aw, bw, ab_type=o.BF16, c_type=ORACLE_OF[output], threads=8)
        np.testing.assert_array_equal(got, want)


def test_k_zero_stores_zeros_and_out_of_range_is_untouched(cuda) -> None:
    torch = cuda
    c = torch.full((20, 32), 3.0, device="cuda", dtype=torch.bfloat16)
    a = torch.zeros((16, 0), device="cuda", dtype=torch.bfloat16)
    b = torch.zeros((8, 0), device="cuda", dtype=torch.bfloat16)
    calls.gemm_tn(a, b, c[:16, :8])
    torch.cuda.synchronize()
    assert not c[:16, :8].any() and bool((c[16:] == 3).all()) and bool((c[:, 8:] == 3).all())
    # a ragged tile must not write past the view either
    aw, bw = operands(50, 40, 72, "bf16", seed=4)
    big = torch.full((64, 64), 3.0, device="cuda", dtype=torch.bfloat16)
    calls.gemm_tn(to_device(torch, aw, "bf16"), to_device(torch, bw, "bf16"), big[:50, :40])
    torch.cuda.synchronize()
    assert bool((big[50:] == 3).all()) and bool((big[:, 40:] == 3).all())


def test_all_ones_known_answer(cuda) -> None:
    """ones(32,16) @ ones(32,16)^T = 16 (tests/compiler/test_tensor_cores.py:404-437)."""
    torch = cuda
    a = torch.ones((32, 16), device="cuda", dtype=torch.float16)
    c = torch.zeros((32, 32), device="cuda", dtype=torch.float32)
    calls.gemm_tn(a, a.clone(), c)
    torch.cuda.synchronize()
    assert bool((c == 16).all())


@pytest.mark.parametrize("m,n,k", [(50, 38, 70), (130, 70, 100), (257, 129, 33), (33, 17, 56), (130, 257, 33), (7, 3, 5)])
@pytest.mark.parametrize("dtype,output", [("bf16", "bf16"), ("f16", "f32"), ("f16", "f16")])
def test_shapes_tma_cannot_describe_match_the_oracle_bit_for_bit(cuda, m, n, k, dtype, output) -> None:
    """The reference's ragged card shapes (tests/compiler/test_tensor_cores.py:314-324) have row pitches that are
    not multiples of 16 bytes; the plain tiled kernel runs the oracle's own k-ordered fma chain, so the bits agree."""
    aw, bw = operands(m, n, k, dtype, seed=0)
    got = run(cuda, aw, bw, dtype, output)
    want = o.gemm(aw, bw, ab_type=ORACLE_OF[dtype], c_type=ORACLE_OF[output])
    np.testing.assert_array_equal(got, want)


def run_nn(torch, aw, bw_kn, dtype, output):
    """`a @ b` with b stored (K, N)."""
    m, n = aw.shape[0], bw_kn.shape[1]
    a, b = to_device(torch, aw, dtype), to_device(torch, np.ascontiguousarray(bw_kn), dtype)
    c = torch.full((m, n), float("nan"), device="cuda", dtype=getattr(torch, TORCH_OF[output]))
    calls.gemm_nn(a, b, c)
    torch.cuda.synchronize()
    return to_words(torch, c, output)


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (384, 512, 1024), (1024, 1024, 1024), (50, 40, 72), (130, 72, 104),
                                   (257, 136, 40), (130, 264, 40), (1, 8, 8), (129, 8, 4096), (300, 520, 328)])
@pytest.mark.parametrize("dtype,output", [("bf16", "bf16"), ("f16", "f32")])
def test_row_major_right_operand_against_oracle(cuda, m, n, k, dtype, output) -> None:
    """`a[rows, ks] @ b[ks, cols]`, the form of examples/04_libraries/01_gemm_tiles.py:35-40: the same numbers as
    the transposed form on the transposed matrix."""
    aw, bw = operands(m, n, k, dtype, seed=1)
    got = run_nn(cuda, aw, bw.T, dtype, output)
    check(got, aw, bw, dtype, output, k)
    # both layouts drive the tensor cores with the same operand values in the same order
    np.testing.assert_array_equal(got, run(cuda, aw, bw, dtype, output))


@pytest.mark.parametrize("m,n,k", [(50, 38, 70), (130, 257, 33), (7, 3, 5)])
def test_row_major_right_operand_unaligned_is_bit_identical_to_the_oracle(cuda, m, n, k) -> None:
    aw, bw = operands(m, n, k, "bf16", seed=2)
    got = run_nn(cuda, aw, bw.T, "bf16", "bf16")
    np.testing.assert_array_equal(got, o.gemm(aw, bw, ab_type=o.BF16, c_type=o.BF16))


def test_row_major_right_operand_exact_and_ragged_views(cuda) -> None:
    torch = cuda
    rng = np.random.default_rng(11)
    m, n, k = 300, 520, 328
    a = rng.integers(-4, 5, (m, k)).astype(np.float32)
    b = rng.integers(-4, 5, (n, k)).astype(np.float32)
    aw, bw = o.bf16_words(a), o.bf16_words(b)
    want = o.gemm(aw, bw, ab_type=o.BF16, c_type=o.F32, threads=8)
    np.testing.assert_array_equal(run_nn(torch, aw, bw.T, "bf16", "f32"), want)
    # b as a column window of a wider (K, N') matrix: the pitch is not the row length
    wide = torch.zeros((k, n + 64), device="cuda", dtype=torch.bfloat16)
    wide[:, 8:8 + n] = to_device(torch, np.ascontiguousarray(bw.T), "bf16")
    big = torch.full((m + 8, n + 8), 3.0, device="cuda", dtype=torch.float32)
    calls.gemm_nn(to_device(torch, aw, "bf16"), wide[:, 8:8 + n], big[:m, :n])
    torch.cuda.synchronize()
    np.testing.assert_array_equal(big[:m, :n].cpu().numpy(), want)
    assert bool((big[m:] == 3).all()) and bool((big[:, n:] == 3).all())


def test_refusals_are_raised_before_launch(cuda) -> None:
    torch = cuda
    b = torch.zeros((8, 12), device="cuda", dtype=torch.bfloat16)
    c = torch.zeros((16, 8), device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="compose"):
        calls.gemm_tn(torch.zeros((16, 16), device="cuda", dtype=torch.bfloat16), b, c)
    with pytest.raises(TypeError, match="same element type"):
        calls.gemm_tn(torch.zeros((16, 12), device="cuda", dtype=torch.float16), b, c)


def test_config_two_statistics_at_full_size(cuda) -> None:
    """bf16 8192^3 from seed 1 (N(0,1)): sampled rows against the oracle, the whole matrix through linearity
    (A @ B^T @ 1 = A @ (B^T @ 1)) and against the relative Frobenius tolerance 1e-2."""
    torch = cuda
    size = 8192
    a_words, b_words = o.config_gemm_bf16(size, size, size, seed=1)  # np.random.default_rng(1): A, then B
    a, b = to_device(torch, a_words, "bf16"), to_device(torch, b_words, "bf16")
    c = torch.empty((size, size), device="cuda", dtype=torch.bfloat16)
    calls.gemm_tn(a, b, c)
    torch.cuda.synchronize()
    rows = [0, 1, 127, 128, 4095, 4096, 8064, 8191]
    want = o.bf16_values(o.gemm(a_words[rows], b_words, ab_type=o.BF16, c_type=o.BF16, threads=8))
    got = o.bf16_values(c[rows].view(torch.int16).cpu().numpy().view(np.uint16))
    assert o.rel_frobenius(got, want) < 1e-2
    assert np.mean(got.view(np.uint32) == want.view(np.uint32)) > 0.95  # same bf16 word almost everywhere
    # linearity over the whole matrix: (A @ B^T) @ 1 = A @ (B^T @ 1). With bf16 output every element carries an
    # independent 2^-9 relative rounding, which leaves about 2e-3 on a row sum; the f32 output carries only
    # accumulation error.
    ones = torch.ones((size, 1), device="cuda", dtype=torch.float64)
    rhs = a.double() @ (b.double().t() @ ones)
    assert float((c.double() @ ones - rhs).norm() / rhs.norm()) < 5e-3
    c32 = torch.empty((size, size), device="cuda", dtype=torch.float32)
    calls.gemm_tn(a, b, c32)
    torch.cuda.synchronize()
    assert float((c32.double() @ ones - rhs).norm() / rhs.norm()) < 1e-5


def test_column_sharded_product_stores_into_every_destination(cuda) -> None:
    """The sharded entry point on one GPU: two "ranks" are two launches on the same device, each storing its column
    block into both destination buffers (which stand in for the ranks' copies of C). Both copies must equal the
    unsharded product bit for bit, and nothing outside a block's columns may be touched by the other launch."""
    torch = cuda
    m, n, k, ranks = 300, 512, 328, 2
    rng = np.random.default_rng(17)
    aw = o.bf16_words(rng.integers(-4, 5, (m, k)).astype(np.float32))
    bw = o.bf16_words(rng.integers(-4, 5, (n, k)).astype(np.float32))
    a, b = to_device(torch, aw, "bf16"), to_device(torch, bw, "bf16")
    copies = [torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(ranks)]
    pointers = [int(c.data_ptr()) for c in copies]
    width = n // ranks
    for rank in range(ranks):
        calls.gemm_tn_gather(a, b[rank * width:(rank + 1) * width], pointers, rank, m, width, n, native.BF16)
        torch.cuda.synchronize()
        other = slice((1 - rank) * width, (2 - rank) * width)
        if rank == 0:
            assert all(bool(torch.isnan(c[:, other].float()).all()) for c in copies)  # the other block is untouched
    want = o.gemm(aw, bw, ab_type=o.BF16, c_type=o.BF16, threads=8)
    for c in copies:
        np.testing.assert_array_equal(to_words(torch, c, "bf16"), want)
    with pytest.raises(Exception, match="whole number of 128-byte store"):
        calls.gemm_tn_gather(a, b[:200], pointers, 0, m, 200, n, native.BF16)
