"""The CPU oracle against the reference's own known answers and against outputs of the reference's own
arithmetic (tests/golden/*.npz, made by tests/golden/make_golden.py). CPU only."""

from __future__ import annotations

import math
from pathlib import Path

import numpy as np
import pytest

from oracle import oracle as o

GOLDEN = Path(__file__).resolve().parent / "golden"
TYPES = {"f32": o.F32, "f16": o.F16, "bf16": o.BF16}


def words(values: np.ndarray, dtype: str) -> np.ndarray:
    if dtype == "f32":
        return values.astype(np.float32)
    if dtype == "f16":
        return values.astype(np.float16).view(np.uint16)
    return o.bf16_words(values)


def values(words_: np.ndarray, dtype: str) -> np.ndarray:
    if dtype == "f32":
        return words_
    if dtype == "f16":
        return words_.view(np.float16).astype(np.float32)
    return o.bf16_values(words_)


# ---- bit-for-bit against the reference emulator's `accumulate` / `_bfloat16` ---------------------------------


@pytest.mark.parametrize("shape", [(50, 38, 70), (16, 8, 8), (33, 17, 56), (64, 64, 64), (130, 70, 100)])
@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("tile", [None, (32, 32, 16), (16, 8, 8), (128, 256, 32)])
def test_product_matches_reference_emulator_bits(shape, dtype, tile) -> None:
    golden = np.load(GOLDEN / "gemm_emulator.npz")
    m, n, k = shape
    key = f"{dtype}_{m}x{n}x{k}"
    a, b = words(golden[f"{key}_a"], dtype), words(golden[f"{key}_b"], dtype)
    c = o.gemm(a, b, ab_type=TYPES[dtype], c_type=o.F32, tile=tile)
    np.testing.assert_array_equal(c.view(np.uint32), golden[f"{key}_c"].view(np.uint32))
    c16 = o.gemm(a, b, ab_type=TYPES[dtype], c_type=o.BF16, tile=tile)
    np.testing.assert_array_equal(o.bf16_values(c16).view(np.uint32), golden[f"{key}_c_bf16"].view(np.uint32))


def test_accumulator_is_reread_between_k_tiles() -> None:
    golden = np.load(GOLDEN / "gemm_emulator.npz")
    a, b = golden["chained_a"], golden["chained_b"]
    for tile in (None, (8, 8, 24), (16, 16, 8)):
        c = o.gemm(a, b, ab_type=o.F32, c_type=o.F32, b_kn=True, tile=tile)
        np.testing.assert_array_equal(c.view(np.uint32), golden["chained_c"].view(np.uint32))


def test_bf16_rounding_matches_reference_emulator() -> None:
    golden = np.load(GOLDEN / "gemm_emulator.npz")
    got = o.bf16_values(o.bf16_words(golden["bf16_in"]))
    np.testing.assert_array_equal(got.view(np.uint32), golden["bf16_out"].view(np.uint32))


# ---- known answers of tests/compiler/test_tensor_cores.py ---------------------------------------------------------


def test_all_ones_known_answers() -> None:
    """ones(32,16) @ ones(16,32) = 16 everywhere; the reference's epilogues then give 33, -496 and 256
    (tests/compiler/test_tensor_cores.py:404-466)."""
    a = np.ones((32, 16), np.float16).view(np.uint16)
    b_kn = np.ones((16, 32), np.float16).view(np.uint16)
    acc = o.gemm(a, b_kn, ab_type=o.F16, c_type=o.F32, b_kn=True, tile=(32, 32, 16))
    assert np.all(acc == 16)
    assert np.all(acc * 2.0 + 1.0 == 33)
    assert np.all(acc - acc.sum(axis=1, keepdims=True) == -496)
    other = o.gemm(acc[:, :16].astype(np.float16).view(np.uint16), np.ones((16, 16), np.float16).view(np.uint16),
                   ab_type=o.F16, c_type=o.F32, b_kn=True, tile=(32, 16, 16))
    assert np.all(other == 256)


def agree(actual: np.ndarray, a: np.ndarray, b_kn: np.ndarray, k: int, output: str) -> None:
    """The reference's acceptance bound (tests/compiler/test_tensor_cores.py:395-401)."""
    reference = a.astype(np.float64) @ b_kn.astype(np.float64)
    bound = o.forward_error_bound(a, b_kn, k)
    if output == "f16":
        bound = bound + np.abs(reference.astype(np.float16).astype(np.float64) - reference)
        bound = bound + np.spacing(np.abs(reference).astype(np.float16))
    assert np.all(np.abs(actual.astype(np.float64) - reference) <= bound)


CARD_SHAPES = [(50, 38, 70, 32, 32, 16), (130, 70, 100, 32, 32, 16), (16, 8, 8, 16, 8, 8), (257, 129, 33, 32, 32, 16),
               (64, 64, 64, 32, 32, 16), (33, 17, 56, 32, 32, 24), (130, 257, 33, 128, 256, 32), (16, 8, 0, 16, 8, 8)]


@pytest.mark.parametrize("m,n,k,bm,bn,bk", CARD_SHAPES)
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("output", ["f16", "f32"])
def test_card_shapes_within_reference_bound(m, n, k, bm, bn, bk, dtype, output) -> None:
    """Seed 0, uniform[-1,1), the eight shapes incl. ragged and K = 0 (tests/compiler/test_tensor_cores.py:314-392)."""
    rng = np.random.default_rng(0)
    a, b = (rng.uniform(-1, 1, shape).astype(np.float32) for shape in ((m, k), (k, n)))
    aw, bw = words(a, dtype), words(b, dtype)
    av, bv = values(aw, dtype), values(bw, dtype)
    c = o.gemm(aw, bw, ab_type=TYPES[dtype], c_type=TYPES[output], b_kn=True, tile=(bm, bn, bk))
    agree(values(c, output), av, bv, k, output)
    if k == 0:
        assert not c.any()


@pytest.mark.parametrize("m,n,k,bm,bn,bk", CARD_SHAPES[:4])
def test_oracles_seed_one(m, n, k, bm, bn, bk) -> None:
    """tests/compiler/test_tensor_cores.py:499-508: f16 operands from seed 1; both loop structures agree."""
    rng = np.random.default_rng(1)
    a, b = (rng.uniform(-1, 1, shape).astype(np.float16) for shape in ((m, k), (k, n)))
    tiled = o.gemm(a.view(np.uint16), b.view(np.uint16), ab_type=o.F16, c_type=o.F32, b_kn=True, tile=(bm, bn, bk))
    fast = o.gemm(a.view(np.uint16), b.view(np.uint16), ab_type=o.F16, c_type=o.F32, b_kn=True)
    np.testing.assert_array_equal(tiled, fast)
    agree(tiled, a, b, k, "f32")


def test_transposed_rhs_product() -> None:
    """`a @ b.transpose()` reads b as (N, K); rows past the edge are not stored (tests/frontend/test_tile_ops.py:90-98)."""
    rng = np.random.default_rng(3)
    a, b = rng.standard_normal((13, 9), np.float32), rng.standard_normal((7, 9), np.float32)
    c = o.gemm(a, b, ab_type=o.F32, c_type=o.F32, tile=(16, 8, 4))
    assert c.shape == (13, 7)
    np.testing.assert_allclose(c, a @ b.T, rtol=1e-5, atol=1e-5)


def test_config_one_f32_256_cubed() -> None:
    """The benchmark's first config: f32 256^3 A @ B^T from seed 0 on the CPU C path."""
    a, b = o.config_gemm_f32()
    c = o.gemm(a, b, ab_type=o.F32, c_type=o.F32, tile=(128, 128, 32))
    np.testing.assert_array_equal(c, o.gemm(a, b, ab_type=o.F32, c_type=o.F32))
    agree(c, a, np.ascontiguousarray(b.T), 256, "f32")
    assert o.rel_frobenius(c, a.astype(np.float64) @ b.T.astype(np.float64)) < 1e-6


# ---- e4m3fn ------------------------------------------------------------------------------------------------------------


def fp8_table(exponent: int, mantissa: int) -> np.ndarray:
    """The independent 256-entry decode table of tests/compiler/test_tensor_cores.py:200-216."""
    result = np.zeros(256, np.float64)
    bias = 2 ** (exponent - 1) - 1
    for code in range(256):
        fraction, power = code & (2**mantissa - 1), (code >> mantissa) & (2**exponent - 1)
        value = (fraction / 2**mantissa * 2.0 ** (1 - bias)) if power == 0 else (1 + fraction / 2**mantissa) * 2.0 ** (power - bias)
        if exponent == 4 and code & 0x7F == 0x7F:
            value = np.nan
        elif exponent == 5 and ((code >> mantissa) & 31) == 31:
            value = np.nan if code & 3 else np.inf
        result[code] = -value if code & 128 else value
    return result


def test_e4m3_decode_tables() -> None:
    golden = np.load(GOLDEN / "e4m3.npz")
    mine = o.e4m3_decode(np.arange(256, dtype=np.uint8))
    np.testing.assert_array_equal(mine.astype(np.float64), fp8_table(4, 3))
    np.testing.assert_array_equal(mine.astype(np.float64), golden["table"])
    np.testing.assert_array_equal(mine, golden["decode"])
    assert float(golden["max"]) == 448.0 == np.nanmax(mine)


def test_e4m3_encode_matches_reference_encode() -> None:
    golden = np.load(GOLDEN / "e4m3.npz")
    np.testing.assert_array_equal(o.e4m3_encode(golden["values"]), golden["codes"])


@pytest.mark.parametrize("a_kind,b_kind", [("e4m3", "e4m3"), ("e4m3", "e5m2"), ("e5m2", "e4m3"), ("e5m2", "e5m2")])
@pytest.mark.parametrize("m,n,k", [(50, 38, 70), (19, 7, 33), (65, 19, 0)])
def test_fp8_codes_product_within_bound(m, n, k, a_kind, b_kind) -> None:
    """Random codes in [0,112)|sign from seed 81, unscaled product of every e4m3 / e5m2 pairing
    (tests/compiler/test_tensor_cores.py:146,219-239), decoded with the test's own independent table."""
    rng = np.random.default_rng(81)
    raw = [rng.integers(0, 112, shape, dtype=np.uint8) | (rng.integers(0, 2, shape, dtype=np.uint8) << 7)
           for shape in ((m, k), (k, n))]
    tables = {"e4m3": fp8_table(4, 3), "e5m2": fp8_table(5, 2)}
    kinds = {"e4m3": o.E4M3, "e5m2": o.E5M2}
    decoded = [tables[a_kind][raw[0]], tables[b_kind][raw[1]]]
    c = o.gemm(raw[0], raw[1], ab_type=kinds[a_kind], b_type=kinds[b_kind], c_type=o.F32, b_kn=True, tile=(32, 32, 32))
    agree(c, decoded[0], decoded[1], k, "f32")


# ---- flash attention --------------------------------------------------------------------------------------------------


@pytest.mark.parametrize("seq", [1, 7, 16, 17, 33, 40])
@pytest.mark.parametrize("heads,d", [(1, 8), (2, 16)])
@pytest.mark.parametrize("causal", [False, True])
def test_flash_attention_against_float64(seq, heads, d, causal) -> None:
    """f16, ragged seq in [1, 40], atol 3e-3 (tests/frontend/test_tile_ops.py:130-154)."""
    rng = np.random.default_rng(seq * 31 + heads)
    q, k, v = (rng.standard_normal((1, heads, seq, d)).astype(np.float16) for _ in range(3))
    out = o.flash_attention(*(x.view(np.uint16) for x in (q, k, v)), dtype=o.F16, scale=math.log2(math.e) / math.sqrt(d),
                            causal=causal, bq=16, bk=16)
    np.testing.assert_allclose(out.view(np.float16).astype(np.float64), o.attention_f64(q, k, v, causal), atol=3e-3)


@pytest.mark.parametrize("d,causal", [(64, False), (128, True)])
def test_flash_attention_example_case(d, causal) -> None:
    """The example's own check: 2 heads, seq 200 (ragged against 16-row tiles), atol 2e-3
    (examples/04_libraries/08_flash_attention.py:72-86)."""
    rng = np.random.default_rng(0)
    q, k, v = (rng.standard_normal((1, 2, 200, d)).astype(np.float16) for _ in range(3))
    out = o.flash_attention(*(x.view(np.uint16) for x in (q, k, v)), dtype=o.F16, scale=math.log2(math.e) / math.sqrt(d),
                            causal=causal)
    np.testing.assert_allclose(out.view(np.float16).astype(np.float64), o.attention_f64(q, k, v, causal), atol=2e-3)


def test_flash_attention_tiling_changes_little_and_gqa_maps_heads() -> None:
    rng = np.random.default_rng(5)
    q = o.bf16_words(rng.standard_normal((2, 4, 50, 16), np.float32))
    k, v = (o.bf16_words(rng.standard_normal((2, 2, 50, 16), np.float32)) for _ in range(2))
    scale = math.log2(math.e) / 4.0
    small = o.flash_attention(q, k, v, dtype=o.BF16, scale=scale, causal=True, bq=16, bk=16)
    large = o.flash_attention(q, k, v, dtype=o.BF16, scale=scale, causal=True, bq=64, bk=32, threads=4)
    want = o.attention_f64(o.bf16_values(q), o.bf16_values(k), o.bf16_values(v), True)
    for got in (small, large):
        assert o.rel_frobenius(o.bf16_values(got), want) < 1e-2


# ---- our own definitions (parity unpinned): internal consistency only ------------------------------------------


def test_blockscaled_fp8_definition_is_consistent() -> None:
    a_codes, sa, b_codes, sb = o.config_gemm_fp8(96, 256, 384, seed=2)
    c = o.bf16_values(o.gemm_fp8_blockscaled(a_codes, sa, b_codes, sb))
    a = o.e4m3_decode(a_codes).astype(np.float64) * np.repeat(sa, 128, axis=1)[:, :384]
    b = o.e4m3_decode(b_codes).astype(np.float64) * np.repeat(np.repeat(sb, 128, axis=0), 128, axis=1)[:256, :384]
    assert o.rel_frobenius(c, a @ b.T) < 5e-3
    rng = np.random.default_rng(2)
    exact_a, exact_b = rng.standard_normal((96, 384), np.float32), rng.standard_normal((256, 384), np.float32)
    assert o.rel_frobenius(c, exact_a.astype(np.float64) @ exact_b.T.astype(np.float64)) < 6e-2  # quantisation noise


def test_paged_decode_definition_is_consistent() -> None:
    q, kp, vp, table, lens, ks, vs = o.config_decode(batch=3, q_heads=4, kv_heads=2, d=32, low=5, high=200, page_size=16)
    scale_log2 = math.log2(math.e) / math.sqrt(32)
    out = o.bf16_values(o.decode_fp8_paged(q, kp, vp, table, lens, ks, vs, scale_log2=scale_log2))
    for b in range(3):
        n = int(lens[b])
        pages = table[b, : -(-n // 16)]
        kk = o.e4m3_decode(kp[pages]).reshape(-1, 2, 32)[:n].astype(np.float64) * ks[b][None, :, None]
        vv = o.e4m3_decode(vp[pages]).reshape(-1, 2, 32)[:n].astype(np.float64) * vs[b][None, :, None]
        for h in range(4):
            s = kk[:, h // 2] @ o.bf16_values(q[b, h]).astype(np.float64) / math.sqrt(32)
            p = np.exp(s - s.max())
            want = (p / p.sum()) @ vv[:, h // 2]
            np.testing.assert_allclose(out[b, h], want, atol=2e-2, rtol=2e-2)


def test_matmul_epilogue_restatement_matches_the_reference_element_functions() -> None:
    """f32 end to end, against numpy written from the emulator's definitions (src/krn/emulator/emulate.py:376-385:
    relu `maximum(x, 0)`, silu `x / (1 + exp(-x))`, gelu `0.5 x (1 + erf(x * 0.7071067811865476))`)."""
    import math

    rng = np.random.default_rng(12)
    a, b = rng.uniform(-1, 1, (9, 40)).astype(np.float32), rng.uniform(-1, 1, (40, 11)).astype(np.float32)
    bias = rng.uniform(-2, 2, 11).astype(np.float32)
    x = (a.astype(np.float64) @ b.astype(np.float64))
    erf = np.vectorize(math.erf)
    for flags, fn in ((0, lambda v: v), (o.EPILOGUE_BIAS, lambda v: v + bias), (o.EPILOGUE_RELU, lambda v: np.maximum(v, 0)),
                      (o.EPILOGUE_BIAS | o.EPILOGUE_GELU, lambda v: 0.5 * (v + bias) * (1 + erf((v + bias) * 0.7071067811865476))),
                      (o.EPILOGUE_SILU, lambda v: v / (1 + np.exp(-v)))):
        got = o.matmul_epilogue(a, b, bias, ab_type=o.F32, c_type=o.F32, flags=flags)
        np.testing.assert_allclose(got, fn(x), rtol=2e-5, atol=2e-6)
    # a bf16 result is the f32 value rounded once
    got = o.matmul_epilogue(a, b, o.bf16_words(bias), ab_type=o.F32, c_type=o.BF16, flags=o.EPILOGUE_BIAS)
    want = o.bf16_words((o.gemm(a, b, ab_type=o.F32, c_type=o.F32, b_kn=True) + o.bf16_values(o.bf16_words(bias))).astype(np.float32))
    np.testing.assert_array_equal(got, want)
