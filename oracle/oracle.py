"""ctypes front of `oracle/krn_oracle.c` plus the seeded synthetic inputs of the five benchmark configs.

TEST INFRASTRUCTURE: the product (`krn_b200`) never imports this module.

The library is rebuilt with `make` whenever it is missing or was built on a machine with different CPU
features (`-march=native` code must not travel between hosts).
"""

from __future__ import annotations

import ctypes
import hashlib
import math
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
F32, F16, BF16, E4M3, E5M2 = 0, 1, 2, 3, 4

_LIB: ctypes.CDLL | None = None


def _cpu_stamp() -> str:
    try:
        flags = next(line for line in Path("/proc/cpuinfo").read_text().splitlines() if line.startswith("flags"))
    except (OSError, StopIteration):
        flags = "unknown"
    source = (HERE / "krn_oracle.c").read_bytes() + (HERE / "Makefile").read_bytes()
    return hashlib.sha256(flags.encode() + source).hexdigest()


def build(force: bool = False) -> Path:
    """Compile the oracle with gcc if it is missing or stale for this machine; returns the library path."""
    library, stamp = HERE / "libkrn_oracle.so", HERE / "libkrn_oracle.stamp"
    want = _cpu_stamp()
    if force or not library.exists() or not stamp.exists() or stamp.read_text() != want:
        subprocess.run(["make", "-B", "-C", str(HERE), "libkrn_oracle.so"], check=True, capture_output=True)
        stamp.write_text(want)
    return library


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        handle = ctypes.CDLL(str(build()))
        i64, i32, ptr, f32 = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_float
        handle.krn_oracle_gemm_blocks.argtypes = [i32, i32, i32, ptr, ptr, ptr, i64, i64, i64, i64, i64, i64, i32, i32, i32, i64, i64]
        handle.krn_oracle_gemm_fast.argtypes = [i32, i32, i32, ptr, ptr, ptr, i64, i64, i64, i64, i64, i64, i64, i64]
        handle.krn_oracle_gemm_fp8_blockscaled.argtypes = [i32, ptr, ptr, ptr, ptr, ptr, i64, i64, i64, i64, i64, i64, i64, i64, i64, i64]
        handle.krn_oracle_gemm_mxfp8.argtypes = [i32, ptr, ptr, ptr, ptr, ptr, i64, i64, i64, i64, i64, i64, i64, i64, i64, i64]
        handle.krn_oracle_gemm_mxfp4.argtypes = [i32, ptr, ptr, ptr, ptr, ptr, i64, i64, i64, i64, i64, i64, i64, i64, i64, i64]
        handle.krn_oracle_gemm_nvfp4.argtypes = [i32, ptr, ptr, ptr, ptr, ctypes.c_float, ptr, i64, i64, i64, i64, i64, i64, i64,
                                                 i64, i64, i64]
        handle.krn_oracle_flash_attention.argtypes = [i32, ptr, ptr, ptr, ptr, i64, i64, i64, i64, i64, i32, f32, i32, i32, i32, i64, i64]
        handle.krn_oracle_decode_fp8_paged.argtypes = [ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, i64, i64, i32, i32, i64, f32, i64, i64]
        handle.krn_oracle_e4m3_encode_array.argtypes = [ptr, ptr, i64]
        handle.krn_oracle_e4m3_decode_array.argtypes = [ptr, ptr, i64]
        handle.krn_oracle_bf16_round_array.argtypes = [ptr, ptr, i64]
        handle.krn_oracle_matmul_epilogue.argtypes = [i32, ptr, ptr, ptr, i64, i64, i32]
        for name in ("gemm_mxfp8", "gemm_nvfp4", "gemm_mxfp4", "matmul_epilogue", "gemm_blocks", "gemm_fast", "gemm_fp8_blockscaled", "flash_attention", "decode_fp8_paged",
                     "e4m3_encode_array", "e4m3_decode_array", "bf16_round_array"):
            getattr(handle, f"krn_oracle_{name}").restype = None
        _LIB = handle
    return _LIB


def _p(array: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(array.ctypes.data)


def _split(count: int, threads: int) -> list[tuple[int, int]]:
    threads = max(1, min(threads, count))
    edges = [count * i // threads for i in range(threads + 1)]
    return [(lo, hi) for lo, hi in zip(edges[:-1], edges[1:]) if hi > lo]


def _run(pieces: list[tuple[int, int]], call) -> None:
    if len(pieces) <= 1:
        for lo, hi in pieces:
            call(lo, hi)
        return
    with ThreadPoolExecutor(len(pieces)) as pool:  # ctypes releases the GIL during the C call
        list(pool.map(lambda piece: call(*piece), pieces))


# ---- storage formats -------------------------------------------------------------------------------------


def bf16_words(values: np.ndarray) -> np.ndarray:
    """float32 -> bf16 words, round to nearest even (tests/compiler/test_tensor_cores.py:305-307)."""
    flat = np.ascontiguousarray(values, np.float32)
    out = np.empty(flat.shape, np.uint16)
    lib().krn_oracle_bf16_round_array(_p(flat), _p(out), flat.size)
    return out


def bf16_values(words: np.ndarray) -> np.ndarray:
    """bf16 words -> the float32 values they stand for (tests/compiler/test_tensor_cores.py:310-311)."""
    return (np.ascontiguousarray(words, np.uint16).astype(np.uint32) << 16).view(np.float32)


def e4m3_encode(values: np.ndarray) -> np.ndarray:
    flat = np.ascontiguousarray(values, np.float32)
    out = np.empty(flat.shape, np.uint8)
    lib().krn_oracle_e4m3_encode_array(_p(flat), _p(out), flat.size)
    return out


def e4m3_decode(codes: np.ndarray) -> np.ndarray:
    flat = np.ascontiguousarray(codes, np.uint8)
    out = np.empty(flat.shape, np.float32)
    lib().krn_oracle_e4m3_decode_array(_p(flat), _p(out), flat.size)
    return out


_NUMPY = {F32: np.float32, F16: np.uint16, BF16: np.uint16, E4M3: np.uint8, E5M2: np.uint8}


# ---- tile product ---------------------------------------------------------------------------------------------


def gemm(a: np.ndarray, b: np.ndarray, *, ab_type: int, c_type: int, b_kn: bool = False, tile: tuple[int, int, int] | None = None,
         threads: int = 1, b_type: int | None = None) -> np.ndarray:
    """C = A @ B^T (b is (N, K)) or A @ B (b_kn, b is (K, N)): the k-ordered fma chain per element.

    With `tile=(bm, bn, bk)` the reference's loop structure runs (staged f32 tiles, block after block); without
    it the vectorised equivalent runs. Both give the same bits. Operands are storage words (uint16 for 16-bit
    types, uint8 for e4m3 / e5m2, float32 for f32); the result is returned in storage words of `c_type`. `b_type`
    names a different storage type for b (the reference multiplies mixed e4m3 / e5m2 pairs,
    tests/compiler/test_tensor_cores.py:146,219-239).
    """
    if b_type is not None:
        ab_type = ab_type | ((b_type + 1) << 8)
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    m, k = a.shape
    n = b.shape[1] if b_kn else b.shape[0]
    c = np.zeros((m, n), _NUMPY[c_type])
    if tile is not None:
        bm, bn, bk = tile
        rows = max(1, -(-m // bm))
        _run(_split(rows, threads), lambda lo, hi: lib().krn_oracle_gemm_blocks(
            ab_type, c_type, int(b_kn), _p(a), _p(b), _p(c), m, n, k, a.shape[1], b.shape[1], n, bm, bn, bk, lo, hi))
    else:
        _run(_split(m, threads), lambda lo, hi: lib().krn_oracle_gemm_fast(
            ab_type, c_type, int(b_kn), _p(a), _p(b), _p(c), m, n, k, a.shape[1], b.shape[1], n, lo, hi))
    return c


EPILOGUE_BIAS, EPILOGUE_RELU, EPILOGUE_GELU, EPILOGUE_SILU = 1, 2, 4, 6


def matmul_epilogue(a: np.ndarray, b: np.ndarray, bias: np.ndarray | None, *, ab_type: int, c_type: int, flags: int,
                    b_kn: bool = True, threads: int = 1) -> np.ndarray:
    """`activation(a @ b + bias)` as the reference's `matmul_epilogue` kernel computes it
    (src/krn/lib/lib_kernels.py:30-48): the k-ordered f32 accumulation of `gemm`, the bias (storage words of the
    output type) and the activation in f32, one rounding to `c_type`. `flags` = EPILOGUE_BIAS | one activation."""
    acc = gemm(a, b, ab_type=ab_type, c_type=F32, b_kn=b_kn, threads=threads)
    m, n = acc.shape
    out = np.zeros((m, n), _NUMPY[c_type])
    words = np.zeros(n, _NUMPY[c_type]) if bias is None else np.ascontiguousarray(bias, _NUMPY[c_type])
    lib().krn_oracle_matmul_epilogue(c_type, _p(acc), _p(words), _p(out), m, n, flags)
    return out


def gemm_fp8_blockscaled(a: np.ndarray, sa: np.ndarray, b: np.ndarray, sb: np.ndarray, *, c_type: int = BF16,
                         threads: int = 1) -> np.ndarray:
    a, b = np.ascontiguousarray(a, np.uint8), np.ascontiguousarray(b, np.uint8)
    sa, sb = np.ascontiguousarray(sa, np.float32), np.ascontiguousarray(sb, np.float32)
    (m, k), n = a.shape, b.shape[0]
    c = np.zeros((m, n), _NUMPY[c_type])
    _run(_split(m, threads), lambda lo, hi: lib().krn_oracle_gemm_fp8_blockscaled(
        c_type, _p(a), _p(sa), _p(b), _p(sb), _p(c), m, n, k, k, k, n, sa.shape[1], sb.shape[1], lo, hi))
    return c


def gemm_mxfp8(a: np.ndarray, sa: np.ndarray, b: np.ndarray, sb: np.ndarray, *, c_type: int = BF16, threads: int = 1) -> np.ndarray:
    """C = sum over 32-wide K blocks of 2^(sa-127) 2^(sb-127) (a8 . b8): a (M, K), b (N, K) e4m3 codes, sa (M, K/32),
    sb (N, K/32) e8m0 bytes."""
    a, b = np.ascontiguousarray(a, np.uint8), np.ascontiguousarray(b, np.uint8)
    sa, sb = np.ascontiguousarray(sa, np.uint8), np.ascontiguousarray(sb, np.uint8)
    (m, k), n = a.shape, b.shape[0]
    c = np.zeros((m, n), _NUMPY[c_type])
    _run(_split(m, threads), lambda lo, hi: lib().krn_oracle_gemm_mxfp8(
        c_type, _p(a), _p(sa), _p(b), _p(sb), _p(c), m, n, k, k, k, n, sa.shape[1], sb.shape[1], lo, hi))
    return c


def quantize_mxfp8(x: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """e4m3 codes + e8m0 scale bytes, one scale per 1 x 32 block of a row, by the OCP MX rule the reference's format
    names (`ScaleRounding.FLOOR`, src/krn/data/formats.py:34-37,138-144): scale = 2^(floor(log2 amax) - 8), 8 being the
    exponent of the largest e4m3 value (448 = 1.75 * 2^8); elements are x / scale rounded to nearest even, saturating.
    A block of zeros gets the scale 2^0."""
    rows, cols = x.shape
    if cols % 32:
        raise ValueError("the row length must be a multiple of 32")
    blocks = np.ascontiguousarray(x, np.float32).reshape(rows, cols // 32, 32)
    amax = np.abs(blocks).max(axis=2)
    exponent = np.where(amax > 0, np.floor(np.log2(np.where(amax > 0, amax, 1.0))) - 8, 0).astype(np.int32)
    exponent = np.clip(exponent, -127, 127)
    scaled = blocks * np.exp2(-exponent.astype(np.float32))[:, :, None]
    return e4m3_encode(scaled.reshape(rows, cols)), (exponent + 127).astype(np.uint8)


def mxfp8_values(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """float64 values of an MXFP8 matrix."""
    return e4m3_decode(codes).astype(np.float64) * np.repeat(np.exp2(scales.astype(np.float64) - 127), 32, axis=1)


E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float32)


def e2m1_decode(codes: np.ndarray) -> np.ndarray:
    """float32 values of 4-bit e2m1 codes (src/krn/data/formats.py:100)."""
    codes = np.asarray(codes, np.uint8)
    return np.where(codes & 8, -E2M1_VALUES[codes & 7], E2M1_VALUES[codes & 7]).astype(np.float32)


def e2m1_encode(x: np.ndarray) -> np.ndarray:
    """Nearest e2m1 code, ties to the code with an even mantissa bit, saturating at 6 (the reference's encoding rule
    for narrow formats, src/krn/compiler/narrow.py:84-110, applied to this format)."""
    x = np.asarray(x, np.float32)
    mag = np.abs(x)
    code = ((mag > 0.25).astype(np.uint8) + (mag >= 0.75) + (mag > 1.25) + (mag >= 1.75) + (mag > 2.5) + (mag >= 3.5) +
            (mag > 5.0)).astype(np.uint8)
    return (code | (np.signbit(x).astype(np.uint8) << 3)).astype(np.uint8)


def pack_nibbles(codes: np.ndarray) -> np.ndarray:
    """Two 4-bit codes per byte along the last axis, the lower index in the low nibble (`Storage.X2`)."""
    codes = np.asarray(codes, np.uint8)
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).astype(np.uint8)


def unpack_nibbles(packed: np.ndarray) -> np.ndarray:
    packed = np.asarray(packed, np.uint8)
    out = np.empty(packed.shape[:-1] + (2 * packed.shape[-1],), np.uint8)
    out[..., 0::2], out[..., 1::2] = packed & 15, packed >> 4
    return out


def quantize_nvfp4(x: np.ndarray) -> tuple[np.ndarray, np.ndarray, float]:
    """(packed e2m1 codes, e4m3 scale bytes per 1 x 16 block, f32 tensor scale) of the reference's NVFP4 format
    (src/krn/data/formats.py:147-154: scale format e4m3fn, tensor scale f32, `ScaleRounding.NEAREST`): the tensor
    scale maps the largest block scale onto 448, a block's scale is amax / 6 / tensor_scale rounded to e4m3, elements
    are x / (scale * tensor_scale) rounded to e2m1."""
    rows, cols = x.shape
    if cols % 16:
        raise ValueError("the row length must be a multiple of 16")
    x = np.ascontiguousarray(x, np.float32)
    amax_all = float(np.abs(x).max()) if x.size else 0.0
    tensor_scale = np.float32(amax_all / (6.0 * 448.0)) if amax_all > 0 else np.float32(1.0)
    blocks = x.reshape(rows, cols // 16, 16)
    amax = np.abs(blocks).max(axis=2)
    scale_codes = e4m3_encode((amax / np.float32(6.0) / tensor_scale).astype(np.float32))
    scale = e4m3_decode(scale_codes).astype(np.float32) * tensor_scale
    safe = np.where(scale > 0, scale, np.float32(1.0))
    codes = e2m1_encode(np.where(scale[:, :, None] > 0, blocks / safe[:, :, None], np.float32(0.0)))
    return pack_nibbles(codes.reshape(rows, cols)), scale_codes.astype(np.uint8), float(tensor_scale)


def nvfp4_values(packed: np.ndarray, scales: np.ndarray, tensor_scale: float) -> np.ndarray:
    """float64 values of an NVFP4 matrix."""
    values = e2m1_decode(unpack_nibbles(packed)).astype(np.float64)
    return values * np.repeat(e4m3_decode(scales).astype(np.float64), 16, axis=1) * float(tensor_scale)


def quantize_mxfp4(x: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """(packed e2m1 codes, e8m0 scale bytes per 1 x 32 block) of the reference's MXFP4 format
    (src/krn/data/formats.py:129-135) by the OCP MX floor rule: scale = 2^(floor(log2 amax) - 2), 2 being the exponent of
    the largest e2m1 value (6 = 1.5 * 2^2); elements are x / scale rounded to e2m1, saturating. A block of zeros gets 2^0."""
    rows, cols = x.shape
    if cols % 32:
        raise ValueError("the row length must be a multiple of 32")
    blocks = np.ascontiguousarray(x, np.float32).reshape(rows, cols // 32, 32)
    amax = np.abs(blocks).max(axis=2)
    exponent = np.where(amax > 0, np.floor(np.log2(np.where(amax > 0, amax, 1.0))) - 2, 0).astype(np.int32)
    exponent = np.clip(exponent, -127, 127)
    scaled = blocks * np.exp2(-exponent.astype(np.float32))[:, :, None]
    return pack_nibbles(e2m1_encode(scaled.reshape(rows, cols))), (exponent + 127).astype(np.uint8)


def mxfp4_values(packed: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """float64 values of an MXFP4 matrix."""
    values = e2m1_decode(unpack_nibbles(packed)).astype(np.float64)
    return values * np.repeat(np.exp2(scales.astype(np.float64) - 127), 32, axis=1)


def gemm_mxfp4(a: np.ndarray, sa: np.ndarray, b: np.ndarray, sb: np.ndarray, *, c_type: int = BF16, threads: int = 1) -> np.ndarray:
    """C = sum over 32-wide K blocks of 2^(sa-127) 2^(sb-127) (a4 . b4): a (M, K/2), b (N, K/2) packed e2m1 codes, sa (M, K/32),
    sb (N, K/32) e8m0 bytes."""
    a, b = np.ascontiguousarray(a, np.uint8), np.ascontiguousarray(b, np.uint8)
    sa, sb = np.ascontiguousarray(sa, np.uint8), np.ascontiguousarray(sb, np.uint8)
    (m, k_bytes), n = a.shape, b.shape[0]
    c = np.zeros((m, n), _NUMPY[c_type])
    _run(_split(m, threads), lambda lo, hi: lib().krn_oracle_gemm_mxfp4(
        c_type, _p(a), _p(sa), _p(b), _p(sb), _p(c), m, n, 2 * k_bytes, k_bytes, k_bytes, n, sa.shape[1], sb.shape[1], lo, hi))
    return c


def gemm_nvfp4(a: np.ndarray, sa: np.ndarray, b: np.ndarray, sb: np.ndarray, alpha: float = 1.0, *, c_type: int = BF16,
               threads: int = 1) -> np.ndarray:
    """C = alpha * sum over 16-wide K blocks of sa sb (a4 . b4): a (M, K/2), b (N, K/2) packed e2m1 codes, sa (M, K/16),
    sb (N, K/16) e4m3 bytes."""
    a, b = np.ascontiguousarray(a, np.uint8), np.ascontiguousarray(b, np.uint8)
    sa, sb = np.ascontiguousarray(sa, np.uint8), np.ascontiguousarray(sb, np.uint8)
    (m, k_bytes), n = a.shape, b.shape[0]
    c = np.zeros((m, n), _NUMPY[c_type])
    _run(_split(m, threads), lambda lo, hi: lib().krn_oracle_gemm_nvfp4(
        c_type, _p(a), _p(sa), _p(b), _p(sb), float(alpha), _p(c), m, n, 2 * k_bytes, k_bytes, k_bytes, n, sa.shape[1],
        sb.shape[1], lo, hi))
    return c


def quantize_blocks(x: np.ndarray, block: tuple[int, int]) -> tuple[np.ndarray, np.ndarray]:
    """e4m3 codes + fp32 scales with each block's absmax mapped to 448 (scale = absmax / 448; 1 for a zero block)."""
    rows, cols = x.shape
    br, bc = block
    nr, nc = -(-rows // br), -(-cols // bc)
    padded = np.zeros((nr * br, nc * bc), np.float32)
    padded[:rows, :cols] = x
    blocks = padded.reshape(nr, br, nc, bc)
    absmax = np.abs(blocks).max(axis=(1, 3))
    scale = np.where(absmax > 0, absmax / np.float32(448.0), np.float32(1.0)).astype(np.float32)
    scaled = (blocks / scale[:, None, :, None]).reshape(nr * br, nc * bc)[:rows, :cols]
    return e4m3_encode(scaled.astype(np.float32)), scale


# ---- attention ---------------------------------------------------------------------------------------------------


def flash_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, *, dtype: int, scale: float, causal: bool,
                    bq: int = 16, bk: int = 16, threads: int = 1) -> np.ndarray:
    """q [B, Hq, Sq, D], k/v [B, Hkv, Skv, D] in storage words; `scale` multiplies the scores (log2e/sqrt(d))."""
    q, k, v = (np.ascontiguousarray(x) for x in (q, k, v))
    batch, hq, sq, d = q.shape
    hkv, skv = k.shape[1], k.shape[2]
    o = np.zeros_like(q)
    _run(_split(batch * hq, threads), lambda lo, hi: lib().krn_oracle_flash_attention(
        dtype, _p(q), _p(k), _p(v), _p(o), batch, hq, hkv, sq, skv, d, scale, int(causal), bq, bk, lo, hi))
    return o


def attention_f64(q: np.ndarray, k: np.ndarray, v: np.ndarray, causal: bool) -> np.ndarray:
    """softmax(Q K^T / sqrt(d)) V in float64 on VALUES (not words): the check the reference's example uses
    (examples/04_libraries/08_flash_attention.py:62-69), extended with batch and grouped heads."""
    q, k, v = (x.astype(np.float64) for x in (q, k, v))
    group = q.shape[1] // k.shape[1]
    k, v = np.repeat(k, group, axis=1), np.repeat(v, group, axis=1)
    s = q @ k.transpose(0, 1, 3, 2) / math.sqrt(q.shape[-1])
    if causal:
        s = np.where(np.tril(np.ones(s.shape[-2:], bool)), s, -np.inf)
    p = np.exp(s - s.max(axis=-1, keepdims=True))
    return (p / p.sum(axis=-1, keepdims=True)) @ v


def decode_fp8_paged(q, k_pages, v_pages, page_table, context_len, k_scale, v_scale, *, scale_log2: float,
                     threads: int = 1) -> np.ndarray:
    q = np.ascontiguousarray(q, np.uint16)
    batch, hq, d = q.shape
    _, page_size, hkv, _ = k_pages.shape
    o = np.zeros_like(q)
    table = np.ascontiguousarray(page_table, np.int32)
    lens = np.ascontiguousarray(context_len, np.int32)
    ks, vs = np.ascontiguousarray(k_scale, np.float32), np.ascontiguousarray(v_scale, np.float32)
    kp, vp = np.ascontiguousarray(k_pages, np.uint8), np.ascontiguousarray(v_pages, np.uint8)
    _run(_split(batch, threads), lambda lo, hi: lib().krn_oracle_decode_fp8_paged(
        _p(q), _p(kp), _p(vp), _p(table), _p(lens), _p(ks), _p(vs), _p(o), hq, hkv, d, page_size, table.shape[1],
        scale_log2, lo, hi))
    return o


# ---- metrics ---------------------------------------------------------------------------------------------------------


def rel_frobenius(actual: np.ndarray, expected: np.ndarray) -> float:
    """||actual - expected||_F / ||expected||_F in float64 — the benchmark's correctness metric."""
    actual, expected = actual.astype(np.float64), expected.astype(np.float64)
    denom = np.linalg.norm(expected)
    return float(np.linalg.norm(actual - expected) / (denom if denom > 0 else 1.0))


def forward_error_bound(a: np.ndarray, b_kn: np.ndarray, k: int) -> np.ndarray:
    """The reference's elementwise bound for a reordered f32 accumulation: 8 * 2^-24 * (k + 8) * |A| @ |B|
    (tests/compiler/test_tensor_cores.py:395-401). `a` (M, K) and `b_kn` (K, N) are VALUES."""
    return 8 * 2.0**-24 * (k + 8) * (np.abs(a.astype(np.float64)) @ np.abs(b_kn.astype(np.float64)))


# ---- seeded synthetic inputs of the benchmark configs ---------------------------------------------------------


def config_gemm_f32(size: int = 256, seed: int = 0) -> tuple[np.ndarray, np.ndarray]:
    """f32 A, B (size, size) uniform[-1, 1) from one generator, A drawn first."""
    rng = np.random.default_rng(seed)
    return (rng.uniform(-1, 1, (size, size)).astype(np.float32), rng.uniform(-1, 1, (size, size)).astype(np.float32))


def config_gemm_bf16(m: int = 8192, n: int = 8192, k: int = 8192, seed: int = 1) -> tuple[np.ndarray, np.ndarray]:
    """bf16 words of A (m, k) and B (n, k), N(0, 1) rounded to nearest even, A drawn first."""
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((m, k), np.float32)
    b = rng.standard_normal((n, k), np.float32)
    return bf16_words(a), bf16_words(b)


def config_gemm_fp8(m: int = 8192, n: int = 28672, k: int = 8192, seed: int = 2):
    """e4m3 codes and fp32 scales: A (m, k) with one scale per 1x128 block, B (n, k) with one per 128x128."""
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((m, k), np.float32)
    b = rng.standard_normal((n, k), np.float32)
    a_codes, sa = quantize_blocks(a, (1, 128))
    b_codes, sb = quantize_blocks(b, (128, 128))
    return a_codes, sa, b_codes, sb


def config_attention(batch: int = 8, q_heads: int = 32, kv_heads: int = 8, seq: int = 4096, d: int = 128, seed: int = 3):
    """bf16 words of Q (B, Hq, S, D), K, V (B, Hkv, S, D), N(0, 1), drawn in that order."""
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((batch, q_heads, seq, d), np.float32)
    k = rng.standard_normal((batch, kv_heads, seq, d), np.float32)
    v = rng.standard_normal((batch, kv_heads, seq, d), np.float32)
    return bf16_words(q), bf16_words(k), bf16_words(v)


def config_decode(batch: int = 64, q_heads: int = 32, kv_heads: int = 8, d: int = 128, low: int = 1024, high: int = 8192,
                  page_size: int = 64, seed: int = 4):
    """Paged e4m3 KV cache: context lengths, then the page table (a random permutation of the pool), then K, V
    per sequence, then Q. K/V are N(0, 1) quantised with one fp32 scale per (sequence, kv head)."""
    rng = np.random.default_rng(seed)
    lens = rng.integers(low, high + 1, batch).astype(np.int32)
    pages_per_seq = -(-lens // page_size)
    max_pages = int(pages_per_seq.max())
    pool = int(pages_per_seq.sum())
    order = rng.permutation(pool).astype(np.int32)
    table = np.zeros((batch, max_pages), np.int32)
    k_pages = np.zeros((pool, page_size, kv_heads, d), np.uint8)
    v_pages = np.zeros((pool, page_size, kv_heads, d), np.uint8)
    k_scale = np.zeros((batch, kv_heads), np.float32)
    v_scale = np.zeros((batch, kv_heads), np.float32)
    cursor = 0
    for i in range(batch):
        count = int(pages_per_seq[i])
        ids = order[cursor:cursor + count]
        cursor += count
        table[i, :count] = ids
        for pages, scales in ((k_pages, k_scale), (v_pages, v_scale)):
            x = rng.standard_normal((count * page_size, kv_heads, d), np.float32)
            x[int(lens[i]):] = 0
            absmax = np.abs(x).max(axis=(0, 2))
            scale = np.where(absmax > 0, absmax / np.float32(448.0), np.float32(1.0)).astype(np.float32)
            scales[i] = scale
            pages[ids] = e4m3_encode(x / scale[None, :, None]).reshape(count, page_size, kv_heads, d)
    q = bf16_words(rng.standard_normal((batch, q_heads, d), np.float32))
    return q, k_pages, v_pages, table, lens, k_scale, v_scale
