"""Typed Python calls over the C ABI for callers that already hold device memory (torch tensors or this
package's device tensors): shape checks, pitch extraction, status → exception. Nothing here computes; a
missing kernel library raises `LibraryNotFound`."""

from __future__ import annotations

import ctypes
import sys
from typing import Any

from krn_b200.runtime import native

_ELEMENT = {"bfloat16": native.BF16, "float16": native.F16, "float32": native.F32, "float8_e4m3fn": native.E4M3,
            "float8_e5m2": native.E5M2, "uint8": native.E4M3}


def _type_of(tensor: Any) -> int:
    name = str(getattr(tensor, "dtype", "")).replace("torch.", "")
    if name not in _ELEMENT:
        raise TypeError(f"no kernel element type for {name!r}")
    return _ELEMENT[name]


def _pointer(tensor: Any) -> int:
    if hasattr(tensor, "data_ptr"):
        return int(tensor.data_ptr())
    return int(tensor.pointer)


def _pitch(tensor: Any) -> int:
    """Row pitch in elements of a rank-2 tensor whose last axis is contiguous."""
    strides = tuple(tensor.stride()) if callable(getattr(tensor, "stride", None)) else tuple(tensor.strides)
    if len(strides) == 2 and 0 in tuple(tensor.shape):
        return max(1, int(tensor.shape[1]))  # an empty tensor has no meaningful strides
    if len(strides) != 2 or (tensor.shape[1] > 1 and strides[1] != 1):
        raise ValueError("expected a rank-2 tensor with a contiguous last axis")
    return int(strides[0]) if tensor.shape[0] > 1 else max(int(strides[0]), int(tensor.shape[1]))


def _stream(stream: Any) -> ctypes.c_void_p:
    """The CUDA stream handle to enqueue on. None means torch's CURRENT stream when torch is loaded (so a call made
    under `with torch.cuda.stream(s)` lands on s like torch's own work), else the legacy default stream."""
    if stream is None:
        torch = sys.modules.get("torch")
        if torch is not None and torch.cuda.is_available():
            return ctypes.c_void_p(int(torch.cuda.current_stream().cuda_stream))
        return ctypes.c_void_p(0)
    if hasattr(stream, "cuda_stream"):
        return ctypes.c_void_p(int(stream.cuda_stream))
    if hasattr(stream, "__cuda_stream__"):
        return ctypes.c_void_p(int(stream.__cuda_stream__()[1]))
    return ctypes.c_void_p(int(stream))


def gemm_tn(a: Any, b: Any, c: Any, stream: Any = None) -> None:
    """c[M, N] = a[M, K] @ b[N, K]^T with f32 accumulation; a, b bf16 or f16 (same type), c bf16/f16/f32."""
    (m, k), (n, kb) = a.shape, b.shape
    if kb != k or tuple(c.shape) != (m, n):
        raise ValueError(f"shapes do not compose: a {tuple(a.shape)}, b {tuple(b.shape)}, c {tuple(c.shape)}")
    if _type_of(a) != _type_of(b):
        raise TypeError("both operands must have the same element type")
    status = native.library().krn_b200_gemm_tn(
        _type_of(a), _type_of(c), _pointer(a), _pointer(b), _pointer(c), m, n, k, _pitch(a), _pitch(b), _pitch(c),
        _stream(stream))
    native.check(status, "tile matrix product")


def gemm_nn(a: Any, b: Any, c: Any, stream: Any = None) -> None:
    """c[M, N] = a[M, K] @ b[K, N] with f32 accumulation (b row-major, not transposed); types as `gemm_tn`."""
    (m, k), (kb, n) = a.shape, b.shape
    if kb != k or tuple(c.shape) != (m, n):
        raise ValueError(f"shapes do not compose: a {tuple(a.shape)}, b {tuple(b.shape)}, c {tuple(c.shape)}")
    if _type_of(a) != _type_of(b):
        raise TypeError("both operands must have the same element type")
    status = native.library().krn_b200_gemm_nn(
        _type_of(a), _type_of(c), _pointer(a), _pointer(b), _pointer(c), m, n, k, _pitch(a), _pitch(b), _pitch(c),
        _stream(stream))
    native.check(status, "tile matrix product")


def gemm_fp8(a: Any, b: Any, c: Any, *, b_kn: bool = False, stream: Any = None) -> None:
    """c = a @ b for two 8-bit float tensors taken as stored (no scales): `b` is (N, K) — the operand of
    `b.transpose()` — or, with `b_kn`, (K, N) row-major. Each operand is e4m3fn or e5m2 on its own; c bf16/f16/f32."""
    (m, k) = a.shape
    kb, n = (b.shape[0], b.shape[1]) if b_kn else (b.shape[1], b.shape[0])
    if kb != k or tuple(c.shape) != (m, n):
        raise ValueError(f"shapes do not compose: a {tuple(a.shape)}, b {tuple(b.shape)}, c {tuple(c.shape)}")
    status = native.library().krn_b200_gemm_fp8(
        _type_of(a), _type_of(b), _type_of(c), int(b_kn), _pointer(a), _pointer(b), _pointer(c), m, n, k, _pitch(a),
        _pitch(b), _pitch(c), _stream(stream))
    native.check(status, "fp8 tile matrix product")


def matmul(a: Any, b: Any, c: Any, *, b_kn: bool = True, epilogue: int = 0, bias: Any = None, stream: Any = None) -> None:
    """c = activation(a @ b + bias): `b` is (K, N) when `b_kn` (the layout `lib.matmul` takes) or (N, K) otherwise;
    `epilogue` holds the KRN_B200_EPILOGUE_* flags (bit 0 bias, bits 1-2 relu / gelu / silu); `bias` is a vector of N
    elements of c's type."""
    (m, k) = a.shape
    kb, n = (b.shape[0], b.shape[1]) if b_kn else (b.shape[1], b.shape[0])
    if kb != k or tuple(c.shape) != (m, n):
        raise ValueError(f"shapes do not compose: a {tuple(a.shape)}, b {tuple(b.shape)}, c {tuple(c.shape)}")
    if _type_of(a) != _type_of(b):
        raise TypeError("both operands must have the same element type")
    if bias is not None and (tuple(bias.shape) != (n,) or _type_of(bias) != _type_of(c)):
        raise TypeError(f"the bias must be a vector of {n} elements of the output type")
    status = native.library().krn_b200_matmul(
        _type_of(a), _type_of(c), int(b_kn), int(epilogue), _pointer(a), _pointer(b),
        _pointer(bias) if bias is not None else None, _pointer(c), m, n, k, _pitch(a), _pitch(b), _pitch(c),
        _stream(stream))
    native.check(status, "tile matrix product with epilogue")


def _sync_array(sync_pointers: list[int] | None, ranks: int):
    if sync_pointers is None:
        return None
    if len(sync_pointers) != ranks:
        raise ValueError(f"{len(sync_pointers)} sync addresses for {ranks} ranks")
    return (ctypes.c_void_p * ranks)(*sync_pointers)


def gemm_tn_gather(a: Any, b_local: Any, c_pointers: list[int], rank: int, m: int, n_local: int, ldc: int, c_type: int,
                   stream: Any = None, sync_pointers: list[int] | None = None, epoch: int = 0) -> None:
    """This rank's column block of c = a @ b^T, stored by the kernel's epilogue into every rank's full C.
    `c_pointers[r]` is the address (valid on this device) of rank r's row-major C[m, len(c_pointers) * n_local].
    `sync_pointers[r]` (optional) is the address of rank r's 9 sync words: with them the kernel itself waits until every
    rank's stores of product number `epoch` have landed; without them the caller runs a cross-rank barrier."""
    (rows, k), (nb, kb) = a.shape, b_local.shape
    if kb != k or rows != m or nb != n_local:
        raise ValueError(f"shapes do not compose: a {tuple(a.shape)}, b {tuple(b_local.shape)}, block {m} x {n_local}")
    ranks = len(c_pointers)
    array = (ctypes.c_void_p * ranks)(*c_pointers)
    status = native.library().krn_b200_gemm_tn_gather(
        _type_of(a), c_type, _pointer(a), _pointer(b_local), array, ranks, rank, m, n_local, k, _pitch(a), _pitch(b_local),
        ldc, _sync_array(sync_pointers, ranks), epoch & 0xFFFFFFFF, _stream(stream))
    native.check(status, "column-sharded tile matrix product")


def gemm_fp8_blockscaled_tn(a: Any, sa: Any, b: Any, sb: Any, c: Any, stream: Any = None) -> None:
    """c = sum_kb sa[:, kb] * sb[n // 128, kb] * (a8[:, kb] @ b8[:, kb]^T); a, b e4m3 codes, scales f32."""
    (m, k), (n, kb) = a.shape, b.shape
    if kb != k or tuple(c.shape) != (m, n):
        raise ValueError(f"shapes do not compose: a {tuple(a.shape)}, b {tuple(b.shape)}, c {tuple(c.shape)}")
    blocks = -(-k // 128)
    if tuple(sa.shape) != (m, blocks) or tuple(sb.shape) != (-(-n // 128), blocks):
        raise ValueError(f"scale shapes {tuple(sa.shape)}, {tuple(sb.shape)} do not match 1x128 / 128x128 blocks")
    status = native.library().krn_b200_gemm_fp8_blockscaled_tn(
        _type_of(c), _pointer(a), _pointer(sa), _pointer(b), _pointer(sb), _pointer(c), m, n, k, _pitch(a), _pitch(b),
        _pitch(c), _pitch(sa), _pitch(sb), _stream(stream))
    native.check(status, "block-scaled FP8 tile matrix product")


def gemm_mxfp8_tn(a: Any, sa: Any, b: Any, sb: Any, c: Any, stream: Any = None) -> None:
    """c = sum over 32-wide K blocks of 2^(sa - 127) * 2^(sb - 127) * (a8 @ b8^T): a [M, K], b [N, K] e4m3 codes, sa [M, K/32]
    and sb [N, K/32] e8m0 bytes (uint8). The tensor cores apply the scales themselves."""
    (m, k), (n, kb) = a.shape, b.shape
    if kb != k or tuple(c.shape) != (m, n):
        raise ValueError(f"shapes do not compose: a {tuple(a.shape)}, b {tuple(b.shape)}, c {tuple(c.shape)}")
    if tuple(sa.shape) != (m, k // 32) or tuple(sb.shape) != (n, k // 32) or k % 32:
        raise ValueError(f"scale shapes {tuple(sa.shape)}, {tuple(sb.shape)} do not match 1x32 blocks of K = {k}")
    if "uint8" not in str(sa.dtype) or "uint8" not in str(sb.dtype):
        raise TypeError("MX scales are e8m0 bytes: pass uint8 tensors")
    status = native.library().krn_b200_gemm_mxfp8_tn(
        _type_of(c), _pointer(a), _pointer(sa), _pointer(b), _pointer(sb), _pointer(c), m, n, k, _pitch(a), _pitch(b),
        _pitch(c), _pitch(sa), _pitch(sb), _stream(stream))
    native.check(status, "MXFP8 tile matrix product")


def gemm_mxfp4_tn(a: Any, sa: Any, b: Any, sb: Any, c: Any, stream: Any = None) -> None:
    """c = sum over 32-wide K blocks of 2^(sa - 127) * 2^(sb - 127) * (a4 @ b4^T): a [M, K/2], b [N, K/2] bytes of packed e2m1
    codes (low nibble first), sa [M, K/32] and sb [N, K/32] e8m0 bytes (uint8). The tensor cores apply the scales."""
    (m, k_bytes), (n, kb_bytes) = a.shape, b.shape
    k = 2 * k_bytes
    if kb_bytes != k_bytes or tuple(c.shape) != (m, n):
        raise ValueError(f"shapes do not compose: a {tuple(a.shape)}, b {tuple(b.shape)}, c {tuple(c.shape)}")
    if tuple(sa.shape) != (m, k // 32) or tuple(sb.shape) != (n, k // 32) or k % 32:
        raise ValueError(f"scale shapes {tuple(sa.shape)}, {tuple(sb.shape)} do not match 1x32 blocks of K = {k}")
    for t in (a, b, sa, sb):
        if "uint8" not in str(t.dtype):
            raise TypeError("MXFP4 codes and scales are bytes: pass uint8 tensors")
    status = native.library().krn_b200_gemm_mxfp4_tn(
        _type_of(c), _pointer(a), _pointer(sa), _pointer(b), _pointer(sb), _pointer(c), m, n, k, _pitch(a), _pitch(b),
        _pitch(c), _pitch(sa), _pitch(sb), _stream(stream))
    native.check(status, "MXFP4 tile matrix product")


def gemm_nvfp4_tn(a: Any, sa: Any, b: Any, sb: Any, c: Any, alpha: float = 1.0, stream: Any = None) -> None:
    """c = alpha * sum over 16-wide K blocks of sa * sb * (a4 @ b4^T): a [M, K/2], b [N, K/2] bytes of packed e2m1 codes (low
    nibble first), sa [M, K/16] and sb [N, K/16] e4m3 bytes (uint8), alpha the product of the two tensor scales. The
    tensor cores apply the block scales themselves."""
    (m, k_bytes), (n, kb_bytes) = a.shape, b.shape
    k = 2 * k_bytes
    if kb_bytes != k_bytes or tuple(c.shape) != (m, n):
        raise ValueError(f"shapes do not compose: a {tuple(a.shape)}, b {tuple(b.shape)}, c {tuple(c.shape)}")
    if tuple(sa.shape) != (m, k // 16) or tuple(sb.shape) != (n, k // 16) or k % 16:
        raise ValueError(f"scale shapes {tuple(sa.shape)}, {tuple(sb.shape)} do not match 1x16 blocks of K = {k}")
    for t in (a, b, sa, sb):
        if "uint8" not in str(t.dtype):
            raise TypeError("NVFP4 codes and scales are bytes: pass uint8 tensors")
    status = native.library().krn_b200_gemm_nvfp4_tn(
        _type_of(c), _pointer(a), _pointer(sa), _pointer(b), _pointer(sb), float(alpha), _pointer(c), m, n, k, _pitch(a),
        _pitch(b), _pitch(c), _pitch(sa), _pitch(sb), _stream(stream))
    native.check(status, "NVFP4 tile matrix product")


def gemm_fp8_blockscaled_tn_gather(a: Any, sa: Any, b_local: Any, sb_local: Any, c_pointers: list[int], rank: int,
                                   n_local: int, ldc: int, c_type: int, stream: Any = None,
                                   sync_pointers: list[int] | None = None, epoch: int = 0) -> None:
    """This rank's column block of the block-scaled FP8 product, stored by the kernel's epilogue into every rank's
    full C (`c_pointers[r]` = address on this device of rank r's row-major C[m, len(c_pointers) * n_local])."""
    (m, k), (nb, kb) = a.shape, b_local.shape
    blocks = -(-k // 128)
    if kb != k or nb != n_local or tuple(sa.shape) != (m, blocks) or tuple(sb_local.shape) != (-(-n_local // 128), blocks):
        raise ValueError(f"shapes do not compose: a {tuple(a.shape)}, b {tuple(b_local.shape)}, scales "
                         f"{tuple(sa.shape)}, {tuple(sb_local.shape)}")
    ranks = len(c_pointers)
    array = (ctypes.c_void_p * ranks)(*c_pointers)
    status = native.library().krn_b200_gemm_fp8_blockscaled_tn_gather(
        c_type, _pointer(a), _pointer(sa), _pointer(b_local), _pointer(sb_local), array, ranks, rank, m, n_local, k,
        _pitch(a), _pitch(b_local), ldc, _pitch(sa), _pitch(sb_local), _sync_array(sync_pointers, ranks),
        epoch & 0xFFFFFFFF, _stream(stream))
    native.check(status, "column-sharded block-scaled FP8 tile matrix product")


def _strides3(tensor: Any) -> Any:
    strides = tuple(tensor.stride()) if callable(getattr(tensor, "stride", None)) else tuple(tensor.strides)
    if len(strides) != 4 or strides[3] != 1:
        raise ValueError("expected a rank-4 tensor [batch, heads, seq, d] with a contiguous last axis")
    return (ctypes.c_int64 * 3)(*strides[:3])


def attention_forward(q: Any, k: Any, v: Any, o: Any, scale_log2: float, causal: bool, stream: Any = None) -> None:
    """o = softmax(scale * q k^T [+ causal mask]) v per (batch, q head); scores carry scale_log2 = log2(e) * scale."""
    batch, hq, sq, d = q.shape
    _, hkv, skv, _ = k.shape
    status = native.library().krn_b200_attn_fwd(
        _type_of(q), _pointer(q), _pointer(k), _pointer(v), _pointer(o), batch, hq, hkv, sq, skv, d, scale_log2,
        int(causal), _strides3(q), _strides3(k), _strides3(v), _strides3(o), _stream(stream))
    native.check(status, "flash attention forward")


def decode_workspace_bytes(batch: int, q_heads: int, d: int, max_context: int) -> int:
    return int(native.library().krn_b200_attn_decode_workspace_bytes(batch, q_heads, d, max_context))


def attention_decode_fp8_paged(q: Any, k_pages: Any, v_pages: Any, page_table: Any, context_len: Any, k_scale: Any,
                               v_scale: Any, o: Any, scale_log2: float, max_context: int, workspace: Any,
                               stream: Any = None) -> None:
    batch, hq, d = q.shape
    num_pages, page_size, hkv, _ = k_pages.shape
    nbytes = workspace.numel() * workspace.element_size() if hasattr(workspace, "numel") else workspace.nbytes
    status = native.library().krn_b200_attn_decode_fp8_paged(
        _pointer(q), _pointer(k_pages), _pointer(v_pages), _pointer(page_table), _pointer(context_len),
        _pointer(k_scale), _pointer(v_scale), _pointer(o), batch, hq, hkv, d, page_size, num_pages, page_table.shape[1],
        max_context, scale_log2, _pointer(workspace), nbytes, _stream(stream))
    native.check(status, "paged FP8 decode attention")


def attention_decode_fp8_paged_noalloc(q: Any, k_pages: Any, v_pages: Any, page_table: Any, context_len: Any,
                                       k_scale: Any, v_scale: Any, o: Any, scale_log2: float, max_context: int,
                                       stream: Any = None) -> None:
    """Paged FP8 decode attention for callers that cannot allocate device memory (no workspace argument: the
    partials go to a 16 MiB array inside the kernel library). Calls on one device must not overlap on the GPU;
    make the first call on a device outside stream capture."""
    batch, hq, d = q.shape
    num_pages, page_size, hkv, _ = k_pages.shape
    status = native.library().krn_b200_attn_decode_fp8_paged_noalloc(
        _pointer(q), _pointer(k_pages), _pointer(v_pages), _pointer(page_table), _pointer(context_len),
        _pointer(k_scale), _pointer(v_scale), _pointer(o), batch, hq, hkv, d, page_size, num_pages, page_table.shape[1],
        max_context, scale_log2, _stream(stream))
    native.check(status, "paged FP8 decode attention (built-in scratch)")


def scatter_columns(slabs: Any, c_full: Any, ranks: int, stream: Any = None) -> None:
    """slabs [ranks, M, n_local] -> c_full [M, ranks * n_local] (row-major)."""
    _, m, n_local = slabs.shape
    element = c_full.element_size() if hasattr(c_full, "element_size") else c_full.itemsize
    status = native.library().krn_b200_scatter_columns(_pointer(slabs), _pointer(c_full), m, n_local, ranks,
                                                       _pitch(c_full), element, _stream(stream))
    native.check(status, "column scatter")


def copy_matrix(dst: Any, src: Any, stream: Any = None) -> None:
    """dst[:, :] = src[:, :] for 2-D tensors of one shape and element type whose rows are contiguous but whose row
    pitches may differ (column slabs of wider matrices); either side may be page-locked host memory."""
    if tuple(dst.shape) != tuple(src.shape) or dst.element_size() != src.element_size() or len(dst.shape) != 2:
        raise ValueError(f"copy of {tuple(src.shape)} into {tuple(dst.shape)}")
    if dst.stride(1) != 1 or src.stride(1) != 1:
        raise ValueError("rows must be contiguous")
    rows, columns = dst.shape
    element = dst.element_size()
    status = native.library().krn_b200_copy_2d(_pointer(dst), dst.stride(0) * element, _pointer(src),
                                               src.stride(0) * element, columns * element, rows, _stream(stream))
    native.check(status, "pitched copy")
