"""Plain-function callers of the hot path for code that is not written as `@kernel` functions — the role
`lib.matmul` plays in the reference (src/krn/lib/lib.py:580-615): typed calls on device tensors that go straight to
the C ABI. Tensors may be this package's `DeviceTensor`s or torch CUDA tensors."""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

import numpy as np

from krn_b200.errors import TargetError
from krn_b200.frontend.types import f8e4m3fn
from krn_b200.runtime import calls
from krn_b200.runtime.device import DeviceTensor, _raw, default_device


def _stream(stream: Any):
    return getattr(stream, "raw", stream)


def matmul_nt(a: Any, b: Any, out: Any, stream: Any = None) -> Any:
    """out[M, N] = a[M, K] @ b[N, K]^T (bf16 or f16 operands; bf16, f16 or f32 output)."""
    calls.gemm_tn(_raw(a), _raw(b), _raw(out), _stream(stream))
    return out


def matmul(a: Any, b: Any, out: Any, stream: Any = None) -> Any:
    """out[M, N] = a[M, K] @ b[K, N], b row-major — the operand order of the reference's `lib.matmul`
    (src/krn/lib/lib.py:580-615)."""
    calls.gemm_nn(_raw(a), _raw(b), _raw(out), _stream(stream))
    return out


@dataclass(frozen=True)
class QMatrix:
    """A block-scaled matrix on the device, with the fields of the reference's `QMatrix[F]` struct
    (src/krn/frontend/memory.py:255-269): the block format `fmt` (a `krn_b200.formats.BlockFormat`: `FP8FN()`,
    `FP8FNWeights()`, `MXFP8()`, `MXFP4()` or `NVFP4()`), the logical `shape`, the `codes` ((rows, K), K contiguous — blocks run
    along the contraction axis; one byte per element, or for the 4-bit formats two codes per byte, low nibble first), the
    `scales` (f32 for the FP8FN formats, e8m0 bytes for MXFP8 and MXFP4, e4m3 bytes for NVFP4; one per block) and the per-tensor
    `tensor_scale` of formats that define one (NVFP4: a float)."""

    fmt: Any
    shape: tuple[int, int]
    codes: Any
    scales: Any
    tensor_scale: Any = None

    @property
    def block(self) -> tuple[int, int]:
        return self.fmt.block


def _e4m3_codes(values: np.ndarray) -> np.ndarray:
    """e4m3fn codes of float32 values: nearest, ties to even, saturating at 448 — the rule of the reference's
    `reference_encode` (src/krn/compiler/narrow.py:94-105). `ml_dtypes` rounds the same way but does not saturate, so
    values are clipped first."""
    import ml_dtypes

    clipped = np.clip(values.astype(np.float32), -448.0, 448.0)
    return clipped.astype(ml_dtypes.float8_e4m3fn).view(np.uint8)


_E2M1_MAX = 6.0


def _e2m1_codes(values: np.ndarray) -> np.ndarray:
    """4-bit e2m1 codes (magnitudes 0, 0.5, 1, 1.5, 2, 3, 4, 6): nearest, ties to the code with an even mantissa bit,
    saturating — the same narrowing rule as `_e4m3_codes`, written as the seven rounding thresholds of the format."""
    mag = np.abs(values.astype(np.float32))
    code = ((mag > 0.25).astype(np.uint8) + (mag >= 0.75) + (mag > 1.25) + (mag >= 1.75) + (mag > 2.5) + (mag >= 3.5) +
            (mag > 5.0)).astype(np.uint8)
    return code | (np.signbit(values).astype(np.uint8) << 3)


def quantize_nvfp4_host(values: np.ndarray) -> tuple[np.ndarray, np.ndarray, float]:
    """(packed codes (rows, K / 2), e4m3 scale bytes (rows, K / 16), tensor scale) of a float32 host matrix in the NVFP4
    format (src/krn/data/formats.py:147-154): the f32 tensor scale maps the largest block scale onto 448 (the largest
    e4m3 value), a block's scale is absmax / 6 / tensor_scale rounded to e4m3 (`ScaleRounding.NEAREST`), and the codes
    are x / (scale * tensor_scale) rounded to e2m1, two per byte with the lower column in the low nibble (`Storage.X2`).
    Blocks whose scale rounds to zero store zero codes."""
    values = np.ascontiguousarray(values, np.float32)
    rows, cols = values.shape
    if cols % 16:
        raise ValueError(f"cannot quantize a {rows} x {cols} matrix to nvfp4: rows must be whole 1 x 16 blocks")
    largest = float(np.abs(values).max()) if values.size else 0.0
    tensor_scale = np.float32(largest / (_E2M1_MAX * 448.0)) if largest > 0 else np.float32(1.0)
    blocks = values.reshape(rows, cols // 16, 16)
    absmax = np.abs(blocks).max(axis=2)
    scale_codes = _e4m3_codes(absmax / np.float32(_E2M1_MAX) / tensor_scale)
    import ml_dtypes

    scale = scale_codes.view(ml_dtypes.float8_e4m3fn).astype(np.float32) * tensor_scale
    safe = np.where(scale > 0, scale, np.float32(1.0))
    codes = _e2m1_codes(np.where(scale[:, :, None] > 0, blocks / safe[:, :, None], np.float32(0.0))).reshape(rows, cols)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    return np.ascontiguousarray(packed), np.ascontiguousarray(scale_codes), float(tensor_scale)


def quantize_mxfp4_host(values: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """(packed codes (rows, K / 2), e8m0 scale bytes (rows, K / 32)) of a float32 host matrix in the MXFP4 format
    (src/krn/data/formats.py:129-135), by the OCP MX floor rule the format names: scale = 2^(floor(log2 absmax) - 2), 2
    being the exponent of the largest e2m1 value; codes = e2m1(x / scale), two per byte, low nibble first."""
    values = np.ascontiguousarray(values, np.float32)
    rows, cols = values.shape
    if cols % 32:
        raise ValueError(f"cannot quantize a {rows} x {cols} matrix to mxfp4: rows must be whole 1 x 32 blocks")
    blocks = values.reshape(rows, cols // 32, 32)
    absmax = np.abs(blocks).max(axis=2)
    exponent = np.where(absmax > 0, np.floor(np.log2(np.where(absmax > 0, absmax, 1.0))) - 2, 0)
    exponent = np.clip(exponent, -127, 127).astype(np.int32)
    codes = _e2m1_codes(blocks * np.exp2(-exponent.astype(np.float32))[:, :, None]).reshape(rows, cols)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    return np.ascontiguousarray(packed), np.ascontiguousarray((exponent + 127).astype(np.uint8))


def quantize_host(values: np.ndarray, fmt: Any) -> tuple[np.ndarray, np.ndarray]:
    """(codes, scales) of a float32 host matrix (rows, K) in block format `fmt`, on the host.

    FP8FN / FP8FNWeights: f32 scale = block absmax / 448 (1 for a block of zeros), codes = e4m3(x / scale).
    MXFP8: e8m0 scale byte of 2^(floor(log2 absmax) - 8) per 1 x 32 block (the OCP MX floor rule the format names, 8
    being the exponent of the largest e4m3 value), codes = e4m3(x / scale)."""
    from krn_b200 import formats

    values = np.ascontiguousarray(values, np.float32)
    rows, cols = values.shape
    br, bc = fmt.block
    if fmt.elem != formats.E4M3FN or rows % br or cols % bc:
        raise ValueError(f"cannot quantize a {rows} x {cols} matrix to {fmt.name}: e4m3fn elements in whole {br} x {bc} blocks")
    blocks = values.reshape(rows // br, br, cols // bc, bc)
    absmax = np.abs(blocks).max(axis=(1, 3))
    if fmt.scale == formats.E8M0:
        exponent = np.where(absmax > 0, np.floor(np.log2(np.where(absmax > 0, absmax, 1.0))) - 8, 0)
        exponent = np.clip(exponent, -127, 127).astype(np.int32)
        scale = np.exp2(exponent.astype(np.float32))
        stored = (exponent + 127).astype(np.uint8)
    elif fmt.scale == formats.FP32:
        scale = np.where(absmax > 0, absmax / np.float32(448.0), np.float32(1.0)).astype(np.float32)
        stored = scale
    else:
        raise ValueError(f"no quantizer for the scale format of {fmt.name}")
    codes = _e4m3_codes((blocks / scale[:, None, :, None]).reshape(rows, cols))
    return codes, np.ascontiguousarray(stored)


def quantize(values: np.ndarray, fmt: Any, device: Any = None) -> QMatrix:
    """Convert a float32 host matrix (rows, K) to `fmt` (see `quantize_host`) and place it on the device — what the
    reference's `Resolution.quantize(weights) -> QMatrix[F]` is declared to do (src/krn/frontend/precision.py:43-45)."""
    from krn_b200 import formats

    device = device or default_device()
    if isinstance(fmt, formats.NVFP4):
        packed, scale_codes, tensor_scale = quantize_nvfp4_host(values)
        return QMatrix(fmt, tuple(values.shape), device.to_device(packed), device.to_device(scale_codes), tensor_scale)
    if isinstance(fmt, formats.MXFP4):
        packed, scale_codes = quantize_mxfp4_host(values)
        return QMatrix(fmt, tuple(values.shape), device.to_device(packed), device.to_device(scale_codes))
    codes, stored = quantize_host(values, fmt)
    return QMatrix(fmt, tuple(values.shape), device.to_device(codes, f8e4m3fn), device.to_device(stored))


def matmul_q(a: QMatrix, b: QMatrix, out: Any, stream: Any = None) -> Any:
    """out[M, N] = a @ b^T for two block-scaled matrices whose blocks run along K (both stored (rows, K)) — the product
    the reference declares as `QTile.__matmul__` (src/krn/frontend/memory.py:173-193). Three pairings have kernels:
    FP8FN activations (1 x 128 f32 scales) with FP8FNWeights (128 x 128 f32 scales), whose partial sums are scaled as they
    are accumulated, and MXFP8 with MXFP8, MXFP4 with MXFP4 and NVFP4 with NVFP4, whose block scales the tensor cores apply
    themselves."""
    from krn_b200 import formats

    if a.shape[1] != b.shape[1]:
        raise ValueError(f"contraction lengths differ: {a.shape} @ {b.shape}^T")
    if isinstance(a.fmt, formats.MXFP8) and isinstance(b.fmt, formats.MXFP8):
        calls.gemm_mxfp8_tn(_raw(a.codes), _raw(a.scales), _raw(b.codes), _raw(b.scales), _raw(out), _stream(stream))
    elif isinstance(a.fmt, formats.MXFP4) and isinstance(b.fmt, formats.MXFP4):
        calls.gemm_mxfp4_tn(_raw(a.codes), _raw(a.scales), _raw(b.codes), _raw(b.scales), _raw(out), _stream(stream))
    elif isinstance(a.fmt, formats.NVFP4) and isinstance(b.fmt, formats.NVFP4):
        alpha = float(a.tensor_scale if a.tensor_scale is not None else 1.0) * float(
            b.tensor_scale if b.tensor_scale is not None else 1.0)
        calls.gemm_nvfp4_tn(_raw(a.codes), _raw(a.scales), _raw(b.codes), _raw(b.scales), _raw(out), alpha, _stream(stream))
    elif a.fmt.block == (1, 128) and b.fmt.block == (128, 128) and a.fmt.scale == formats.FP32 and b.fmt.scale == formats.FP32:
        calls.gemm_fp8_blockscaled_tn(_raw(a.codes), _raw(a.scales), _raw(b.codes), _raw(b.scales), _raw(out), _stream(stream))
    else:
        raise TargetError(f"the product {a.fmt.name} @ {b.fmt.name}", "sm_100a", "no prebuilt kernel multiplies this pair "
                          "of block formats", "use FP8FN activations with FP8FNWeights, MXFP8 with MXFP8, MXFP4 with MXFP4, or NVFP4 with NVFP4")
    return out


def matmul_fp8_blockscaled(a: QMatrix, b: QMatrix, out: Any, stream: Any = None) -> Any:
    """out = sum over 128-wide K blocks of sa * sb * (a8 @ b8^T); a has 1x128 scales, b 128x128 scales."""
    if a.block != (1, 128) or b.block != (128, 128):
        raise ValueError("matmul_fp8_blockscaled takes 1x128-scaled activations and 128x128-scaled weights")
    return matmul_q(a, b, out, stream)


def attention(q: Any, k: Any, v: Any, out: Any, *, causal: bool = False, scale: float | None = None,
              stream: Any = None) -> Any:
    """out = softmax(scale * q k^T [+ causal mask]) v over [batch, heads, seq, d] tensors; `scale` defaults to
    1/sqrt(d). Grouped-query attention when k/v have fewer heads than q."""
    d = q.shape[-1]
    scale = (1.0 / math.sqrt(d)) if scale is None else scale
    calls.attention_forward(_raw(q), _raw(k), _raw(v), _raw(out), scale * math.log2(math.e), causal, _stream(stream))
    return out


def decode_attention_workspace(batch: int, q_heads: int, d: int, max_context: int) -> int:
    return calls.decode_workspace_bytes(batch, q_heads, d, max_context)


def decode_attention(q: Any, k_pages: Any, v_pages: Any, page_table: Any, context_len: Any, k_scale: Any, v_scale: Any,
                     out: Any, *, max_context: int, workspace: Any = None, scale: float | None = None,
                     stream: Any = None) -> Any:
    """One-token attention over a paged e4m3 KV cache. With `workspace=None` the allocation-free entry point is
    used (partials in the library's built-in scratch; calls on one device must then not overlap)."""
    d = q.shape[-1]
    scale = (1.0 / math.sqrt(d)) if scale is None else scale
    args = [_raw(x) for x in (q, k_pages, v_pages, page_table, context_len, k_scale, v_scale, out)]
    if workspace is None:
        calls.attention_decode_fp8_paged_noalloc(*args, scale * math.log2(math.e), max_context, _stream(stream))
    else:
        calls.attention_decode_fp8_paged(*args, scale * math.log2(math.e), max_context, _raw(workspace), _stream(stream))
    return out


__all__ = ["DeviceTensor", "QMatrix", "attention", "decode_attention", "decode_attention_workspace", "matmul", "matmul_fp8_blockscaled",
           "matmul_nt", "matmul_q", "quantize", "quantize_host"]
