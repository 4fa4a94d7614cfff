"""Plain-function callers of the hot path for code that is not written as `@kernel` functions — the role
`lib.matmul` plays in the reference (src/krn/lib/lib.py:580-615): typed calls on device tensors that go straight to
the C ABI. Tensors may be this package's `DeviceTensor`s or torch CUDA tensors."""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

from krn_b200.runtime import calls
from krn_b200.runtime.device import DeviceTensor, _raw


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
    """A block-scaled FP8 matrix on the device: e4m3fn `codes` (rows, K) and fp32 `scales` with one scale per
    `block` (1x128 for activations, 128x128 for weights) — the wire format the reference sketches as
    `QMatrix[FP8FN]` (src/krn/frontend/memory.py:257-269)."""

    codes: Any
    scales: Any
    block: tuple[int, int]


def matmul_fp8_blockscaled(a: QMatrix, b: QMatrix, out: Any, stream: Any = None) -> Any:
    """out = sum over 128-wide K blocks of sa * sb * (a8 @ b8^T); a has 1x128 scales, b 128x128 scales."""
    if a.block != (1, 128) or b.block != (128, 128):
        raise ValueError("matmul_fp8_blockscaled takes 1x128-scaled activations and 128x128-scaled weights")
    calls.gemm_fp8_blockscaled_tn(_raw(a.codes), _raw(a.scales), _raw(b.codes), _raw(b.scales), _raw(out), _stream(stream))
    return out


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


__all__ = ["DeviceTensor", "QMatrix", "attention", "decode_attention", "decode_attention_workspace", "matmul_fp8_blockscaled",
           "matmul_nt"]
