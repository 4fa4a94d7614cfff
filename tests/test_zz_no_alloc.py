"""The allocation-free decode entry point against the workspace one.

Some callers of the kernel library cannot allocate device memory where they need attention (a serving loop whose
KV-cache pool owns the rest of HBM, a plugin living inside another runtime's memory budget), so
`krn_b200_attn_decode_fp8_paged_noalloc` keeps its split-KV partials in an array built into the library. This
test calls it through the C ABI twice in a row — the array is shared between calls and keeps the previous call's
contents, so the second call runs over stale partials of a different problem — and wants the same bits as the
workspace entry point both times. The file sorts last on purpose: a run that stops at the first failure has
already run every other test."""

from __future__ import annotations

import math

import numpy as np
import pytest

from oracle import oracle as o
from krn_b200.runtime import calls, native

pytestmark = pytest.mark.gpu


def to_device(torch, config):
    q, kp, vp, table, lens, ks, vs = config
    tensors = [torch.from_numpy(x).cuda() for x in (q.view(np.int16), kp, vp, table, lens, ks, vs)]
    tensors[0] = tensors[0].view(torch.bfloat16)
    return tensors


def test_noalloc_matches_workspace_entry_on_two_calls_in_a_row(cuda) -> None:
    torch = cuda
    scale = math.log2(math.e) / math.sqrt(128)
    first = o.config_decode(batch=5, q_heads=32, kv_heads=8, d=128, low=900, high=2500, page_size=64, seed=21)
    second = o.config_decode(batch=3, q_heads=8, kv_heads=2, d=128, low=1, high=700, page_size=64, seed=22)
    for config in (first, second):
        tensors = to_device(torch, config)
        max_context = int(config[3].shape[1]) * 64
        want = torch.full(tensors[0].shape, float("nan"), device="cuda", dtype=torch.bfloat16)
        workspace = torch.empty(calls.decode_workspace_bytes(*tensors[0].shape, max_context), device="cuda",
                                dtype=torch.uint8)
        calls.attention_decode_fp8_paged(*tensors, want, scale, max_context, workspace)
        torch.cuda.synchronize()
        got = torch.full(tensors[0].shape, float("nan"), device="cuda", dtype=torch.bfloat16)
        torch.cuda.synchronize()
        held = torch.cuda.memory_allocated()
        calls.attention_decode_fp8_paged_noalloc(*tensors, got, scale, max_context)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == held  # no torch allocation on the way either
        assert bool(torch.isfinite(got.float()).all())
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
        reference = o.bf16_values(o.decode_fp8_paged(*config, scale_log2=scale, threads=8))
        assert o.rel_frobenius(o.bf16_values(got.view(torch.int16).cpu().numpy().view(np.uint16)), reference) < 1e-2
    native.raise_device_status()


def test_noalloc_refuses_problems_beyond_its_scratch(cuda) -> None:
    torch = cuda
    config = o.config_decode(batch=2, q_heads=4, kv_heads=1, d=128, low=10, high=60, page_size=64, seed=23)
    tensors = to_device(torch, config)
    out = torch.empty_like(tensors[0])
    # a page table wide enough for 70 Mi tokens per sequence would need far more than 16 MiB of partials
    wide = torch.zeros((2, 1 << 20), device="cuda", dtype=torch.int32)
    wide[:, : tensors[3].shape[1]] = tensors[3]
    tensors[3] = wide
    with pytest.raises(Exception, match="built-in scratch holds"):
        calls.attention_decode_fp8_paged_noalloc(*tensors, out, 1.0, (1 << 20) * 64)
