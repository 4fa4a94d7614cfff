"""Paged FP8 decode attention on the GPU, through the C ABI, against the CPU oracle.

PARITY UNPINNED: the reference has no paged decode attention (neither code nor test); the oracle evaluates our
definition (K, V = e4m3 code * per-(sequence, kv head) scale, softmax in float64) and the acceptance tolerance is
the benchmark's 3e-2 relative Frobenius error."""

from __future__ import annotations

import math

import numpy as np
import pytest

from oracle import oracle as o
from krn_b200.runtime import calls

pytestmark = pytest.mark.gpu


def run(torch, q, kp, vp, table, lens, ks, vs):
    d = q.shape[-1]
    dq = torch.from_numpy(q.view(np.int16)).cuda().view(torch.bfloat16)
    dk = torch.from_numpy(kp).cuda()
    dv = torch.from_numpy(vp).cuda()
    dt, dl = torch.from_numpy(table).cuda(), torch.from_numpy(lens).cuda()
    dks, dvs = torch.from_numpy(ks).cuda(), torch.from_numpy(vs).cuda()
    out = torch.full(dq.shape, float("nan"), device="cuda", dtype=torch.bfloat16)
    max_context = int(table.shape[1]) * kp.shape[1]
    nbytes = calls.decode_workspace_bytes(q.shape[0], q.shape[1], d, max_context)
    workspace = torch.empty(nbytes, device="cuda", dtype=torch.uint8)
    calls.attention_decode_fp8_paged(dq, dk, dv, dt, dl, dks, dvs, out, math.log2(math.e) / math.sqrt(d), max_context,
                                     workspace)
    torch.cuda.synchronize()
    return o.bf16_values(out.view(torch.int16).cpu().numpy().view(np.uint16))


@pytest.mark.parametrize("batch,hq,hkv,low,high", [(3, 4, 1, 1, 64), (4, 8, 2, 60, 130), (5, 32, 8, 100, 1500),
                                                   (2, 4, 4, 1024, 1024), (6, 16, 8, 1000, 4000), (2, 8, 8, 1, 300)])
def test_decode_against_oracle(cuda, batch, hq, hkv, low, high) -> None:
    q, kp, vp, table, lens, ks, vs = o.config_decode(batch=batch, q_heads=hq, kv_heads=hkv, d=128, low=low, high=high,
                                                     page_size=64, seed=4)
    got = run(cuda, q, kp, vp, table, lens, ks, vs)
    want = o.bf16_values(o.decode_fp8_paged(q, kp, vp, table, lens, ks, vs, scale_log2=math.log2(math.e) / math.sqrt(128),
                                            threads=8))
    assert np.isfinite(got).all()
    assert o.rel_frobenius(got, want) < 3e-2   # the benchmark's tolerance
    assert o.rel_frobenius(got, want) < 1e-2   # what the hi/lo FP8 split actually delivers


def test_garbage_after_the_context_end_is_ignored(cuda) -> None:
    """Slots of the last page past context_len, and unused page-table entries, may hold anything (NaN codes)."""
    q, kp, vp, table, lens, ks, vs = o.config_decode(batch=3, q_heads=8, kv_heads=2, d=128, low=70, high=200, seed=8)
    clean = run(cuda, q, kp, vp, table, lens, ks, vs)
    kp2, vp2 = kp.copy(), vp.copy()
    for b in range(3):
        last = int(lens[b]) // 64
        used = -(-int(lens[b]) // 64)
        if int(lens[b]) % 64:
            kp2[table[b, last], int(lens[b]) % 64:] = 0x7F
            vp2[table[b, last], int(lens[b]) % 64:] = 0x7F
        table[b, used:] = 0
    dirty = run(cuda, q, kp2, vp2, table, lens, ks, vs)
    np.testing.assert_array_equal(clean, dirty)


def test_refusals_and_workspace(cuda) -> None:
    torch = cuda
    q, kp, vp, table, lens, ks, vs = o.config_decode(batch=2, q_heads=4, kv_heads=1, d=128, low=10, high=100, seed=1)
    args = [torch.from_numpy(x).cuda() for x in (q.view(np.int16), kp, vp, table, lens, ks, vs)]
    args[0] = args[0].view(torch.bfloat16)
    out = torch.empty_like(args[0])
    small = torch.empty(16, device="cuda", dtype=torch.uint8)
    with pytest.raises(Exception, match="KRN_B200_ERR_WORKSPACE"):
        calls.attention_decode_fp8_paged(*args, out, 1.0, int(table.shape[1]) * 64, small)
    assert calls.decode_workspace_bytes(2, 4, 128, 128) == 2 * 4 * 1 * 130 * 4
