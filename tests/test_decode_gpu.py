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


def run(torch, q, kp, vp, table, lens, ks, vs, max_context=None):
    d = q.shape[-1]
    dq = torch.from_numpy(q.view(np.int16)).cuda().view(torch.bfloat16)
    dk = torch.from_numpy(kp).cuda()
    dv = torch.from_numpy(vp).cuda()
    dt, dl = torch.from_numpy(table).cuda(), torch.from_numpy(lens).cuda()
    dks, dvs = torch.from_numpy(ks).cuda(), torch.from_numpy(vs).cuda()
    out = torch.full(dq.shape, float("nan"), device="cuda", dtype=torch.bfloat16)
    max_context = max_context or int(table.shape[1]) * kp.shape[1]
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


def test_context_lengths_are_clamped_to_max_context(cuda) -> None:
    """A context_len beyond max_context (a caller bug, or a stale value) must not make the kernel read past the page
    table row: it is clamped, so the result is that of the first max_context tokens. A negative one counts as 0."""
    q, kp, vp, table, lens, ks, vs = o.config_decode(batch=4, q_heads=8, kv_heads=2, d=128, low=200, high=300, seed=9)
    assert table.shape[1] == 5
    max_context = 128  # two pages per sequence
    narrow = np.ascontiguousarray(table[:, :2])
    wild = lens.copy()
    wild[1], wild[2], wild[3] = 1000, 2**30, -5
    got = run(cuda, q, kp, vp, narrow, wild, ks, vs, max_context=max_context)
    clamped = np.clip(wild, 0, max_context).astype(np.int32)
    want = o.bf16_values(o.decode_fp8_paged(q, kp, vp, narrow, clamped, ks, vs,
                                            scale_log2=math.log2(math.e) / math.sqrt(128)))
    assert np.isfinite(got).all() and not got[3].any()  # the empty sequence's rows are zeros
    assert o.rel_frobenius(got[:3], want[:3]) < 1e-2


def test_page_ids_outside_the_pool_are_never_fetched(cuda) -> None:
    """Ids of num_pages and -1: in table slots past the context they are not looked at; inside the context the page is
    not fetched — its 64 tokens read as zero codes, exactly as if the table pointed at a page of zeros — and the status
    word says so."""
    from krn_b200.runtime import native

    q, kp, vp, table, lens, ks, vs = o.config_decode(batch=3, q_heads=8, kv_heads=2, d=128, low=300, high=1400, seed=10)
    scale = math.log2(math.e) / math.sqrt(128)
    clean = run(cuda, q, kp, vp, table, lens, ks, vs)
    unused = table.copy()
    for b in range(3):
        used = -(-int(lens[b]) // 64)
        unused[b, used:] = kp.shape[0] if b % 2 else -1
    np.testing.assert_array_equal(run(cuda, q, kp, vp, unused, lens, ks, vs), clean)
    assert native.device_status()[0] == 0

    # sequence 0 loses its third page, sequence 2 its first; the oracle sees a pool with one more page, all zero codes
    broken, zeroed = table.copy(), table.copy()
    broken[0, 2], broken[2, 0] = kp.shape[0], -1
    zeroed[0, 2] = zeroed[2, 0] = kp.shape[0]
    pad = np.zeros((1,) + kp.shape[1:], np.uint8)
    got = run(cuda, q, kp, vp, broken, lens, ks, vs)
    code, site, _ = native.device_status()  # reads and clears the word
    assert code == native.ERR_DEVICE_INDEX and site == 36
    want = o.bf16_values(o.decode_fp8_paged(q, np.concatenate([kp, pad]), np.concatenate([vp, pad]), zeroed, lens, ks, vs,
                                            scale_log2=scale))
    assert np.isfinite(got).all()
    assert o.rel_frobenius(got, want) < 1e-2


def test_config_five_as_configured(cuda) -> None:
    """The benchmark configuration itself: 64 sequences, 32 / 8 heads, contexts U[1024, 8192] from seed 4, random page
    table over a pool of ~4.6k pages — every sequence against the oracle, the shortest and the longest singled out."""
    config = o.config_decode(batch=64, q_heads=32, kv_heads=8, d=128, low=1024, high=8192, page_size=64, seed=4)
    lens = config[4]
    got = run(cuda, *config)
    want = o.bf16_values(o.decode_fp8_paged(*config, scale_log2=math.log2(math.e) / math.sqrt(128), threads=16))
    assert np.isfinite(got).all()
    assert o.rel_frobenius(got, want) < 1e-2
    for b in (int(lens.argmin()), int(lens.argmax())):
        assert o.rel_frobenius(got[b], want[b]) < 1e-2, (b, int(lens[b]))
    worst = max(o.rel_frobenius(got[b], want[b]) for b in range(64))
    assert worst < 3e-2, worst


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
