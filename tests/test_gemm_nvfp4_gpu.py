"""NVFP4 tile product on the GPU (block scales applied by the tensor cores), through the C ABI, against the CPU oracle.

PARITY UNPINNED for the product: the reference declares the NVFP4 format (src/krn/data/formats.py:147-154) and the
`QTile @ QTile` product (src/krn/frontend/memory.py:173-193) but implements neither, so the oracle's definition
(oracle/krn_oracle.c) is ours; the FORMAT's value tables are pinned (tests/test_quantize_cpu.py). The tensor cores add
the 64 scaled products of an instruction in an order of their own, so agreement with the oracle's f32 chain is up to f32
rounding, and exact where every term is exactly representable."""

from __future__ import annotations

import numpy as np
import pytest

import krn_b200 as krn
from krn_b200 import ops
from krn_b200.runtime import calls
from oracle import oracle as o

pytestmark = pytest.mark.gpu


def run(torch, a, sa, b, sb, alpha=1.0, out="bf16"):
    m, n = a.shape[0], b.shape[0]
    dtype = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[out]
    c = torch.full((m, n), float("nan"), device="cuda", dtype=dtype)
    calls.gemm_nvfp4_tn(torch.from_numpy(a).cuda(), torch.from_numpy(sa).cuda(), torch.from_numpy(b).cuda(),
                        torch.from_numpy(sb).cuda(), c, alpha)
    torch.cuda.synchronize()
    return c.float().cpu().numpy()


def draw(m, n, k, seed):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((m, k), np.float32) * np.exp2(rng.integers(-3, 4, (m, 1))).astype(np.float32)
    b = rng.standard_normal((n, k), np.float32) * np.exp2(rng.integers(-3, 4, (n, 1))).astype(np.float32)
    return o.quantize_nvfp4(a), o.quantize_nvfp4(b)


def test_small_integer_codes_and_power_of_two_scales_are_exact(cuda) -> None:
    """Codes of small magnitudes with power-of-two scales that differ per 16-wide block: every term and every partial sum
    is exactly representable, so the result must equal the oracle bit for bit — and any mix-up of nibbles, scale bytes
    (row, block, which instruction's column) or operand halves shows as a wrong value."""
    rng = np.random.default_rng(23)
    m, n, k = 300, 520, 768
    a_codes = o.e2m1_encode(rng.choice([-2.0, -1.0, -0.5, 0.0, 0.5, 1.0, 2.0, 3.0], (m, k)).astype(np.float32))
    b_codes = o.e2m1_encode(rng.choice([-3.0, -1.5, -1.0, 0.0, 0.5, 1.0, 2.0, 4.0], (n, k)).astype(np.float32))
    sa = o.e4m3_encode(np.exp2(rng.integers(-3, 4, (m, k // 16))).astype(np.float32))
    sb = o.e4m3_encode(np.exp2(rng.integers(-3, 4, (n, k // 16))).astype(np.float32))
    a, b = o.pack_nibbles(a_codes), o.pack_nibbles(b_codes)
    got = run(cuda, a, sa, b, sb, 0.25, "f32")
    want = o.gemm_nvfp4(a, sa, b, sb, 0.25, c_type=o.F32, threads=8)
    np.testing.assert_array_equal(got, want)
    np.testing.assert_array_equal(got, (o.nvfp4_values(a, sa, 0.25) @ o.nvfp4_values(b, sb, 1.0).T).astype(np.float32))


@pytest.mark.parametrize("m,n,k", [(128, 256, 256), (128, 256, 1024), (256, 512, 2048), (384, 768, 1280), (1024, 1024, 4096),
                                   (100, 200, 768), (130, 264, 512), (16, 8, 256), (257, 136, 2304)])
@pytest.mark.parametrize("out", ["bf16", "f32"])
def test_nvfp4_product_against_oracle(cuda, m, n, k, out) -> None:
    (a, sa, ta), (b, sb, tb) = draw(m, n, k, seed=m + n + k)
    got = run(cuda, a, sa, b, sb, ta * tb, out)
    want_words = o.gemm_nvfp4(a, sa, b, sb, ta * tb, c_type=o.BF16 if out == "bf16" else o.F32, threads=8)
    want = o.bf16_values(want_words) if out == "bf16" else want_words
    exact = o.nvfp4_values(a, sa, ta) @ o.nvfp4_values(b, sb, tb).T
    assert np.isfinite(got).all()
    assert o.rel_frobenius(got, exact) < (1e-2 if out == "bf16" else 1e-5)
    assert o.rel_frobenius(got, want) < (1e-2 if out == "bf16" else 1e-5)


def test_ragged_edges_leave_neighbours_alone(cuda) -> None:
    torch = cuda
    (a, sa, ta), (b, sb, tb) = draw(33, 24, 512, seed=5)
    c = torch.full((40, 48), 5.0, device="cuda", dtype=torch.bfloat16)
    calls.gemm_nvfp4_tn(torch.from_numpy(a).cuda(), torch.from_numpy(sa).cuda(), torch.from_numpy(b).cuda(),
                        torch.from_numpy(sb).cuda(), c[:33, :24], ta * tb)
    torch.cuda.synchronize()
    assert bool((c[33:] == 5).all()) and bool((c[:, 24:] == 5).all())
    want = o.bf16_values(o.gemm_nvfp4(a, sa, b, sb, ta * tb))
    assert o.rel_frobenius(c[:33, :24].float().cpu().numpy(), want) < 1e-2


def test_quantised_containers_and_refusals(cuda) -> None:
    """`ops.quantize` + `ops.matmul_q` for `QMatrix[NVFP4]`, and the refusals of the entry point."""
    torch = cuda
    device = krn.host.Device.current()
    rng = np.random.default_rng(9)
    x, w = rng.standard_normal((256, 512), np.float32), rng.standard_normal((384, 512), np.float32)
    exact = x.astype(np.float64) @ w.astype(np.float64).T
    qx, qw = ops.quantize(x, krn.formats.NVFP4()), ops.quantize(w, krn.formats.NVFP4())
    assert qx.shape == (256, 512) and tuple(qx.codes.shape) == (256, 256) and tuple(qx.scales.shape) == (256, 32)
    assert qx.fmt.name == "nvfp4" and qx.tensor_scale > 0
    out = device.empty(krn.bf16, 256, 384)
    ops.matmul_q(qx, qw, out)
    torch.cuda.synchronize()
    assert o.rel_frobenius(o.bf16_values(out.to_host().view(np.uint16)), exact) < 0.2  # two 4-bit quantisations of N(0,1) data
    with pytest.raises(krn.TargetError, match="no prebuilt kernel multiplies this pair"):
        ops.matmul_q(qx, ops.quantize(w, krn.formats.MXFP8()), out)
    a = torch.zeros((128, 64), device="cuda", dtype=torch.uint8)
    s = torch.zeros((128, 8), device="cuda", dtype=torch.uint8)
    with pytest.raises(Exception, match="K = 128 is not available on sm_100a"):
        calls.gemm_nvfp4_tn(a, s, a, s, torch.zeros((128, 128), device="cuda", dtype=torch.bfloat16))


def test_calls_in_flight_on_two_streams_keep_their_own_scale_copies(cuda) -> None:
    """Each call rewrites its scale bytes into scratch memory that lives for the call, in stream order. Calls of different
    sizes queued back to back on two streams, with nothing waited for in between, must each read their own copy: every
    result is compared with the oracle bit for bit (exactly representable inputs)."""
    torch = cuda
    rng = np.random.default_rng(77)
    cases = []
    for m, n, k in [(256, 512, 1024), (384, 256, 2048), (130, 264, 512), (512, 768, 1280)] * 3:
        a_codes = o.e2m1_encode(rng.choice([-2.0, -1.0, 0.0, 0.5, 1.0, 3.0], (m, k)).astype(np.float32))
        b_codes = o.e2m1_encode(rng.choice([-1.5, -1.0, 0.0, 0.5, 2.0, 4.0], (n, k)).astype(np.float32))
        sa = o.e4m3_encode(np.exp2(rng.integers(-2, 3, (m, k // 16))).astype(np.float32))
        sb = o.e4m3_encode(np.exp2(rng.integers(-2, 3, (n, k // 16))).astype(np.float32))
        a, b = o.pack_nibbles(a_codes), o.pack_nibbles(b_codes)
        dev = [torch.from_numpy(x).cuda() for x in (a, sa, b, sb)]
        cases.append((a, sa, b, sb, dev, torch.full((m, n), float("nan"), device="cuda", dtype=torch.float32)))
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    for i, (_, _, _, _, dev, c) in enumerate(cases):
        calls.gemm_nvfp4_tn(dev[0], dev[1], dev[2], dev[3], c, 0.5, streams[i % 2])
    torch.cuda.synchronize()
    for a, sa, b, sb, _, c in cases:
        np.testing.assert_array_equal(c.cpu().numpy(), o.gemm_nvfp4(a, sa, b, sb, 0.5, c_type=o.F32, threads=8))
