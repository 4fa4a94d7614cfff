"""MXFP4 tile product on the GPU (e8m0 block scales applied by the tensor cores), through the C ABI, against the CPU oracle.

PARITY UNPINNED for the product: the reference declares the MXFP4 format (src/krn/data/formats.py:129-135) and the
`QTile @ QTile` product (src/krn/frontend/memory.py:173-193) but implements neither, so the oracle's definition
(oracle/krn_oracle.c) is ours; the FORMAT's value tables are pinned (tests/test_quantize_cpu.py). Scales are powers of
two and e2m1 products are exact, so agreement with the oracle is up to the order of f32 additions only."""

from __future__ import annotations

import numpy as np
import pytest

import krn_b200 as krn
from krn_b200 import ops
from krn_b200.runtime import calls
from oracle import oracle as o

pytestmark = pytest.mark.gpu


def run(torch, a, sa, b, sb, out="bf16"):
    m, n = a.shape[0], b.shape[0]
    dtype = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[out]
    c = torch.full((m, n), float("nan"), device="cuda", dtype=dtype)
    calls.gemm_mxfp4_tn(torch.from_numpy(a).cuda(), torch.from_numpy(sa).cuda(), torch.from_numpy(b).cuda(),
                        torch.from_numpy(sb).cuda(), c)
    torch.cuda.synchronize()
    return c.float().cpu().numpy()


def draw(m, n, k, seed):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((m, k), np.float32) * np.exp2(rng.integers(-3, 4, (m, 1))).astype(np.float32)
    b = rng.standard_normal((n, k), np.float32) * np.exp2(rng.integers(-3, 4, (n, 1))).astype(np.float32)
    return o.quantize_mxfp4(a), o.quantize_mxfp4(b)


def test_small_codes_with_scales_that_differ_per_block_are_exact(cuda) -> None:
    """Every term and every partial sum exactly representable, scales differing per 32-wide block: bit for bit equal to
    the oracle — any mix-up of nibbles, scale bytes (row, block, which half of a tensor-memory column an instruction
    reads) or operand halves shows as a wrong value."""
    rng = np.random.default_rng(29)
    m, n, k = 300, 520, 1536
    a_codes = o.e2m1_encode(rng.choice([-2.0, -1.0, -0.5, 0.0, 0.5, 1.0, 2.0, 3.0], (m, k)).astype(np.float32))
    b_codes = o.e2m1_encode(rng.choice([-3.0, -1.5, -1.0, 0.0, 0.5, 1.0, 2.0, 4.0], (n, k)).astype(np.float32))
    sa = (127 + rng.integers(-3, 4, (m, k // 32))).astype(np.uint8)
    sb = (127 + rng.integers(-3, 4, (n, k // 32))).astype(np.uint8)
    a, b = o.pack_nibbles(a_codes), o.pack_nibbles(b_codes)
    got = run(cuda, a, sa, b, sb, "f32")
    want = o.gemm_mxfp4(a, sa, b, sb, c_type=o.F32, threads=8)
    np.testing.assert_array_equal(got, want)
    np.testing.assert_array_equal(got, (o.mxfp4_values(a, sa) @ o.mxfp4_values(b, sb).T).astype(np.float32))


@pytest.mark.parametrize("m,n,k", [(128, 256, 512), (128, 256, 1024), (256, 512, 2048), (384, 768, 2560), (1024, 1024, 4096),
                                   (100, 200, 1536), (130, 264, 512), (16, 8, 512), (257, 136, 3584)])
@pytest.mark.parametrize("out", ["bf16", "f32"])
def test_mxfp4_product_against_oracle(cuda, m, n, k, out) -> None:
    (a, sa), (b, sb) = draw(m, n, k, seed=m + n + k)
    got = run(cuda, a, sa, b, sb, out)
    want_words = o.gemm_mxfp4(a, sa, b, sb, c_type=o.BF16 if out == "bf16" else o.F32, threads=8)
    want = o.bf16_values(want_words) if out == "bf16" else want_words
    exact = o.mxfp4_values(a, sa) @ o.mxfp4_values(b, sb).T
    assert np.isfinite(got).all()
    assert o.rel_frobenius(got, exact) < (1e-2 if out == "bf16" else 1e-5)
    assert o.rel_frobenius(got, want) < (1e-2 if out == "bf16" else 1e-5)


def test_quantised_containers_and_refusals(cuda) -> None:
    torch = cuda
    device = krn.host.Device.current()
    rng = np.random.default_rng(9)
    x, w = rng.standard_normal((256, 512), np.float32), rng.standard_normal((384, 512), np.float32)
    exact = x.astype(np.float64) @ w.astype(np.float64).T
    qx, qw = ops.quantize(x, krn.formats.MXFP4()), ops.quantize(w, krn.formats.MXFP4())
    assert qx.shape == (256, 512) and tuple(qx.codes.shape) == (256, 256) and tuple(qx.scales.shape) == (256, 16)
    assert qx.fmt.name == "mxfp4" and qx.tensor_scale is None
    out = device.empty(krn.bf16, 256, 384)
    ops.matmul_q(qx, qw, out)
    torch.cuda.synchronize()
    assert o.rel_frobenius(o.bf16_values(out.to_host().view(np.uint16)), exact) < 0.25  # two 4-bit quantisations of N(0,1) data
    a = torch.zeros((128, 128), device="cuda", dtype=torch.uint8)
    s = torch.zeros((128, 8), device="cuda", dtype=torch.uint8)
    with pytest.raises(Exception, match="K = 256 is not available on sm_100a"):
        calls.gemm_mxfp4_tn(a, s, a, s, torch.zeros((128, 128), device="cuda", dtype=torch.bfloat16))
