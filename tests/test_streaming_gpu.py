"""Host-resident operands streamed through the device in panels give the bits of the one-shot device calls."""

from __future__ import annotations

import math

import numpy as np
import pytest

from krn_b200 import streaming
from krn_b200.runtime import calls
from oracle import oracle as o

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k,axis", [(1100, 520, 264, "m"), (520, 1100, 264, "n"), (300, 300, 64, None)])
def test_streamed_product_equals_the_device_call_and_the_oracle(cuda, m, n, k, axis) -> None:
    torch = cuda
    aw, bw = o.config_gemm_bf16(m, n, k, seed=21)
    a_host = torch.from_numpy(aw.view(np.int16)).view(torch.bfloat16).pin_memory()
    b_host = torch.from_numpy(bw.view(np.int16)).view(torch.bfloat16).pin_memory()
    c_host = torch.full((m, n), float("nan"), dtype=torch.bfloat16).pin_memory()
    product = streaming.StreamedProduct(m, n, k, torch.bfloat16, panels=3, axis=axis)
    assert len(product.ranges) > 1 or max(m, n) <= 256
    for _ in range(2):  # a second run reuses the device buffers and the events
        product.run(a_host, b_host, c_host)
    torch.cuda.synchronize()
    direct = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
    calls.gemm_tn(a_host.cuda(), b_host.cuda(), direct)
    torch.cuda.synchronize()
    assert torch.equal(c_host, direct.cpu())
    want = o.bf16_values(o.gemm(aw, bw, ab_type=o.BF16, c_type=o.BF16, threads=8))
    assert o.rel_frobenius(c_host.float().numpy(), want) < 1e-2
    with pytest.raises(ValueError, match="compose"):
        product.run(a_host[:-1], b_host, c_host)


def test_streamed_fp8_product_equals_the_device_call(cuda) -> None:
    torch = cuda
    m, n, k = 384, 1280, 512
    a_codes, sa, b_codes, sb = o.config_gemm_fp8(m, n, k, seed=22)
    hosts = [torch.from_numpy(x).pin_memory() for x in (a_codes, sa, b_codes, sb)]
    c_host = torch.full((m, n), float("nan"), dtype=torch.bfloat16).pin_memory()
    product = streaming.StreamedFp8Product(m, n, k, torch.bfloat16, panels=3)
    assert len(product.ranges) == 3
    product.run(*hosts, c_host)
    torch.cuda.synchronize()
    fp8 = torch.float8_e4m3fn
    direct = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
    calls.gemm_fp8_blockscaled_tn(hosts[0].cuda().view(fp8), hosts[1].cuda(), hosts[2].cuda().view(fp8), hosts[3].cuda(),
                                  direct)
    torch.cuda.synchronize()
    assert torch.equal(c_host, direct.cpu())
    want = o.bf16_values(o.gemm_fp8_blockscaled(a_codes, sa, b_codes, sb, threads=8))
    assert o.rel_frobenius(c_host.float().numpy(), want) < 1e-2


def test_streamed_attention_equals_the_device_call(cuda) -> None:
    torch = cuda
    batch, hq, hkv, seq, d = 3, 4, 2, 256, 128
    gen = torch.Generator().manual_seed(23)
    q, k, v = (torch.randn(shape, generator=gen).to(torch.bfloat16).pin_memory()
               for shape in ((batch, hq, seq, d), (batch, hkv, seq, d), (batch, hkv, seq, d)))
    o_host = torch.full((batch, hq, seq, d), float("nan"), dtype=torch.bfloat16).pin_memory()
    scale = math.log2(math.e) / math.sqrt(d)
    attention = streaming.StreamedAttention(batch, hq, hkv, seq, d, torch.bfloat16, groups=3)
    attention.run(q, k, v, o_host, scale, True)
    torch.cuda.synchronize()
    direct = torch.empty((batch, hq, seq, d), device="cuda", dtype=torch.bfloat16)
    calls.attention_forward(q.cuda(), k.cuda(), v.cuda(), direct, scale, True)
    torch.cuda.synchronize()
    assert torch.equal(o_host, direct.cpu())


@pytest.mark.parametrize("form", ["mxfp8", "nvfp4", "mxfp4"])
def test_streamed_scaled_product_matches_the_resident_call(cuda, form) -> None:
    """Host codes and scale bytes through `StreamedScaledProduct` (panels of b, column slabs of c) give the same bytes as
    one call on device-resident operands."""
    torch = cuda
    from krn_b200.runtime import calls
    from oracle import oracle as o

    m, n, k = 384, 1280, 2048
    rng = np.random.default_rng(11)
    x = rng.standard_normal((m, k), np.float32)
    y = rng.standard_normal((n, k), np.float32)
    alpha = 1.0
    if form == "mxfp8":
        (a, sa), (b, sb) = o.quantize_mxfp8(x), o.quantize_mxfp8(y)
    elif form == "nvfp4":
        (a, sa, ta), (b, sb, tb) = o.quantize_nvfp4(x), o.quantize_nvfp4(y)
        alpha = ta * tb
    else:
        (a, sa), (b, sb) = o.quantize_mxfp4(x), o.quantize_mxfp4(y)
    host = [torch.from_numpy(np.ascontiguousarray(t).view(np.uint8)).pin_memory() for t in (a, sa, b, sb)]
    out = torch.empty((m, n), dtype=torch.bfloat16).pin_memory()
    streamed = streaming.StreamedScaledProduct(form, m, n, k, torch.bfloat16, panels=4)
    streamed.run(*host, out, alpha)
    torch.cuda.synchronize()
    dev = [t.cuda() for t in host]
    want = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
    if form == "mxfp8":
        calls.gemm_mxfp8_tn(dev[0].view(torch.float8_e4m3fn), dev[1], dev[2].view(torch.float8_e4m3fn), dev[3], want)
    elif form == "nvfp4":
        calls.gemm_nvfp4_tn(dev[0], dev[1], dev[2], dev[3], want, alpha)
    else:
        calls.gemm_mxfp4_tn(dev[0], dev[1], dev[2], dev[3], want)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), want.cpu().view(torch.int16))
