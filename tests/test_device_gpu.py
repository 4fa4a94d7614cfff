"""The kernel-language surface on the GPU: `@kernel` functions launched through `host.Device.current()` reach the
prebuilt kernels through the C ABI and agree with the CPU oracle. Mirrors the call forms of the reference's
launcher tests (tests/frontend/test_launch_inference.py:202-217, tests/runtime/test_cuda_backend.py)."""

from __future__ import annotations

import asyncio
import math

import numpy as np
import pytest

import krn_b200 as krn
from krn_b200 import Blocks, TargetError, Tiles, ops
from oracle import oracle as o
from tests.kernels import tile_kernels as K

pytestmark = pytest.mark.gpu
TIMEOUT = 60  # every wait is time-boxed, as in the reference's device tests


@pytest.fixture()
def device(cuda):
    return krn.host.Device.current()


def test_configured_gemm_call_forms_and_ragged_shapes(device) -> None:
    """Every call form of a configured kernel computes the same ragged product (the reference's 50 x 38 x 70)."""
    aw, bw = o.config_gemm_bf16(50, 38, 70, seed=5)
    a, b = device.to_device(aw, krn.bf16), device.to_device(bw, krn.bf16)
    outputs = [device.empty(krn.bf16, 50, 38) for _ in range(6)]
    t = K.Tiling(bm=16, bn=16, bk=8)
    launch = Tiles((50, 38), (16, 16))
    K.matmul_nt(a, b, outputs[0])
    K.matmul_nt[t](a, b, outputs[1])
    K.matmul_nt(t, a, b, outputs[2], launch=launch)
    K.matmul_nt(t, a, b, outputs[3])
    device.launcher(K.matmul_nt, launch.blocks)(t, a, b, outputs[4])
    device.launcher(K.matmul_nt).bind(t, a, b, outputs[5])()
    device.default_stream.record().wait(TIMEOUT)
    want = o.gemm(aw, bw, ab_type=o.BF16, c_type=o.BF16)
    for output in outputs:
        got = output.to_host().view(np.uint16)
        assert o.rel_frobenius(o.bf16_values(got), o.bf16_values(want)) < 1e-2
        np.testing.assert_array_equal(got, outputs[0].to_host().view(np.uint16))


def test_reference_example_form_with_row_major_b(device) -> None:
    """`acc += a[rows, ks] @ b[ks, cols]` on the reference example's 50 x 38 x 70 f16 shapes
    (examples/04_libraries/01_gemm_tiles.py:35-52) and on an aligned shape that takes the tensor-core kernel."""
    rng = np.random.default_rng(3)
    for m, n, k in ((50, 38, 70), (260, 136, 72)):
        a16 = rng.uniform(-1, 1, (m, k)).astype(np.float16)
        b16 = rng.uniform(-1, 1, (k, n)).astype(np.float16)
        a, b, c = device.to_device(a16), device.to_device(b16), device.empty(krn.f16, m, n)
        t = K.Tiling(bm=16, bn=16, bk=8)
        assert "krn_b200_gemm_nn" in str(K.matmul_nn.explain(t, a, b, c))
        K.matmul_nn(t, a, b, c)
        ops.matmul(a, b, c2 := device.empty(krn.f16, m, n))
        device.default_stream.record().wait(TIMEOUT)
        want = o.gemm(a16.view(np.uint16), np.ascontiguousarray(b16.T).view(np.uint16), ab_type=o.F16, c_type=o.F16)
        got = c.to_host().view(np.uint16)
        assert o.rel_frobenius(got.view(np.float16).astype(np.float32), want.view(np.float16).astype(np.float32)) < 1e-2
        np.testing.assert_array_equal(got, c2.to_host().view(np.uint16))


def test_family_launches_the_tensor_memory_variant(device) -> None:
    """Calling a family runs the variant selected for the current device (src/krn/frontend/variants.py:114-126)."""
    rng = np.random.default_rng(4)
    m, n, k = 200, 136, 72
    a16, b16 = rng.uniform(-1, 1, (m, k)).astype(np.float16), rng.uniform(-1, 1, (k, n)).astype(np.float16)
    a, b = device.to_device(a16), device.to_device(b16)
    c1, c2 = device.empty(krn.f32, m, n), device.empty(krn.f32, m, n)
    assert K.gemm.select(device.target).name == "gemm_tensor_memory"
    assert "krn_b200_gemm_nn" in str(K.gemm.explain(a, b, c1))
    K.gemm(a, b, c1)
    K.gemm[K.FamilyTiling(bm=64, bn=64, bk=32)](a, b, c2)
    device.default_stream.record().wait(TIMEOUT)
    exact = a16.astype(np.float64) @ b16.astype(np.float64)
    assert np.all(np.abs(c1.to_host() - exact) <= o.forward_error_bound(a16, b16, k))
    np.testing.assert_array_equal(c1.to_host(), c2.to_host())


def test_range_loop_f16_f32_and_explain(device) -> None:
    rng = np.random.default_rng(2)
    a16, b16 = rng.uniform(-1, 1, (130, 104)).astype(np.float16), rng.uniform(-1, 1, (72, 104)).astype(np.float16)
    a, b, c = device.to_device(a16), device.to_device(b16), device.empty(krn.f32, 130, 72)
    text = str(K.matmul_nt_f16_f32.explain(a, b, c))
    assert "krn_b200_gemm_tn" in text and "Blocks(x=2, y=5" in text
    event = device.launcher(K.matmul_nt_f16_f32).submit(a, b, c)
    event.wait(TIMEOUT)
    assert event.done() and event.error is None
    want = o.gemm(a16.view(np.uint16), b16.view(np.uint16), ab_type=o.F16, c_type=o.F32)
    exact = a16.astype(np.float64) @ b16.astype(np.float64).T
    got = c.to_host()
    assert np.all(np.abs(got - exact) <= o.forward_error_bound(a16, b16.T, 104))
    assert o.rel_frobenius(got, want) < 1e-5


def test_flash_attention_example_through_the_kernel_language(device) -> None:
    """The reference example's own run: 2 heads, 200 tokens, launch=Tiles((heads, seq), (1, 16)), f16, atol 2e-3
    (examples/04_libraries/08_flash_attention.py:72-86)."""
    rng = np.random.default_rng(0)
    heads, seq = 2, 200
    for d, causal in ((64, False), (128, True)):
        host = [rng.standard_normal((heads, seq, d)).astype(np.float16) for _ in range(3)]
        q, k, v = (device.to_device(x) for x in host)
        out = device.empty(krn.T.f16, heads, seq, d)
        scale = math.log2(math.e) / math.sqrt(d)
        K.flash_attention(K.Heads(d=d, causal=causal), q, k, v, out, scale, launch=Tiles((heads, seq), (1, 16)))
        asyncio.run(device.synchronize())
        want = o.attention_f64(*(x[None] for x in host), causal)[0]
        np.testing.assert_allclose(out.to_host().astype(np.float64), want, atol=2e-3)


def test_grouped_batched_causal_attention_kernel(device) -> None:
    batch, hq, hkv, seq, d = 2, 8, 2, 300, 128
    qw, kw, vw = o.config_attention(batch, hq, hkv, seq, d, seed=3)
    q, k, v = (device.to_device(x, krn.bf16) for x in (qw, kw, vw))
    out = device.empty(krn.bf16, batch, hq, seq, d)
    K.grouped_causal_attention(q, k, v, out, krn.T.f32(math.log2(math.e) / math.sqrt(d)),
                               launch=Blocks(math.ceil(seq / 128), hq, batch))
    device.default_stream.record().wait(TIMEOUT)
    exact = o.attention_f64(o.bf16_values(qw), o.bf16_values(kw), o.bf16_values(vw), True)
    assert o.rel_frobenius(o.bf16_values(out.to_host().view(np.uint16)), exact) < 1e-2


def test_streams_bound_rebind_and_graph_replay(device) -> None:
    aw, bw = o.config_gemm_bf16(256, 128, 64, seed=9)
    a, b = device.to_device(aw, krn.bf16), device.to_device(bw, krn.bf16)
    c1, c2 = device.empty(krn.bf16, 256, 128), device.empty(krn.bf16, 256, 128)
    bound = device.launcher(K.matmul_nt).bind(K.Tiling(), a, b, c1)
    stream = device.stream()
    with stream:
        first = bound.submit()
        bound.rebind(K.Tiling(), a, b, c2)
        second = bound.submit()
    second.wait(TIMEOUT)
    assert first.done() and second.elapsed_since(first) >= 0.0
    np.testing.assert_array_equal(c1.to_host().view(np.uint16), c2.to_host().view(np.uint16))
    c1.data.zero_()
    graph = device.graph(lambda: K.matmul_nt(a, b, c1))
    c1.data.zero_()
    graph()
    graph.submit().wait(TIMEOUT)
    np.testing.assert_array_equal(c1.to_host().view(np.uint16), c2.to_host().view(np.uint16))


def test_refusals_happen_before_any_launch(device) -> None:
    a, c = device.empty(krn.f32, 32, 32), device.empty(krn.f32, 32, 32)
    with pytest.raises(TargetError, match="no code generator"):
        K.row_scale(a, c)
    aw, bw = o.config_gemm_bf16(64, 64, 64, seed=1)
    x, y, z = device.to_device(aw, krn.bf16), device.to_device(bw, krn.bf16), device.empty(krn.bf16, 64, 64)
    with pytest.raises(TargetError, match="computes the whole output"):
        K.matmul_nt(K.Tiling(bm=16, bn=16), x, y, z, launch=Blocks(1, 1))
    with pytest.raises(TypeError, match="declared bf16"):
        K.matmul_nt(device.empty(krn.f16, 64, 64), y, z)
    with pytest.raises(ValueError, match="do not compose"):
        K.matmul_nt(x, device.empty(krn.bf16, 64, 32), z)


def test_plain_function_callers(device) -> None:
    torch = pytest.importorskip("torch")
    a_codes, sa, b_codes, sb = o.config_gemm_fp8(128, 256, 256, seed=2)
    qa = ops.QMatrix(krn.formats.FP8FN(), a_codes.shape, device.to_device(a_codes, krn.f8e4m3fn), device.to_device(sa))
    qb = ops.QMatrix(krn.formats.FP8FNWeights(), b_codes.shape, device.to_device(b_codes, krn.f8e4m3fn), device.to_device(sb))
    out = device.empty(krn.bf16, 128, 256)
    ops.matmul_fp8_blockscaled(qa, qb, out)
    torch.cuda.synchronize()
    want = o.bf16_values(o.gemm_fp8_blockscaled(a_codes, sa, b_codes, sb))
    assert o.rel_frobenius(o.bf16_values(out.to_host().view(np.uint16)), want) < 1e-2
    config = o.config_decode(batch=3, q_heads=8, kv_heads=2, d=128, low=50, high=400, seed=6)
    tensors = [device.to_device(x, krn.bf16 if i == 0 else None) for i, x in enumerate(config)]
    result = device.empty(krn.bf16, 3, 8, 128)
    ops.decode_attention(*tensors, result, max_context=int(config[3].shape[1]) * 64)
    torch.cuda.synchronize()
    want = o.bf16_values(o.decode_fp8_paged(*config, scale_log2=math.log2(math.e) / math.sqrt(128)))
    assert o.rel_frobenius(o.bf16_values(result.to_host().view(np.uint16)), want) < 1e-2
