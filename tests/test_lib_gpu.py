"""`lib.matmul` with fused epilogues on the GPU against the oracle's restatement of the reference's `matmul_epilogue`
kernel (src/krn/lib/lib_kernels.py:30-48; call forms as tests of src/krn/lib/lib.py:580-615 use them)."""

from __future__ import annotations

import numpy as np
import pytest

import krn_b200 as krn
from krn_b200 import lib
from krn_b200.runtime import calls
from oracle import oracle as o
from tests.kernels import tile_kernels as K

pytestmark = pytest.mark.gpu

ORACLE_OF = {"bf16": o.BF16, "f16": o.F16, "f32": o.F32}
TYPE_OF = {"bf16": krn.bf16, "f16": krn.f16, "f32": krn.f32}


def words(x: np.ndarray, dtype: str) -> np.ndarray:
    return x.astype(np.float32) if dtype == "f32" else (x.astype(np.float16).view(np.uint16) if dtype == "f16" else o.bf16_words(x))


def values(w: np.ndarray, dtype: str) -> np.ndarray:
    return w.astype(np.float32) if dtype == "f32" else (w.view(np.float16).astype(np.float32) if dtype == "f16" else o.bf16_values(w))


def on_device(device, w: np.ndarray, dtype: str):
    """Storage words to a device tensor of element type `dtype`."""
    if dtype == "bf16":
        return device.to_device(w, krn.bf16)
    return device.to_device(w.view(np.float16) if dtype == "f16" else w)


def ulp(x: np.ndarray, dtype: str) -> np.ndarray:
    """Spacing of the output type at |x| (bf16: 8 significand bits)."""
    if dtype == "f32":
        return np.spacing(np.abs(x).astype(np.float32))
    if dtype == "f16":
        return np.spacing(np.abs(x).astype(np.float16)).astype(np.float32)
    return np.spacing(np.abs(x).astype(np.float32)) * 2.0**16


def close(got: np.ndarray, want: np.ndarray, dtype: str, k: int) -> None:
    """The tensor cores add in another order than the k-ordered fma chain: within the reordering bound of the f32
    sum (8 * 2^-24 * (k + 8) * |a||b| ~ a few 1e-5 here) plus one rounding step of the output type."""
    slack = 1e-4 * max(1.0, float(np.abs(want).max())) * (1 + k / 1024) + 1.01 * ulp(want, dtype)
    assert np.all(np.abs(got - want) <= slack), float(np.abs(got - want).max())
    assert o.rel_frobenius(got, want) < 4e-3


@pytest.mark.parametrize("epilogue", list(lib.Epilogue))
@pytest.mark.parametrize("ab,out", [("f16", "f16"), ("bf16", "bf16"), ("bf16", "f32")])
@pytest.mark.parametrize("m,n,k", [(300, 520, 328), (50, 38, 70)])
def test_matmul_epilogues_against_the_oracle(cuda, epilogue, ab, out, m, n, k) -> None:
    device = krn.host.Device.current()
    rng = np.random.default_rng(31)
    a, b = rng.uniform(-1, 1, (m, k)).astype(np.float32), rng.uniform(-1, 1, (k, n)).astype(np.float32)
    aw, bw = words(a, ab), words(b, ab)
    flags = lib.FLAGS[epilogue]
    bias_words = words(rng.uniform(-2, 2, n).astype(np.float32), out) if flags & 1 else None
    da, db = on_device(device, aw, ab), on_device(device, bw, ab)
    dbias = on_device(device, bias_words, out) if bias_words is not None else None
    result = device.empty(TYPE_OF[out], m, n)
    returned = lib.matmul(da, db, epilogue=epilogue, bias=dbias, out=result)
    assert returned is result
    device.default_stream.record().wait(60)
    host = result.to_host()
    got = values(host if out == "f32" else host.view(np.uint16), out)
    want = values(o.matmul_epilogue(aw, bw, bias_words, ab_type=ORACLE_OF[ab], c_type=ORACLE_OF[out], flags=flags,
                                    threads=8), out)
    close(got, want, out, k)


def test_matmul_allocates_the_result_and_refuses_what_it_cannot_run(cuda) -> None:
    device = krn.host.Device.current()
    rng = np.random.default_rng(32)
    a16, b16 = rng.uniform(-1, 1, (64, 72)).astype(np.float16), rng.uniform(-1, 1, (72, 40)).astype(np.float16)
    da, db = device.to_device(a16), device.to_device(b16)
    c = lib.matmul(da, db, epilogue=lib.Epilogue.RELU)
    device.default_stream.record().wait(60)
    assert c.element == krn.f16 and tuple(c.shape) == (64, 40)
    want = o.matmul_epilogue(a16.view(np.uint16), b16.view(np.uint16), None, ab_type=o.F16, c_type=o.F16, flags=o.EPILOGUE_RELU)
    close(values(c.to_host().view(np.uint16), "f16"), values(want, "f16"), "f16", 72)
    assert float(c.to_host().min()) >= 0.0
    with pytest.raises(ValueError, match="needs a bias"):
        lib.matmul(da, db, epilogue=lib.Epilogue.BIAS)
    with pytest.raises(ValueError, match="takes no bias"):
        lib.matmul(da, db, bias=device.empty(krn.f16, 40))
    with pytest.raises(ValueError, match="bias must be a vector of 40 f16"):
        lib.matmul(da, db, epilogue=lib.Epilogue.BIAS, bias=device.empty(krn.f32, 40))
    with pytest.raises(ValueError, match="compose"):
        lib.matmul(da, da)
    with pytest.raises(lib.NoCandidate, match="b200: the tensor-memory product multiplies two bf16 or two f16"):
        lib.matmul(device.to_device(a16.astype(np.float32)), device.to_device(b16.astype(np.float32)))
    with pytest.raises(krn.TargetError, match="tf32"):
        lib.matmul(da, db, precision=lib.Compute.TF32)


def test_an_empty_sum_still_gets_its_epilogue(cuda) -> None:
    """K = 0: the accumulator is zero, so the result is activation(bias) in every row."""
    torch = cuda
    bias = torch.linspace(-3, 3, 48, device="cuda").to(torch.bfloat16)
    out = torch.full((20, 48), float("nan"), device="cuda", dtype=torch.bfloat16)
    calls.matmul(torch.zeros((20, 0), device="cuda", dtype=torch.bfloat16),
                 torch.zeros((0, 48), device="cuda", dtype=torch.bfloat16), out, epilogue=1 | 6, bias=bias)
    torch.cuda.synchronize()
    x = bias.float()
    want = (x / (1 + torch.exp(-x))).to(torch.bfloat16)
    assert bool((out.float() - want.float()).abs().max() <= 0.02) and bool((out == out[0]).all())


@pytest.mark.parametrize("flags", [{}, {"bias": True}, {"bias": True, "gelu": True}, {"silu": True}, {"relu": True}])
def test_the_reference_library_kernel_runs_as_written(cuda, flags) -> None:
    """`matmul_epilogue[tiling](a, b, bias, out)` as the reference's own candidate launches it
    (src/krn/lib/lib_ours.py:70-75)."""
    device = krn.host.Device.current()
    rng = np.random.default_rng(33)
    m, n, k = 130, 136, 104
    a16, b16 = rng.uniform(-1, 1, (m, k)).astype(np.float16), rng.uniform(-1, 1, (k, n)).astype(np.float16)
    bias16 = rng.uniform(-2, 2, n).astype(np.float16)
    da, db, dbias = device.to_device(a16), device.to_device(b16), device.to_device(bias16)
    out = device.empty(krn.f16, m, n)
    tiling = K.MatmulTiling(**flags)
    assert ("krn_b200_matmul" if flags else "krn_b200_gemm_nn") in str(K.matmul_epilogue.explain(tiling, da, db, dbias, out))
    K.matmul_epilogue[tiling](da, db, dbias, out)
    device.default_stream.record().wait(60)
    code = (1 if flags.get("bias") else 0) | (2 if flags.get("relu") else 4 if flags.get("gelu") else 6 if flags.get("silu") else 0)
    want = o.matmul_epilogue(a16.view(np.uint16), b16.view(np.uint16), bias16.view(np.uint16), ab_type=o.F16, c_type=o.F16,
                             flags=code)
    close(values(out.to_host().view(np.uint16), "f16"), values(want, "f16"), "f16", k)
