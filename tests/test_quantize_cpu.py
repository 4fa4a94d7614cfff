"""Host-side quantisers of the block formats against the oracle's: same codes, same scales. CPU only."""

from __future__ import annotations

import numpy as np
import pytest

import krn_b200 as krn
from krn_b200 import ops
from oracle import oracle as o


def sample(rows: int, cols: int, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, cols), np.float32) * np.exp2(rng.integers(-9, 9, (rows, 1))).astype(np.float32)
    x[3, 32:64] = 0  # a block of zeros
    x[5, 7] = 1e6    # far beyond its block-mates
    return x


def test_fp8fn_quantisers_match_the_oracle() -> None:
    x = sample(256, 384, 1)
    codes, scales = ops.quantize_host(x, krn.formats.FP8FN())
    want_codes, want_scales = o.quantize_blocks(x, (1, 128))
    np.testing.assert_array_equal(codes, want_codes)
    np.testing.assert_array_equal(scales, want_scales)
    codes, scales = ops.quantize_host(x, krn.formats.FP8FNWeights())
    want_codes, want_scales = o.quantize_blocks(x, (128, 128))
    np.testing.assert_array_equal(codes, want_codes)
    np.testing.assert_array_equal(scales, want_scales)


def test_mxfp8_quantiser_matches_the_oracle_and_the_format_tables() -> None:
    x = sample(64, 256, 2)
    codes, scales = ops.quantize_host(x, krn.formats.MXFP8())
    want_codes, want_scales = o.quantize_mxfp8(x)
    np.testing.assert_array_equal(codes, want_codes)
    np.testing.assert_array_equal(scales, want_scales)
    assert scales.dtype == np.uint8 and scales.shape == (64, 8)
    # decoded through the format definitions themselves (E4M3FN and E8M0 tables) the values are the oracle's, and
    # every block's largest element lands in the top binade of e4m3 or below (the floor rule never overflows by more
    # than the saturation it allows)
    e4m3, e8m0 = np.array(krn.formats.E4M3FN.table), np.array(krn.formats.E8M0.table)
    values = e4m3[codes] * np.repeat(e8m0[scales], 32, axis=1)
    np.testing.assert_array_equal(values, o.mxfp8_values(codes, scales))
    live = np.abs(x).reshape(64, 8, 32).max(axis=2) > 0
    error = np.abs(values - x).reshape(64, 8, 32).max(axis=2)[live] / np.abs(x).reshape(64, 8, 32).max(axis=2)[live]
    assert error.max() < 0.13  # half a step of a 3-bit mantissa in the top binade, plus saturation from 480 to 448


def test_quantiser_refusals() -> None:
    with pytest.raises(ValueError, match="whole 1 x 32 blocks"):
        ops.quantize_host(np.zeros((4, 48), np.float32), krn.formats.MXFP8())
    with pytest.raises(ValueError, match="e4m3fn elements"):
        ops.quantize_host(np.zeros((4, 64), np.float32), krn.formats.NVFP4())


def test_nvfp4_quantiser_matches_the_oracle_and_the_format_tables() -> None:
    """The product side's NVFP4 quantiser and the oracle's agree code for code; the e2m1 and e4m3 values both use are the
    format tables (`krn.formats.E2M1`, `E4M3FN`: the reference's src/krn/data/formats.py:95,100)."""
    x = np.random.default_rng(14).standard_normal((24, 256)).astype(np.float32) * 3
    packed, scales, tensor_scale = ops.quantize_nvfp4_host(x)
    want_packed, want_scales, want_tensor = o.quantize_nvfp4(x)
    np.testing.assert_array_equal(packed, want_packed)
    np.testing.assert_array_equal(scales, want_scales)
    assert tensor_scale == want_tensor
    assert [float(v) for v in o.e2m1_decode(np.arange(16))] == [float(v) for v in krn.formats.E2M1.table]
    codes = o.unpack_nibbles(packed)
    table = np.array(krn.formats.E2M1.table)
    scale_table = np.array(krn.formats.E4M3FN.table)
    values = table[codes] * np.repeat(scale_table[scales], 16, axis=1) * tensor_scale
    np.testing.assert_allclose(values, o.nvfp4_values(packed, scales, tensor_scale), rtol=1e-7)
    # 4-bit elements with an e4m3 scale per 16: the block maximum is reproduced to the scale's precision (6.25 %), the rest
    # to half a step of the element grid
    assert np.linalg.norm(values - x) / np.linalg.norm(x) < 0.12
    # every e2m1 magnitude is its own code, ties go to the even mantissa bit
    grid = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float32)
    np.testing.assert_array_equal(o.e2m1_decode(o.e2m1_encode(grid)), grid)
    np.testing.assert_array_equal(o.e2m1_decode(o.e2m1_encode(np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -9.0], np.float32))),
                                  np.array([0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, -6.0], np.float32))
    with pytest.raises(ValueError, match="whole 1 x 16 blocks"):
        ops.quantize_nvfp4_host(np.zeros((4, 24), np.float32))


def test_mxfp4_quantiser_matches_the_oracle() -> None:
    x = np.random.default_rng(15).standard_normal((24, 256)).astype(np.float32) * 5
    packed, scales = ops.quantize_mxfp4_host(x)
    want_packed, want_scales = o.quantize_mxfp4(x)
    np.testing.assert_array_equal(packed, want_packed)
    np.testing.assert_array_equal(scales, want_scales)
    table = np.array(krn.formats.E2M1.table)
    values = table[o.unpack_nibbles(packed)] * np.repeat(np.exp2(scales.astype(np.float64) - 127), 32, axis=1)
    np.testing.assert_array_equal(values, o.mxfp4_values(packed, scales))
    assert np.abs(values).max() <= np.abs(x).max() * 1.51  # the floor rule may leave the block maximum up to 1.5x above 6 * scale: it saturates
    assert np.linalg.norm(values - x) / np.linalg.norm(x) < 0.16
    with pytest.raises(ValueError, match="whole 1 x 32 blocks"):
        ops.quantize_mxfp4_host(np.zeros((4, 48), np.float32))
