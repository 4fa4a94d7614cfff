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
