"""Number formats as data: what the block-scaled FP8 path needs of src/krn/data/formats.py (E4M3FN: bias 7, finite,
0x7F/0xFF NaN, max 448, :59-95; FP8FN: e4m3 elements with one fp32 scale per 1x128 block, :157-164)."""

from __future__ import annotations

import math
from dataclasses import dataclass
from functools import cached_property


@dataclass(frozen=True)
class FloatFormat:
    exp_bits: int
    man_bits: int
    finite_only: bool = False

    @property
    def bits(self) -> int:
        return 1 + self.exp_bits + self.man_bits

    @property
    def exp_bias(self) -> int:
        return 2 ** (self.exp_bits - 1) - 1

    def decode(self, code: int) -> float:
        man = code & ((1 << self.man_bits) - 1)
        exp = (code >> self.man_bits) & ((1 << self.exp_bits) - 1)
        sign = -1.0 if code >> (self.man_bits + self.exp_bits) else 1.0
        top = (1 << self.exp_bits) - 1
        if self.finite_only:
            if exp == top and man == (1 << self.man_bits) - 1:
                return math.nan
        elif exp == top:
            return math.nan if man else sign * math.inf
        if exp == 0:
            return sign * man * 2.0 ** (1 - self.exp_bias - self.man_bits)
        return sign * (1 + man / (1 << self.man_bits)) * 2.0 ** (exp - self.exp_bias)

    @cached_property
    def table(self) -> tuple:
        return tuple(self.decode(code) for code in range(1 << self.bits))

    @property
    def max(self) -> float:
        return max(v for v in self.table if math.isfinite(v))


E4M3FN = FloatFormat(4, 3, finite_only=True)
E5M2 = FloatFormat(5, 2)


@dataclass(frozen=True)
class BlockFormat:
    """Elements of `element` with one `scale` per `block` (rows x columns) of the matrix."""

    element: FloatFormat
    block: tuple
    scale: str = "f32"


def FP8FN() -> BlockFormat:
    """e4m3fn elements, one fp32 scale per 1x128 block: the activation-side format of the block-scaled product."""
    return BlockFormat(E4M3FN, (1, 128))


def FP8FN_WEIGHTS() -> BlockFormat:
    """e4m3fn elements, one fp32 scale per 128x128 block: the weight-side format of the block-scaled product."""
    return BlockFormat(E4M3FN, (128, 128))
