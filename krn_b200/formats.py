"""Number formats as plain data, for the block-scaled part of the path.

The names and constructor fields follow the reference's format module (src/krn/data/formats.py:41-164) so that code
written against `krn.formats` keeps working: `FloatFormat(exp_bits, man_bits, signed, special, bias, subnormals)` with
`.bits / .exp_bias / .decode / .table / .max`, and `BlockFormat(elem, scale, block, storage, tensor_scale,
scale_rounding)` with the named block formats below. The decoding itself is written from the formats' definitions:

* a code is split into sign | exponent field E | mantissa field M;
* the top exponent field is special in a way that depends on the family — IEEE: inf (M = 0) or NaN; FN ("finite,
  NaN only"): just the all-ones code is NaN, e.g. e4m3fn 0x7F / 0xFF; FNU: the same for unsigned formats (e8m0's 0xFF);
  FNUZ: only sign-bit-alone is NaN, there is no negative zero and the bias is one larger; NONE: every code is a number;
* otherwise the value is (-1)^s * 2^(E - bias) * (1 + M / 2^m), or, when E = 0 and the format has subnormals,
  (-1)^s * 2^(1 - bias) * (M / 2^m).

Formats the kernels of this package consume: `FP8FN` (e4m3fn codes, one f32 scale per 1 x 128 block, the activation
side of the block-scaled product), `FP8FNWeights` (the same with 128 x 128 blocks: the weight side of that product,
which is NOT one of the reference's formats) and `MXFP8` (e4m3fn codes, one e8m0 power-of-two scale per 1 x 32
block, which the tensor cores apply themselves).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from enum import StrEnum, auto
from functools import cached_property
from typing import ClassVar


class Special(StrEnum):
    """What the all-ones exponent field (or, for FNUZ, the lone sign bit) means."""

    IEEE = auto()
    FN = auto()
    FNUZ = auto()
    FNU = auto()
    NONE = auto()


class Rounding(StrEnum):
    NEAREST_EVEN = auto()
    STOCHASTIC = auto()
    TOWARD_ZERO = auto()


class ScaleRounding(StrEnum):
    """How a block's scale is derived from its largest magnitude."""

    FLOOR = auto()    # 2^(floor(log2 amax) - emax of the element format): the OCP MX rule
    CEIL = auto()     # the next power of two up, so no element can overflow
    NEAREST = auto()  # amax / element max rounded into a scale format that has mantissa bits


class Storage(StrEnum):
    """How codes sit in bytes."""

    BYTE = auto()       # one code per byte
    X2 = auto()         # two 4-bit codes per byte, low nibble first
    BITPACKED = auto()  # codes packed bit by bit along the block axis


@dataclass(frozen=True)
class FloatFormat:
    exp_bits: int
    man_bits: int
    signed: bool = True
    special: Special = Special.IEEE
    bias: int | None = None
    subnormals: bool = True

    @property
    def bits(self) -> int:
        return self.exp_bits + self.man_bits + (1 if self.signed else 0)

    @property
    def exp_bias(self) -> int:
        if self.bias is not None:
            return self.bias
        ieee_bias = (1 << (self.exp_bits - 1)) - 1
        return ieee_bias + 1 if self.special is Special.FNUZ else ieee_bias

    def _fields(self, code: int) -> tuple[int, int, int]:
        """(sign bit, exponent field, mantissa field) of a code."""
        rest, mantissa = divmod(code, 1 << self.man_bits)
        sign, exponent = divmod(rest, 1 << self.exp_bits)
        return (sign & 1 if self.signed else 0), exponent, mantissa

    def _is_nan(self, code: int, exponent: int, mantissa: int) -> bool:
        all_ones_exponent = exponent == (1 << self.exp_bits) - 1
        all_ones_mantissa = mantissa == (1 << self.man_bits) - 1
        if self.special is Special.IEEE:
            return all_ones_exponent and mantissa != 0
        if self.special in (Special.FN, Special.FNU):
            return all_ones_exponent and all_ones_mantissa
        if self.special is Special.FNUZ:
            return code == 1 << (self.bits - 1)
        return False

    def decode(self, code: int) -> float:
        """The real number (or inf / NaN) that `code` stands for."""
        sign, exponent, mantissa = self._fields(code)
        if self._is_nan(code, exponent, mantissa):
            return math.nan
        negate = -1.0 if sign else 1.0
        if self.special is Special.IEEE and exponent == (1 << self.exp_bits) - 1:
            return negate * math.inf
        fraction = mantissa / (1 << self.man_bits)
        if exponent == 0 and self.subnormals:
            return negate * math.ldexp(fraction, 1 - self.exp_bias)
        return negate * math.ldexp(1.0 + fraction, exponent - self.exp_bias)

    @cached_property
    def table(self) -> tuple[float, ...]:
        """Every code's value, indexed by code."""
        return tuple(map(self.decode, range(1 << self.bits)))

    @property
    def max(self) -> float:
        """The largest finite value."""
        return max(filter(math.isfinite, self.table))


@dataclass(frozen=True)
class IntFormat:
    bits: int
    signed: bool = True


E5M2 = FloatFormat(5, 2)
E4M3 = FloatFormat(4, 3)
E4M3FN = FloatFormat(4, 3, special=Special.FN)
E4M3FNUZ = FloatFormat(4, 3, special=Special.FNUZ)
E5M2FNUZ = FloatFormat(5, 2, special=Special.FNUZ)
E8M0 = FloatFormat(8, 0, signed=False, special=Special.FNU, bias=127, subnormals=False)
UE5M3 = FloatFormat(5, 3, signed=False, special=Special.FNU)
E2M1 = FloatFormat(2, 1, special=Special.NONE)
E2M3 = FloatFormat(2, 3, special=Special.NONE)
E3M2 = FloatFormat(3, 2, special=Special.NONE)
FP32 = FloatFormat(8, 23)
BF16 = FloatFormat(8, 7)
FP16 = FloatFormat(5, 10)


@dataclass(frozen=True, slots=True)
class BlockFormat:
    """Codes of `elem` with one `scale` per `block` = (rows, columns) of the matrix; (1, 32) is 32 consecutive
    values of a row. `scale=None` means unscaled storage of `elem`."""

    name: ClassVar[str] = "custom"
    elem: FloatFormat | IntFormat
    scale: FloatFormat | None
    block: tuple[int, int]
    storage: Storage = Storage.BYTE
    tensor_scale: FloatFormat | None = None
    scale_rounding: ScaleRounding = ScaleRounding.FLOOR

    @property
    def bits_per_value(self) -> float:
        """Storage cost of one value including its share of the block scale."""
        rows, columns = self.block
        overhead = self.scale.bits / (rows * columns) if self.scale is not None else 0.0
        return self.elem.bits + overhead


@dataclass(frozen=True, slots=True)
class MXFP4(BlockFormat):
    name: ClassVar[str] = "mxfp4"
    elem: FloatFormat = E2M1
    scale: FloatFormat = E8M0
    block: tuple[int, int] = (1, 32)
    storage: Storage = Storage.X2


@dataclass(frozen=True, slots=True)
class MXFP8(BlockFormat):
    """OCP MX: e4m3fn codes and one e8m0 (power of two) scale per 32 consecutive values of a row."""

    name: ClassVar[str] = "mxfp8"
    elem: FloatFormat = E4M3FN
    scale: FloatFormat = E8M0
    block: tuple[int, int] = (1, 32)


@dataclass(frozen=True, slots=True)
class NVFP4(BlockFormat):
    name: ClassVar[str] = "nvfp4"
    elem: FloatFormat = E2M1
    scale: FloatFormat = E4M3FN
    block: tuple[int, int] = (1, 16)
    storage: Storage = Storage.X2
    tensor_scale: FloatFormat | None = FP32
    scale_rounding: ScaleRounding = ScaleRounding.NEAREST


@dataclass(frozen=True, slots=True)
class FP8FN(BlockFormat):
    """e4m3fn codes with one float32 scale per 1 x 128 block."""

    name: ClassVar[str] = "fp8-fn"
    elem: FloatFormat = E4M3FN
    scale: FloatFormat | None = FP32
    block: tuple[int, int] = (1, 128)


@dataclass(frozen=True, slots=True)
class FP8FNWeights(BlockFormat):
    """e4m3fn codes with one float32 scale per 128 x 128 block: the weight operand of this package's block-scaled
    product. Not a format of the reference (its FP8FN is 1 x 128 on both sides)."""

    name: ClassVar[str] = "fp8-fn-128x128"
    elem: FloatFormat = E4M3FN
    scale: FloatFormat | None = FP32
    block: tuple[int, int] = (128, 128)


@dataclass(frozen=True, slots=True)
class FP8FNUZ(BlockFormat):
    name: ClassVar[str] = "fp8-fnuz"
    elem: FloatFormat = E4M3FNUZ
    scale: FloatFormat | None = FP32
    block: tuple[int, int] = (1, 128)


@dataclass(frozen=True, slots=True)
class Plain16(BlockFormat):
    name: ClassVar[str] = "fp16"
    elem: FloatFormat = FP16
    scale: FloatFormat | None = None
    block: tuple[int, int] = (1, 1)


@dataclass(frozen=True, slots=True)
class PlainBF16(BlockFormat):
    name: ClassVar[str] = "bf16"
    elem: FloatFormat = BF16
    scale: FloatFormat | None = None
    block: tuple[int, int] = (1, 1)


@dataclass(frozen=True, slots=True)
class Plain32(BlockFormat):
    name: ClassVar[str] = "fp32"
    elem: FloatFormat = FP32
    scale: FloatFormat | None = None
    block: tuple[int, int] = (1, 1)


FP8FN_WEIGHTS = FP8FNWeights  # earlier spelling of the same constructor
