"""Element types and tensor annotations.

`bf16 = fp[8, 7]`, `f8e4m3fn = fp[4, 3, fn]` in the reference (src/krn/frontend/numerics.py:376-387); here each is a
`Dtype` singleton that also acts as a host scalar constructor (`T.f32(2.5)` boxes a value,
src/krn/frontend/numerics.py:52-69). `Matrix[T]` is rank 2, `Vector[T]` rank 1, `Tensor[T, int, int, int]` takes its
rank from the arity (src/krn/compiler/source.py:280-294)."""

from __future__ import annotations

from dataclasses import dataclass
from types import SimpleNamespace


@dataclass(frozen=True)
class Scalar:
    """A boxed host scalar: `T.f32(2.5)`."""

    dtype: "Dtype"
    value: float | int | bool

    def __float__(self) -> float:
        return float(self.value)

    def __int__(self) -> int:
        return int(self.value)


@dataclass(frozen=True)
class Dtype:
    name: str
    bits: int
    kind: str  # "f" float, "i" signed, "u" unsigned, "b" bool
    native: int | None = None  # element code of the kernel library (include/krn_b200.h), if it has one

    def __call__(self, value: float | int | bool) -> Scalar:
        return Scalar(self, value)

    def __repr__(self) -> str:
        return self.name

    @property
    def floating(self) -> bool:
        return self.kind == "f"


f64 = Dtype("f64", 64, "f")
f32 = Dtype("f32", 32, "f", native=0)
f16 = Dtype("f16", 16, "f", native=1)
bf16 = Dtype("bf16", 16, "f", native=2)
f8e4m3fn = Dtype("f8e4m3fn", 8, "f", native=3)
f8e5m2 = Dtype("f8e5m2", 8, "f")
i64, i32, i16, i8 = Dtype("i64", 64, "i"), Dtype("i32", 32, "i"), Dtype("i16", 16, "i"), Dtype("i8", 8, "i")
u64, u32, u16, u8 = Dtype("u64", 64, "u"), Dtype("u32", 32, "u"), Dtype("u16", 16, "u"), Dtype("u8", 8, "u")
boolean = Dtype("bool", 8, "b")

ALL = (f64, f32, f16, bf16, f8e4m3fn, f8e5m2, i64, i32, i16, i8, u64, u32, u16, u8, boolean)
T = SimpleNamespace(**{d.name: d for d in ALL})
BY_NAME = {d.name: d for d in ALL}


@dataclass(frozen=True)
class TensorType:
    """The annotation of a tensor parameter: element type and rank."""

    dtype: Dtype
    rank: int
    quantized: bool = False

    def __repr__(self) -> str:
        return f"Tensor[{self.dtype}, rank {self.rank}]"


class _Annotation:
    """`Matrix[T.bf16]`-style subscription producing a TensorType."""

    def __init__(self, name: str, rank: int | None, quantized: bool = False) -> None:
        self.name, self.rank, self.quantized = name, rank, quantized

    def __getitem__(self, item) -> TensorType:
        items = item if isinstance(item, tuple) else (item,)
        dtype = items[0]
        if not isinstance(dtype, Dtype):
            raise TypeError(f"{self.name}[...] takes an element type first, got {dtype!r}")
        rank = self.rank if self.rank is not None else len(items) - 1
        if rank < 1:
            raise TypeError(f"{self.name}[{dtype}, ...] needs one `int` per axis")
        return TensorType(dtype, rank, self.quantized)

    def __repr__(self) -> str:
        return self.name


Vector = _Annotation("Vector", 1)
Matrix = _Annotation("Matrix", 2)
Tensor = _Annotation("Tensor", None)
Tile = _Annotation("Tile", None)
QMatrix = _Annotation("QMatrix", 2, quantized=True)
QTile = _Annotation("QTile", None, quantized=True)
