"""A small typed IR for tile kernels: just what the tile matrix product and the flash-attention pattern need.

Names follow the reference's IR where the meaning is the same (`Accumulate`, `Transpose`, `TileLoad`, `TileStore`,
`For(pipelined, stages)`, `Reduce`, `Select`, `Arange`, `Axis`; src/krn/compiler/ir.py:231-427). Scalars are
capture-time Python values whenever they can be (configuration `Const` fields, literals), otherwise `Scalar`
expression nodes evaluated on the host for geometry or passed to the device as parameters."""

from __future__ import annotations

from dataclasses import dataclass, field

from krn_b200.errors import Span
from krn_b200.frontend.types import Dtype

# ---- scalar expressions ------------------------------------------------------------------------------------------


@dataclass(frozen=True)
class Expr:
    pass


@dataclass(frozen=True)
class Const(Expr):
    value: int | float | bool


@dataclass(frozen=True)
class Param(Expr):
    """A scalar kernel parameter, or a field of a struct parameter (`path` = parameter name, then field names)."""

    path: tuple[str, ...]
    dtype: Dtype | None = None


@dataclass(frozen=True)
class Dim(Expr):
    """`tensor.shape[axis]`."""

    tensor: str
    axis: int


@dataclass(frozen=True)
class BlockIndex(Expr):
    """`block.index().x/.y/.z`."""

    axis: str


@dataclass(frozen=True)
class LoopVar(Expr):
    name: str


@dataclass(frozen=True)
class Binary(Expr):
    op: str  # + - * // % < <= > >= == !=
    lhs: Expr
    rhs: Expr


@dataclass(frozen=True)
class SliceExpr(Expr):
    """`[start, start + extent)` with a capture-time constant extent."""

    start: Expr
    extent: int


# ---- tile expressions --------------------------------------------------------------------------------------------------


@dataclass(frozen=True)
class TileExpr:
    pass


@dataclass(frozen=True)
class TileLoad(TileExpr):
    tensor: str
    index: tuple[Expr, ...]  # SliceExpr for sliced axes, scalar Expr for squeezed ones
    dtype: Dtype
    shape: tuple[int, ...]


@dataclass(frozen=True)
class Var(TileExpr):
    name: str
    dtype: Dtype
    shape: tuple[int, ...]


@dataclass(frozen=True)
class Zeros(TileExpr):
    dtype: Dtype
    shape: tuple[int, ...]
    value: float = 0.0


@dataclass(frozen=True)
class Transpose(TileExpr):
    operand: TileExpr
    dtype: Dtype
    shape: tuple[int, ...]


@dataclass(frozen=True)
class Cast(TileExpr):
    operand: TileExpr
    dtype: Dtype
    shape: tuple[int, ...]


@dataclass(frozen=True)
class Math(TileExpr):
    """Elementwise arithmetic with broadcasting: fn in add, sub, mul, div, maximum, minimum, exp2, exp, neg."""

    fn: str
    operands: tuple["TileExpr | Expr", ...]
    dtype: Dtype
    shape: tuple[int, ...]


@dataclass(frozen=True)
class Compare(TileExpr):
    op: str
    lhs: "TileExpr | Expr"
    rhs: "TileExpr | Expr"
    dtype: Dtype
    shape: tuple[int, ...]


@dataclass(frozen=True)
class Select(TileExpr):
    cond: TileExpr
    then: "TileExpr | Expr"
    orelse: "TileExpr | Expr"
    dtype: Dtype
    shape: tuple[int, ...]


@dataclass(frozen=True)
class Arange(TileExpr):
    extent: int
    axis: int
    rank: int
    start: Expr
    dtype: Dtype
    shape: tuple[int, ...]


@dataclass(frozen=True)
class Reduce(TileExpr):
    op: str  # max, sum, min
    operand: TileExpr
    axis: int
    keepdims: bool
    dtype: Dtype
    shape: tuple[int, ...]


@dataclass(frozen=True)
class Product(TileExpr):
    """A fresh matrix product `lhs @ rhs` (f32 result)."""

    lhs: TileExpr
    rhs: TileExpr
    dtype: Dtype
    shape: tuple[int, ...]


# ---- statements ------------------------------------------------------------------------------------------------------------


@dataclass(frozen=True)
class Stmt:
    pass


@dataclass(frozen=True)
class Assign(Stmt):
    var: Var
    value: TileExpr
    span: Span | None = field(default=None, compare=False)


@dataclass(frozen=True)
class Accumulate(Stmt):
    """`acc += lhs @ rhs`: f32 accumulator of shape (m, n) (src/krn/compiler/ir.py:308-314)."""

    acc: Var
    lhs: TileExpr
    rhs: TileExpr
    span: Span | None = field(default=None, compare=False)


@dataclass(frozen=True)
class For(Stmt):
    var: str
    start: Expr
    stop: Expr
    step: int
    body: tuple[Stmt, ...]
    pipelined: bool = False
    stages: int = 0
    schedule: object = None
    span: Span | None = field(default=None, compare=False)


@dataclass(frozen=True)
class TileStore(Stmt):
    tensor: str
    index: tuple[Expr, ...]
    value: TileExpr
    span: Span | None = field(default=None, compare=False)


# ---- kernel --------------------------------------------------------------------------------------------------------------


@dataclass(frozen=True)
class Axis:
    """One axis of the iteration space: grid axis `grid` covers `tile` elements per block of the dimensions in
    `extents` (src/krn/compiler/ir.py:399-412)."""

    grid: str
    tile: int
    extents: tuple[Expr, ...]
    strided: bool = False


@dataclass(frozen=True)
class TensorParam:
    name: str
    dtype: Dtype
    rank: int


@dataclass(frozen=True)
class Kernel:
    name: str
    params: tuple[tuple[str, object], ...]  # (name, TensorParam | Dtype (scalar) | "config")
    body: tuple[Stmt, ...]
    space: tuple[Axis, ...]
    file: str = ""

    def tensor(self, name: str) -> TensorParam:
        for param_name, kind in self.params:
            if param_name == name and isinstance(kind, TensorParam):
                return kind
        raise KeyError(name)


def walk(body: tuple[Stmt, ...]):
    """Every statement, outer before inner."""
    for statement in body:
        yield statement
        if isinstance(statement, For):
            yield from walk(statement.body)


def children(e):
    """The tile/scalar sub-expressions of an expression node."""
    if isinstance(e, (Transpose, Cast)):
        return (e.operand,)
    if isinstance(e, Math):
        return e.operands
    if isinstance(e, Compare):
        return (e.lhs, e.rhs)
    if isinstance(e, Select):
        return (e.cond, e.then, e.orelse)
    if isinstance(e, Reduce):
        return (e.operand,)
    if isinstance(e, Product):
        return (e.lhs, e.rhs)
    if isinstance(e, Arange):
        return (e.start,)
    if isinstance(e, Binary):
        return (e.lhs, e.rhs)
    if isinstance(e, SliceExpr):
        return (e.start,)
    if isinstance(e, TileLoad):
        return e.index
    return ()


def nested(e):
    """The expression and every expression inside it."""
    yield e
    for child in children(e):
        yield from nested(child)


def expressions(statement: Stmt):
    """The expressions a statement holds directly."""
    if isinstance(statement, Assign):
        yield statement.value
    elif isinstance(statement, Accumulate):
        yield statement.lhs
        yield statement.rhs
    elif isinstance(statement, TileStore):
        yield from statement.index
        yield statement.value
    elif isinstance(statement, For):
        yield statement.start
        yield statement.stop
