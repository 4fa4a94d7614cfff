"""What the body of a kernel says about its launch: the iteration space.

The block tiles are found in the slices that load and store tensors: a slice that starts at
`block.index.<axis> * size` with extent `size` makes grid axis `axis` cover `size` elements of the dimension it
slices; extents are taken from the tensors the body STORES with that axis, else from those it loads; blocks are the
ceiling quotient, at least one; mixed tile sizes on one grid axis and tensors of different lengths along one axis are
`LaunchError`s (src/krn/compiler/space.py:93-213)."""

from __future__ import annotations

from collections import defaultdict
from typing import Any, Mapping, Sequence

from krn_b200.compiler import ir
from krn_b200.errors import LaunchError
from krn_b200.frontend.geometry import Blocks, Items, ceildiv
from krn_b200.frontend.types import Scalar


class Unreadable(Exception):
    """An extent reads something only the device has."""


def block_axis(tile: ir.SliceExpr) -> str | None:
    """The grid axis a slice follows when it is the tile of a block, `[block.index.<axis> * size, + size)`."""
    start = tile.start
    if isinstance(start, ir.Binary) and start.op == "*" and isinstance(start.lhs, ir.BlockIndex) \
            and isinstance(start.rhs, ir.Const):
        return start.lhs.axis if start.rhs.value == tile.extent else None
    if isinstance(start, ir.BlockIndex):
        return start.axis if tile.extent == 1 else None
    return None


def tile_uses(body: tuple[ir.Stmt, ...]):
    """Every tile of a global tensor the body loads or stores: (tensor, index, written)."""
    for statement in ir.walk(body):
        if isinstance(statement, ir.TileStore):
            yield statement.tensor, statement.index, True
        for expression in ir.expressions(statement):
            for found in ir.nested(expression):
                if isinstance(found, ir.TileLoad):
                    yield found.tensor, found.index, False


def iteration_space(body: tuple[ir.Stmt, ...]) -> tuple[ir.Axis, ...]:
    stored: dict[tuple[str, int], dict[ir.Expr, None]] = defaultdict(dict)
    loaded: dict[tuple[str, int], dict[ir.Expr, None]] = defaultdict(dict)
    for tensor, index, writes in tile_uses(body):
        for dimension, item in enumerate(index):
            if isinstance(item, ir.SliceExpr) and (grid := block_axis(item)) is not None:
                (stored if writes else loaded)[grid, item.extent][ir.Dim(tensor, dimension)] = None
    keys = dict.fromkeys((*stored, *loaded))
    return tuple(ir.Axis(grid, tile, tuple(stored.get((grid, tile)) or loaded[grid, tile])) for grid, tile in keys)


def operand(arguments: Mapping[str, Any], path: tuple[str, ...]) -> Any:
    value = arguments[path[0]]
    for name in path[1:]:
        value = value[name] if isinstance(value, Mapping) else getattr(value, name)
    return value


def evaluate(expression: ir.Expr, arguments: Mapping[str, Any]) -> int:
    """An extent on the arguments: constants, scalar parameters, tensor dimensions and integer arithmetic."""
    if isinstance(expression, ir.Const):
        return int(expression.value)
    if isinstance(expression, ir.Param):
        value = operand(arguments, expression.path)
        if isinstance(value, Scalar):
            return int(value.value)
        if hasattr(value, "shape"):
            raise Unreadable(f"the tensor `{expression.path[0]}`")
        return int(value)
    if isinstance(expression, ir.Dim):
        return int(arguments[expression.tensor].shape[expression.axis])
    if isinstance(expression, ir.Binary):
        a, b = evaluate(expression.lhs, arguments), evaluate(expression.rhs, arguments)
        return int({"+": a + b, "-": a - b, "*": a * b, "//": a // b if b else 0, "%": a % b if b else 0,
                    "<": a < b, "<=": a <= b, ">": a > b, ">=": a >= b, "==": a == b, "!=": a != b}[expression.op])
    if isinstance(expression, ir.LoopVar):
        raise Unreadable(f"the local variable `{expression.name}`")
    raise Unreadable(f"a {type(expression).__name__}")


def extent(kernel: ir.Kernel, axis: ir.Axis, arguments: Mapping[str, Any]) -> int:
    try:
        lengths = {evaluate(each, arguments) for each in axis.extents}
    except Unreadable as unreadable:
        raise LaunchError(kernel.name, f"its extent reads {unreadable}, which the host cannot evaluate") from None
    if len(lengths) > 1:
        raise LaunchError(kernel.name, f"the tensors it tiles along grid axis {axis.grid} have lengths {sorted(lengths)}")
    return lengths.pop()


def geometry(kernel: ir.Kernel, values: Sequence[Any]) -> Items | Blocks:
    """The launch the body of `kernel` asks for, from `values`, the arguments in parameter order."""
    strided = [axis for axis in kernel.space if axis.strided]
    tiled = [axis for axis in kernel.space if not axis.strided]
    if not kernel.space:
        raise LaunchError(kernel.name, "its body has no `items(n)` loop and slices no tensor with `block.tile`")
    if strided and tiled:
        raise LaunchError(kernel.name, "its body mixes `items(n)` loops with `block.tile` slices")
    arguments = dict(zip((name for name, _ in kernel.params), values, strict=True))
    if strided:
        return Items(max(1, *(extent(kernel, axis, arguments) for axis in strided)))
    blocks: dict[str, int] = {}
    for axis in tiled:
        if axis.grid in blocks:
            raise LaunchError(kernel.name, f"its body tiles grid axis {axis.grid} by more than one size")
        blocks[axis.grid] = max(1, ceildiv(extent(kernel, axis, arguments), axis.tile))
    return Blocks(blocks.get("x", 1), blocks.get("y", 1), blocks.get("z", 1))
