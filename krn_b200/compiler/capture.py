"""Capture: read a `@kernel` function's source with `ast` (the function is never run), type-check the tile
subset and build the IR of `krn_b200.compiler.ir`.

The reference does the same in one pass over the AST (src/krn/compiler/source.py:96-321,
src/krn/compiler/capture.py:427-457); this capture covers what the tile matrix product and the flash-attention
pattern are written with: `block.tile`, `block.index`, `zeros`, `pipelined`/`range` loops, tensor slicing with
capture-time extents (src/krn/compiler/capture.py:925-997), `@`, `.transpose()`, `.to()`, elementwise arithmetic,
`exp2`, `.relu()` / `.gelu()` / `.silu()`, row reductions, `where`, `arange`, `maximum`, static `if` on configuration
constants, tile stores.
Anything else is refused with a `CaptureError` at the user's line."""

from __future__ import annotations

import ast
import inspect
import textwrap
from dataclasses import fields, is_dataclass
from typing import Any

from krn_b200.compiler import ir
from krn_b200.compiler.space import iteration_space
from krn_b200.errors import CaptureError, Span, TargetError
from krn_b200.frontend import device_functions as df
from krn_b200.frontend.records import AUTO, is_configuration, is_const
from krn_b200.frontend.types import Dtype, Scalar, TensorType, boolean, f32, f64, i32

FLOAT_OPERANDS = {"f16", "bf16", "f32", "f8e4m3fn", "f8e5m2"}


class _Shape:
    """`tensor.shape`: indexing gives a `Dim`."""

    def __init__(self, tensor: str, rank: int) -> None:
        self.tensor, self.rank = tensor, rank


class _Tensor:
    def __init__(self, param: ir.TensorParam) -> None:
        self.param = param


class _Index3:
    """`block.index()`."""


def _is_tile(value: Any) -> bool:
    return isinstance(value, ir.TileExpr)


def _fold(op: str, a: Any, b: Any) -> Any:
    """Scalar arithmetic: Python numbers fold, anything symbolic builds a Binary."""
    if isinstance(a, Scalar):
        a = a.value
    if isinstance(b, Scalar):
        b = b.value
    numeric = (int, float, bool)
    if isinstance(a, numeric) and isinstance(b, numeric):
        return {"+": lambda: a + b, "-": lambda: a - b, "*": lambda: a * b, "//": lambda: a // b, "%": lambda: a % b,
                "/": lambda: a / b, "<": lambda: a < b, "<=": lambda: a <= b, ">": lambda: a > b, ">=": lambda: a >= b,
                "==": lambda: a == b, "!=": lambda: a != b}[op]()
    lhs = a if isinstance(a, ir.Expr) else ir.Const(a)
    rhs = b if isinstance(b, ir.Expr) else ir.Const(b)
    if op == "+" and rhs == ir.Const(0):
        return lhs
    if op == "+" and lhs == ir.Const(0):
        return rhs
    if op == "*" and rhs == ir.Const(1):
        return lhs
    return ir.Binary(op, lhs, rhs)


def _as_expr(value: Any) -> ir.Expr:
    if isinstance(value, ir.Expr):
        return value
    if isinstance(value, Scalar):
        return ir.Const(value.value)
    return ir.Const(value)


def _difference(stop: Any, start: Any) -> int | None:
    """`stop - start` when it is a capture-time constant: both numbers, or `stop` spelled `start + C`."""
    if isinstance(stop, (int, bool)) and isinstance(start, (int, bool)):
        return int(stop) - int(start)
    if isinstance(stop, ir.Binary) and stop.op == "+":
        if stop.lhs == _as_expr(start) and isinstance(stop.rhs, ir.Const):
            return int(stop.rhs.value)
        if stop.rhs == _as_expr(start) and isinstance(stop.lhs, ir.Const):
            return int(stop.lhs.value)
    return None


def _broadcast(a: tuple[int, ...], b: tuple[int, ...]) -> tuple[int, ...] | None:
    """numpy's rule: shapes align at the last axis, missing leading axes count as 1 (`acc += bias[cols]` adds a row
    vector to every row of the accumulator, src/krn/lib/lib_kernels.py:40-41)."""
    rank = max(len(a), len(b))
    a, b = (1,) * (rank - len(a)) + tuple(a), (1,) * (rank - len(b)) + tuple(b)
    out = []
    for x, y in zip(a, b):
        if x == y or y == 1:
            out.append(x)
        elif x == 1:
            out.append(y)
        else:
            return None
    return tuple(out)


class Builder:
    def __init__(self, fn, config: Any | None) -> None:
        self.fn = fn
        self.file = inspect.getsourcefile(fn) or "<kernel>"
        source, first_line = inspect.getsourcelines(fn)
        tree = ast.parse(textwrap.dedent("".join(source)))
        ast.increment_lineno(tree, first_line - 1)
        self.node = next(n for n in ast.walk(tree) if isinstance(n, ast.FunctionDef) and n.name == fn.__name__)
        self.globals = dict(fn.__globals__)
        if fn.__closure__:
            self.globals.update({name: cell.cell_contents for name, cell in zip(fn.__code__.co_freevars, fn.__closure__)})
        self.env: dict[str, Any] = {}
        self.config = config
        self.params: list[tuple[str, object]] = []
        self.temporaries = 0

    # ---- diagnostics -----------------------------------------------------------------------------------------------

    def span(self, node: ast.AST) -> Span:
        return Span.of(self.file, node)

    def error(self, node: ast.AST, message: str) -> CaptureError:
        return CaptureError(self.span(node), message)

    # ---- entry -------------------------------------------------------------------------------------------------------

    def kernel(self) -> ir.Kernel:
        signature = inspect.signature(self.fn)
        for index, (name, parameter) in enumerate(signature.parameters.items()):
            annotation = parameter.annotation
            if isinstance(annotation, str):
                annotation = eval(annotation, self.globals)  # noqa: S307 - the user's own annotation text
            if isinstance(annotation, TensorType):
                param = ir.TensorParam(name, annotation.dtype, annotation.rank)
                self.params.append((name, param))
                self.env[name] = _Tensor(param)
            elif isinstance(annotation, Dtype):
                self.params.append((name, annotation))
                self.env[name] = ir.Param((name,), annotation)
            elif index == 0 and is_configuration(annotation):
                if self.config is None:
                    try:
                        self.config = annotation()
                    except TypeError:
                        raise TypeError(f"{self.fn.__name__}: configuration needs arguments; write "
                                        f"{self.fn.__name__}[Config(...)](...)") from None
                if not isinstance(self.config, annotation):
                    raise TypeError(f"{self.fn.__name__}: expected a {annotation.__name__} configuration")
                self.params.append((name, "config"))
                self.env[name] = self.config
            else:
                raise CaptureError(Span(self.file, self.node.lineno, 1),
                                   f"parameter `{name}` needs a tensor, scalar or configuration annotation")
        body = self.block(self.node.body)
        return ir.Kernel(self.fn.__name__, tuple(self.params), body, iteration_space(body), self.file)

    # ---- statements ------------------------------------------------------------------------------------------------

    def block(self, statements: list[ast.stmt]) -> tuple[ir.Stmt, ...]:
        out: list[ir.Stmt] = []
        for statement in statements:
            out.extend(self.statement(statement))
        return tuple(out)

    def statement(self, s: ast.stmt) -> list[ir.Stmt]:
        if isinstance(s, ast.Expr) and isinstance(s.value, ast.Constant):
            return []  # docstring
        if isinstance(s, ast.Pass):
            return []
        if isinstance(s, ast.Return):
            if s.value is not None and not (isinstance(s.value, ast.Constant) and s.value.value is None):
                raise self.error(s, "an entry kernel returns None")
            return []
        if isinstance(s, ast.Assign):
            if len(s.targets) != 1:
                raise self.error(s, "chained assignment is not supported in a tile kernel")
            return self.assign(s.targets[0], self.expr(s.value), s)
        if isinstance(s, ast.AnnAssign) and s.value is not None:
            return self.assign(s.target, self.expr(s.value), s)
        if isinstance(s, ast.AugAssign):
            return self.augmented(s)
        if isinstance(s, ast.For):
            return [self.loop(s)]
        if isinstance(s, ast.If):
            condition = self.expr(s.test)
            if isinstance(condition, Scalar):
                condition = condition.value
            if not isinstance(condition, (bool, int)):
                raise self.error(s.test, "an `if` in a tile kernel must test a capture-time constant "
                                         "(a Const field of the configuration); use `where` for data")
            return list(self.block(s.body if condition else s.orelse))
        raise self.error(s, f"{type(s).__name__} statements are not part of the tile subset")

    def assign(self, target: ast.expr, value: Any, node: ast.stmt) -> list[ir.Stmt]:
        if isinstance(target, ast.Tuple):
            if not isinstance(value, tuple) or len(value) != len(target.elts):
                raise self.error(node, "cannot unpack this value")
            out: list[ir.Stmt] = []
            for element, item in zip(target.elts, value):
                out.extend(self.assign(element, item, node))
            return out
        if isinstance(target, ast.Name):
            if _is_tile(value):
                previous = self.env.get(target.id)
                if isinstance(previous, ir.Var) and (previous.dtype, previous.shape) != (value.dtype, value.shape):
                    raise self.error(node, f"`{target.id}` was a {previous.dtype}{list(previous.shape)} tile and is "
                                           f"assigned a {value.dtype}{list(value.shape)} tile")
                var = ir.Var(target.id, value.dtype, value.shape)
                self.env[target.id] = var
                return [ir.Assign(var, value, self.span(node))]
            self.env[target.id] = value
            return []
        if isinstance(target, ast.Subscript):
            tensor = self.expr(target.value)
            if not isinstance(tensor, _Tensor):
                raise self.error(target, "only a global tensor can be stored into")
            index, shape = self.index(tensor, target.slice, target)
            if not _is_tile(value):
                raise self.error(node, "a tile store needs a tile on the right")
            if value.shape != shape:
                raise self.error(node, f"a {list(value.shape)} tile does not fit the {list(shape)} slice")
            if value.dtype != tensor.param.dtype:
                raise self.error(node, f"`{tensor.param.name}` holds {tensor.param.dtype}, the tile is {value.dtype}: "
                                       f"convert it with .to({tensor.param.dtype})")
            return [ir.TileStore(tensor.param.name, index, value, self.span(node))]
        raise self.error(target, "unsupported assignment target")

    def augmented(self, s: ast.AugAssign) -> list[ir.Stmt]:
        if not isinstance(s.target, ast.Name):
            raise self.error(s, "augmented assignment needs a plain name on the left")
        current = self.env.get(s.target.id)
        value = self.expr(s.value)
        if isinstance(s.op, ast.Add) and isinstance(value, ir.Product) and isinstance(current, ir.Var):
            if current.dtype != f32 or current.shape != value.shape:
                raise self.error(s, f"the accumulator of a matrix product must be an f32 {list(value.shape)} tile, "
                                    f"`{current.name}` is {current.dtype}{list(current.shape)}")
            return [ir.Accumulate(current, value.lhs, value.rhs, self.span(s))]
        op = {ast.Add: "add", ast.Sub: "sub", ast.Mult: "mul", ast.Div: "div"}.get(type(s.op))
        if op is None:
            raise self.error(s, "this augmented operator is not supported on tiles")
        if _is_tile(current):
            return self.assign(s.target, self.math(op, [current, value], s), s)
        symbol = {"add": "+", "sub": "-", "mul": "*", "div": "/"}[op]
        self.env[s.target.id] = _fold(symbol, current, value)
        return []

    def loop(self, s: ast.For) -> ir.For:
        if not isinstance(s.target, ast.Name) or s.orelse:
            raise self.error(s, "a tile loop has one loop variable and no else clause")
        if not isinstance(s.iter, ast.Call):
            raise self.error(s.iter, "loop over `pipelined(extent, tile)` or `range(start, stop, step)`")
        callee = self.expr(s.iter.func)
        args = [self.expr(a) for a in s.iter.args]
        keywords = {k.arg: self.expr(k.value) for k in s.iter.keywords}
        name = s.target.id
        if callee is df.pipelined or callee is df.chunks:
            if len(args) != 2 or not isinstance(args[1], int):
                raise self.error(s.iter, "pipelined(extent, tile): the tile size must be a capture-time constant")
            stages = keywords.get("stages", AUTO)
            schedule = keywords.get("schedule", AUTO)
            if stages is not AUTO and (not isinstance(stages, int) or stages < 2 or stages > 8):
                raise self.error(s.iter, "stages must be AUTO or an integer from 2 to 8")
            self.env[name] = ir.SliceExpr(ir.LoopVar(name), args[1])
            body = self.block(s.body)
            return ir.For(name, ir.Const(0), _as_expr(args[0]), args[1], body, callee is df.pipelined,
                          0 if stages is AUTO else stages, None if schedule is AUTO else schedule, self.span(s))
        if callee is range:
            if len(args) == 1:
                args = [0, args[0], 1]
            elif len(args) == 2:
                args = [args[0], args[1], 1]
            if len(args) != 3 or not isinstance(args[2], int) or args[2] <= 0:
                raise self.error(s.iter, "range(start, stop, step) needs a positive capture-time step")
            self.env[name] = ir.LoopVar(name)
            body = self.block(s.body)
            return ir.For(name, _as_expr(args[0]), _as_expr(args[1]), args[2], body, False, 0, None, self.span(s))
        raise self.error(s.iter, "loop over `pipelined(extent, tile)` or `range(start, stop, step)`")

    # ---- expressions -----------------------------------------------------------------------------------------------

    def expr(self, e: ast.expr) -> Any:
        if isinstance(e, ast.Constant):
            return e.value
        if isinstance(e, ast.Name):
            if e.id in self.env:
                return self.env[e.id]
            if e.id in self.globals:
                return self.globals[e.id]
            if e.id in ("range", "slice", "min", "max", "int", "float", "bool", "len"):
                return {"range": range, "slice": slice, "min": min, "max": max, "int": int, "float": float,
                        "bool": bool, "len": len}[e.id]
            raise self.error(e, f"unknown name `{e.id}`")
        if isinstance(e, ast.Tuple):
            return tuple(self.expr(x) for x in e.elts)
        if isinstance(e, ast.Attribute):
            return self.attribute(e)
        if isinstance(e, ast.Subscript):
            return self.subscript(e)
        if isinstance(e, ast.Call):
            return self.call(e)
        if isinstance(e, ast.BinOp):
            return self.binary(e)
        if isinstance(e, ast.UnaryOp):
            operand = self.expr(e.operand)
            if isinstance(e.op, ast.USub):
                if _is_tile(operand):
                    return self.math("neg", [operand], e)
                return _fold("-", 0, operand)
            if isinstance(e.op, ast.Not) and isinstance(operand, (bool, int)):
                return not operand
            raise self.error(e, "unsupported unary operator")
        if isinstance(e, ast.Compare):
            if len(e.ops) != 1:
                raise self.error(e, "chained comparisons are not supported")
            op = {ast.Lt: "<", ast.LtE: "<=", ast.Gt: ">", ast.GtE: ">=", ast.Eq: "==", ast.NotEq: "!="}.get(type(e.ops[0]))
            if op is None:
                raise self.error(e, "unsupported comparison")
            lhs, rhs = self.expr(e.left), self.expr(e.comparators[0])
            if _is_tile(lhs) or _is_tile(rhs):
                shape = self.common_shape(lhs, rhs, e)
                return ir.Compare(op, lhs, rhs, boolean, shape)
            return _fold(op, lhs, rhs)
        if isinstance(e, ast.Slice):
            raise self.error(e, "a bare slice is only meaningful as a tensor index")
        raise self.error(e, f"{type(e).__name__} expressions are not part of the tile subset")

    def attribute(self, e: ast.Attribute) -> Any:
        base = self.expr(e.value)
        if isinstance(base, _Tensor):
            if e.attr == "shape":
                return _Shape(base.param.name, base.param.rank)
            raise self.error(e, f"a tensor has no device-side attribute `{e.attr}`")
        if isinstance(base, _Index3):
            if e.attr in ("x", "y", "z"):
                return ir.BlockIndex(e.attr)
            raise self.error(e, "block.index() has .x, .y and .z")
        if _is_tile(base):
            return ("method", base, e.attr)
        if base is self.config and is_dataclass(base):
            if e.attr not in {f.name for f in fields(base)}:
                raise self.error(e, f"the configuration has no field `{e.attr}`")
            hints = type(base).__annotations__
            if not is_const(hints.get(e.attr)):
                raise self.error(e, f"`{e.attr}` is not a Const field: only compile-time fields can shape tiles")
            return getattr(base, e.attr)
        try:
            return getattr(base, e.attr)
        except AttributeError:
            raise self.error(e, f"`{e.attr}` is not available here") from None

    def subscript(self, e: ast.Subscript) -> Any:
        base = self.expr(e.value)
        if isinstance(base, _Shape):
            axis = self.expr(e.slice)
            if not isinstance(axis, int) or not -base.rank <= axis < base.rank:
                raise self.error(e, f"`shape` of a rank-{base.rank} tensor is indexed by a constant in range")
            return ir.Dim(base.tensor, axis % base.rank)
        if isinstance(base, _Tensor):
            index, shape = self.index(base, e.slice, e)
            if not shape:
                raise self.error(e, "element loads are not part of the tile subset: slice at least one axis")
            return ir.TileLoad(base.param.name, index, base.param.dtype, shape)
        if isinstance(base, tuple):
            return base[self.expr(e.slice)]
        raise self.error(e, "only tensors, shapes and tuples can be indexed")

    def index(self, tensor: _Tensor, node: ast.expr, at: ast.AST) -> tuple[tuple[ir.Expr, ...], tuple[int, ...]]:
        """All-scalar index = element; any slice = tile; a scalar among slices is squeezed. A slice extent must be a
        capture-time constant: `lo : lo + C`, `0 : C`, `slice(lo, lo + C)`, a `block.tile` slice or a loop slice
        (src/krn/compiler/capture.py:925-997)."""
        items = node.elts if isinstance(node, ast.Tuple) else [node]
        if len(items) != tensor.param.rank:
            raise self.error(at, f"`{tensor.param.name}` has rank {tensor.param.rank}, got {len(items)} indices")
        index: list[ir.Expr] = []
        shape: list[int] = []
        for item in items:
            if isinstance(item, ast.Slice):
                if item.step is not None:
                    raise self.error(item, "strided slices are not supported")
                start = self.expr(item.lower) if item.lower is not None else 0
                if item.upper is None:
                    raise self.error(item, "a slice needs an upper bound that is `lower + constant`")
                extent = _difference(self.expr(item.upper), start)
                if extent is None or extent <= 0:
                    raise self.error(item, "the extent of a slice must be a capture-time constant: write lo : lo + C")
                index.append(ir.SliceExpr(_as_expr(start), extent))
                shape.append(extent)
                continue
            value = self.expr(item)
            if isinstance(value, slice):
                start = value.start or 0
                extent = _difference(value.stop, start)
                if value.step is not None or extent is None or extent <= 0:
                    raise self.error(item, "the extent of a slice must be a capture-time constant")
                index.append(ir.SliceExpr(_as_expr(start), extent))
                shape.append(extent)
            elif isinstance(value, ir.SliceExpr):
                index.append(value)
                shape.append(value.extent)
            elif isinstance(value, (int, ir.Expr)) and not isinstance(value, bool):
                index.append(_as_expr(value))
            else:
                raise self.error(item, "a tensor is indexed by integers and slices")
        return tuple(index), tuple(shape)

    def binary(self, e: ast.BinOp) -> Any:
        lhs, rhs = self.expr(e.left), self.expr(e.right)
        if isinstance(e.op, ast.MatMult):
            return self.product(lhs, rhs, e)
        op = {ast.Add: "add", ast.Sub: "sub", ast.Mult: "mul", ast.Div: "div"}.get(type(e.op))
        if _is_tile(lhs) or _is_tile(rhs):
            if op is None:
                raise self.error(e, "this operator is not supported on tiles")
            return self.math(op, [lhs, rhs], e)
        symbol = {ast.Add: "+", ast.Sub: "-", ast.Mult: "*", ast.Div: "/", ast.FloorDiv: "//", ast.Mod: "%"}.get(type(e.op))
        if symbol is None:
            raise self.error(e, "unsupported scalar operator")
        return _fold(symbol, lhs, rhs)

    def product(self, lhs: Any, rhs: Any, node: ast.AST) -> ir.Product:
        """`a @ b`: (m, k) @ (k, n) → f32 (m, n); operands f16/bf16/f32 or an fp8 pair that is loaded directly
        (src/krn/compiler/capture.py:3157-3211)."""
        if not (_is_tile(lhs) and _is_tile(rhs)) or len(lhs.shape) != 2 or len(rhs.shape) != 2:
            raise self.error(node, "`@` multiplies two rank-2 tiles")
        if lhs.shape[1] != rhs.shape[0]:
            raise self.error(node, f"shapes {list(lhs.shape)} @ {list(rhs.shape)} do not compose")
        for operand in (lhs, rhs):
            if operand.dtype.name not in FLOAT_OPERANDS:
                raise self.error(node, f"`@` needs floating-point tiles, got {operand.dtype}")
        narrow = [o for o in (lhs, rhs) if o.dtype.bits == 8]
        if narrow and len(narrow) != 2:
            raise self.error(node, "an fp8 product needs both operands in fp8")
        for operand in narrow:
            inner = operand.operand if isinstance(operand, ir.Transpose) else operand
            if not isinstance(inner, ir.TileLoad):
                raise self.error(node, "fp8 operands of `@` must be loaded directly from a tensor")
        return ir.Product(lhs, rhs, f32, (lhs.shape[0], rhs.shape[1]))

    def common_shape(self, a: Any, b: Any, node: ast.AST) -> tuple[int, ...]:
        if _is_tile(a) and _is_tile(b):
            shape = _broadcast(a.shape, b.shape)
            if shape is None:
                raise self.error(node, f"tiles of shapes {list(a.shape)} and {list(b.shape)} do not broadcast")
            return shape
        return a.shape if _is_tile(a) else b.shape

    def math(self, fn: str, operands: list[Any], node: ast.AST) -> ir.Math:
        tiles = [o for o in operands if _is_tile(o)]
        shape = tiles[0].shape
        for other in tiles[1:]:
            shape = _broadcast(shape, other.shape)
            if shape is None:
                raise self.error(node, "tile shapes do not broadcast")
        dtypes = {t.dtype for t in tiles}
        if len(dtypes) > 1:
            raise self.error(node, f"mixed tile types {sorted(d.name for d in dtypes)}: convert with .to(...) first")
        dtype = tiles[0].dtype
        if fn in ("exp2", "exp") and dtype not in (f32, f64):
            raise self.error(node, f"{fn} needs an f32 or f64 tile, got {dtype}")
        cleaned = tuple(o if _is_tile(o) else _as_expr(o) for o in operands)
        return ir.Math(fn, cleaned, dtype, shape)

    def reduce(self, op: str, tile: ir.TileExpr, args: list[Any], keywords: dict[str, Any], node: ast.AST) -> ir.Reduce:
        axis = args[0] if args else keywords.get("axis", -1)
        keepdims = bool(keywords.get("keepdims", False))
        if not isinstance(axis, int) or not -len(tile.shape) <= axis < len(tile.shape):
            raise self.error(node, "the reduction axis must be a constant in range")
        axis %= len(tile.shape)
        if len(tile.shape) == 1 and not keepdims:
            raise self.error(node, "reducing a rank-1 tile to a scalar is not supported: use keepdims=True")
        shape = tuple(1 if a == axis else n for a, n in enumerate(tile.shape)) if keepdims else \
            tuple(n for a, n in enumerate(tile.shape) if a != axis)
        return ir.Reduce(op, tile, axis, keepdims, tile.dtype, shape)

    def call(self, e: ast.Call) -> Any:
        callee = self.expr(e.func)
        args = [self.expr(a) for a in e.args]
        keywords = {k.arg: self.expr(k.value) for k in e.keywords}
        if isinstance(callee, tuple) and callee and callee[0] == "method":
            return self.method(callee[1], callee[2], args, keywords, e)
        if callee is df.block.tile:
            if not args or len(args) > 2 or not all(isinstance(a, int) and a > 0 for a in args):
                raise self.error(e, "block.tile takes one or two positive capture-time sizes")
            if len(args) == 1:
                return ir.SliceExpr(_fold("*", ir.BlockIndex("x"), args[0]), args[0])
            return (ir.SliceExpr(_fold("*", ir.BlockIndex("y"), args[0]), args[0]),
                    ir.SliceExpr(_fold("*", ir.BlockIndex("x"), args[1]), args[1]))
        if callee is df.block.index:
            return _Index3()
        if callee in (df.WarpSpecialized, df.PingPong, df.Uniform):
            # a schedule is an intent attached to `pipelined(..., schedule=)`: built here, carried on the loop
            if not all(isinstance(v, int) for v in [*args, *keywords.values()]):
                raise self.error(e, "a schedule is built from capture-time integers")
            return callee(*args, **keywords)
        if callee is df.zeros or callee is df.full:
            dtype = args[0]
            value, extent = (0.0, args[1:]) if callee is df.zeros else (float(args[1]), args[2:])
            if "space" in keywords and keywords["space"] not in (df.Space.REGISTERS, df.Space.TENSOR_MEMORY):
                raise TargetError("zeros(space=SHARED)", "sm_100a", "accumulators of the prebuilt kernels live in "
                                  "tensor memory", "leave `space` at its default", span=self.span(e))
            if not isinstance(dtype, Dtype) or not extent or not all(isinstance(x, int) and x > 0 for x in extent):
                raise self.error(e, "zeros(dtype, *extent) needs an element type and capture-time extents")
            return ir.Zeros(dtype, tuple(extent), value)
        if callee is df.arange:
            extent = args[0]
            axis = args[1] if len(args) > 1 else keywords.get("axis", 0)
            rank = keywords.get("rank", 1)
            start = keywords.get("start", 0)
            if not all(isinstance(x, int) for x in (extent, axis, rank)) or not 0 <= axis < rank:
                raise self.error(e, "arange(extent, axis, rank=, start=) needs capture-time extent, axis and rank")
            shape = tuple(extent if a == axis else 1 for a in range(rank))
            return ir.Arange(extent, axis, rank, _as_expr(start), i32, shape)
        if callee is df.where:
            if len(args) != 3 or not _is_tile(args[0]) or args[0].dtype != boolean:
                raise self.error(e, "where(condition, x, y) needs a boolean tile first")
            tiles = [a for a in args[1:] if _is_tile(a)]
            if not tiles:
                raise self.error(e, "where needs a tile among x and y")
            shape = args[0].shape
            for t in tiles:
                shape = _broadcast(shape, t.shape) or shape
            then, orelse = (a if _is_tile(a) else _as_expr(a) for a in args[1:])
            return ir.Select(args[0], then, orelse, tiles[0].dtype, shape)
        if callee is df.maximum or callee is df.minimum:
            return self.math("maximum" if callee is df.maximum else "minimum", args, e)
        if callee is slice:
            return slice(*args)
        if callee in (min, max) and all(isinstance(a, (int, float)) for a in args):
            return callee(*args)
        if callee in (int, float, bool) and len(args) == 1 and isinstance(args[0], (int, float, bool)):
            return callee(args[0])
        if isinstance(callee, Dtype) and len(args) == 1 and isinstance(args[0], (int, float)):
            return args[0]
        raise self.error(e, "this call is not part of the tile subset")

    def method(self, tile: ir.TileExpr, name: str, args: list[Any], keywords: dict[str, Any], node: ast.AST) -> Any:
        if name == "transpose":
            if len(tile.shape) != 2 or args:
                raise self.error(node, ".transpose() swaps the axes of a rank-2 tile")
            return ir.Transpose(tile, tile.dtype, (tile.shape[1], tile.shape[0]))
        if name == "to":
            if len(args) != 1 or not isinstance(args[0], Dtype):
                raise self.error(node, ".to(dtype) takes one element type")
            return tile if args[0] == tile.dtype else ir.Cast(tile, args[0], tile.shape)
        if name in ("mul", "sub", "add", "div", "maximum", "minimum"):
            if len(args) != 1:
                raise self.error(node, f".{name}(other) takes one operand")
            return self.math(name, [tile, args[0]], node)
        if name in ("exp2", "exp"):
            return self.math(name, [tile], node)
        if name in ("relu", "gelu", "silu"):  # the tile activations (src/krn/frontend/_ops.py:185-205)
            if args or keywords:
                raise self.error(node, f".{name}() takes no operands")
            return self.math(name, [tile], node)
        if name in ("max", "sum", "min"):
            return self.reduce(name, tile, args, keywords, node)
        raise self.error(node, f"tiles have no method `{name}` in the tile subset")


def capture(fn, config: Any | None = None) -> ir.Kernel:
    """The IR of kernel function `fn`, specialised on `config` (an instance of its configuration struct, or None)."""
    return Builder(fn, config).kernel()
