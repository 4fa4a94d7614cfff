"""Pattern recogniser: captured IR → which prebuilt sm_100a kernel runs it.

The reference renders every IR statement as CUDA text (src/krn/compiler/emit.py); the B200 path has no code
generator, so a kernel either IS one of the contractions the library implements or it is refused before anything is
launched ("never ignore it silently", the reference's refusal policy, AGENTS.md:17). Two patterns:

* tile matrix product — `acc = zeros(f32, bm, bn)`, one K loop of `acc += a[rows, ks] @ b[ks, cols]`
  (examples/04_libraries/01_gemm_tiles.py:35-40) or of `acc += a[rows, ks] @ b[cols, ks].transpose()`, optionally the
  library epilogue `acc += bias[cols].to(f32)` and one of `acc = acc.relu()` / `.gelu()` / `.silu()`
  (src/krn/lib/lib_kernels.py:30-48), then `c[rows, cols] = acc.to(T)`;
* flash attention — the statement sequence of examples/04_libraries/08_flash_attention.py:44-59, optionally with a
  leading batch axis and grouped kv heads (`k[head // g, ...]`)."""

from __future__ import annotations

from dataclasses import dataclass

from krn_b200.compiler import ir
from krn_b200.errors import TargetError
from krn_b200.frontend.types import Dtype, f32

TARGET = "sm_100a"


@dataclass(frozen=True)
class GemmPlan:
    """`c = a @ b^T` with a (M, K), b (N, K), or — `transposed_b` False — `c = a @ b` with b (K, N); c (M, N)."""

    a: str
    b: str
    c: str
    operand: Dtype
    output: Dtype
    tile: tuple[int, int, int]
    transposed_b: bool = True
    bias: str | None = None        # vector added to every row of the accumulator before the store
    activation: str | None = None  # "relu", "gelu" or "silu", applied after the bias
    operand_b: Dtype | None = None  # b's element type for an fp8 pair (which may mix e4m3 and e5m2), else None


@dataclass(frozen=True)
class AttentionPlan:
    """`o = softmax(scale * q k^T [+ causal]) v`; tensors are (heads, seq, d) or (batch, heads, seq, d)."""

    q: str
    k: str
    v: str
    o: str
    scale: tuple[str, ...]
    dtype: Dtype
    d: int
    causal: bool
    batched: bool
    group: int  # q heads per kv head, from `head // group`
    tile: tuple[int, int]


Plan = GemmPlan | AttentionPlan


def refuse(kernel: ir.Kernel, reason: str, instead: str, span=None) -> TargetError:
    return TargetError(f"kernel `{kernel.name}`", TARGET, reason, instead, span=span)


def _block_tile(e: ir.Expr, axis: str) -> int | None:
    """`size` if `e` is the slice [block.index.<axis> * size, + size)."""
    if isinstance(e, ir.SliceExpr) and isinstance(e.start, ir.Binary) and e.start.op == "*" \
            and e.start.lhs == ir.BlockIndex(axis) and e.start.rhs == ir.Const(e.extent):
        return e.extent
    return None


def _loop_slice(e: ir.Expr, loop: ir.For) -> bool:
    return isinstance(e, ir.SliceExpr) and e.start == ir.LoopVar(loop.var) and e.extent == loop.step


def _epilogue(kernel: ir.Kernel, acc: ir.Var, statements: list[ir.Stmt], bn: int) -> tuple[str | None, str | None] | None:
    """(bias tensor, activation) of the statements between the K loop and the store — `acc += bias[cols].to(f32)` and
    `acc = acc.relu()` / `.gelu()` / `.silu()` (src/krn/lib/lib_kernels.py:40-47) — or None when they are something else."""
    bias = activation = None
    for s in statements:
        if not (isinstance(s, ir.Assign) and s.var == acc and isinstance(s.value, ir.Math)):
            return None
        fn, operands = s.value.fn, s.value.operands
        if fn == "add" and len(operands) == 2 and operands[0] == acc and bias is None and activation is None:
            vector = operands[1].operand if isinstance(operands[1], ir.Cast) else operands[1]
            if not (isinstance(vector, ir.TileLoad) and len(vector.index) == 1 and _block_tile(vector.index[0], "x") == bn):
                return None
            bias = vector.tensor
        elif fn in ("relu", "gelu", "silu") and operands == (acc,):
            if activation is not None:
                raise refuse(kernel, f"{activation} followed by {fn}: the library epilogue applies one activation",
                             "keep one of relu, gelu, silu (the reference's Epilogue values name one each)", span=s.span)
            activation = fn
        else:
            return None
    return bias, activation


def _gemm(kernel: ir.Kernel) -> GemmPlan | None:
    body = kernel.body
    if len(body) < 3 or not isinstance(body[0], ir.Assign) or not isinstance(body[1], ir.For) \
            or not isinstance(body[-1], ir.TileStore):
        return None
    tail = list(body[2:-1])
    body = (body[0], body[1], body[-1])
    init, loop, store = body
    if not (isinstance(init.value, ir.Zeros) and init.value.value == 0.0 and init.value.dtype == f32
            and len(init.value.shape) == 2):
        return None
    bm, bn = init.value.shape
    if len(loop.body) != 1 or not isinstance(loop.body[0], ir.Accumulate) or loop.start != ir.Const(0):
        return None
    step = loop.body[0]
    if step.acc != init.var or not isinstance(step.lhs, ir.TileLoad):
        return None
    a = step.lhs
    if len(a.index) != 2 or _block_tile(a.index[0], "y") != bm or not _loop_slice(a.index[1], loop) \
            or loop.stop != ir.Dim(a.tensor, 1):
        return None
    rhs = step.rhs
    if isinstance(rhs, ir.TileLoad):
        # `a[rows, ks] @ b[ks, cols]`: b is (K, N) and reaches the tensor cores as an MN-major operand
        b, transposed_b = rhs, False
        if len(b.index) != 2 or not _loop_slice(b.index[0], loop) or _block_tile(b.index[1], "x") != bn:
            return None
    elif isinstance(rhs, ir.Transpose) and isinstance(rhs.operand, ir.TileLoad):
        b, transposed_b = rhs.operand, True
        if len(b.index) != 2 or _block_tile(b.index[0], "x") != bn or not _loop_slice(b.index[1], loop):
            return None
    else:
        return None
    value = store.value
    if isinstance(value, ir.Cast):
        value = value.operand
    if value != init.var or len(store.index) != 2 or _block_tile(store.index[0], "y") != bm \
            or _block_tile(store.index[1], "x") != bn:
        return None
    fp8 = ("f8e4m3fn", "f8e5m2")
    if a.dtype.name in fp8 and b.dtype.name in fp8:
        # fp8 pairs loaded directly multiply as stored, each operand in its own format
        # (src/krn/compiler/capture.py:3185-3192, src/krn/compiler/cuda.py:207-227)
        pass
    elif a.dtype != b.dtype:
        raise refuse(kernel, f"mixed operand types {a.dtype} @ {b.dtype} have no tcgen05 kind",
                     "convert one operand so both are bf16, both f16, or both 8-bit floats", span=step.span)
    elif a.dtype.name not in ("bf16", "f16"):
        raise refuse(kernel, f"{a.dtype} operands are not a tensor-core kind",
                     "use bf16, f16 or fp8 (f8e4m3fn / f8e5m2) operands; block-scaled FP8 goes through "
                     "krn_b200.ops.matmul_fp8_blockscaled", span=step.span)
    output = kernel.tensor(store.tensor).dtype
    if output.name not in ("bf16", "f16", "f32"):
        raise refuse(kernel, f"{output} outputs are not supported", "store bf16, f16 or f32", span=store.span)
    epilogue = _epilogue(kernel, init.var, tail, bn)
    if epilogue is None:
        return None
    bias, activation = epilogue
    if bias is not None and kernel.tensor(bias).dtype != output:
        raise refuse(kernel, f"a {kernel.tensor(bias).dtype} bias on a {output} result: the library epilogue reads the "
                             "bias in the type of the result", "declare bias and out with one element type",
                     span=store.span)
    if a.dtype.name in fp8 and (bias is not None or activation is not None):
        raise refuse(kernel, "the library epilogue (bias / activation) on an fp8 product has no prebuilt kernel",
                     "store the product and apply the epilogue to 16-bit operands", span=store.span)
    return GemmPlan(a.tensor, b.tensor, store.tensor, a.dtype, output, (bm, bn, loop.step), transposed_b, bias, activation,
                    b.dtype if a.dtype.name in fp8 else None)


def _head_index(e: ir.Expr) -> int | None:
    """1 for `block.index().y`, g for `block.index().y // g`."""
    if e == ir.BlockIndex("y"):
        return 1
    if isinstance(e, ir.Binary) and e.op == "//" and e.lhs == ir.BlockIndex("y") and isinstance(e.rhs, ir.Const):
        return int(e.rhs.value)
    return None


def _attention(kernel: ir.Kernel) -> AttentionPlan | None:
    statements = list(kernel.body)
    loops = [s for s in statements if isinstance(s, ir.For)]
    if len(loops) != 1 or not isinstance(statements[-1], ir.TileStore):
        return None
    loop = loops[0]
    before = statements[: statements.index(loop)]
    store = statements[-1]
    assigns = {s.var.name: s.value for s in before if isinstance(s, ir.Assign)}

    products = [s for s in loop.body if isinstance(s, ir.Assign) and isinstance(s.value, ir.Math) and s.value.fn == "mul"
                and isinstance(s.value.operands[0], ir.Product)]
    accumulates = [s for s in loop.body if isinstance(s, ir.Accumulate)]
    if len(products) != 1 or len(accumulates) != 1:
        return None
    score, pv = products[0], accumulates[0]
    product = score.value.operands[0]
    scale = score.value.operands[1]
    if not isinstance(scale, ir.Param):
        return None
    # q tile: loaded once before the loop; k tile: transposed load inside the loop
    qt = product.lhs
    if isinstance(qt, ir.Var):
        qt = assigns.get(qt.name)
    if not (isinstance(qt, ir.TileLoad) and isinstance(product.rhs, ir.Transpose)
            and isinstance(product.rhs.operand, ir.TileLoad)):
        return None
    kt = product.rhs.operand
    vt = pv.rhs
    if not isinstance(vt, ir.TileLoad) or not isinstance(pv.lhs, ir.Cast):
        return None
    rank = len(qt.index)
    if rank not in (3, 4) or any(len(t.index) != rank for t in (kt, vt)) or len(store.index) != rank:
        return None
    batched = rank == 4
    offset = 1 if batched else 0
    if batched and any(t.index[0] != ir.BlockIndex("z") for t in (qt, kt, vt)) or (batched and store.index[0] != ir.BlockIndex("z")):
        return None
    bq = _block_tile(qt.index[offset + 1], "x")
    d = qt.shape[1]
    if bq is None or _head_index(qt.index[offset]) != 1 or store.index[offset] != ir.BlockIndex("y") \
            or _block_tile(store.index[offset + 1], "x") != bq:
        return None
    group = _head_index(kt.index[offset])
    if group is None or _head_index(vt.index[offset]) != group:
        return None
    for t in (kt, vt):
        rows, cols = t.index[offset + 1], t.index[offset + 2]
        if not _loop_slice(rows, loop) or not (isinstance(cols, ir.SliceExpr) and cols.start == ir.Const(0) and cols.extent == d):
            return None
    if loop.start != ir.Const(0) or loop.stop != ir.Dim(kt.tensor, offset + 1):
        return None

    # the online-softmax statements, in the example's order
    names = {"s": score.var.name}
    body = [s for s in loop.body if s is not score]
    causal = False
    if body and isinstance(body[0], ir.Assign) and isinstance(body[0].value, ir.Select):
        select = body.pop(0)
        cond = select.value.cond
        ok = (select.var.name == names["s"] and isinstance(cond, ir.Compare) and cond.op == "<="
              and isinstance(cond.lhs, ir.Arange) and cond.lhs.axis == 1 and cond.lhs.start == ir.LoopVar(loop.var)
              and isinstance(select.value.orelse, ir.Const) and select.value.orelse.value <= -1.0e29)
        q_pos = cond.rhs if ok else None
        if isinstance(q_pos, ir.Var):
            q_pos = assigns.get(q_pos.name)
        if not (ok and isinstance(q_pos, ir.Arange) and q_pos.axis == 0
                and q_pos.start == ir.Binary("*", ir.BlockIndex("x"), ir.Const(bq))):
            return None
        causal = True
    kinds = []
    for s in body:
        if isinstance(s, ir.Accumulate):
            kinds.append("accumulate")
        elif isinstance(s, ir.Assign) and isinstance(s.value, ir.Math):
            inner = s.value.operands[0]
            kinds.append(s.value.fn + (":" + inner.fn if isinstance(inner, ir.Math) else ""))
        elif isinstance(s, ir.Assign) and isinstance(s.value, ir.Var):
            kinds.append("copy")
        else:
            return None
    if kinds != ["maximum", "exp2:sub", "exp2:sub", "mul", "add", "mul", "accumulate", "copy"]:
        return None
    m_new, p, corr, total_scale, total_add, acc_scale, _, m_copy = body
    s_var, m_var = score.var, m_copy.var  # the scores and the running maximum (`m = m_new` names it)
    l_var, acc_var = total_add.var, pv.acc

    def is_sub(e, lhs, rhs) -> bool:
        return isinstance(e, ir.Math) and e.fn == "sub" and e.operands == (lhs, rhs)

    row_max, row_sum = m_new.value.operands[1], total_add.value.operands[1]
    checks = (
        # m_new = maximum(m, max(s, axis=1)): the running maximum first, the row maximum of THE SCORES second
        m_new.value.operands[0] == m_var,
        isinstance(row_max, ir.Reduce) and row_max.op == "max" and row_max.operand == s_var and row_max.axis == 1,
        # p = exp2(s - m_new), corr = exp2(m - m_new): against the NEW maximum, from the OLD one
        is_sub(p.value.operands[0], s_var, m_new.var),
        is_sub(corr.value.operands[0], m_var, m_new.var),
        # l = l * corr + sum(p, axis=1); acc = acc * corr + p.to(T) @ v; m = m_new
        total_scale.var == l_var and total_scale.value.operands == (l_var, corr.var),
        total_add.value.operands[0] == l_var,
        isinstance(row_sum, ir.Reduce) and row_sum.op == "sum" and row_sum.operand == p.var and row_sum.axis == 1,
        acc_scale.var == acc_var and acc_scale.value.operands == (acc_var, corr.var),
        pv.lhs.operand == p.var,
        m_copy.value == m_new.var,
        # both sums start from zero
        isinstance(assigns.get(l_var.name), ir.Zeros) and assigns[l_var.name].value == 0.0,
        isinstance(assigns.get(acc_var.name), ir.Zeros) and assigns[acc_var.name].value == 0.0,
    )
    if not all(checks):
        return None
    if causal and select.value.then != s_var:
        return None  # the mask keeps something other than the score itself
    final = store.value
    if not (isinstance(final, ir.Cast) and isinstance(final.operand, ir.Math) and final.operand.fn == "div"
            and final.operand.operands[0] == pv.acc and final.operand.operands[1] == total_add.var):
        return None
    start = assigns.get(m_copy.var.name)  # the running maximum starts at 0 - 1e30 (or lower)
    if not (isinstance(start, ir.Math) and start.fn == "sub" and isinstance(start.operands[0], ir.Zeros)
            and start.operands[0].value == 0.0 and isinstance(start.operands[1], ir.Const) and start.operands[1].value >= 1.0e29):
        return None
    dtype = qt.dtype
    if dtype.name not in ("bf16", "f16") or any(t.dtype != dtype for t in (kt, vt)) or pv.lhs.dtype != dtype:
        raise refuse(kernel, f"attention over {dtype} tiles has no prebuilt kernel", "use bf16 or f16 tensors",
                     span=score.span)
    if d not in (64, 128):
        raise refuse(kernel, f"head dimension {d} is not built from 128-byte rows", "use d = 64 or d = 128",
                     span=score.span)
    return AttentionPlan(qt.tensor, kt.tensor, vt.tensor, store.tensor, scale.path, dtype, d, causal, batched, group,
                         (bq, loop.step))


def recognise(kernel: ir.Kernel) -> Plan:
    """The plan for `kernel`, or a `TargetError` naming what to write instead."""
    plan = _gemm(kernel) or _attention(kernel)
    if plan is None:
        raise refuse(kernel,
                     "its body is neither the tile matrix product `acc += a[rows, ks] @ b[cols, ks].transpose()` nor the "
                     "flash-attention statement sequence, and this device has no code generator for other bodies",
                     "write the contraction in one of those two forms, or run other kernels on a device with a compiler")
    return plan
