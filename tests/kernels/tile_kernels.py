"""Kernel sources the front-end tests capture (capture reads source files, so kernels live in a module)."""

from krn_b200 import (Const, Feature, Matrix, PingPong, Space, T, Tensor, Vector, WarpSpecialized, arange, bf16, block, f16,
                      f32, family, full, kernel, pipelined, struct, targets, where, zeros)


@struct
class Tiling:
    bm: Const[int] = 128
    bn: Const[int] = 128
    bk: Const[int] = 32


@kernel
def matmul_nt(t: Tiling, a: Matrix[bf16], b: Matrix[bf16], c: Matrix[bf16]) -> None:
    rows, cols = block.tile(t.bm, t.bn)
    acc = zeros(f32, t.bm, t.bn)
    for ks in pipelined(a.shape[1], t.bk):
        acc += a[rows, ks] @ b[cols, ks].transpose()
    c[rows, cols] = acc.to(bf16)


@kernel
def matmul_nt_f16_f32(a: Matrix[f16], b: Matrix[f16], c: Matrix[f32]) -> None:
    rows, cols = block.tile(32, 64)
    acc = zeros(f32, 32, 64)
    for ks in range(0, a.shape[1], 16):
        acc += a[rows, slice(ks, ks + 16)] @ b[cols, slice(ks, ks + 16)].transpose()
    c[rows, cols] = acc


@kernel
def matmul_nn(t: Tiling, a: Matrix[f16], b: Matrix[f16], c: Matrix[f16]) -> None:
    """The reference example's row-major-B form (examples/04_libraries/01_gemm_tiles.py:35-40)."""
    rows, cols = block.tile(t.bm, t.bn)
    acc = zeros(f32, t.bm, t.bn)
    for ks in pipelined(a.shape[1], t.bk):
        acc += a[rows, ks] @ b[ks, cols]
    c[rows, cols] = acc.to(f16)


@struct
class MatmulTiling:
    """The configuration of the reference's library kernel (src/krn/lib/lib_kernels.py:18-28)."""

    bm: Const[int] = 64
    bn: Const[int] = 64
    bk: Const[int] = 32
    bias: Const[bool] = False
    relu: Const[bool] = False
    gelu: Const[bool] = False
    silu: Const[bool] = False


@kernel
def matmul_epilogue(t: MatmulTiling, a: Matrix[f16], b: Matrix[f16], bias: Vector[f16], out: Matrix[f16]) -> None:
    """`out = activation(a @ b + bias)`, the statements of src/krn/lib/lib_kernels.py:30-48."""
    rows, cols = block.tile(t.bm, t.bn)
    acc = zeros(f32, t.bm, t.bn)
    for ks in pipelined(a.shape[1], t.bk):
        acc += a[rows, ks] @ b[ks, cols]
    if t.bias:
        acc += bias[cols].to(f32)
    if t.relu:
        acc = acc.relu()
    if t.gelu:
        acc = acc.gelu()
    if t.silu:
        acc = acc.silu()
    out[rows, cols] = acc.to(f16)


@kernel
def matmul_mixed(t: Tiling, a: Matrix[bf16], b: Matrix[f16], c: Matrix[f32]) -> None:
    """Mixed 16-bit operand types: no tensor-core kind multiplies them."""
    rows, cols = block.tile(t.bm, t.bn)
    acc = zeros(f32, t.bm, t.bn)
    for ks in pipelined(a.shape[1], t.bk):
        acc += a[rows, ks] @ b[cols, ks].transpose()
    c[rows, cols] = acc.to(f32)


@struct
class Heads:
    bq: Const[int] = 16
    bk: Const[int] = 16
    d: Const[int] = 64
    causal: Const[bool] = False


@kernel
def flash_attention(t: Heads, q: Tensor[T.f16, int, int, int], k: Tensor[T.f16, int, int, int],
                    v: Tensor[T.f16, int, int, int], o: Tensor[T.f16, int, int, int], scale: T.f32) -> None:
    """The reference's example kernel, statement for statement (examples/04_libraries/08_flash_attention.py:35-59)."""
    rows, head = block.tile(t.bq), block.index().y
    q_pos = arange(t.bq, 0, rank=2, start=block.index().x * t.bq)
    m, total, acc = zeros(T.f32, t.bq, 1).sub(1.0e30), zeros(T.f32, t.bq, 1), zeros(T.f32, t.bq, t.d)
    qt = q[head, rows, slice(0, t.d)]
    for c in range(0, k.shape[1], t.bk):
        s = (qt @ k[head, c : c + t.bk, slice(0, t.d)].transpose()).mul(scale)
        if t.causal:
            s = where(arange(t.bk, 1, rank=2, start=c) <= q_pos, s, -1.0e30)
        m_new = m.maximum(s.max(keepdims=True))
        p, corr = (s - m_new).exp2(), (m - m_new).exp2()
        total *= corr
        total += p.sum(keepdims=True)
        acc *= corr
        acc += p.to(T.f16) @ v[head, c : c + t.bk, slice(0, t.d)]
        m = m_new
    o[head, rows, slice(0, t.d)] = (acc / total).to(T.f16)


# ---- near misses of the attention pattern: each differs from the example in ONE operand and must be refused, not run
# as standard attention


@kernel
def attention_old_maximum_in_exponent(t: Heads, q: Tensor[T.f16, int, int, int], k: Tensor[T.f16, int, int, int],
                                      v: Tensor[T.f16, int, int, int], o: Tensor[T.f16, int, int, int], scale: T.f32) -> None:
    rows, head = block.tile(t.bq), block.index().y
    m, total, acc = zeros(T.f32, t.bq, 1).sub(1.0e30), zeros(T.f32, t.bq, 1), zeros(T.f32, t.bq, t.d)
    qt = q[head, rows, slice(0, t.d)]
    for c in range(0, k.shape[1], t.bk):
        s = (qt @ k[head, c : c + t.bk, slice(0, t.d)].transpose()).mul(scale)
        m_new = m.maximum(s.max(keepdims=True))
        p, corr = (s - m).exp2(), (m - m_new).exp2()  # exponent against the OLD maximum
        total *= corr
        total += p.sum(keepdims=True)
        acc *= corr
        acc += p.to(T.f16) @ v[head, c : c + t.bk, slice(0, t.d)]
        m = m_new
    o[head, rows, slice(0, t.d)] = (acc / total).to(T.f16)


@kernel
def attention_sum_starts_at_one(t: Heads, q: Tensor[T.f16, int, int, int], k: Tensor[T.f16, int, int, int],
                                v: Tensor[T.f16, int, int, int], o: Tensor[T.f16, int, int, int], scale: T.f32) -> None:
    rows, head = block.tile(t.bq), block.index().y
    m, total, acc = zeros(T.f32, t.bq, 1).sub(1.0e30), full(T.f32, 1.0, t.bq, 1), zeros(T.f32, t.bq, t.d)
    qt = q[head, rows, slice(0, t.d)]
    for c in range(0, k.shape[1], t.bk):
        s = (qt @ k[head, c : c + t.bk, slice(0, t.d)].transpose()).mul(scale)
        m_new = m.maximum(s.max(keepdims=True))
        p, corr = (s - m_new).exp2(), (m - m_new).exp2()
        total *= corr
        total += p.sum(keepdims=True)
        acc *= corr
        acc += p.to(T.f16) @ v[head, c : c + t.bk, slice(0, t.d)]
        m = m_new
    o[head, rows, slice(0, t.d)] = (acc / total).to(T.f16)


@kernel
def attention_correction_swapped(t: Heads, q: Tensor[T.f16, int, int, int], k: Tensor[T.f16, int, int, int],
                                 v: Tensor[T.f16, int, int, int], o: Tensor[T.f16, int, int, int], scale: T.f32) -> None:
    rows, head = block.tile(t.bq), block.index().y
    m, total, acc = zeros(T.f32, t.bq, 1).sub(1.0e30), zeros(T.f32, t.bq, 1), zeros(T.f32, t.bq, t.d)
    qt = q[head, rows, slice(0, t.d)]
    for c in range(0, k.shape[1], t.bk):
        s = (qt @ k[head, c : c + t.bk, slice(0, t.d)].transpose()).mul(scale)
        m_new = m.maximum(s.max(keepdims=True))
        p, corr = (s - m_new).exp2(), (m_new - m).exp2()  # the correction's operands swapped
        total *= corr
        total += p.sum(keepdims=True)
        acc *= corr
        acc += p.to(T.f16) @ v[head, c : c + t.bk, slice(0, t.d)]
        m = m_new
    o[head, rows, slice(0, t.d)] = (acc / total).to(T.f16)


@struct
class Grouped:
    bq: Const[int] = 128
    bk: Const[int] = 128
    d: Const[int] = 128
    group: Const[int] = 4


@kernel
def grouped_causal_attention(t: Grouped, q: Tensor[T.bf16, int, int, int, int], k: Tensor[T.bf16, int, int, int, int],
                             v: Tensor[T.bf16, int, int, int, int], o: Tensor[T.bf16, int, int, int, int],
                             scale: T.f32) -> None:
    """Batched, grouped-query, causal: batch on grid z, `head // group` selects the kv head."""
    rows, head, batch = block.tile(t.bq), block.index().y, block.index().z
    q_pos = arange(t.bq, 0, rank=2, start=block.index().x * t.bq)
    m, total, acc = zeros(T.f32, t.bq, 1).sub(1.0e30), zeros(T.f32, t.bq, 1), zeros(T.f32, t.bq, t.d)
    qt = q[batch, head, rows, slice(0, t.d)]
    for c in range(0, k.shape[2], t.bk):
        s = (qt @ k[batch, head // t.group, c : c + t.bk, slice(0, t.d)].transpose()).mul(scale)
        s = where(arange(t.bk, 1, rank=2, start=c) <= q_pos, s, -1.0e30)
        m_new = m.maximum(s.max(keepdims=True))
        p, corr = (s - m_new).exp2(), (m - m_new).exp2()
        total *= corr
        total += p.sum(keepdims=True)
        acc *= corr
        acc += p.to(T.bf16) @ v[batch, head // t.group, c : c + t.bk, slice(0, t.d)]
        m = m_new
    o[batch, head, rows, slice(0, t.d)] = (acc / total).to(T.bf16)


@kernel
def row_scale(a: Matrix[f32], c: Matrix[f32]) -> None:
    """Not a contraction: the B200 device has no kernel for it."""
    rows, cols = block.tile(16, 16)
    c[rows, cols] = a[rows, cols] * 2.0


@kernel
def conflicting_tiles(a: Matrix[f32], c: Matrix[f32]) -> None:
    rows = block.tile(8)
    wide = block.tile(16)
    c[rows, slice(0, 4)] = a[rows, slice(0, 4)]
    c[wide, slice(4, 8)] = a[wide, slice(4, 8)]


@kernel
def mismatched_extents(a: Matrix[f32], b: Matrix[f32], c: Matrix[f32], d: Matrix[f32]) -> None:
    rows, cols = block.tile(8, 8)
    c[rows, cols] = a[rows, cols]
    d[rows, cols] = b[rows, cols]


@kernel
def data_dependent_branch(a: Matrix[f32], c: Matrix[f32]) -> None:
    rows, cols = block.tile(8, 8)
    if a.shape[0] > 4:
        c[rows, cols] = a[rows, cols]


@kernel
def fp8_pair_kn(a: Matrix[T.f8e4m3fn], b: Matrix[T.f8e5m2], c: Matrix[f32]) -> None:
    """An fp8 pair loaded directly, b row-major as (K, N): the form of the reference's fp8 kernels
    (tests/compiler/test_tensor_cores.py:47-78 with dtype / rhs fp8). The two operands have different formats."""
    rows, cols = block.tile(32, 32)
    acc = zeros(f32, 32, 32)
    for ks in pipelined(a.shape[1], 32):
        acc += a[rows, ks] @ b[ks, cols]
    c[rows, cols] = acc


@kernel
def fp8_pair_nt(a: Matrix[T.f8e4m3fn], b: Matrix[T.f8e4m3fn], c: Matrix[bf16]) -> None:
    """The same product with b stored (N, K): `a8[rows, ks] @ b8[cols, ks].transpose()`."""
    rows, cols = block.tile(128, 128)
    acc = zeros(f32, 128, 128)
    for ks in pipelined(a.shape[1], 128):
        acc += a[rows, ks] @ b[cols, ks].transpose()
    c[rows, cols] = acc.to(bf16)


@kernel
def fp8_needs_direct_loads(a: Matrix[T.f8e4m3fn], b: Matrix[T.f8e4m3fn], c: Matrix[f32]) -> None:
    rows, cols = block.tile(32, 32)
    acc = zeros(f32, 32, 32)
    for ks in pipelined(a.shape[1], 32):
        acc += a[rows, ks] @ (b[cols, ks] + b[cols, ks]).transpose()
    c[rows, cols] = acc


# ---- a kernel family: one contract, the variant chosen by what the target can do ------------------------------------
# (the shape of examples/04_libraries/03_gemm_variants.py:43-90)


@struct
class FamilyTiling:
    bm: Const[int] = 128
    bn: Const[int] = 128
    bk: Const[int] = 64


@family
def gemm(t: FamilyTiling, a: Matrix[T.f16], b: Matrix[T.f16], c: Matrix[T.f32]) -> None:
    """Portable: C = A @ B on whatever matrix unit the target has."""
    rows, cols = block.tile(t.bm, t.bn)
    acc = zeros(T.f32, t.bm, t.bn)
    for ks in pipelined(a.shape[1], t.bk):
        acc += a[rows, ks] @ b[ks, cols]
    c[rows, cols] = acc


@gemm.variant(targets.Nvidia, requires={Feature.TENSOR_MEMORY})
def gemm_tensor_memory(t: FamilyTiling, a: Matrix[T.f16], b: Matrix[T.f16], c: Matrix[T.f32]) -> None:
    """The accumulator lives in tensor memory; one producer, one consumer."""
    rows, cols = block.tile(t.bm, t.bn)
    acc = zeros(T.f32, t.bm, t.bn, space=Space.TENSOR_MEMORY)
    for ks in pipelined(a.shape[1], t.bk, schedule=WarpSpecialized(producers=1, consumers=1)):
        acc += a[rows, ks] @ b[ks, cols]
    c[rows, cols] = acc


@gemm.variant(arch={"sm_90a"})
def gemm_hopper(t: FamilyTiling, a: Matrix[T.f16], b: Matrix[T.f16], c: Matrix[T.f32]) -> None:
    rows, cols = block.tile(t.bm, t.bn)
    acc = zeros(T.f32, t.bm, t.bn)
    for ks in pipelined(a.shape[1], t.bk, schedule=WarpSpecialized(producers=1, consumers=2)):
        acc += a[rows, ks] @ b[ks, cols]
    c[rows, cols] = acc


@gemm.variant(targets.AMD, requires={Feature.ASYNC_COPY})
def gemm_amd(t: FamilyTiling, a: Matrix[T.f16], b: Matrix[T.f16], c: Matrix[T.f32]) -> None:
    rows, cols = block.tile(t.bm, t.bn)
    acc = zeros(T.f32, t.bm, t.bn)
    for ks in pipelined(a.shape[1], t.bk, stages=2, schedule=PingPong()):
        acc += a[rows, ks] @ b[ks, cols]
    c[rows, cols] = acc
