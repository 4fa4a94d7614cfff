"""Host-resident operands streamed through the device in panels.

The reference's host path is three separate steps — `device.to_device(array)`, the launch, `tensor.to_host()`
(src/krn/runtime/host.py:78-118) — and a caller whose operands live in host memory pays them back to back: at PCIe
rates the copies of a large product take ten times longer than the product itself. The classes here are the same
three steps cut into panels and overlapped on three CUDA streams (host→device, the caller's compute stream,
device→host): while panel i is multiplied, panel i+1 arrives and panel i-1 leaves. PCIe is full duplex, so the
elapsed time tends to max(bytes in, bytes out) / link rate plus one panel of tail, instead of the sum.

Operands and results are torch CPU tensors; pinned memory is what makes the copies asynchronous
(`torch.Tensor.pin_memory`). Every `run` only enqueues; the caller's current stream is made to wait for the last
device→host copy, so synchronising that stream (or an event recorded on it) makes the result visible."""

from __future__ import annotations

from typing import Any

from krn_b200.runtime import calls


def _torch():
    import torch

    return torch


def _panels(extent: int, count: int, multiple: int) -> list[tuple[int, int]]:
    """`count` contiguous [begin, end) ranges covering `extent`, boundaries on multiples of `multiple`."""
    units = -(-extent // multiple)
    count = max(1, min(count, units))
    bounds = [min(extent, (units * i // count) * multiple) for i in range(count + 1)]
    bounds[-1] = extent
    return [(bounds[i], bounds[i + 1]) for i in range(count) if bounds[i + 1] > bounds[i]]


def _copy_out(target: Any, source: Any, stream: Any) -> None:
    """Device → host copy of one panel on `stream`. Row panels are contiguous and go through torch; a column slab is a
    pitched copy, which torch would stage through temporaries, so it goes to the library's cudaMemcpy2DAsync."""
    torch = _torch()
    if target.is_contiguous() and source.is_contiguous():
        with torch.cuda.stream(stream):
            target.copy_(source, non_blocking=True)
    else:
        calls.copy_matrix(target, source, stream)


class _Streams:
    """Two side streams and an event pool shared by the streamed operations of one device."""

    def __init__(self) -> None:
        torch = _torch()
        self.h2d = torch.cuda.Stream()
        self.d2h = torch.cuda.Stream()
        self.events: list[Any] = []

    def event(self, index: int):
        torch = _torch()
        while len(self.events) <= index:
            self.events.append(torch.cuda.Event())
        return self.events[index]


class StreamedProduct:
    """`c_host = a_host @ b_host^T` (bf16 or f16 operands) with all three matrices in host memory.

    Panels run over `axis` ("m": row panels of `a`, contiguous row panels of `c`; "n": row panels of `b`, column
    slabs of `c`), and the OTHER operand is copied whole first. `axis=None` picks the longer of M and N, which keeps
    the whole-operand copy — the part nothing overlaps — short."""

    def __init__(self, m: int, n: int, k: int, dtype: Any, out_dtype: Any = None, panels: int = 16,
                 axis: str | None = None) -> None:
        torch = _torch()
        self.m, self.n, self.k = m, n, k
        self.axis = axis or ("n" if n > m else "m")
        self.a = torch.empty((m, k), device="cuda", dtype=dtype)
        self.b = torch.empty((n, k), device="cuda", dtype=dtype)
        self.c = torch.empty((m, n), device="cuda", dtype=out_dtype or dtype)
        # 256-row panels keep every panel a whole number of CTA-pair tiles
        self.ranges = _panels(m if self.axis == "m" else n, panels, 256)
        self.streams = _Streams()

    def run(self, a_host: Any, b_host: Any, c_host: Any) -> None:
        torch = _torch()
        if tuple(a_host.shape) != (self.m, self.k) or tuple(b_host.shape) != (self.n, self.k) \
                or tuple(c_host.shape) != (self.m, self.n):
            raise ValueError(f"shapes do not compose: a {tuple(a_host.shape)}, b {tuple(b_host.shape)}, "
                             f"c {tuple(c_host.shape)} for a ({self.m}, {self.n}, {self.k}) product")
        current = torch.cuda.current_stream()
        s = self.streams
        s.h2d.wait_stream(current)  # earlier work on the caller's stream may still read the device buffers
        whole, paneled, whole_host, paneled_host = (self.b, self.a, b_host, a_host) if self.axis == "m" else \
            (self.a, self.b, a_host, b_host)
        with torch.cuda.stream(s.h2d):
            whole.copy_(whole_host, non_blocking=True)
            for index, (lo, hi) in enumerate(self.ranges):
                paneled[lo:hi].copy_(paneled_host[lo:hi], non_blocking=True)
                s.event(2 * index).record(s.h2d)
        for index, (lo, hi) in enumerate(self.ranges):
            current.wait_event(s.event(2 * index))
            if self.axis == "m":
                calls.gemm_tn(self.a[lo:hi], self.b, self.c[lo:hi], current)
                source, target = self.c[lo:hi], c_host[lo:hi]
            else:
                calls.gemm_tn(self.a, self.b[lo:hi], self.c[:, lo:hi], current)
                source, target = self.c[:, lo:hi], c_host[:, lo:hi]
            s.event(2 * index + 1).record(current)
            s.d2h.wait_event(s.event(2 * index + 1))
            _copy_out(target, source, s.d2h)
        current.wait_stream(s.d2h)


class ShardedStreamedProduct:
    """The column-sharded product of a node with host operands: rank r of G returns `c_host[:, block r] = a_host @
    b_host[block r]^T` (its rows of `b`, its column block of `c`).

    Every rank needs all of `a`, but `a` should cross PCIe once per node, not once per GPU (eight GPUs pulling the
    same 128 MiB through the host at once were slower end to end than one GPU alone). So rank r copies only rows
    [r M/G, (r+1) M/G) of `a_host`, the row blocks are all-gathered between the GPUs over NVLink (NCCL, in place in
    the device copy of `a`), and the rank's rows of `b` stream in panels behind it with the products and the
    device→host copies of the finished column slabs overlapped as in `StreamedProduct`. M must divide by G."""

    def __init__(self, m: int, n_local: int, k: int, dtype: Any, out_dtype: Any = None, panels: int = 8,
                 group: Any = None) -> None:
        torch = _torch()
        import torch.distributed as dist

        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if m % self.world:
            raise ValueError(f"{m} rows of a do not divide over {self.world} ranks")
        self.m, self.n, self.k = m, n_local, k
        self.rows = (self.rank * (m // self.world), (self.rank + 1) * (m // self.world))
        self.a = torch.empty((m, k), device="cuda", dtype=dtype)
        self.b = torch.empty((n_local, k), device="cuda", dtype=dtype)
        self.c = torch.empty((m, n_local), device="cuda", dtype=out_dtype or dtype)
        self.ranges = _panels(n_local, panels, 256)
        self.streams = _Streams()

    def run(self, a_host: Any, b_host: Any, c_host: Any) -> None:
        torch = _torch()
        import torch.distributed as dist

        current = torch.cuda.current_stream()
        s = self.streams
        lo_a, hi_a = self.rows
        s.h2d.wait_stream(current)
        with torch.cuda.stream(s.h2d):
            self.a[lo_a:hi_a].copy_(a_host[lo_a:hi_a], non_blocking=True)
            s.event(0).record(s.h2d)
            for index, (lo, hi) in enumerate(self.ranges):
                self.b[lo:hi].copy_(b_host[lo:hi], non_blocking=True)
                s.event(2 * index + 2).record(s.h2d)
        current.wait_event(s.event(0))
        dist.all_gather_into_tensor(self.a, self.a[lo_a:hi_a], group=self.group)  # in place: the slice is the input
        for index, (lo, hi) in enumerate(self.ranges):
            current.wait_event(s.event(2 * index + 2))
            calls.gemm_tn(self.a, self.b[lo:hi], self.c[:, lo:hi], current)
            s.event(2 * index + 3).record(current)
            s.d2h.wait_event(s.event(2 * index + 3))
            _copy_out(c_host[:, lo:hi], self.c[:, lo:hi], s.d2h)
        current.wait_stream(s.d2h)


class StreamedFp8Product:
    """The block-scaled FP8 product with host operands: codes and scales of `a` (1x128 blocks) go first, then row
    panels of `b` (codes + their 128x128 block scales, panel boundaries on multiples of 256 rows); column slabs of
    `c` return as they finish. N is the streamed axis because weights outnumber activations in this product."""

    def __init__(self, m: int, n: int, k: int, out_dtype: Any, panels: int = 16) -> None:
        torch = _torch()
        self.m, self.n, self.k = m, n, k
        blocks_k = -(-k // 128)
        self.a = torch.empty((m, k), device="cuda", dtype=torch.uint8)
        self.sa = torch.empty((m, blocks_k), device="cuda", dtype=torch.float32)
        self.b = torch.empty((n, k), device="cuda", dtype=torch.uint8)
        self.sb = torch.empty((-(-n // 128), blocks_k), device="cuda", dtype=torch.float32)
        self.c = torch.empty((m, n), device="cuda", dtype=out_dtype)
        self.ranges = _panels(n, panels, 256)
        self.streams = _Streams()

    def run(self, a_host: Any, sa_host: Any, b_host: Any, sb_host: Any, c_host: Any) -> None:
        """Codes are uint8 views of the e4m3 bytes (`tensor.view(torch.uint8)`)."""
        torch = _torch()
        current = torch.cuda.current_stream()
        s = self.streams
        s.h2d.wait_stream(current)
        with torch.cuda.stream(s.h2d):
            self.a.copy_(a_host, non_blocking=True)
            self.sa.copy_(sa_host, non_blocking=True)
            for index, (lo, hi) in enumerate(self.ranges):
                self.b[lo:hi].copy_(b_host[lo:hi], non_blocking=True)
                self.sb[lo // 128:-(-hi // 128)].copy_(sb_host[lo // 128:-(-hi // 128)], non_blocking=True)
                s.event(2 * index).record(s.h2d)
        fp8 = torch.float8_e4m3fn
        for index, (lo, hi) in enumerate(self.ranges):
            current.wait_event(s.event(2 * index))
            calls.gemm_fp8_blockscaled_tn(self.a.view(fp8), self.sa, self.b[lo:hi].view(fp8),
                                          self.sb[lo // 128:-(-hi // 128)], self.c[:, lo:hi], current)
            s.event(2 * index + 1).record(current)
            s.d2h.wait_event(s.event(2 * index + 1))
            _copy_out(c_host[:, lo:hi], self.c[:, lo:hi], s.d2h)
        current.wait_stream(s.d2h)


class StreamedScaledProduct:
    """The MXFP8 / NVFP4 / MXFP4 product (block scales applied by the tensor cores) with host operands: codes and scale
    bytes of `a` go first, then row panels of `b` (codes + their scale rows, panel boundaries on multiples of 256 rows);
    column slabs of `c` return as they finish. `form` is "mxfp8", "nvfp4" or "mxfp4"; codes and scales are uint8 tensors
    as `krn_b200.ops.quantize` lays them out (4-bit codes two per byte)."""

    FORMS = {"mxfp8": (1, 32), "nvfp4": (2, 16), "mxfp4": (2, 32)}  # codes per byte, codes per scale byte

    def __init__(self, form: str, m: int, n: int, k: int, out_dtype: Any, panels: int = 16) -> None:
        torch = _torch()
        if form not in self.FORMS:
            raise ValueError(f"block format {form!r} is not available: use one of {sorted(self.FORMS)}")
        per_byte, per_scale = self.FORMS[form]
        self.form, self.m, self.n, self.k = form, m, n, k
        self.a = torch.empty((m, k // per_byte), device="cuda", dtype=torch.uint8)
        self.sa = torch.empty((m, k // per_scale), device="cuda", dtype=torch.uint8)
        self.b = torch.empty((n, k // per_byte), device="cuda", dtype=torch.uint8)
        self.sb = torch.empty((n, k // per_scale), device="cuda", dtype=torch.uint8)
        self.c = torch.empty((m, n), device="cuda", dtype=out_dtype)
        self.ranges = _panels(n, panels, 256)
        self.streams = _Streams()

    def run(self, a_host: Any, sa_host: Any, b_host: Any, sb_host: Any, c_host: Any, alpha: float = 1.0) -> None:
        """`alpha` (the product of the two tensor scales) applies to NVFP4 only."""
        torch = _torch()
        current = torch.cuda.current_stream()
        s = self.streams
        s.h2d.wait_stream(current)
        with torch.cuda.stream(s.h2d):
            self.a.copy_(a_host, non_blocking=True)
            self.sa.copy_(sa_host, non_blocking=True)
            for index, (lo, hi) in enumerate(self.ranges):
                self.b[lo:hi].copy_(b_host[lo:hi], non_blocking=True)
                self.sb[lo:hi].copy_(sb_host[lo:hi], non_blocking=True)
                s.event(2 * index).record(s.h2d)
        for index, (lo, hi) in enumerate(self.ranges):
            current.wait_event(s.event(2 * index))
            if self.form == "mxfp8":
                fp8 = torch.float8_e4m3fn
                calls.gemm_mxfp8_tn(self.a.view(fp8), self.sa, self.b[lo:hi].view(fp8), self.sb[lo:hi], self.c[:, lo:hi], current)
            elif self.form == "nvfp4":
                calls.gemm_nvfp4_tn(self.a, self.sa, self.b[lo:hi], self.sb[lo:hi], self.c[:, lo:hi], alpha, current)
            else:
                calls.gemm_mxfp4_tn(self.a, self.sa, self.b[lo:hi], self.sb[lo:hi], self.c[:, lo:hi], current)
            s.event(2 * index + 1).record(current)
            s.d2h.wait_event(s.event(2 * index + 1))
            _copy_out(c_host[:, lo:hi], self.c[:, lo:hi], s.d2h)
        current.wait_stream(s.d2h)


class ShardedStreamedFp8Product:
    """The column-sharded block-scaled FP8 product with host operands, as `ShardedStreamedProduct`: rank r copies only
    its M/G rows of `a` (codes and 1x128 scales), NCCL all-gathers both over NVLink, and the rank's rows of `b` (codes
    and 128x128 scales) stream in panels with the column slabs of its block of `c` returning as they finish."""

    def __init__(self, m: int, n_local: int, k: int, out_dtype: Any, panels: int = 8, group: Any = None) -> None:
        torch = _torch()
        import torch.distributed as dist

        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if m % self.world:
            raise ValueError(f"{m} rows of a do not divide over {self.world} ranks")
        self.m, self.n, self.k = m, n_local, k
        self.rows = (self.rank * (m // self.world), (self.rank + 1) * (m // self.world))
        blocks_k = -(-k // 128)
        self.a = torch.empty((m, k), device="cuda", dtype=torch.uint8)
        self.sa = torch.empty((m, blocks_k), device="cuda", dtype=torch.float32)
        self.b = torch.empty((n_local, k), device="cuda", dtype=torch.uint8)
        self.sb = torch.empty((-(-n_local // 128), blocks_k), device="cuda", dtype=torch.float32)
        self.c = torch.empty((m, n_local), device="cuda", dtype=out_dtype)
        self.ranges = _panels(n_local, panels, 256)
        self.streams = _Streams()

    def run(self, a_host: Any, sa_host: Any, b_host: Any, sb_host: Any, c_host: Any) -> None:
        torch = _torch()
        import torch.distributed as dist

        current = torch.cuda.current_stream()
        s = self.streams
        lo_a, hi_a = self.rows
        s.h2d.wait_stream(current)
        with torch.cuda.stream(s.h2d):
            self.a[lo_a:hi_a].copy_(a_host[lo_a:hi_a], non_blocking=True)
            self.sa[lo_a:hi_a].copy_(sa_host[lo_a:hi_a], non_blocking=True)
            s.event(0).record(s.h2d)
            for index, (lo, hi) in enumerate(self.ranges):
                self.b[lo:hi].copy_(b_host[lo:hi], non_blocking=True)
                self.sb[lo // 128:-(-hi // 128)].copy_(sb_host[lo // 128:-(-hi // 128)], non_blocking=True)
                s.event(2 * index + 2).record(s.h2d)
        current.wait_event(s.event(0))
        dist.all_gather_into_tensor(self.a, self.a[lo_a:hi_a], group=self.group)
        dist.all_gather_into_tensor(self.sa, self.sa[lo_a:hi_a], group=self.group)
        fp8 = torch.float8_e4m3fn
        for index, (lo, hi) in enumerate(self.ranges):
            current.wait_event(s.event(2 * index + 2))
            calls.gemm_fp8_blockscaled_tn(self.a.view(fp8), self.sa, self.b[lo:hi].view(fp8),
                                          self.sb[lo // 128:-(-hi // 128)], self.c[:, lo:hi], current)
            s.event(2 * index + 3).record(current)
            s.d2h.wait_event(s.event(2 * index + 3))
            _copy_out(c_host[:, lo:hi], self.c[:, lo:hi], s.d2h)
        current.wait_stream(s.d2h)


class StreamedAttention:
    """Flash-attention forward over host tensors q, o (batch, q_heads, seq, d) and k, v (batch, kv_heads, seq, d),
    streamed one group of batches at a time (batches are independent, so nothing is copied whole)."""

    def __init__(self, batch: int, q_heads: int, kv_heads: int, seq: int, d: int, dtype: Any, groups: int = 8) -> None:
        torch = _torch()
        self.shape_q, self.shape_kv = (batch, q_heads, seq, d), (batch, kv_heads, seq, d)
        self.q = torch.empty(self.shape_q, device="cuda", dtype=dtype)
        self.k = torch.empty(self.shape_kv, device="cuda", dtype=dtype)
        self.v = torch.empty(self.shape_kv, device="cuda", dtype=dtype)
        self.o = torch.empty(self.shape_q, device="cuda", dtype=dtype)
        self.ranges = _panels(batch, groups, 1)
        self.streams = _Streams()

    def run(self, q_host: Any, k_host: Any, v_host: Any, o_host: Any, scale_log2: float, causal: bool) -> None:
        torch = _torch()
        current = torch.cuda.current_stream()
        s = self.streams
        s.h2d.wait_stream(current)
        with torch.cuda.stream(s.h2d):
            for index, (lo, hi) in enumerate(self.ranges):
                for device, host in ((self.q, q_host), (self.k, k_host), (self.v, v_host)):
                    device[lo:hi].copy_(host[lo:hi], non_blocking=True)
                s.event(2 * index).record(s.h2d)
        for index, (lo, hi) in enumerate(self.ranges):
            current.wait_event(s.event(2 * index))
            calls.attention_forward(self.q[lo:hi], self.k[lo:hi], self.v[lo:hi], self.o[lo:hi], scale_log2, causal, current)
            s.event(2 * index + 1).record(current)
            s.d2h.wait_event(s.event(2 * index + 1))
            with torch.cuda.stream(s.d2h):
                o_host[lo:hi].copy_(self.o[lo:hi], non_blocking=True)
        current.wait_stream(s.d2h)
