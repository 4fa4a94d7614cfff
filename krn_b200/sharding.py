"""How the path is split over the GPUs of one node (one process per GPU, `torch.distributed`).

* Tile matrix product: output COLUMN blocks. Rank r multiplies A by rows [r*N/G, (r+1)*N/G) of B (and its slab of
  block scales), producing C[:, block r]; one all-gather of the column blocks is the path's only exchange, followed
  by a re-layout of the gathered slabs into one row-major C.
* Flash attention: (batch, kv head) units, contiguous per rank, so the q heads of a kv head stay together. No
  collective.
* Paged decode: sequences, balanced by context length (longest first onto the least loaded rank). No collective.

The reference has no multi-device path; nothing here has a counterpart in it."""

from __future__ import annotations

from typing import Any, Sequence


def column_block(n: int, rank: int, world: int, multiple: int = 128) -> tuple[int, int]:
    """[begin, end) of the output columns rank `rank` owns: equal blocks, each a multiple of `multiple` columns so
    that 128-column scale blocks and 256-column tiles are not split between ranks."""
    if n % (world * multiple) != 0:
        raise ValueError(f"N = {n} does not split into {world} blocks of a multiple of {multiple} columns")
    width = n // world
    return rank * width, (rank + 1) * width


def contiguous_units(count: int, rank: int, world: int) -> range:
    """Unit indices [begin, end) of `rank` when `count` independent units are dealt in contiguous runs."""
    return range(count * rank // world, count * (rank + 1) // world)


def balanced_by_length(lengths: Sequence[int], world: int) -> list[list[int]]:
    """Longest-processing-time assignment of sequences to ranks: indices sorted by length, longest first, each to the
    rank with the least total so far (ties to the lower rank). Deterministic, so every rank computes the same table."""
    loads = [0] * world
    assignment: list[list[int]] = [[] for _ in range(world)]
    for index in sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i)):
        rank = min(range(world), key=lambda r: (loads[r], r))
        assignment[rank].append(index)
        loads[rank] += int(lengths[index])
    return [sorted(indices) for indices in assignment]


def gather_columns(c_local: Any, slabs: Any, c_full: Any, world: int, group: Any = None, stream: Any = None) -> None:
    """All-gather every rank's [M, N/G] column block into `slabs` [G, M, N/G] and lay them out as the row-major
    `c_full` [M, N]. On CUDA tensors the re-layout is the library's `krn_b200_scatter_columns` kernel; on CPU tensors
    (gloo, used by the host-logic tests) it is a strided copy."""
    import torch.distributed as dist

    dist.all_gather_into_tensor(slabs.view(-1, slabs.shape[-1]), c_local, group=group)  # concatenation along rows
    if c_full.is_cuda:
        from krn_b200.runtime import calls

        calls.scatter_columns(slabs, c_full, world, stream)
    else:
        m, width = c_local.shape
        c_full.view(m, world, width).copy_(slabs.permute(1, 0, 2))


class GatherSchedule:
    """Which copy of C a product writes and what number it carries, for a `GatheredProduct` with `buffers` copies.

    Product i (1, 2, 3, ...) writes copy (i - 1) % buffers and signals number i. With two copies a rank that starts
    product i + 2 has finished product i + 1, whose completion means every rank had launched i + 1, i.e. every rank's
    stream is past whatever read copy i % buffers after product i: peers' stores can never land in a copy that is still
    being read, without any extra barrier. With one copy the caller must keep all ranks from starting a product until
    every rank has consumed the previous one."""

    def __init__(self, buffers: int = 2) -> None:
        if buffers < 1:
            raise ValueError("at least one copy of C is needed")
        self.buffers, self.count = buffers, 0

    def next(self) -> tuple[int, int]:
        """(copy to write, product number) of the next product."""
        self.count += 1
        return (self.count - 1) % self.buffers, self.count


SYNC_WORDS = 16  # per rank: 8 flags + the arrival counter (+ padding), 32-bit each


class GatheredProduct:
    """C = A @ B^T sharded by output columns with the all-gather AND the cross-rank completion inside the product kernel.

    Every rank allocates `buffers` full copies of C and a few sync words in symmetric memory (torch's
    `_symmetric_memory`: CUDA virtual-memory allocations mapped into every peer over NVLink; multicast binding is
    switched off because only unicast peer stores are used) and calls `run(a, b_local)`: the kernel stores this rank's
    column block into all ranks' C from its epilogue, tile by tile, and its last CTA exchanges "my stores have landed"
    flags with the peers, waiting — for at most about two seconds — until all have said so. When `run`'s kernel has
    completed on a stream, the returned tensor holds the whole product on this rank; there is no barrier kernel and no
    host round trip. A peer that never launches shows up as KRN_B200_ERR_DEVICE_TIMEOUT in the status word
    (`native.raise_device_status()` after a synchronisation), not as a hang.

    Consecutive products alternate between the copies of C (see `GatherSchedule`), so the tensor returned by product
    i stays valid until product i + `buffers` is enqueued."""

    def __init__(self, m: int, n: int, dtype: Any, group: Any = None, multiple: int = 64, buffers: int = 2) -> None:
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.m, self.n = m, n
        begin, end = column_block(n, self.rank, self.world, multiple)
        self.n_local = end - begin
        device = torch.device("cuda", torch.cuda.current_device())
        self.schedule = GatherSchedule(buffers)
        self.copies, self.handles, self.pointers = [], [], []
        for _ in range(buffers):
            c = symm.empty((m, n), dtype=dtype, device=device)
            handle = symm.rendezvous(c, self.group)
            self.copies.append(c)
            self.handles.append(handle)
            self.pointers.append([int(p) for p in handle.buffer_ptrs])
        self.sync = symm.empty((SYNC_WORDS,), dtype=torch.int32, device=device)
        self.sync_handle = symm.rendezvous(self.sync, self.group)
        self.sync_pointers = [int(p) for p in self.sync_handle.buffer_ptrs]
        self.sync.zero_()
        torch.cuda.synchronize()
        dist.barrier(self.group)  # every rank's sync words are zero before anyone's kernel can write a flag
        from krn_b200.runtime import native

        self.c_type = {torch.bfloat16: native.BF16, torch.float16: native.F16, torch.float32: native.F32}[dtype]

    @property
    def c(self) -> Any:
        """The copy of C the most recent product wrote (the first copy before any product)."""
        return self.copies[(max(self.schedule.count, 1) - 1) % self.schedule.buffers]

    def run(self, a: Any, b_local: Any, stream: Any = None) -> Any:
        """Enqueue the product on `stream` (torch's current stream when None) and return the copy of C it fills."""
        from krn_b200.runtime import calls

        copy, epoch = self.schedule.next()
        calls.gemm_tn_gather(a, b_local, self.pointers[copy], self.rank, self.m, self.n_local, self.n, self.c_type, stream,
                             sync_pointers=self.sync_pointers, epoch=epoch)
        return self.copies[copy]

    def run_fp8(self, a: Any, sa: Any, b_local: Any, sb_local: Any, stream: Any = None) -> Any:
        """The block-scaled FP8 product through the same destinations (construct with `multiple=128`: a column block
        must end on a scale block of b)."""
        from krn_b200.runtime import calls

        copy, epoch = self.schedule.next()
        calls.gemm_fp8_blockscaled_tn_gather(a, sa, b_local, sb_local, self.pointers[copy], self.rank, self.n_local, self.n,
                                             self.c_type, stream, sync_pointers=self.sync_pointers, epoch=epoch)
        return self.copies[copy]
