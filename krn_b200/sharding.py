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
