"""The N > 1 host logic on CPU: two gloo ranks shard the tile product by output column blocks, all-gather and
re-lay-out, and must reproduce the unsharded oracle product; unit and length-balanced sharding tables agree across
ranks. (The kernels themselves need a GPU; here each rank's block is computed by the oracle.)"""

from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

from krn_b200 import sharding

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results) -> None:
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist

    from oracle import oracle as o

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, n, k = 96, 512, 160
        aw, bw = o.config_gemm_bf16(m, n, k, seed=1)
        begin, end = sharding.column_block(n, rank, world)
        local = o.gemm(aw, bw[begin:end], ab_type=o.BF16, c_type=o.BF16)
        c_local = torch.from_numpy(local.astype(np.int32))  # gloo has no 16-bit integer type: widen the words
        slabs = torch.empty((world, m, end - begin), dtype=torch.int32)
        c_full = torch.empty((m, n), dtype=torch.int32)
        sharding.gather_columns(c_local, slabs, c_full, world)
        want = o.gemm(aw, bw, ab_type=o.BF16, c_type=o.BF16)
        ok = np.array_equal(c_full.numpy().astype(np.uint16), want)
        lengths = np.random.default_rng(4).integers(1024, 8193, 64)
        table = sharding.balanced_by_length(lengths, world)
        gathered = [None] * world
        dist.all_gather_object(gathered, table)
        results.put((rank, ok, all(t == table for t in gathered)))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_unsharded_product() -> None:
    import torch.multiprocessing as mp

    context = mp.get_context("spawn")
    results = context.Queue()
    port = _free_port()
    workers = [context.Process(target=_worker, args=(rank, 2, port, results)) for rank in range(2)]
    for w in workers:
        w.start()
    for w in workers:
        w.join(timeout=120)
        assert w.exitcode == 0
    got = sorted(results.get(timeout=10) for _ in range(2))
    assert got == [(0, True, True), (1, True, True)]


def test_sharding_tables() -> None:
    assert sharding.column_block(8192, 3, 8) == (3072, 4096)
    assert sharding.column_block(28672, 7, 8) == (25088, 28672)
    with pytest.raises(ValueError):
        sharding.column_block(8192 + 128, 0, 8)
    units = [list(sharding.contiguous_units(64, r, 8)) for r in range(8)]
    assert sum(units, []) == list(range(64)) and all(len(u) == 8 for u in units)
    assert [list(sharding.contiguous_units(10, r, 4)) for r in range(4)] == [[0, 1], [2, 3, 4], [5, 6], [7, 8, 9]]
    lengths = np.random.default_rng(4).integers(1024, 8193, 64)
    table = sharding.balanced_by_length(lengths, 8)
    assert sorted(sum(table, [])) == list(range(64))
    loads = [int(lengths[t].sum()) for t in table]
    assert max(loads) - min(loads) <= int(lengths.max())  # the LPT bound
    assert max(loads) <= 1.05 * sum(loads) / 8


def test_gather_schedule_alternates_copies_and_numbers_products() -> None:
    """Product i writes copy (i - 1) % buffers and carries number i: the bookkeeping that keeps a peer's stores out of a
    copy of C that is still being read."""
    schedule = sharding.GatherSchedule(2)
    assert [schedule.next() for _ in range(5)] == [(0, 1), (1, 2), (0, 3), (1, 4), (0, 5)]
    single = sharding.GatherSchedule(1)
    assert [single.next() for _ in range(3)] == [(0, 1), (0, 2), (0, 3)]
    with pytest.raises(ValueError):
        sharding.GatherSchedule(0)
