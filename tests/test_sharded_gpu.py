"""Two ranks on two GPUs: the column-sharded product with the all-gather fused into the kernel's epilogue, and the
sharded host-operand path whose `a` is all-gathered over NVLink. Skipped on a machine with one GPU (the sharded entry
points themselves are also exercised on one GPU in tests/test_gemm_gpu.py and tests/test_gemm_fp8_gpu.py)."""

from __future__ import annotations

import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank: int, world: int, port: int, failures) -> None:
    import torch
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from krn_b200 import sharding, streaming
        from krn_b200.runtime import calls

        m, n, k = 512, 1024, 328
        gen = torch.Generator().manual_seed(5)
        a_host = torch.randint(-4, 5, (m, k), generator=gen).to(torch.bfloat16).pin_memory()
        b_host = torch.randint(-4, 5, (n, k), generator=gen).to(torch.bfloat16).pin_memory()
        a, b = a_host.cuda(), b_host.cuda()
        whole = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
        calls.gemm_tn(a, b, whole)
        begin, end = sharding.column_block(n, rank, world, 64)

        from krn_b200.runtime import native

        fused = sharding.GatheredProduct(m, n, torch.bfloat16)
        for c in fused.copies:
            c.fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()
        # three products in a row on a side stream, each read back (on that stream) before the next is enqueued: the
        # kernel's own tail is the only cross-rank synchronisation
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        sums = []
        with torch.cuda.stream(side):
            for scale in (1, 2, 4):  # powers of two: scaling commutes with the bf16 rounding of the output
                result = fused.run(a * scale, b[begin:end])
                sums.append((result.float() - whole.float() * scale).abs().max())
        side.synchronize()
        native.raise_device_status()
        if any(float(x) != 0.0 for x in sums):
            failures.put(f"rank {rank}: the fused gather does not hold the whole product: {[float(x) for x in sums]}")

        streamed = streaming.ShardedStreamedProduct(m, end - begin, k, torch.bfloat16, panels=2)
        c_host = torch.full((m, end - begin), float("nan"), dtype=torch.bfloat16).pin_memory()
        zeros = torch.zeros_like(a_host)
        zeros[streamed.rows[0]:streamed.rows[1]] = a_host[streamed.rows[0]:streamed.rows[1]]
        streamed.run(zeros, b_host[begin:end], c_host)  # only this rank's rows of a are read from ITS host copy
        torch.cuda.synchronize()
        if not torch.equal(c_host, whole[:, begin:end].cpu()):
            failures.put(f"rank {rank}: the sharded host-operand product differs from the one-GPU product")

        import numpy as np
        from oracle import oracle as o

        a_codes, sa, b_codes, sb = o.config_gemm_fp8(256, 1024, 512, seed=6)
        hosts = [torch.from_numpy(x).pin_memory() for x in (a_codes, sa, b_codes, sb)]
        fp8 = torch.float8_e4m3fn
        whole8 = torch.empty((256, 1024), device="cuda", dtype=torch.bfloat16)
        calls.gemm_fp8_blockscaled_tn(hosts[0].cuda().view(fp8), hosts[1].cuda(), hosts[2].cuda().view(fp8), hosts[3].cuda(),
                                      whole8)
        begin8, end8 = sharding.column_block(1024, rank, world, 256)
        product8 = streaming.ShardedStreamedFp8Product(256, end8 - begin8, 512, torch.bfloat16, panels=2)
        c8 = torch.full((256, end8 - begin8), float("nan"), dtype=torch.bfloat16).pin_memory()
        product8.run(hosts[0], hosts[1], hosts[2][begin8:end8], hosts[3][begin8 // 128:end8 // 128], c8)
        torch.cuda.synchronize()
        if not torch.equal(c8, whole8[:, begin8:end8].cpu()):
            failures.put(f"rank {rank}: the sharded host-operand FP8 product differs from the one-GPU product")
    except Exception as error:  # reported to the parent, which fails the test
        failures.put(f"rank {rank}: {type(error).__name__}: {error}")
    finally:
        dist.destroy_process_group()


def test_two_ranks_fused_gather_and_sharded_streaming(cuda) -> None:
    torch = cuda
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    context = mp.get_context("spawn")
    failures = context.Queue()
    port = _free_port()
    workers = [context.Process(target=_rank, args=(rank, 2, port, failures)) for rank in range(2)]
    for w in workers:
        w.start()
    for w in workers:
        w.join(timeout=180)
    hung = [w for w in workers if w.is_alive()]
    for w in hung:
        w.terminate()  # our own children, by handle
    problems = []
    while not failures.empty():
        problems.append(failures.get())
    assert not hung and not problems and all(w.exitcode == 0 for w in workers), problems
