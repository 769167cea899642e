"""Two ranks on two GPUs (skipped on a single-GPU box): each computes its row shard with the
CUDA GEMM, the optional NCCL all-gather rebuilds C, and the result equals the single-GPU
product bit for bit.  Ranks are child processes; NVLS is switched off for them."""

import os
import socket

import numpy as np
import pytest

from aster_b200 import _native as nat

pytestmark = pytest.mark.gpu


def _rank(rank, world, port, M, N, K, out):
    try:
        _rank_body(rank, world, port, M, N, K, out)
    except Exception:  # report instead of leaving the parent to time out
        import traceback

        out.put(("error", f"rank {rank}: {traceback.format_exc()}"))
        raise


def _rank_body(rank, world, port, M, N, K, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist

    from aster_b200.dtypes import from_f32
    from aster_b200.gemm import gemm
    from aster_b200.sharding import allgather_rows, shard_rows, sharded_uniform_rows

    torch.cuda.set_device(rank)
    nat.call("b200_init", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        first, rows = shard_rows(M, world, rank)
        a = from_f32(sharded_uniform_rows(4, first, rows, K, block_rows=256), "bf16")
        b = from_f32(np.random.default_rng(5).uniform(-1, 1, (N, K)).astype(np.float32), "bf16")
        c = gemm(a, b, dtype_ab="bf16", dtype_c="bf16", tile_n=128)
        shard = torch.from_numpy(c.view(np.int16)).cuda()
        full = allgather_rows(shard, M).cpu().numpy().view(np.uint16)
        if rank == 0:
            a_full = from_f32(sharded_uniform_rows(4, 0, M, K, block_rows=256), "bf16")
            whole = gemm(a_full, b, dtype_ab="bf16", dtype_c="bf16", tile_n=128)
            out.put((bool(np.array_equal(full, whole)), tuple(full.shape)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_row_shards_allgathered_equal_the_whole(gpu):
    if nat.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    M, N, K = 1024 + 128, 512, 768  # ragged: 5 + 4 row blocks of 128
    procs = [ctx.Process(target=_rank, args=(r, 2, port, M, N, K, out)) for r in range(2)]
    for p in procs:
        p.start()
    ok, shape = out.get(timeout=180)
    assert ok != "error", shape
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert ok is True and shape == (M, N)


def _rank_pipeline(rank, world, port, M, N, K, out):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        import torch
        import torch.distributed as dist

        from aster_b200.dtypes import from_f32
        from aster_b200.gemm import GemmPlan, gemm
        from aster_b200.sharding import ShardedHostGemmPipeline, bind_to_gpu_numa_node, shard_rows, sharded_uniform_rows

        torch.cuda.set_device(rank)
        nat.call("b200_init", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        try:
            bind_to_gpu_numa_node(rank)  # a no-op where the platform names no node
            first, rows = shard_rows(M, world, rank)
            a = from_f32(sharded_uniform_rows(4, first, rows, K, block_rows=256), "bf16")
            b = from_f32(np.random.default_rng(5).uniform(-1, 1, (N, K)).astype(np.float32), "bf16")
            plan = GemmPlan(rows, N, K, "bf16", "bf16", tile_n=128)
            pipe = ShardedHostGemmPipeline(plan, rank, world, depth=2)
            hA, hB = pipe.pinned_operands()
            hA.array[...] = a
            hB.array[...] = b[pipe.b_row_slice]  # this rank's share of B only
            assert pipe.h2d_bytes_per_problem == a.nbytes + b.nbytes // world
            results = []
            for _ in range(3):  # both slots, and a slot reused
                slot = pipe.submit(hA, hB)
                results.append(pipe.result(slot).copy())
            pipe.close()
            hA.free(), hB.free()
            whole = gemm(a, b, dtype_ab="bf16", dtype_c="bf16", tile_n=128)  # all of B uploaded the plain way
            out.put((rank, all(bool(np.array_equal(r, whole)) for r in results)))
            dist.barrier()
        finally:
            dist.destroy_process_group()
    except Exception:
        import traceback

        out.put(("error", f"rank {rank}: {traceback.format_exc()}"))
        raise


def test_sharded_host_pipeline_rebuilds_b_over_nvlink(gpu):
    """End to end on two ranks: each uploads its rows of A and half of B, the all-gather rebuilds B
    on both GPUs, and every rank's C equals what it gets with all of B uploaded."""
    if nat.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_rank_pipeline, args=(r, 2, port, 1024, 512, 768, out)) for r in range(2)]
    for p in procs:
        p.start()
    got = [out.get(timeout=180) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
    assert sorted(got) == [(0, True), (1, True)], got
    assert all(p.exitcode == 0 for p in procs)


def test_single_process_gather_through_the_c_abi(gpu):
    """One process drives both GPUs: a plan per GPU computes its row shard, the NCCL entry
    points of the C ABI put all of C on both, and both copies equal the one-GPU product."""
    if nat.device_count() < 2:
        pytest.skip("needs two GPUs")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from aster_b200.dtypes import from_f32
    from aster_b200.execution import GpuBuffer
    from aster_b200.gemm import GemmPlan, gemm
    from aster_b200.sharding import NcclRowGather

    M, N, K = 512, 384, 256
    rows = M // 2
    rng = np.random.default_rng(8)
    a = from_f32(rng.uniform(-1, 1, (M, K)).astype(np.float32), "bf16")
    b = from_f32(rng.uniform(-1, 1, (N, K)).astype(np.float32), "bf16")
    assert NcclRowGather.version() >= 21800
    keep, fulls, shards = [], [], []
    try:
        for d in (0, 1):
            nat.call("b200_set_device", d)
            da, db, full = GpuBuffer(rows * K * 2), GpuBuffer(N * K * 2), GpuBuffer(M * N * 2)
            da.copy_from_host(a[d * rows:(d + 1) * rows])
            db.copy_from_host(b)
            full.zero()
            plan = GemmPlan(rows, N, K, "bf16", "bf16", tile_n=128)
            if d == 0:  # rank 0 writes its shard straight into its slot of the destination
                plan.run(da, db, full.ptr_value)
                shards.append(full.ptr_value)
            else:       # rank 1 gathers from a separate buffer
                shard = GpuBuffer(rows * N * 2)
                plan.run(da, db, shard)
                shards.append(shard)
                keep.append(shard)
            nat.call("b200_device_synchronize")
            keep += [da, db, plan]
            fulls.append(full)
        with NcclRowGather([0, 1]) as gather:
            with pytest.raises(nat.B200Error, match="overlaps"):  # refused before NCCL sees any rank
                gather.allgather([fulls[0].ptr_value + 64, shards[1]], fulls, rows * N * 2)
            gather.allgather(shards, fulls, rows * N * 2)
            got = []
            for d in (0, 1):
                nat.call("b200_set_device", d)
                nat.call("b200_device_synchronize")
                host = np.empty((M, N), dtype=np.uint16)
                fulls[d].copy_to_host(host)
                got.append(host)
    finally:
        nat.call("b200_set_device", 0)
    whole = gemm(a, b, dtype_ab="bf16", dtype_c="bf16", tile_n=128).view(np.uint16)
    assert np.array_equal(got[0], whole) and np.array_equal(got[1], whole)
