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
