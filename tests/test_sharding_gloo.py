"""Host-side multi-rank logic on CPU ranks (gloo, world size 2): row partitioning, identical
global operands for every world size, and the optional all-gather of C shards.  The shard
"compute" here is the oracle -- the point is the partition and the exchange, not the kernel."""

import os
import socket

import numpy as np
import pytest

from aster_b200.sharding import shard_rows, sharded_uniform_rows


@pytest.mark.parametrize("M", [1, 100, 128, 4096, 65536, 65536 + 5, 1000])
@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_partition_covers_rows_once(M, world):
    spans = [shard_rows(M, world, r) for r in range(world)]
    assert spans[0][0] == 0 and sum(n for _, n in spans) == M
    for (f0, n0), (f1, _) in zip(spans, spans[1:]):
        assert f0 + n0 == f1
    for f, n in spans:
        assert f % 128 == 0 or n == 0
    sizes = [n for _, n in spans]
    assert max(sizes) - min(sizes) < 2 * 128 or M < 128 * world


def test_partition_of_the_configured_sweep():
    for g in (1, 2, 4, 8):
        assert [shard_rows(65536, g, r)[1] for r in range(g)] == [65536 // g] * g
    with pytest.raises(ValueError):
        shard_rows(10, 2, 2)


def test_global_operand_is_world_size_independent():
    whole = sharded_uniform_rows(4, 0, 600, 16, block_rows=256)
    for g in (2, 3):
        parts = []
        for r in range(g):
            f, n = shard_rows(600, g, r)
            parts.append(sharded_uniform_rows(4, f, n, 16, block_rows=256))
        assert np.array_equal(np.concatenate(parts), whole)
    assert whole.min() >= -1 and whole.max() < 1


def _rank_main(rank, world, port, M, N, K, out):
    import torch
    import torch.distributed as dist

    from aster_b200.sharding import allgather_rows
    from oracle import gemm_oracle as orc

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        first, rows = shard_rows(M, world, rank)
        a = orc.encode(sharded_uniform_rows(4, first, rows, K, block_rows=256), "bf16")
        b = orc.encode(np.random.default_rng(5).uniform(-1, 1, (N, K)).astype(np.float32), "bf16")
        c_bits = orc.gemm(a, b, "bf16", "bf16")  # bf16 bit patterns, as the GPU path returns them
        full_bits = allgather_rows(torch.from_numpy(c_bits.view(np.int16)), M)  # 16-bit ints travel as bytes
        full = allgather_rows(torch.from_numpy(orc.decode(c_bits, "bf16")), M)
        a_full = orc.encode(sharded_uniform_rows(4, 0, M, K, block_rows=256), "bf16")
        want_bits = orc.gemm(a_full, b, "bf16", "bf16")
        ok = np.array_equal(full.numpy(), orc.decode(want_bits, "bf16")) and np.array_equal(full_bits.numpy().view(np.uint16), want_bits)
        out.put((rank, bool(ok), tuple(full.shape)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("M", [512, 640 + 3])
def test_allgather_of_row_shards_world2(M):
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, M, 48, 64, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == [0, 1]
    assert all(ok and shape == (M, 48) for _, ok, shape in results)
