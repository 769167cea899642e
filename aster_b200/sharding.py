"""M-row sharding of a GEMM over the GPUs of one box.

Output rows are independent, so ``C = A . B^T`` splits into contiguous row blocks of A and C
with B replicated: each rank runs the single-GPU kernel on its block and no collective is on
the compute path.  :func:`allgather_rows` is the optional exchange for callers that need the
whole C on every rank (NCCL over NVLink when the tensors are on GPUs, gloo on CPU).

The reference only fans independent configs out over GPUs
(contrib/kittens/test/bench/bench_harness.py:999-1053); per-shard results here are defined to
be the corresponding row slices of the single-GPU result.
"""

from __future__ import annotations

import numpy as np

ROW_ALIGN = 128  # rows per CTA tile: shard boundaries on tile boundaries keep shards bit-identical slices


def shard_rows(M: int, world_size: int, rank: int, align: int = ROW_ALIGN) -> tuple[int, int]:
    """``(first_row, num_rows)`` of ``rank``'s block.  Blocks are contiguous, cover ``[0, M)``
    exactly once, start on multiples of ``align`` and differ by at most one aligned unit."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of {world_size}")
    units = -(-M // align)
    base, extra = divmod(units, world_size)
    first_unit = rank * base + min(rank, extra)
    n_units = base + (1 if rank < extra else 0)
    first = min(first_unit * align, M)
    last = min((first_unit + n_units) * align, M)
    return first, last - first


def sharded_uniform_rows(seed: int, first_row: int, num_rows: int, K: int, block_rows: int = 8192) -> np.ndarray:
    """Rows ``[first_row, first_row + num_rows)`` of the global operand whose fixed
    ``block_rows``-row blocks are drawn U(-1, 1) from ``default_rng([seed, block])``: every
    world size sees the same global matrix.  float32."""
    out = np.empty((num_rows, K), dtype=np.float32)
    row = first_row
    while row < first_row + num_rows:
        block = row // block_rows
        lo = row - block * block_rows
        take = min(block_rows - lo, first_row + num_rows - row)
        vals = np.random.default_rng([seed, block]).uniform(-1.0, 1.0, size=(block_rows, K)).astype(np.float32)
        out[row - first_row: row - first_row + take] = vals[lo: lo + take]
        row += take
    return out


def allgather_rows(c_shard, M: int, group=None):
    """All-gather the row shards of C (torch tensors, any device) into the full ``[M, N]``
    tensor on every rank.  Shards may be ragged (the last ranks may hold fewer rows)."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    sizes = [shard_rows(M, world, r)[1] for r in range(world)]
    # The exchange moves bytes: bf16 bit patterns held as 16-bit integers (a type NCCL's
    # process group rejects) travel as uint8 and are viewed back afterwards.
    dtype = c_shard.dtype
    if dtype in (torch.int16, torch.uint16):
        return allgather_rows(c_shard.contiguous().view(torch.uint8), M, group).view(dtype)
    n = c_shard.shape[1]
    if len(set(sizes)) == 1:
        full = torch.empty((M, n), dtype=c_shard.dtype, device=c_shard.device)
        dist.all_gather_into_tensor(full, c_shard.contiguous(), group=group)
        return full
    pad = max(sizes)
    padded = torch.zeros((pad, n), dtype=c_shard.dtype, device=c_shard.device)
    padded[: c_shard.shape[0]] = c_shard
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[:s] for p, s in zip(parts, sizes)], dim=0)


class NcclRowGather:
    """One process, several GPUs: gathers byte shards onto every GPU through the C ABI
    (``b200_nccl_init_all`` / ``b200_allgather_rows_all``), without torch.

    ``devices`` lists the CUDA device of each rank.  :meth:`allgather` takes, per rank, the
    device address of its shard and of its full-size destination (both on that rank's GPU)
    and enqueues the exchange on each GPU's default stream (or on ``streams``); it returns
    once the work is enqueued.  The shard may already sit in its own slot of the destination.
    """

    def __init__(self, devices) -> None:
        import ctypes as C

        from . import _native as nat

        self._nat, self._C = nat, C
        self.devices = [int(d) for d in devices]
        self._comm = None
        comm = C.c_void_p()
        nat.call("b200_nccl_init_all", len(self.devices), (C.c_int * len(self.devices))(*self.devices), C.byref(comm))
        self._comm = comm.value

    @staticmethod
    def version() -> int:
        import ctypes as C

        from . import _native as nat

        v = C.c_int(0)
        nat.call("b200_nccl_version", C.byref(v))
        return v.value

    def allgather(self, c_shards, c_fulls, bytes_per_rank: int, streams=None) -> None:
        C, n = self._C, len(self.devices)
        if self._comm is None:
            raise RuntimeError("communicator already destroyed")
        if len(c_shards) != n or len(c_fulls) != n or (streams is not None and len(streams) != n):
            raise ValueError(f"expected {n} shard, destination and stream entries")

        def addr(x):
            return getattr(x, "ptr_value", None) or int(getattr(x, "value", x) or 0)

        arr = C.c_void_p * n
        self._nat.call(
            "b200_allgather_rows_all", C.c_void_p(self._comm), arr(*[addr(x) for x in c_shards]),
            arr(*[addr(x) for x in c_fulls]), int(bytes_per_rank),
            None if streams is None else arr(*[addr(s) for s in streams]),
        )

    def destroy(self) -> None:
        if self._comm is not None:
            comm, self._comm = self._comm, None
            self._nat.call("b200_nccl_destroy", self._C.c_void_p(comm))

    def __enter__(self):
        return self

    def __exit__(self, *_):
        self.destroy()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass
