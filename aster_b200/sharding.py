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


def sharded_uniform_rows(seed: int, first_row: int, num_rows: int, K: int, block_rows: int = 8192, threads: int = 1) -> np.ndarray:
    """Rows ``[first_row, first_row + num_rows)`` of the global operand whose fixed
    ``block_rows``-row blocks are drawn U(-1, 1) from ``default_rng([seed, block])``: every
    world size sees the same global matrix.  float32.  ``threads`` > 1 draws the blocks
    concurrently (they are independent streams, so the values do not depend on it)."""
    out = np.empty((num_rows, K), dtype=np.float32)
    spans = []
    row = first_row
    while row < first_row + num_rows:
        block = row // block_rows
        lo = row - block * block_rows
        take = min(block_rows - lo, first_row + num_rows - row)
        spans.append((block, lo, take, row - first_row))
        row += take

    def fill(span):
        block, lo, take, dst = span
        vals = np.random.default_rng([seed, block]).uniform(-1.0, 1.0, size=(block_rows, K)).astype(np.float32)
        out[dst: dst + take] = vals[lo: lo + take]

    if threads > 1 and len(spans) > 1:
        from concurrent.futures import ThreadPoolExecutor

        with ThreadPoolExecutor(max_workers=min(threads, len(spans))) as pool:
            list(pool.map(fill, spans))
    else:
        for span in spans:
            fill(span)
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


def gpu_numa_node(device: int):
    """NUMA node of the host memory closest to CUDA device ``device`` (from the PCI device's
    ``numa_node`` entry in sysfs), or None when the platform does not say."""
    from . import _native as nat

    try:
        bus = nat.device_pci_bus_id(device).lower()
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        return node if node >= 0 else None
    except Exception:
        return None


def numa_node_cpus(node: int) -> set:
    """CPUs of a NUMA node, from ``/sys/devices/system/node/nodeN/cpulist`` ("0-15,32-47")."""
    with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
        return parse_cpulist(f.read())


def parse_cpulist(text: str) -> set:
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def bind_to_gpu_numa_node(device: int):
    """Pin the calling process to the CPUs of the NUMA node next to ``device`` so that the
    pinned host buffers it allocates afterwards (first touch) live in the memory that GPU's PCIe
    root is attached to.  With one rank per GPU this spreads the ranks' uploads over the host's
    memory controllers instead of funnelling them through one node.  Returns the node, or None
    when nothing was changed (single-node host, no sysfs entry, affinity not permitted)."""
    import os

    node = gpu_numa_node(device)
    if node is None:
        return None
    try:
        cpus = numa_node_cpus(node) & os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return node
    except Exception:
        return None


class ShardedHostGemmPipeline:
    """:class:`aster_b200.gemm.HostGemmPipeline` for one rank of an M-sharded job whose operands
    arrive from the host every step: the rank uploads its rows of A and only *its share* of the
    replicated B (rows ``[rank * N / world, (rank + 1) * N / world)``); an all-gather over
    NVLink (NCCL through ``torch.distributed``) then rebuilds B on every GPU, so B crosses each
    PCIe link once per ``world`` steps' worth of bytes instead of once per step.  Needs an
    initialised process group and ``N % world == 0``; every rank must submit in the same order.
    """

    def __init__(self, plan, rank: int, world: int, depth: int = 2, bias=None, scale_a=None, scale_b=None, group=None) -> None:
        import torch

        from . import _native as nat
        from .dtypes import STORAGE
        from .execution import GpuBuffer, GpuStream
        from .gemm import PinnedArray

        if plan.direct_b:
            raise ValueError("ShardedHostGemmPipeline takes row-major B")
        if plan.N % world != 0:
            raise ValueError(f"N={plan.N} does not split evenly over {world} ranks")
        self.plan, self.rank, self.world, self.depth, self.group = plan, rank, world, depth, group
        self._torch, self._nat = torch, nat
        res = plan.resources()
        eb_ab = np.dtype(STORAGE[plan.dtype_ab]).itemsize
        eb_c = np.dtype(STORAGE[plan.dtype_c]).itemsize
        self.b_rows = plan.N // world
        self.b_row_slice = slice(rank * self.b_rows, (rank + 1) * self.b_rows)
        self.a_bytes = plan.M * plan.K * eb_ab
        self.b_shard_bytes = self.b_rows * plan.K * eb_ab
        self.c_bytes = plan.M * plan.N * eb_c
        self._b_dtype = STORAGE[plan.dtype_ab]
        nat.init_current()
        self.streams = [GpuStream() for _ in range(depth)]
        self._tstreams = [torch.cuda.ExternalStream(s.handle.value) for s in self.streams]
        self.dA = [GpuBuffer(self.a_bytes) for _ in range(depth)]
        self.dC = [GpuBuffer(self.c_bytes) for _ in range(depth)]
        # B and its uploaded share are torch tensors (bytes) because the collective takes tensors.
        self.dB = [torch.empty(self.b_shard_bytes * world, dtype=torch.uint8, device="cuda") for _ in range(depth)]
        self.dB_shard = [torch.empty(self.b_shard_bytes, dtype=torch.uint8, device="cuda") for _ in range(depth)]
        ws_bytes = res.workspace_bytes or res.optional_workspace_bytes
        self.ws = [GpuBuffer(ws_bytes) if ws_bytes else None for _ in range(depth)]
        self.hC = [PinnedArray((plan.M, plan.N), STORAGE[plan.dtype_c]) for _ in range(depth)]
        self._small = []
        self.bias = self._upload_small(np.ascontiguousarray(bias, dtype=np.float32)) if bias is not None else None
        self.scale_a = self._upload_small(np.array([scale_a], np.float32)) if scale_a is not None else None
        self.scale_b = self._upload_small(np.array([scale_b], np.float32)) if scale_b is not None else None
        self._next = 0

    def _upload_small(self, arr):
        from .execution import GpuBuffer

        buf = GpuBuffer(arr.nbytes)
        buf.copy_from_host(arr)
        self._small.append(buf)
        return buf

    def pinned_operands(self):
        """Pinned host arrays for this rank's rows of A and its share of B's rows."""
        from .dtypes import STORAGE
        from .gemm import PinnedArray

        return (PinnedArray((self.plan.M, self.plan.K), STORAGE[self.plan.dtype_ab]),
                PinnedArray((self.b_rows, self.plan.K), self._b_dtype))

    @property
    def h2d_bytes_per_problem(self) -> int:
        return self.a_bytes + self.b_shard_bytes

    @property
    def d2h_bytes_per_problem(self) -> int:
        return self.c_bytes

    def submit(self, hA, hB_shard) -> int:
        import ctypes as C

        import torch.distributed as dist

        torch, nat = self._torch, self._nat
        slot = self._next
        self._next = (self._next + 1) % self.depth
        s = self.streams[slot]
        s.synchronize()  # the slot's previous problem must have left its buffers
        nat.call("b200_memcpy_h2d_async", self.dA[slot].ptr, hA.ptr, self.a_bytes, s.handle)
        nat.call("b200_memcpy_h2d_async", C.c_void_p(self.dB_shard[slot].data_ptr()), hB_shard.ptr, self.b_shard_bytes, s.handle)
        with torch.cuda.stream(self._tstreams[slot]):  # the collective is ordered after the uploads and before the GEMM
            dist.all_gather_into_tensor(self.dB[slot], self.dB_shard[slot], group=self.group)
        self.plan.run(self.dA[slot], self.dB[slot].data_ptr(), self.dC[slot], self.bias, self.scale_a, self.scale_b,
                      self.ws[slot], stream=s.handle)
        nat.call("b200_memcpy_d2h_async", self.hC[slot].ptr, self.dC[slot].ptr, self.c_bytes, s.handle)
        return slot

    def result(self, slot: int) -> np.ndarray:
        self.streams[slot].synchronize()
        return self.hC[slot].array

    def drain(self) -> None:
        for s in self.streams:
            s.synchronize()

    def close(self) -> None:
        self.drain()
        self._torch.cuda.synchronize()
        for group in (self.dA, self.dC, self.ws, self._small):
            for buf in group:
                if buf is not None:
                    buf.free()
        self.dB, self.dB_shard = [], []
        for h in self.hC:
            h.free()
        for s in self.streams:
            s.destroy()
