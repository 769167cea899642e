"""GEMM operator: plan objects over the C ABI and the host-buffer entry point.

``GemmPlan`` wraps ``b200_gemm_plan_*`` / ``b200_gemm_run``.  :func:`gemm` is the call a user
of the reference makes through ``execute_multitile_hsaco(cfg, artifact, iters, A, B)``
(contrib/kittens/test/test_102_gemm_python_multitile_lds_cdna3.py:417-436): host arrays in,
host array out, with the uploads and the download inside.
"""

from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import _native as nat
from .dtypes import STORAGE
from .execution import GpuBuffer

DTYPE_CODES = {"f16": nat.F16, "bf16": nat.BF16, "e4m3": nat.E4M3, "f32": nat.F32, "e5m2": nat.E5M2, "i8": nat.I8,
               "i32": nat.I32, "e5m2_e4m3": nat.E5M2_E4M3, "e4m3_e5m2": nat.E4M3_E5M2, "mxe4m3": nat.MXE4M3,
               "mxe5m2": nat.MXE5M2}
B_LAYOUT_CODES = {"row_major": nat.B_ROW_MAJOR_NK, "ref_preshuffled": nat.B_REF_PRESHUFFLED, "packed": nat.B_PACKED}
EPILOGUE_CODES = {"none": nat.EPI_NONE, "bias_relu": nat.EPI_BIAS_RELU, "bias": nat.EPI_BIAS, "relu": nat.EPI_RELU}
BIAS_AXIS_CODES = {"n": nat.BIAS_AXIS_N, "m": nat.BIAS_AXIS_M}


def _ptr(x) -> Optional[C.c_void_p]:
    if x is None:
        return None
    if isinstance(x, GpuBuffer):
        return x.ptr
    if isinstance(x, C.c_void_p):
        return x
    return C.c_void_p(int(x))


class GemmPlan:
    """A validated problem description bound to a kernel instance.

    Parameters mirror ``b200_gemm_desc``.  ``tile_n``, ``stages``, ``split_k`` = 0 let the
    library choose (``split_k=-1``: choose a K split for skinny problems).  ``static_b=True``
    declares that nothing enqueued before a launch in its stream writes B (a weight matrix):
    the kernel may then request its first B tiles while the previous kernel is still finishing.
    ``workspace_exchange=True`` makes a tail split meet in the lent workspace even where the
    parts of a tile could form a cluster and meet in its shared memory (same sums, same order).
    """

    def __init__(
        self,
        M: int,
        N: int,
        K: int,
        dtype_ab: str = "f16",
        dtype_c: str = "f32",
        *,
        b_layout: str = "row_major",
        epilogue: str = "none",
        bias_axis: str = "n",
        tile_m: int = 0,
        tile_n: int = 0,
        tile_k: int = 0,
        stages: int = 0,
        cta_group: int = 0,
        split_k: int = 0,
        max_ctas: int = 0,
        raster_group: int = 0,
        label: str = "",
        debug_mode: int = 0,
        no_tail_split: bool = False,
        wait_limit_ms: int = 0,
        static_b: bool = False,
        workspace_exchange: bool = False,
    ) -> None:
        self._handle = None
        desc = nat.GemmDesc()
        desc.M, desc.N, desc.K = int(M), int(N), int(K)
        try:
            desc.dtype_ab = DTYPE_CODES[dtype_ab]
            desc.dtype_c = DTYPE_CODES[dtype_c]
            desc.b_layout = B_LAYOUT_CODES[b_layout]
            desc.epilogue = EPILOGUE_CODES[epilogue]
            desc.bias_axis = BIAS_AXIS_CODES[bias_axis]
        except KeyError as e:
            raise ValueError(f"unknown enum value {e.args[0]!r}") from None
        desc.tile_m, desc.tile_n, desc.tile_k = tile_m, tile_n, tile_k
        desc.stages, desc.cta_group, desc.split_k = stages, cta_group, split_k
        desc.max_ctas, desc.raster_group = max_ctas, raster_group
        desc.reserved[0] = debug_mode  # 8 = wait-limit fault injection, 16 = no dependent launch (others: bring-up builds only)
        desc.reserved[1] = (1 if no_tail_split else 0) | (2 if static_b else 0) | (4 if workspace_exchange else 0)
        desc.reserved[2] = wait_limit_ms
        desc.label = label.encode()[:255]
        handle = C.c_void_p()
        nat.call("b200_gemm_plan_create", C.byref(desc), C.byref(handle))
        self._handle = handle.value
        self.M, self.N, self.K = int(M), int(N), int(K)
        self.dtype_ab, self.dtype_c = dtype_ab, dtype_c
        self.b_layout, self.epilogue, self.bias_axis = b_layout, epilogue, bias_axis
        self.label = label

    def __del__(self) -> None:
        try:
            self.destroy()
        except Exception:
            pass

    def destroy(self) -> None:
        if getattr(self, "_handle", None):
            h, self._handle = self._handle, None
            nat.call("b200_gemm_plan_destroy", C.c_void_p(h))

    @property
    def handle(self) -> C.c_void_p:
        if not self._handle:
            raise RuntimeError("plan was destroyed")
        return C.c_void_p(self._handle)

    @property
    def total_flops(self) -> int:
        return 2 * self.M * self.N * self.K

    def resources(self) -> nat.GemmResources:
        r = nat.GemmResources()
        nat.call("b200_gemm_plan_resources", self.handle, C.byref(r))
        return r

    @property
    def direct_b(self) -> bool:
        return self.b_layout != "row_major"

    def pack_b(self, b_in, b_packed, stream=None) -> None:
        nat.call("b200_pack_b", self.handle, _ptr(b_in), _ptr(b_packed), _ptr(stream))

    def set_mx_scales(self, scales_a_packed, scales_b_packed) -> None:
        """Attach the packed E8M0 scales of A and B (device addresses, see
        :func:`pack_mx_scales`) to a block-scaled plan; they must outlive its launches."""
        nat.call("b200_gemm_plan_set_mx_scales", self.handle, _ptr(scales_a_packed), _ptr(scales_b_packed))

    def run(self, A, B, Cbuf, bias=None, scale_a=None, scale_b=None, workspace=None, workspace_bytes=0, stream=None) -> None:
        """Enqueue one launch.  All pointers are device addresses (GpuBuffer, int or c_void_p)."""
        if isinstance(workspace, GpuBuffer) and not workspace_bytes:
            workspace_bytes = workspace.size_bytes
        nat.call(
            "b200_gemm_run", self.handle, _ptr(A), _ptr(B), _ptr(Cbuf), _ptr(bias), _ptr(scale_a), _ptr(scale_b),
            _ptr(workspace), workspace_bytes, _ptr(stream),
        )

    def bind(self, A, B, Cbuf, bias=None, scale_a=None, scale_b=None, workspace=None, workspace_bytes=0, stream=None):
        """A zero-argument callable that enqueues one launch with these arguments.  The ctypes
        argument objects are built once, which takes the host-side cost of a launch from about
        8 us (``run``) to about 3 us -- the difference shows on problems as small as 512^3,
        where the kernel itself is shorter than that."""
        if isinstance(workspace, GpuBuffer) and not workspace_bytes:
            workspace_bytes = workspace.size_bytes
        fn = nat.lib().b200_gemm_run
        args = (self.handle, _ptr(A), _ptr(B), _ptr(Cbuf), _ptr(bias), _ptr(scale_a), _ptr(scale_b), _ptr(workspace),
                C.c_size_t(workspace_bytes), _ptr(stream))
        keep = (A, B, Cbuf, bias, scale_a, scale_b, workspace)  # the buffers outlive the closure's launches
        check = nat.check

        def launch(_fn=fn, _args=args, _check=check, _keep=keep) -> None:
            _check(_fn(*_args))

        return launch

    def time(self, A, B, Cbuf, bias=None, scale_a=None, scale_b=None, workspace=None, workspace_bytes=0,
             iters: int = 100, flush_l2: bool = False) -> np.ndarray:
        """Per-launch event-timed loop run natively; returns milliseconds per iteration."""
        if isinstance(workspace, GpuBuffer) and not workspace_bytes:
            workspace_bytes = workspace.size_bytes
        out = (C.c_float * iters)()
        nat.call(
            "b200_gemm_time", self.handle, _ptr(A), _ptr(B), _ptr(Cbuf), _ptr(bias), _ptr(scale_a), _ptr(scale_b),
            _ptr(workspace), workspace_bytes, iters, int(flush_l2), out,
        )
        return np.frombuffer(out, dtype=np.float32).copy()

    def time_batch(self, A, B, Cbuf, bias=None, scale_a=None, scale_b=None, workspace=None, workspace_bytes=0,
                   iters: int = 100) -> float:
        """Milliseconds for ``iters`` back-to-back launches (one event pair)."""
        if isinstance(workspace, GpuBuffer) and not workspace_bytes:
            workspace_bytes = workspace.size_bytes
        ms = C.c_float(0.0)
        nat.call(
            "b200_gemm_time_batch", self.handle, _ptr(A), _ptr(B), _ptr(Cbuf), _ptr(bias), _ptr(scale_a), _ptr(scale_b),
            _ptr(workspace), workspace_bytes, iters, C.byref(ms),
        )
        return ms.value

    def last_sm_mhz(self) -> float:
        """SM clock (MHz) the last launch actually ran at (cycles / nanoseconds of CTA 0)."""
        mhz = C.c_float(0.0)
        nat.call("b200_gemm_last_sm_mhz", self.handle, C.byref(mhz))
        return mhz.value

    def clock_totals(self) -> tuple:
        """``(SM cycles, nanoseconds, launches)`` summed over all launches of the plan so far
        (CTA 0 of each launch).  Take it before and after a timed region and use
        :func:`mean_sm_mhz` on the two readings."""
        cyc, ns, n = C.c_uint64(0), C.c_uint64(0), C.c_uint64(0)
        nat.call("b200_gemm_clock_totals", self.handle, C.byref(cyc), C.byref(ns), C.byref(n))
        return cyc.value, ns.value, n.value

    def status(self) -> Sequence[int]:
        """Device status words of the last launch; raises ``B200Error`` (TIMEOUT) if a wait gave up."""
        words = (C.c_uint32 * 4)()
        nat.call("b200_status_read", self.handle, words)
        return list(words)


def mean_sm_mhz(before: tuple, after: tuple) -> float:
    """Average SM clock (MHz) of the launches between two :meth:`GemmPlan.clock_totals` readings."""
    cycles, ns = after[0] - before[0], after[1] - before[1]
    return cycles / ns * 1000.0 if ns > 0 else 0.0


def gemm_splitk_noalloc(A, B, Cbuf, M: int, N: int, K: int, dtype_ab: str = "bf16", dtype_c: str = "bf16",
                        split_k: int = 4, stream=None) -> None:
    """Enqueue a split-K GEMM whose partial sums live in the library's built-in 16 MiB scratch.

    For hosts that cannot allocate device memory when they need the GEMM (their own pool owns
    all of it, or they cannot afford the synchronisation an allocation implies).  ``A``, ``B``,
    ``Cbuf`` are device addresses.  ``split_k * M * N * 4`` must not exceed 16 MiB.  Calls on
    one device share the scratch: keep them ordered on one stream.  The first call per device
    performs a one-time host-side set-up and should be made before any stream capture starts.
    """
    nat.call("b200_gemm_splitk_noalloc", _ptr(A), _ptr(B), _ptr(Cbuf), int(M), int(N), int(K), DTYPE_CODES[dtype_ab],
             DTYPE_CODES[dtype_c], int(split_k), _ptr(stream))


def gemm_splitk_noalloc_status() -> Sequence[int]:
    """Status words of the :func:`gemm_splitk_noalloc` calls made so far on the current device
    (synchronises it; allocates nothing).  Raises ``B200Error`` (TIMEOUT) when a bounded
    device-side wait of the most recent call gave up -- that call left its C unwritten."""
    words = (C.c_uint32 * 4)()
    nat.call("b200_gemm_splitk_noalloc_status", words)
    return list(words)


def mx_scales_bytes(rows: int, K: int) -> int:
    """Bytes of the packed scale array for ``rows`` rows of ``K`` block-scaled elements."""
    n = C.c_size_t(0)
    nat.call("b200_mx_scales_bytes", int(rows), int(K), C.byref(n))
    return n.value


def pack_mx_scales(scales_in, scales_packed, rows: int, K: int, stream=None) -> None:
    """Device-side reorder of row-major scales ``[rows][K/32]`` into the kernel's streaming order."""
    nat.call("b200_pack_mx_scales", _ptr(scales_in), _ptr(scales_packed), int(rows), int(K), _ptr(stream))


def _check_operand(name: str, arr: np.ndarray, shape, dtype: str) -> np.ndarray:
    want = STORAGE[dtype]
    if not isinstance(arr, np.ndarray):
        raise TypeError(f"{name}: expected numpy array, got {type(arr)}")
    if arr.dtype != want:
        raise TypeError(f"{name}: dtype {arr.dtype} does not store {dtype} (expected {np.dtype(want)})")
    if int(np.prod(arr.shape)) != int(np.prod(shape)):
        raise ValueError(f"{name}: {arr.shape} does not hold {tuple(shape)}")
    return np.ascontiguousarray(arr)


def gemm(
    A: np.ndarray,
    B: np.ndarray,
    *,
    dtype_ab: str = "f16",
    dtype_c: str = "f32",
    bias: Optional[np.ndarray] = None,
    relu: bool = False,
    bias_axis: str = "n",
    scale_a: Optional[float] = None,
    scale_b: Optional[float] = None,
    shape: Optional[tuple] = None,
    plan: Optional[GemmPlan] = None,
    b_layout: str = "row_major",
    tail_split: bool = False,
    block_scales_a: Optional[np.ndarray] = None,
    block_scales_b: Optional[np.ndarray] = None,
    **plan_kw,
) -> np.ndarray:
    """``C = epilogue(A . B^T)`` on the GPU with host arrays in and a host array out.

    A is ``[M, K]``, B is ``[N, K]`` (both K-contiguous), stored as float16, as bf16 / e4m3 /
    e5m2 bit patterns (uint16 / uint8; see :mod:`aster_b200.dtypes`) or as int8.  ``B`` in a direct-B
    layout ("ref_preshuffled" or "packed" = row-major to be packed) is packed on the device
    first.  ``tail_split=True`` lends the plan its optional workspace so that a mostly idle
    last round of tiles is cut along K (changes the fp32 summation order of those tiles).
    For the block-scaled types ("mxe4m3", "mxe5m2") ``block_scales_a`` / ``block_scales_b`` are
    the E8M0 scale bytes ``[M, K/32]`` / ``[N, K/32]`` (see :func:`aster_b200.dtypes.quantize_mx`).
    Returns ``[M, N]`` float32, bf16 bit patterns (uint16) for ``dtype_c="bf16"``, or the int32
    sums for int8 inputs with ``dtype_c="i32"``.
    """
    if shape is None:
        M, K = A.shape
        N = B.shape[0]
    else:
        M, N, K = shape
    type_a, type_b = dtype_ab.split("_")[0], dtype_ab.split("_")[-1]  # "e5m2_e4m3": A e5m2, B e4m3
    A = _check_operand("A", A, (M, K), type_a)
    B = _check_operand("B", B, (N, K), type_b)
    if plan is None:
        epilogue = {(False, False): "none", (True, True): "bias_relu", (True, False): "bias", (False, True): "relu"}[
            (bias is not None, bool(relu))
        ]
        plan = GemmPlan(M, N, K, dtype_ab, dtype_c, b_layout=b_layout, epilogue=epilogue, bias_axis=bias_axis, **plan_kw)
    res = plan.resources()
    nat.init_current()
    bufs = []

    def dev(arr: np.ndarray) -> GpuBuffer:
        b = GpuBuffer(arr.nbytes)
        bufs.append(b)
        b.copy_from_host(arr)
        return b

    try:
        dA, dB = dev(A), dev(B)
        if plan.direct_b:
            packed = GpuBuffer(res.packed_b_bytes)
            bufs.append(packed)
            plan.pack_b(dB, packed)
            dB = packed
        if dtype_ab.startswith("mx"):
            if block_scales_a is None or block_scales_b is None:
                raise ValueError(f"{dtype_ab} needs block_scales_a and block_scales_b")
            packed_scales = []
            for name, sc, rows in (("block_scales_a", block_scales_a, M), ("block_scales_b", block_scales_b, N)):
                sc = _check_operand(name, sc, (rows, K // 32), "e4m3")  # stored as uint8, one per 32 elements
                out_buf = GpuBuffer(mx_scales_bytes(rows, K))
                bufs.append(out_buf)
                pack_mx_scales(dev(sc), out_buf, rows, K)
                packed_scales.append(out_buf)
            plan.set_mx_scales(*packed_scales)
        elif block_scales_a is not None or block_scales_b is not None:
            raise ValueError(f"block scales given for dtype_ab={dtype_ab!r}, which is not block-scaled")
        dbias = dev(np.ascontiguousarray(bias, dtype=np.float32)) if bias is not None else None
        dsa = dev(np.array([scale_a], dtype=np.float32)) if scale_a is not None else None
        dsb = dev(np.array([scale_b], dtype=np.float32)) if scale_b is not None else None
        out = np.empty((M, N), dtype=STORAGE[dtype_c])
        dC = GpuBuffer(out.nbytes)
        bufs.append(dC)
        ws = None
        ws_bytes = res.workspace_bytes or (res.optional_workspace_bytes if tail_split else 0)
        if ws_bytes:
            ws = GpuBuffer(ws_bytes)
            bufs.append(ws)
        plan.run(dA, dB, dC, dbias, dsa, dsb, ws)
        plan.status()
        dC.copy_to_host(out)
        return out
    finally:
        for b in bufs:
            b.free()


class PinnedArray:
    """A numpy array backed by page-locked host memory (``b200_host_alloc``)."""

    def __init__(self, shape, dtype) -> None:
        self._freed = True
        self.nbytes = int(np.prod(shape)) * np.dtype(dtype).itemsize
        p = C.c_void_p()
        nat.call("b200_host_alloc", C.byref(p), self.nbytes)
        self._ptr = p.value
        self._freed = False
        raw = (C.c_char * max(self.nbytes, 1)).from_address(self._ptr)
        self.array = np.frombuffer(raw, dtype=dtype, count=int(np.prod(shape))).reshape(shape)

    @property
    def ptr(self) -> C.c_void_p:
        return C.c_void_p(self._ptr)

    def free(self) -> None:
        if not getattr(self, "_freed", True):
            self._freed = True
            self.array = None
            nat.call("b200_host_free", C.c_void_p(self._ptr))

    def __del__(self) -> None:
        try:
            self.free()
        except Exception:
            pass


class HostGemmPipeline:
    """Back-to-back GEMMs on host buffers with transfers overlapped with compute.

    Each :meth:`submit` takes the host operands of one problem (pinned arrays from
    :meth:`pinned_operands`) and enqueues upload -> GEMM -> download on one of ``depth``
    streams, so the upload of problem i+1 and the download of problem i-1 overlap the GEMM of
    problem i.  :meth:`result` waits for a slot and returns its pinned C array.  This is the
    end-to-end path: every byte of A, B and C crosses PCIe for every problem.
    """

    def __init__(self, plan: GemmPlan, depth: int = 2, bias: Optional[np.ndarray] = None,
                 scale_a: Optional[float] = None, scale_b: Optional[float] = None) -> None:
        from .execution import GpuStream

        if plan.direct_b:
            raise ValueError("HostGemmPipeline takes row-major B")
        self.plan = plan
        self.depth = depth
        res = plan.resources()
        eb_ab = np.dtype(STORAGE[plan.dtype_ab]).itemsize
        eb_c = np.dtype(STORAGE[plan.dtype_c]).itemsize
        self.a_bytes, self.b_bytes = plan.M * plan.K * eb_ab, plan.N * plan.K * eb_ab
        self.c_bytes = plan.M * plan.N * eb_c
        nat.init_current()
        self.streams = [GpuStream() for _ in range(depth)]
        self.dA = [GpuBuffer(self.a_bytes) for _ in range(depth)]
        self.dB = [GpuBuffer(self.b_bytes) for _ in range(depth)]
        self.dC = [GpuBuffer(self.c_bytes) for _ in range(depth)]
        ws_bytes = res.workspace_bytes or res.optional_workspace_bytes
        self.ws = [GpuBuffer(ws_bytes) if ws_bytes else None for _ in range(depth)]
        self.hC = [PinnedArray((plan.M, plan.N), STORAGE[plan.dtype_c]) for _ in range(depth)]
        self._small = []
        self.bias = self._upload_small(np.ascontiguousarray(bias, dtype=np.float32)) if bias is not None else None
        self.scale_a = self._upload_small(np.array([scale_a], np.float32)) if scale_a is not None else None
        self.scale_b = self._upload_small(np.array([scale_b], np.float32)) if scale_b is not None else None
        self._next = 0

    def _upload_small(self, arr: np.ndarray) -> GpuBuffer:
        buf = GpuBuffer(arr.nbytes)
        buf.copy_from_host(arr)
        self._small.append(buf)
        return buf

    def pinned_operands(self):
        """Allocate pinned host arrays for one problem's A and B."""
        return (PinnedArray((self.plan.M, self.plan.K), STORAGE[self.plan.dtype_ab]),
                PinnedArray((self.plan.N, self.plan.K), STORAGE[self.plan.dtype_ab]))

    @property
    def h2d_bytes_per_problem(self) -> int:
        return self.a_bytes + self.b_bytes

    @property
    def d2h_bytes_per_problem(self) -> int:
        return self.c_bytes

    def submit(self, hA: PinnedArray, hB: PinnedArray) -> int:
        """Enqueue one problem; returns the slot to pass to :meth:`result`."""
        slot = self._next
        self._next = (self._next + 1) % self.depth
        s = self.streams[slot]
        s.synchronize()  # the slot's previous problem must have left its buffers
        nat.call("b200_memcpy_h2d_async", self.dA[slot].ptr, hA.ptr, self.a_bytes, s.handle)
        nat.call("b200_memcpy_h2d_async", self.dB[slot].ptr, hB.ptr, self.b_bytes, s.handle)
        self.plan.run(self.dA[slot], self.dB[slot], self.dC[slot], self.bias, self.scale_a, self.scale_b,
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
        for group in (self.dA, self.dB, self.dC, self.ws, self._small):
            for buf in group:
                if buf is not None:
                    buf.free()
        for h in self.hC:
            h.free()
        for s in self.streams:
            s.destroy()


def _current_device() -> int:
    d = C.c_int(0)
    nat.call("b200_get_device", C.byref(d))
    return d.value
