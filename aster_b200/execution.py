"""Execution runtime: device buffers, events, streams and the event-timed launch loop.

Mirrors the reference's ``aster.execution.core`` (python/aster/execution/core.py:59-717) name
for name -- ``GpuBuffer``, ``GpuStream``, ``GpuEvent``, ``MemoryManager``, ``InputArray`` /
``OutputArray`` / ``InOutArray``, the ``_TimedLaunch`` protocol -- on top of the C ABI instead
of a nanobind HIP module.  :func:`execute_hsaco` keeps the reference's signature: the artifact
path and the kernel name select one of the library's kernels (there is no code object to load),
and the upload / timed-launch / download loop is :func:`execute_launch`, which times any
callable that enqueues work on the default stream.
"""

from __future__ import annotations

import ctypes as C
import dataclasses
from typing import Any, Callable, List, Optional, Tuple

import numpy as np

from . import _native as nat


def system_has_gpu(arch: str = "sm_100a") -> bool:
    """True when a device of the requested architecture family is visible.

    Stands in for the reference's ``rocminfo`` probe (python/aster/execution/utils.py:7-37).
    """
    try:
        if nat.device_count() < 1:
            return False
        props = nat.device_props(0)
    except (RuntimeError, OSError):
        return False
    want_major = 10 if arch.startswith("sm_100") else int(arch.split("_")[1][:-1] or 0)
    return props.cc_major == want_major


def hip_init(device: int = 0) -> None:  # name kept for drop-in callers of the reference API
    nat.call("b200_init", device)


init = hip_init


class GpuBuffer:
    """RAII device allocation (python/aster/execution/core.py:59-136)."""

    def __init__(self, size_bytes: int) -> None:
        self._freed = True  # guard against partial construction
        self._size_bytes = int(size_bytes)
        ptr = C.c_void_p()
        nat.call("b200_malloc", C.byref(ptr), self._size_bytes)
        if not ptr.value:
            raise RuntimeError(f"Failed to allocate GPU memory of size {size_bytes}")
        self._ptr_value = ptr.value
        self._freed = False

    def __del__(self) -> None:
        try:
            self.free()
        except Exception:
            pass

    def free(self) -> None:
        """Release the buffer; safe to call more than once."""
        if not getattr(self, "_freed", True):
            self._freed = True
            nat.call("b200_free", C.c_void_p(self._ptr_value))

    @property
    def ptr(self) -> C.c_void_p:
        return C.c_void_p(self._ptr_value)

    @property
    def ptr_value(self) -> int:
        return self._ptr_value

    @property
    def size_bytes(self) -> int:
        return self._size_bytes

    def copy_from_host(self, array: np.ndarray) -> None:
        if not isinstance(array, np.ndarray):
            raise TypeError(f"expected numpy array, got {type(array)}")
        if array.nbytes > self._size_bytes:
            raise ValueError(f"array ({array.nbytes} bytes) exceeds buffer ({self._size_bytes} bytes)")
        src = np.ascontiguousarray(array)
        nat.call("b200_memcpy_h2d", self.ptr, C.c_void_p(src.ctypes.data), src.nbytes)

    def copy_to_host(self, array: np.ndarray) -> None:
        if not isinstance(array, np.ndarray):
            raise TypeError(f"expected numpy array, got {type(array)}")
        if array.nbytes > self._size_bytes:
            raise ValueError(f"array ({array.nbytes} bytes) exceeds buffer ({self._size_bytes} bytes)")
        if not array.flags["C_CONTIGUOUS"]:
            raise ValueError("copy_to_host needs a C-contiguous destination")
        nat.call("b200_memcpy_d2h", C.c_void_p(array.ctypes.data), self.ptr, array.nbytes)

    def zero(self) -> None:
        nat.call("b200_memset", self.ptr, 0, self._size_bytes)


class GpuStream:
    """RAII stream (python/aster/execution/core.py:139-176)."""

    def __init__(self) -> None:
        self._destroyed = True
        h = C.c_void_p()
        nat.call("b200_stream_create", C.byref(h))
        self._handle = h.value
        self._destroyed = False

    def __del__(self) -> None:
        try:
            self.destroy()
        except Exception:
            pass

    def destroy(self) -> None:
        if not getattr(self, "_destroyed", True):
            self._destroyed = True
            nat.call("b200_stream_destroy", C.c_void_p(self._handle))

    def synchronize(self) -> None:
        nat.call("b200_stream_synchronize", C.c_void_p(self._handle))

    @property
    def handle(self) -> C.c_void_p:
        return C.c_void_p(self._handle)


class GpuEvent:
    """RAII event (python/aster/execution/core.py:179-232)."""

    def __init__(self) -> None:
        self._destroyed = True
        h = C.c_void_p()
        nat.call("b200_event_create", C.byref(h))
        self._handle = h.value
        self._destroyed = False

    def __del__(self) -> None:
        try:
            self.destroy()
        except Exception:
            pass

    def destroy(self) -> None:
        if not getattr(self, "_destroyed", True):
            self._destroyed = True
            nat.call("b200_event_destroy", C.c_void_p(self._handle))

    def record(self, stream: Optional[GpuStream] = None) -> None:
        nat.call("b200_event_record", C.c_void_p(self._handle), stream.handle if stream else None)

    def synchronize(self) -> None:
        nat.call("b200_event_synchronize", C.c_void_p(self._handle))

    def elapsed_ms(self, start: "GpuEvent") -> float:
        ms = C.c_float(0.0)
        nat.call("b200_event_elapsed_ms", C.c_void_p(start._handle), C.c_void_p(self._handle), C.byref(ms))
        return ms.value

    def elapsed_ns(self, start: "GpuEvent") -> int:
        return int(self.elapsed_ms(start) * 1_000_000)

    @property
    def handle(self) -> C.c_void_p:
        return C.c_void_p(self._handle)


@dataclasses.dataclass
class InputArray:
    """Read-only kernel input: copied host-to-device before the first launch only."""

    array: Any


@dataclasses.dataclass
class OutputArray:
    """Kernel output: allocated but not uploaded; copied back after the first iteration."""

    array: Any


@dataclasses.dataclass
class InOutArray:
    """Uploaded before the first launch and copied back after the first iteration."""

    array: Any


class MemoryManager:
    """Pairs numpy arrays with device buffers by object identity
    (python/aster/execution/core.py:384-464)."""

    def __init__(self) -> None:
        self._buffers: dict = {}

    def register(self, array: np.ndarray, upload: bool = True) -> GpuBuffer:
        if not isinstance(array, np.ndarray):
            raise TypeError(f"expected numpy array, got {type(array)}")
        key = id(array)
        if key in self._buffers:
            return self._buffers[key][0]
        buf = GpuBuffer(array.nbytes)
        if upload:
            buf.copy_from_host(array)
        self._buffers[key] = (buf, array)
        return buf

    def sync_to_gpu(self, array: np.ndarray) -> None:
        self._entry(array)[0].copy_from_host(array)

    def sync_from_gpu(self, array: np.ndarray) -> None:
        self._entry(array)[0].copy_to_host(array)

    def get_buffer(self, array: np.ndarray) -> GpuBuffer:
        return self._entry(array)[0]

    def release(self, array: np.ndarray) -> None:
        key = id(array)
        if key not in self._buffers:
            raise KeyError("array is not registered with this MemoryManager")
        self._buffers.pop(key)[0].free()

    def release_all(self) -> None:
        for buf, _ in self._buffers.values():
            buf.free()
        self._buffers.clear()

    def _entry(self, array: np.ndarray):
        key = id(array)
        if key not in self._buffers:
            raise KeyError("array is not registered with this MemoryManager")
        return self._buffers[key]


class FlushL2:
    """L2 eviction between timed launches; the reference's ``FlushLLC`` protocol
    (initialize / flush_llc / cleanup, python/aster/execution/flush_llc.py:25-204)."""

    def initialize(self) -> None:
        nat.call("b200_flush_l2", None)

    def flush_llc(self) -> None:
        nat.call("b200_flush_l2", None)

    def cleanup(self) -> None:
        pass


class _TimedLaunch:
    """Brackets a launch with events on the default stream and synchronises on exit
    (python/aster/execution/core.py:562-597)."""

    elapsed_ns: int

    def __init__(self, start_event: GpuEvent, stop_event: GpuEvent, flush_llc=None):
        self._start = start_event
        self._stop = stop_event
        self._flush_llc = flush_llc

    def __enter__(self):
        if self._flush_llc is not None:
            self._flush_llc.flush_llc()
        self._start.record()
        return self

    def __exit__(self, *_):
        self._stop.record()
        self._stop.synchronize()
        self.elapsed_ns = self._stop.elapsed_ns(self._start)


def execute_launch(
    launch_fn: Callable[..., None],
    arguments: list,
    num_iterations: int = 1,
    device_id: Optional[int] = None,
    flush_llc: Optional[Any] = None,
    verify_fn: Optional[Callable] = None,
    memory_manager: Optional[MemoryManager] = None,
) -> List[int]:
    """Upload, launch ``num_iterations`` times with per-launch event timing, download.

    The argument handling and the loop are the reference's ``execute_hsaco``
    (python/aster/execution/core.py:605-717): ``InputArray`` is uploaded, ``OutputArray`` is
    only allocated, raw ndarrays count as ``InOutArray``; outputs are copied back after
    iteration 0 and ``verify_fn(arguments)`` runs then.  ``launch_fn`` receives one positional
    argument per entry of ``arguments``: the :class:`GpuBuffer` for array wrappers, the value
    itself for scalars.  Returns the per-iteration times in nanoseconds.
    """
    if device_id is None:
        nat.init_current()  # keep the caller's device, as the reference does
    else:
        nat.call("b200_init", device_id)
    nat.call("b200_clear_last_error")
    arguments = [InOutArray(a) if isinstance(a, np.ndarray) else a for a in arguments]
    owns_mm = memory_manager is None
    mm = MemoryManager() if owns_mm else memory_manager
    times_ns: List[int] = []
    try:
        for arg in arguments:
            if isinstance(arg, (InputArray, InOutArray)):
                mm.register(arg.array, upload=True)
            elif isinstance(arg, OutputArray):
                mm.register(arg.array, upload=False)
        launch_args = [
            mm.get_buffer(a.array) if isinstance(a, (InputArray, OutputArray, InOutArray)) else a for a in arguments
        ]
        start_event, stop_event = GpuEvent(), GpuEvent()
        if flush_llc is not None:
            flush_llc.initialize()
        try:
            for it in range(num_iterations):
                with _TimedLaunch(start_event, stop_event, flush_llc) as t:
                    launch_fn(*launch_args)
                times_ns.append(t.elapsed_ns)
                if it == 0:
                    for arg in arguments:
                        if isinstance(arg, (OutputArray, InOutArray)):
                            mm.sync_from_gpu(arg.array)
                    if verify_fn is not None:
                        verify_fn(arguments)
        finally:
            if flush_llc is not None:
                flush_llc.cleanup()
    finally:
        if owns_mm:
            mm.release_all()
    return times_ns


# ---------------------------------------------------------------------------------------------
# execute_hsaco: the reference's entry point, kernel chosen by name
# ---------------------------------------------------------------------------------------------
def _host_array(arg) -> np.ndarray:
    if isinstance(arg, (InputArray, OutputArray, InOutArray)):
        return arg.array
    raise TypeError(f"expected an array argument, got {type(arg).__name__}")


def _elementwise_launcher(entry_i32: Optional[str], entry_f32: str):
    def build(_artifact: Optional[dict], arguments: list):
        arrays = [_host_array(a) for a in arguments[:3]]
        if len(arrays) != 3 or len({a.size for a in arrays}) != 1:
            raise ValueError("expected three arrays of equal size: two inputs and the output")
        dt = arrays[0].dtype
        if any(a.dtype != dt for a in arrays):
            raise TypeError("the three arrays must share one dtype")
        if dt == np.int32 and entry_i32 is not None:
            entry = entry_i32
        elif dt == np.float32:
            entry = entry_f32
        else:
            raise TypeError(f"unsupported element type {dt}")
        n = arrays[0].size

        def launch(a, b, c, *_scalars):
            nat.call(entry, a.ptr, b.ptr, c.ptr, n, None)

        return launch

    return build


def _copy_2d_padded_launcher(artifact: Optional[dict], arguments: list):
    src, dst = _host_array(arguments[0]), _host_array(arguments[1])
    if src.ndim != 2 or src.shape != dst.shape or src.dtype != np.float32 or dst.dtype != np.float32:
        raise ValueError("copy_2d_padded expects two float32 arrays of one 2-D shape")
    m, n = src.shape
    depth = int((artifact or {}).get("depth", 2))

    def launch(s, d, *_scalars):
        nat.call("b200_copy_2d_padded_f32", s.ptr, d.ptr, m, n, depth, 0, None)

    return launch


def _gemm_launcher(artifact: Optional[dict], arguments: list):
    from .gemm import GemmPlan

    if not artifact or "plan" not in artifact:
        raise RuntimeError("gemm_multitile needs the plan artifact that compile_multitile_gemm wrote as its hsaco_path")
    kw = dict(artifact["plan"])
    if kw.get("b_layout", "row_major") != "row_major":
        raise RuntimeError("execute_hsaco runs row-major B; direct-B configs go through execute_multitile_hsaco, which packs B first")
    plan = GemmPlan(**kw)
    res = plan.resources()
    ws_bytes = res.workspace_bytes or res.optional_workspace_bytes
    ws = GpuBuffer(ws_bytes) if ws_bytes else None

    def launch(a, b, c, *_scalars):
        plan.run(a, b, c, workspace=ws)

    def finish():
        try:
            plan.status()
        finally:
            if ws is not None:
                ws.free()
            plan.destroy()

    launch.finish = finish
    return launch


# kernel name -> builder(artifact dict or None, normalised arguments) -> launch callable.
# The names are the reference's: "kernel" is examples/03_vector_add (run.py:26), "copy_2d_padded"
# examples/06_copy_layout (copy_2d_padded.py:26), "fused" examples/07_simple_fusion
# (simple_fusion.py:27), "gemm_multitile" the GEMM generators (test_102_..._lds_cdna3.py:571-579).
HSACO_KERNELS = {
    "kernel": _elementwise_launcher("b200_vector_add_i32", "b200_vector_add_f32"),
    "vector_add": _elementwise_launcher("b200_vector_add_i32", "b200_vector_add_f32"),
    "fused": _elementwise_launcher(None, "b200_add_relu_f32"),
    "add_relu": _elementwise_launcher(None, "b200_add_relu_f32"),
    "copy_2d_padded": _copy_2d_padded_launcher,
    "gemm_multitile": _gemm_launcher,
}


def _read_artifact(path: Optional[str]) -> Optional[dict]:
    """The JSON artifact at ``path`` if there is one (the GEMM plan; optional parameters such as
    ``{"depth": 4}`` for the bandwidth kernels); any other file -- e.g. a real HSACO of the
    reference -- carries nothing this library can use and is ignored."""
    import json
    import os

    if not path or not os.path.isfile(path):
        return None
    try:
        with open(path) as f:
            art = json.load(f)
    except (OSError, UnicodeDecodeError, ValueError):
        return None
    return art if isinstance(art, dict) else None


def execute_hsaco(
    hsaco_path: Optional[str],
    kernel_name: str,
    arguments: list,
    grid_dim: Tuple[int, int, int] = (1, 1, 1),
    block_dim: Tuple[int, int, int] = (64, 1, 1),
    cluster_dim: Optional[Tuple[int, int, int]] = None,
    num_iterations: int = 1,
    device_id: Optional[int] = None,
    flush_llc: Optional[Any] = None,
    verify_fn: Optional[Callable] = None,
    memory_manager: Optional[MemoryManager] = None,
) -> List[int]:
    """The reference's execution entry point (python/aster/execution/core.py:605-717), same
    signature and return value: upload the arguments, launch ``kernel_name`` ``num_iterations``
    times with an event pair and a synchronise around each launch, copy outputs back after the
    first iteration, call ``verify_fn(arguments)``, return the times in nanoseconds.

    There is no code object to load here: ``kernel_name`` selects one of the library's kernels
    (:data:`HSACO_KERNELS`) and ``hsaco_path`` names its artifact -- the plan that
    ``compile_multitile_gemm`` wrote for ``"gemm_multitile"``, optional for the bandwidth
    kernels.  ``grid_dim``, ``block_dim`` and ``cluster_dim`` are accepted and ignored: every
    kernel sizes its own persistent grid.  Argument wrappers, raw arrays (in/out) and scalars
    are handled as in the reference; scalars are passed through to kernels that take none.
    """
    try:
        build = HSACO_KERNELS[kernel_name]
    except KeyError:
        raise RuntimeError(f"no kernel named {kernel_name!r} in this library (known: {sorted(HSACO_KERNELS)})") from None
    if device_id is None:
        nat.init_current()
    else:
        nat.call("b200_init", device_id)
    normalised = [InOutArray(a) if isinstance(a, np.ndarray) else a for a in arguments]
    launch = build(_read_artifact(hsaco_path), normalised)
    try:
        return execute_launch(launch, arguments, num_iterations=num_iterations, device_id=device_id, flush_llc=flush_llc,
                              verify_fn=verify_fn, memory_manager=memory_manager)
    finally:
        finish = getattr(launch, "finish", None)
        if finish is not None:
            finish()
