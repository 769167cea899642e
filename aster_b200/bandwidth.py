"""Bandwidth kernels of the hot path with host arrays in and out.

``vector_add`` (examples/03_vector_add/run.py:44-54), ``copy_2d_padded``
(examples/06_copy_layout/copy_2d_padded.py:101-151) and ``add_relu``
(examples/07_simple_fusion/simple_fusion.py:133-144) of the reference, each as one call that
uploads, launches the CUDA kernel through the C ABI and downloads.  ``*_device`` variants take
device buffers and only enqueue the launch.
"""

from __future__ import annotations

import ctypes as C

import numpy as np

from . import _native as nat
from .execution import GpuBuffer

SENTINEL = -999.0  # value the reference pre-fills dst with (copy_2d_padded.py:31,133)


def vector_add_device(a: GpuBuffer, b: GpuBuffer, c: GpuBuffer, n: int, dtype=np.int32, stream=None) -> None:
    fn = "b200_vector_add_i32" if np.dtype(dtype) == np.int32 else "b200_vector_add_f32"
    nat.call(fn, a.ptr, b.ptr, c.ptr, int(n), stream)


def add_relu_device(a: GpuBuffer, b: GpuBuffer, out: GpuBuffer, n: int, stream=None) -> None:
    nat.call("b200_add_relu_f32", a.ptr, b.ptr, out.ptr, int(n), stream)


def copy_2d_padded_device(src: GpuBuffer, dst: GpuBuffer, m: int, n: int, depth: int = 2, num_ctas: int = 0, stream=None) -> None:
    nat.call("b200_copy_2d_padded_f32", src.ptr, dst.ptr, int(m), int(n), int(depth), int(num_ctas), stream)


def _elementwise(fn_name: str, a: np.ndarray, b: np.ndarray, dtype) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=dtype)
    b = np.ascontiguousarray(b, dtype=dtype)
    if a.shape != b.shape:
        raise ValueError(f"shape mismatch: {a.shape} vs {b.shape}")
    out = np.empty_like(a)
    if a.size == 0:
        return out
    nat.init_current()
    da, db, dc = GpuBuffer(a.nbytes), GpuBuffer(a.nbytes), GpuBuffer(a.nbytes)
    try:
        da.copy_from_host(a)
        db.copy_from_host(b)
        nat.call(fn_name, da.ptr, db.ptr, dc.ptr, a.size, None)
        dc.copy_to_host(out)
    finally:
        for buf in (da, db, dc):
            buf.free()
    return out


def vector_add(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """``c = a + b`` for int32 (wrapping) or float32 arrays of equal shape."""
    dt = np.result_type(a, b)
    if dt == np.int32:
        return _elementwise("b200_vector_add_i32", a, b, np.int32)
    if dt == np.float32:
        return _elementwise("b200_vector_add_f32", a, b, np.float32)
    raise TypeError(f"vector_add supports int32 and float32, got {dt}")


def add_relu(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """``out = max(a + b, 0)`` in float32."""
    return _elementwise("b200_add_relu_f32", a, b, np.float32)


def copy_2d_padded(src: np.ndarray, dst: np.ndarray | None = None, *, depth: int = 2, num_ctas: int = 0) -> np.ndarray:
    """Copy a row-major float32 ``[M, N]`` matrix (``N % 4 == 0``) through the GPU.

    ``dst`` (default: a new array filled with the sentinel) is uploaded first, so whatever the
    kernel does not write is returned unchanged -- the reference checks exactly that.
    """
    src = np.ascontiguousarray(src, dtype=np.float32)
    if src.ndim != 2:
        raise ValueError("copy_2d_padded expects a 2-D array")
    m, n = src.shape
    if dst is None:
        dst = np.full_like(src, SENTINEL)
    if dst.shape != src.shape or dst.dtype != np.float32 or not dst.flags["C_CONTIGUOUS"]:
        raise ValueError("dst must be a C-contiguous float32 array of src's shape")
    if n % 4 != 0:
        raise ValueError(f"N={n} must be a multiple of 4 (a 16-byte access must not straddle a row)")
    if src.size == 0:
        return dst
    nat.init_current()
    ds, dd = GpuBuffer(src.nbytes), GpuBuffer(dst.nbytes)
    try:
        ds.copy_from_host(src)
        dd.copy_from_host(dst)
        nat.call("b200_copy_2d_padded_f32", ds.ptr, dd.ptr, m, n, depth, num_ctas, None)
        dd.copy_to_host(dst)
    finally:
        ds.free()
        dd.free()
    return dst
