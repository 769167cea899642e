"""ctypes binding of the C ABI in ``include/aster_b200.h``.

Loads the in-tree ``libaster_b200.so`` (built by :mod:`aster_b200.build`); there is no
fallback implementation: if the library is missing, :func:`lib` raises.  Every wrapper checks
the returned status and raises ``RuntimeError`` carrying ``b200_last_error()``, which is how
the reference surfaces native failures (``std::runtime_error`` -> ``RuntimeError``,
python/lib/RuntimeModule.cpp:126-134).
"""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

LIB_NAME = "libaster_b200.so"
LIB_PATH = Path(__file__).resolve().parent / LIB_NAME

# Status codes (include/aster_b200.h).
OK, ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED, ERR_TIMEOUT, ERR_NO_DEVICE, ERR_WORKSPACE = range(7)
STATUS_NAMES = {
    OK: "B200_OK",
    ERR_INVALID: "B200_ERR_INVALID",
    ERR_CUDA: "B200_ERR_CUDA",
    ERR_UNSUPPORTED: "B200_ERR_UNSUPPORTED",
    ERR_TIMEOUT: "B200_ERR_TIMEOUT",
    ERR_NO_DEVICE: "B200_ERR_NO_DEVICE",
    ERR_WORKSPACE: "B200_ERR_WORKSPACE",
}

# Element types and enums.
F16, BF16, E4M3, F32, E5M2, I8, I32, E5M2_E4M3, E4M3_E5M2, MXE4M3, MXE5M2 = range(11)
B_ROW_MAJOR_NK, B_REF_PRESHUFFLED, B_PACKED = 0, 1, 2
EPI_NONE, EPI_BIAS_RELU, EPI_BIAS, EPI_RELU = 0, 1, 2, 3
BIAS_AXIS_N, BIAS_AXIS_M = 0, 1


class B200Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status
        self.message = message


class Props(C.Structure):
    _fields_ = [
        ("name", C.c_char * 128),
        ("cc_major", C.c_int32),
        ("cc_minor", C.c_int32),
        ("sm_count", C.c_int32),
        ("max_smem_per_block_optin", C.c_int32),
        ("smem_per_sm", C.c_int32),
        ("regs_per_sm", C.c_int32),
        ("l2_bytes", C.c_int32),
        ("sm_clock_khz", C.c_int32),
        ("mem_clock_khz", C.c_int32),
        ("mem_bus_bits", C.c_int32),
        ("total_mem_bytes", C.c_int64),
    ]


class GemmDesc(C.Structure):
    _fields_ = [
        ("M", C.c_int64),
        ("N", C.c_int64),
        ("K", C.c_int64),
        ("dtype_ab", C.c_int32),
        ("dtype_c", C.c_int32),
        ("b_layout", C.c_int32),
        ("epilogue", C.c_int32),
        ("bias_axis", C.c_int32),
        ("tile_m", C.c_int32),
        ("tile_n", C.c_int32),
        ("tile_k", C.c_int32),
        ("stages", C.c_int32),
        ("cta_group", C.c_int32),
        ("split_k", C.c_int32),
        ("max_ctas", C.c_int32),
        ("raster_group", C.c_int32),
        ("reserved", C.c_int32 * 3),
        ("label", C.c_char * 256),
    ]


class GemmResources(C.Structure):
    _fields_ = [
        ("tile_m", C.c_int32),
        ("tile_n", C.c_int32),
        ("tile_k", C.c_int32),
        ("stages", C.c_int32),
        ("cta_group", C.c_int32),
        ("split_k", C.c_int32),
        ("grid_ctas", C.c_int32),
        ("block_threads", C.c_int32),
        ("smem_bytes", C.c_int32),
        ("tmem_columns", C.c_int32),
        ("regs_per_thread", C.c_int32),
        ("ctas_per_sm", C.c_int32),
        ("num_tiles", C.c_int64),
        ("workspace_bytes", C.c_int64),
        ("packed_b_bytes", C.c_int64),
        ("optional_workspace_bytes", C.c_int64),
        ("tail_tiles", C.c_int32),
        ("tail_parts", C.c_int32),
        ("tail_exchange", C.c_int32),
        ("reserved0", C.c_int32),
    ]


_P = C.c_void_p
_SZ = C.c_size_t
_FP = C.POINTER(C.c_float)

# name -> argtypes; every function returns int status unless listed in _NON_STATUS.
SIGNATURES = {
    "b200_init": [C.c_int],
    "b200_device_count": [C.POINTER(C.c_int)],
    "b200_set_device": [C.c_int],
    "b200_get_device": [C.POINTER(C.c_int)],
    "b200_device_props": [C.c_int, C.POINTER(Props)],
    "b200_device_pci_bus_id": [C.c_int, C.c_char_p, C.c_int],
    "b200_clear_last_error": [],
    "b200_device_synchronize": [],
    "b200_device_reset": [],
    "b200_malloc": [C.POINTER(_P), _SZ],
    "b200_free": [_P],
    "b200_memcpy_h2d": [_P, _P, _SZ],
    "b200_memcpy_d2h": [_P, _P, _SZ],
    "b200_memcpy_d2d": [_P, _P, _SZ],
    "b200_memset": [_P, C.c_int, _SZ],
    "b200_host_alloc": [C.POINTER(_P), _SZ],
    "b200_host_free": [_P],
    "b200_memcpy_h2d_async": [_P, _P, _SZ, _P],
    "b200_memcpy_d2h_async": [_P, _P, _SZ, _P],
    "b200_event_create": [C.POINTER(_P)],
    "b200_event_destroy": [_P],
    "b200_event_record": [_P, _P],
    "b200_event_synchronize": [_P],
    "b200_event_elapsed_ms": [_P, _P, _FP],
    "b200_stream_create": [C.POINTER(_P)],
    "b200_stream_destroy": [_P],
    "b200_stream_synchronize": [_P],
    "b200_flush_l2": [_P],
    "b200_gemm_plan_create": [C.POINTER(GemmDesc), C.POINTER(_P)],
    "b200_gemm_plan_destroy": [_P],
    "b200_gemm_plan_resources": [_P, C.POINTER(GemmResources)],
    "b200_pack_b": [_P, _P, _P, _P],
    "b200_gemm_run": [_P, _P, _P, _P, _P, _P, _P, _P, _SZ, _P],
    "b200_gemm_time": [_P, _P, _P, _P, _P, _P, _P, _P, _SZ, C.c_int, C.c_int, _FP],
    "b200_gemm_time_batch": [_P, _P, _P, _P, _P, _P, _P, _P, _SZ, C.c_int, _FP],
    "b200_gemm_splitk_noalloc": [_P, _P, _P, C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.c_int32, _P],
    "b200_gemm_splitk_noalloc_status": [C.POINTER(C.c_uint32)],
    "b200_status_read": [_P, C.POINTER(C.c_uint32)],
    "b200_gemm_last_sm_mhz": [_P, _FP],
    "b200_gemm_clock_totals": [_P, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)],
    "b200_launch_count": [C.POINTER(C.c_int64)],
    "b200_vector_add_i32": [_P, _P, _P, _SZ, _P],
    "b200_vector_add_f32": [_P, _P, _P, _SZ, _P],
    "b200_copy_2d_padded_f32": [_P, _P, C.c_int64, C.c_int64, C.c_int, C.c_int, _P],
    "b200_add_relu_f32": [_P, _P, _P, _SZ, _P],
    "b200_mx_scales_bytes": [C.c_int64, C.c_int64, C.POINTER(_SZ)],
    "b200_pack_mx_scales": [_P, _P, C.c_int64, C.c_int64, _P],
    "b200_gemm_plan_set_mx_scales": [_P, _P, _P],
    "b200_nccl_version": [C.POINTER(C.c_int)],
    "b200_nccl_init_all": [C.c_int, C.POINTER(C.c_int), C.POINTER(_P)],
    "b200_nccl_destroy": [_P],
    "b200_nccl_group_start": [],
    "b200_nccl_group_end": [],
    "b200_allgather_rows": [_P, C.c_int, _P, _P, _SZ, _P],
    "b200_allgather_rows_all": [_P, C.POINTER(_P), C.POINTER(_P), _SZ, C.POINTER(_P)],
}
_NON_STATUS = {"b200_last_error": C.c_char_p, "b200_version": C.c_char_p}
# Present only in a bring-up build of the library (include/aster_b200_bringup.h).
BRINGUP_SIGNATURES = {"b200_gemm_debug_timeline": [_P, _P]}

_lib = None


def lib() -> C.CDLL:
    """The loaded native library.  Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is None:
        path = Path(os.environ.get("ASTER_B200_LIB", LIB_PATH))
        if not path.exists():
            raise RuntimeError(
                f"{path} is missing: build it with `python -m aster_b200.build` "
                "(the CUDA kernels have no CPU or library fallback)"
            )
        handle = C.CDLL(str(path))
        for name, argtypes in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = C.c_int
        for name, restype in _NON_STATUS.items():
            fn = getattr(handle, name)
            fn.argtypes = []
            fn.restype = restype
        for name, argtypes in BRINGUP_SIGNATURES.items():
            fn = getattr(handle, name, None)
            if fn is not None:
                fn.argtypes = argtypes
                fn.restype = C.c_int
        _lib = handle
    return _lib


def is_bringup_build() -> bool:
    """Was the loaded library built with -DB200_BRINGUP (work-skipping modes, per-CTA timeline)?"""
    return hasattr(lib(), "b200_gemm_debug_timeline")


def last_error() -> str:
    return lib().b200_last_error().decode(errors="replace")


def check(status: int) -> None:
    if status != OK:
        raise B200Error(status, last_error())


def call(name: str, *args) -> None:
    """Call a status-returning entry point and raise :class:`B200Error` on failure."""
    check(getattr(lib(), name)(*args))


def init_current() -> int:
    """Initialise the runtime on the device that is current for this thread (device 0 when
    none has been chosen yet) and return its index.  Host-buffer helpers call this instead of
    selecting a device themselves, so that a rank that picked its GPU keeps it."""
    d = C.c_int(0)
    if lib().b200_get_device(C.byref(d)) != OK:
        d.value = 0
    call("b200_init", d.value)
    return d.value


def launch_count() -> int:
    n = C.c_int64(0)
    call("b200_launch_count", C.byref(n))
    return n.value


def device_count() -> int:
    """Number of visible CUDA devices; 0 when there is no driver or GPU."""
    n = C.c_int(0)
    status = lib().b200_device_count(C.byref(n))
    return n.value if status == OK else 0


def device_props(device: int = 0) -> Props:
    p = Props()
    call("b200_device_props", device, C.byref(p))
    return p


def device_pci_bus_id(device: int = 0) -> str:
    buf = C.create_string_buffer(64)
    call("b200_device_pci_bus_id", device, buf, 64)
    return buf.value.decode()
