"""Builds the in-tree native library ``aster_b200/libaster_b200.so`` with nvcc for sm_100a.

Run as ``python -m aster_b200.build [--force] [--verbose] [--bringup]``.  The library carries
every CUDA kernel and the C ABI declared in ``include/aster_b200.h``; nothing is JIT-compiled at
run time.  ``--bringup`` builds a second library, ``libaster_b200_bringup.so``, with
``-DB200_BRINGUP``: the work-skipping kernel modes and the per-CTA timeline of
``include/aster_b200_bringup.h``.  It is never loaded by default; point ``ASTER_B200_LIB`` at it.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libaster_b200.so"
BRINGUP_LIB_PATH = PKG_DIR / "libaster_b200_bringup.so"
SOURCES = ["runtime.cpp", "nccl_rows.cpp", "bandwidth.cu", "gemm_sm100.cu", "gemm_noalloc.cu"]
HEADERS = ["common.h", "ptx_sm100.cuh", "gemm_kernel.cuh", "../../include/aster_b200.h", "../../include/aster_b200_bringup.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
    "-cudart", "static",
    "--threads", "0",
]


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the native library cannot be built")
    return nvcc


def is_stale(lib_path: Path = LIB_PATH) -> bool:
    if not lib_path.exists():
        return True
    built = lib_path.stat().st_mtime
    deps = [CSRC / s for s in SOURCES] + [(CSRC / h).resolve() for h in HEADERS]
    return any(d.stat().st_mtime > built for d in deps)


def build(force: bool = False, verbose: bool = False, bringup: bool = False) -> Path:
    """Compile the library if it is missing or older than its sources; return its path."""
    lib_path = BRINGUP_LIB_PATH if bringup else LIB_PATH
    if not force and not is_stale(lib_path):
        return lib_path
    cmd = [find_nvcc(), *NVCC_FLAGS]
    if bringup:
        cmd += ["-DB200_BRINGUP"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [str(CSRC / s) for s in SOURCES] + ["-o", str(lib_path)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed with exit code {proc.returncode}")
    return lib_path


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, bringup="--bringup" in sys.argv)
    print(path)
