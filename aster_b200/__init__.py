"""B200-native GEMM hot path behind ASTER's operator surface.

The compute lives in ``libaster_b200.so`` (hand-written CUDA for sm_100a behind the C ABI of
``include/aster_b200.h``); this package is the ctypes binding plus the host-side mirror of the
reference's interfaces for the path: ``gemm_config`` (problem + mapping + label grammar),
``kittens_helpers`` (preshuffle, pipeline strategies), ``execution`` (buffers, events, the
timed launch loop) and ``bench_harness`` (input initialisation, statistics, hooks).
"""

__version__ = "0.1.0"
