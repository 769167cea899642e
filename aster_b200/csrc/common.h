// Shared host-side helpers for the aster_b200 C ABI: thread-local error text, CUDA status
// checks that turn failures into status codes (nothing throws across the ABI), and the
// process-wide launch counter.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/aster_b200.h"

namespace b200 {

// Store a printf-style message as the calling thread's last error and return `code`.
int fail(int code, const char* fmt, ...);
void clear_error();

// Count of kernel launches issued by this library in this process.
extern std::atomic<int64_t> g_launches;
inline void count_launch(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// TMA descriptor of a row-major [rows, cols] operand (element type B200_*), read in boxes of
// box_rows x 128 bytes with the 128-byte swizzle; out-of-range parts of a box read as zero.
// Defined in gemm_sm100.cu.
int make_operand_map(CUtensorMap* map, const void* base, int dtype, uint64_t rows, uint64_t cols, uint32_t box_rows);

}  // namespace b200

// Mirrors the reference's hipCheck text "HIP error at file:line - msg"
// (python/lib/RuntimeModule.cpp:126-134), but returns a status instead of throwing.
#define B200_CUDA_OK(expr)                                                                   \
  do {                                                                                       \
    cudaError_t _e = (expr);                                                                 \
    if (_e != cudaSuccess) {                                                                 \
      return b200::fail(B200_ERR_CUDA, "CUDA error at %s:%d - %s (%s)", __FILE__, __LINE__,  \
                        cudaGetErrorString(_e), #expr);                                      \
    }                                                                                        \
  } while (0)

#define B200_REQUIRE(cond, ...)                                  \
  do {                                                           \
    if (!(cond)) return b200::fail(B200_ERR_INVALID, __VA_ARGS__); \
  } while (0)
