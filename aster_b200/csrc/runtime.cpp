// Runtime half of the aster_b200 C ABI: device, memory, event and stream calls.
//
// Stands in for the reference's nanobind module over a dlopen'd HIP runtime
// (python/lib/RuntimeModule.cpp:38-418).  Differences by design: status codes instead of
// exceptions, the CUDA runtime is linked statically (no dlopen table), and device reset is
// refused because the GPU is shared.
#include "common.h"

#include <cstring>
#include <mutex>

namespace b200 {

static thread_local char t_error[512] = {0};
std::atomic<int64_t> g_launches{0};

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
  return code;
}

void clear_error() { t_error[0] = 0; }

}  // namespace b200

using b200::as_stream;
using b200::fail;

extern "C" {

const char* b200_last_error(void) { return b200::t_error; }
const char* b200_version(void) { return "aster_b200 0.1 (sm_100a)"; }

int b200_init(int device) {
  // The reference initialises once and selects device 0 (RuntimeModule.cpp:143-150); here the
  // device is explicit and re-selecting it is harmless.
  static std::once_flag once;
  static cudaError_t init_err = cudaSuccess;
  std::call_once(once, [] { init_err = cudaFree(nullptr); });
  if (init_err != cudaSuccess) {
    return fail(B200_ERR_NO_DEVICE, "CUDA runtime not available - %s", cudaGetErrorString(init_err));
  }
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
    cudaGetLastError();
    return fail(B200_ERR_NO_DEVICE, "no CUDA device visible");
  }
  B200_REQUIRE(device >= 0 && device < n, "device %d out of range [0,%d)", device, n);
  B200_CUDA_OK(cudaSetDevice(device));
  return B200_OK;
}

int b200_device_count(int* count) {
  B200_REQUIRE(count != nullptr, "count is NULL");
  cudaError_t e = cudaGetDeviceCount(count);
  if (e != cudaSuccess) {
    *count = 0;
    cudaGetLastError();
    return fail(B200_ERR_NO_DEVICE, "cudaGetDeviceCount failed - %s", cudaGetErrorString(e));
  }
  return B200_OK;
}

int b200_set_device(int device) {
  B200_CUDA_OK(cudaSetDevice(device));
  return B200_OK;
}

int b200_get_device(int* device) {
  B200_REQUIRE(device != nullptr, "device is NULL");
  B200_CUDA_OK(cudaGetDevice(device));
  return B200_OK;
}

int b200_device_props(int device, b200_props* p) {
  B200_REQUIRE(p != nullptr, "props is NULL");
  cudaDeviceProp dp;
  B200_CUDA_OK(cudaGetDeviceProperties(&dp, device));
  std::memset(p, 0, sizeof(*p));
  std::strncpy(p->name, dp.name, sizeof(p->name) - 1);
  p->cc_major = dp.major;
  p->cc_minor = dp.minor;
  p->sm_count = dp.multiProcessorCount;
  p->max_smem_per_block_optin = static_cast<int32_t>(dp.sharedMemPerBlockOptin);
  p->smem_per_sm = static_cast<int32_t>(dp.sharedMemPerMultiprocessor);
  p->regs_per_sm = dp.regsPerMultiprocessor;
  p->l2_bytes = dp.l2CacheSize;
  int v = 0;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, device) == cudaSuccess) p->sm_clock_khz = v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMemoryClockRate, device) == cudaSuccess) p->mem_clock_khz = v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrGlobalMemoryBusWidth, device) == cudaSuccess) p->mem_bus_bits = v;
  cudaGetLastError();
  p->total_mem_bytes = static_cast<int64_t>(dp.totalGlobalMem);
  return B200_OK;
}

int b200_device_pci_bus_id(int device, char* buf, int len) {
  B200_REQUIRE(buf != nullptr && len >= 16, "device_pci_bus_id: buffer of at least 16 bytes needed");
  B200_CUDA_OK(cudaDeviceGetPCIBusId(buf, len, device));
  return B200_OK;
}

int b200_clear_last_error(void) {
  // Clears the runtime's sticky-free error slot and this thread's message, like
  // hip_clear_last_error before each execute (python/aster/execution/core.py:656-662).
  cudaGetLastError();
  b200::clear_error();
  return B200_OK;
}

int b200_device_synchronize(void) {
  B200_CUDA_OK(cudaDeviceSynchronize());
  return B200_OK;
}

int b200_device_reset(void) {
  return fail(B200_ERR_UNSUPPORTED, "device reset is refused: the GPU is shared with other jobs");
}

int b200_malloc(void** dptr, size_t bytes) {
  B200_REQUIRE(dptr != nullptr, "dptr is NULL");
  *dptr = nullptr;
  if (bytes == 0) bytes = 16;  // keep a distinct, freeable handle for empty arrays
  B200_CUDA_OK(cudaMalloc(dptr, bytes));
  return B200_OK;
}

int b200_free(void* dptr) {
  if (dptr == nullptr) return B200_OK;
  B200_CUDA_OK(cudaFree(dptr));
  return B200_OK;
}

int b200_memcpy_h2d(void* dst, const void* src, size_t bytes) {
  if (bytes == 0) return B200_OK;
  B200_REQUIRE(dst && src, "memcpy_h2d: NULL pointer");
  B200_CUDA_OK(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice));
  return B200_OK;
}

int b200_memcpy_d2h(void* dst, const void* src, size_t bytes) {
  if (bytes == 0) return B200_OK;
  B200_REQUIRE(dst && src, "memcpy_d2h: NULL pointer");
  B200_CUDA_OK(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost));
  return B200_OK;
}

int b200_memcpy_d2d(void* dst, const void* src, size_t bytes) {
  if (bytes == 0) return B200_OK;
  B200_REQUIRE(dst && src, "memcpy_d2d: NULL pointer");
  B200_CUDA_OK(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToDevice));
  return B200_OK;
}

int b200_memset(void* dst, int value, size_t bytes) {
  if (bytes == 0) return B200_OK;
  B200_REQUIRE(dst != nullptr, "memset: NULL pointer");
  B200_CUDA_OK(cudaMemset(dst, value, bytes));
  return B200_OK;
}

int b200_host_alloc(void** hptr, size_t bytes) {
  B200_REQUIRE(hptr != nullptr, "hptr is NULL");
  *hptr = nullptr;
  if (bytes == 0) bytes = 16;
  B200_CUDA_OK(cudaHostAlloc(hptr, bytes, cudaHostAllocDefault));
  return B200_OK;
}

int b200_host_free(void* hptr) {
  if (hptr == nullptr) return B200_OK;
  B200_CUDA_OK(cudaFreeHost(hptr));
  return B200_OK;
}

int b200_memcpy_h2d_async(void* dst, const void* src, size_t bytes, void* stream) {
  if (bytes == 0) return B200_OK;
  B200_REQUIRE(dst && src, "memcpy_h2d_async: NULL pointer");
  B200_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
  return B200_OK;
}

int b200_memcpy_d2h_async(void* dst, const void* src, size_t bytes, void* stream) {
  if (bytes == 0) return B200_OK;
  B200_REQUIRE(dst && src, "memcpy_d2h_async: NULL pointer");
  B200_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
  return B200_OK;
}

int b200_event_create(void** event) {
  B200_REQUIRE(event != nullptr, "event is NULL");
  cudaEvent_t e = nullptr;
  B200_CUDA_OK(cudaEventCreate(&e));
  *event = e;
  return B200_OK;
}

int b200_event_destroy(void* event) {
  if (event == nullptr) return B200_OK;
  B200_CUDA_OK(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
  return B200_OK;
}

int b200_event_record(void* event, void* stream) {
  B200_REQUIRE(event != nullptr, "event is NULL");
  B200_CUDA_OK(cudaEventRecord(static_cast<cudaEvent_t>(event), as_stream(stream)));
  return B200_OK;
}

int b200_event_synchronize(void* event) {
  B200_REQUIRE(event != nullptr, "event is NULL");
  B200_CUDA_OK(cudaEventSynchronize(static_cast<cudaEvent_t>(event)));
  return B200_OK;
}

int b200_event_elapsed_ms(void* start, void* stop, float* ms) {
  B200_REQUIRE(start && stop && ms, "event_elapsed_ms: NULL argument");
  B200_CUDA_OK(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop)));
  return B200_OK;
}

int b200_stream_create(void** stream) {
  B200_REQUIRE(stream != nullptr, "stream is NULL");
  cudaStream_t s = nullptr;
  B200_CUDA_OK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *stream = s;
  return B200_OK;
}

int b200_stream_destroy(void* stream) {
  if (stream == nullptr) return B200_OK;
  B200_CUDA_OK(cudaStreamDestroy(as_stream(stream)));
  return B200_OK;
}

int b200_stream_synchronize(void* stream) {
  B200_CUDA_OK(cudaStreamSynchronize(as_stream(stream)));
  return B200_OK;
}

int b200_launch_count(int64_t* count) {
  B200_REQUIRE(count != nullptr, "count is NULL");
  *count = b200::g_launches.load(std::memory_order_relaxed);
  return B200_OK;
}

}  // extern "C"
