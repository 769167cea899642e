// Split-K GEMM entry point that performs no device allocation.
//
// Who needs this: a host process that cannot call cudaMalloc when it wants a GEMM -- an
// inference server that has already handed every byte of HBM to its own memory pool, or a
// latency-critical loop that must not pay for the device-wide synchronisation cudaMalloc and
// cudaFree imply.  The regular path (b200_gemm_run with split_k > 1) needs the caller to
// bring an fp32 workspace for the partial sums; such callers have nowhere to get one from.
// Here the workspace is a fixed array that is part of the library image itself, so it exists
// on every GPU that loads the library, from load until the process exits, and costs
// kNoAllocScratchBytes of device memory there whether or not the entry point is ever called.
//
// What the caller must know:
//  * The array is shared by every call on a device and keeps the previous call's contents.
//    The kernels overwrite every partial sum before reading it, and the status words are
//    cleared on the stream at the start of each call, so stale contents are never consumed;
//    but two calls that overlap on the GPU (different streams, or the same stream from two
//    threads without ordering) race on the array and produce garbage.  Serialise them.
//  * The first call on each device looks up the array's device address and sets the kernel's
//    shared-memory attribute.  That set-up is host-side and happens once per device; make that
//    first call before starting any stream capture.
//  * Problems whose partial sums do not fit (split_k * M * N * 4 bytes > kNoAllocScratchBytes)
//    are rejected with B200_ERR_WORKSPACE.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstring>
#include <mutex>

#include "common.h"
#include "gemm_kernel.cuh"

namespace {

constexpr size_t kNoAllocScratchBytes = 16u << 20;  // 16 MiB of fp32 partial sums
constexpr int kMaxDevices = 64;
constexpr int kTileN = 64;
constexpr int kStages = 8;

// In host code these names are only handles for cudaGetSymbolAddress; they are not device
// addresses and must never be passed to a kernel directly.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
static __device__ __align__(256) uint32_t g_noalloc_status[64];

struct DeviceSetup {
  bool ready = false;
  float* scratch = nullptr;    // device address of g_noalloc_scratch on this device
  uint32_t* status = nullptr;  // device address of g_noalloc_status on this device
  int sm_count = 148;
};
DeviceSetup g_setup[kMaxDevices];
std::mutex g_setup_mu;

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encode_operand(CUtensorMap* map, const void* base, int dtype, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      return b200::fail(B200_ERR_CUDA, "gemm_splitk_noalloc: cuTensorMapEncodeTiled is not available from this driver");
    }
    fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  const uint32_t eb = dtype == B200_E4M3 ? 1u : 2u;
  const CUtensorMapDataType dt = dtype == B200_F16    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                 : dtype == B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                      : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * eb};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(gemm::kRowBytes / eb), box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return b200::fail(B200_ERR_CUDA, "gemm_splitk_noalloc: cuTensorMapEncodeTiled failed (%d)", (int)r);
  return B200_OK;
}

int setup_device(int dev, DeviceSetup** out) {
  std::lock_guard<std::mutex> lock(g_setup_mu);
  DeviceSetup& s = g_setup[dev];
  if (!s.ready) {
    int cc_major = 0;
    B200_CUDA_OK(cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    if (cc_major != 10) return b200::fail(B200_ERR_NO_DEVICE, "gemm_splitk_noalloc: device %d is not an sm_100 part", dev);
    // The symbol names are host-side stand-ins: ask the runtime for the device addresses.
    void* p = nullptr;
    B200_CUDA_OK(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    s.scratch = static_cast<float*>(p);
    B200_CUDA_OK(cudaGetSymbolAddress(&p, g_noalloc_status));
    s.status = static_cast<uint32_t*>(p);
    B200_CUDA_OK(cudaDeviceGetAttribute(&s.sm_count, cudaDevAttrMultiProcessorCount, dev));
    const int smem = gemm::smem_bytes(kTileN, kStages, 1);
    B200_CUDA_OK(cudaFuncSetAttribute(reinterpret_cast<const void*>(gemm::gemm_tn_kernel<kTileN, float, 1>),
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    B200_CUDA_OK(cudaFuncSetAttribute(reinterpret_cast<const void*>(gemm::gemm_tn_kernel<kTileN, __nv_bfloat16, 1>),
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    s.ready = true;
  }
  *out = &s;
  return B200_OK;
}

}  // namespace

extern "C" int b200_gemm_splitk_noalloc(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                                         int32_t dtype_ab, int32_t dtype_c, int32_t split_k, void* stream) {
  B200_REQUIRE(A && B && C, "gemm_splitk_noalloc: A, B and C must be non-NULL");
  B200_REQUIRE(((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15u) == 0,
               "gemm_splitk_noalloc: A, B and C must be 16-byte aligned");
  B200_REQUIRE(M >= 1 && N >= 1 && K >= 1 && M < (1ll << 31) - 256 && N < (1ll << 31) - 256 && K < (1ll << 31) - 256,
               "gemm_splitk_noalloc: M, N, K must be in [1, 2^31)");
  B200_REQUIRE(dtype_ab == B200_F16 || dtype_ab == B200_BF16 || dtype_ab == B200_E4M3,
               "gemm_splitk_noalloc: dtype_ab=%d is not f16, bf16 or e4m3", dtype_ab);
  B200_REQUIRE(dtype_c == B200_F32 || dtype_c == B200_BF16, "gemm_splitk_noalloc: dtype_c=%d is not f32 or bf16", dtype_c);
  B200_REQUIRE(split_k >= 1 && split_k <= 64, "gemm_splitk_noalloc: split_k=%d outside [1,64]", split_k);
  const int eb = dtype_ab == B200_E4M3 ? 1 : 2;
  B200_REQUIRE((K * eb) % 16 == 0, "gemm_splitk_noalloc: K=%lld gives a row pitch that is not a multiple of 16 bytes", (long long)K);
  const int kb_elems = gemm::kRowBytes / eb;
  const int k_blocks = static_cast<int>((K + kb_elems - 1) / kb_elems);
  int split = split_k > k_blocks ? k_blocks : split_k;
  const unsigned long long need = split > 1 ? static_cast<unsigned long long>(split) * M * N * 4ull : 0ull;
  if (need > kNoAllocScratchBytes) {
    return b200::fail(B200_ERR_WORKSPACE,
                      "gemm_splitk_noalloc: split_k * M * N * 4 = %llu bytes of partial sums exceed the built-in %zu-byte scratch; "
                      "use b200_gemm_run with a caller workspace for this size",
                      need, kNoAllocScratchBytes);
  }
  int dev = 0;
  B200_CUDA_OK(cudaGetDevice(&dev));
  B200_REQUIRE(dev >= 0 && dev < kMaxDevices, "gemm_splitk_noalloc: device index %d not supported", dev);
  DeviceSetup* setup = nullptr;
  int rc = setup_device(dev, &setup);
  if (rc != B200_OK) return rc;

  CUtensorMap map_a, map_b;
  const CUtensorMap no_scales = {};  // block scales are not part of this entry point
  rc = encode_operand(&map_a, A, dtype_ab, static_cast<uint64_t>(M), static_cast<uint64_t>(K), gemm::kBM);
  if (rc != B200_OK) return rc;
  rc = encode_operand(&map_b, B, dtype_ab, static_cast<uint64_t>(N), static_cast<uint64_t>(K), kTileN);
  if (rc != B200_OK) return rc;

  gemm::Params p;
  std::memset(&p, 0, sizeof(p));
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.K = static_cast<int>(K);
  p.m_blocks = static_cast<int>((M + gemm::kBM - 1) / gemm::kBM);
  p.n_blocks = static_cast<int>((N + kTileN - 1) / kTileN);
  p.num_tiles = p.m_blocks * p.n_blocks;
  p.num_kb = (k_blocks + split - 1) / split;
  p.kb_elems = kb_elems;
  p.split_k = split;
  p.stages = kStages;
  p.raster_group = 8;
  p.idesc = sm100::make_idesc(1u, dtype_ab == B200_BF16 ? 1u : 0u, dtype_ab == B200_BF16 ? 1u : 0u, gemm::kBM, kTileN);
  p.mma_kind = dtype_ab == B200_E4M3 ? sm100::kKindF8 : sm100::kKindF16;
  p.C = C;
  p.workspace = setup->scratch;  // the device address from cudaGetSymbolAddress, never the symbol itself
  p.status = setup->status;

  cudaStream_t s = b200::as_stream(stream);
  // The status words must start at zero for this launch; the partial sums need no clearing
  // (every element the reduction reads is written by this launch first).
  B200_CUDA_OK(cudaMemsetAsync(setup->status, 0, 8 * sizeof(uint32_t), s));
  const int items = p.num_tiles * split;
  const int grid = items < setup->sm_count ? items : setup->sm_count;
  const int smem = gemm::smem_bytes(kTileN, kStages, 1);
  if (dtype_c == B200_F32) {
    gemm::gemm_tn_kernel<kTileN, float, 1><<<grid, gemm::kThreads, smem, s>>>(map_a, map_b, no_scales, no_scales, p);
  } else {
    gemm::gemm_tn_kernel<kTileN, __nv_bfloat16, 1><<<grid, gemm::kThreads, smem, s>>>(map_a, map_b, no_scales, no_scales, p);
  }
  b200::count_launch();
  B200_CUDA_OK(cudaGetLastError());
  if (split > 1) {
    const size_t vecs = static_cast<size_t>(M) * N / 4 + 1;
    size_t blocks = (vecs + 255) / 256;
    const size_t cap = static_cast<size_t>(setup->sm_count) * 8;
    if (blocks > cap) blocks = cap;
    if (dtype_c == B200_F32) {
      gemm::splitk_reduce_kernel<float><<<static_cast<int>(blocks), 256, 0, s>>>(p);
    } else {
      gemm::splitk_reduce_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, s>>>(p);
    }
    b200::count_launch();
    B200_CUDA_OK(cudaGetLastError());
  }
  return B200_OK;
}
