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
//  * Every device-side wait is bounded.  If one gives up, the kernel records where in the
//    status words, the reduction that follows sees them and leaves C untouched (it does not sum
//    the previous call's partial sums), and b200_gemm_splitk_noalloc_status -- which allocates
//    nothing either -- reports B200_ERR_TIMEOUT for the calls made since the last clear.
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

// Kernel instance for a problem: skinny problems (M <= 64) stage only 32 or 64 rows of A, as the
// regular plan does, so that the ring holds more of B; `stages` is the ring depth that goes with it.
using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, const gemm::Params);
struct Variant {
  KernelFn fn;
  int am;      // rows of A per stage
  int stages;
};
constexpr int kMaxSmemOptin = 232448;  // 227 KB: the sm_100 per-block opt-in limit
constexpr int stages_short_a(int am) {  // as many short-A stages as fit, up to the ring's maximum
  const int fit = (kMaxSmemOptin - gemm::kBarrierBytes - 1024 - gemm::a_overrun_bytes(kTileN, 1, false, am)) / gemm::stage_bytes(kTileN, 1, false, am);
  return fit < gemm::kMaxStages ? fit : gemm::kMaxStages;
}
Variant variant_for(int64_t M, bool f32) {
  if (M <= 32) return {f32 ? gemm::gemm_tn_kernel<kTileN, float, 1, false, 32> : gemm::gemm_tn_kernel<kTileN, __nv_bfloat16, 1, false, 32>, 32, stages_short_a(32)};
  if (M <= 64) return {f32 ? gemm::gemm_tn_kernel<kTileN, float, 1, false, 64> : gemm::gemm_tn_kernel<kTileN, __nv_bfloat16, 1, false, 64>, 64, stages_short_a(64)};
  return {f32 ? gemm::gemm_tn_kernel<kTileN, float, 1> : gemm::gemm_tn_kernel<kTileN, __nv_bfloat16, 1>, gemm::kBM, kStages};
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
    for (int64_t m : {int64_t{32}, int64_t{64}, int64_t{128}}) {
      for (bool f32 : {false, true}) {
        const Variant v = variant_for(m, f32);
        // The per-block limit rather than this variant's footprint: the instance is shared with the
        // plans of b200_gemm_run, which set the same ceiling.
        B200_CUDA_OK(cudaFuncSetAttribute(reinterpret_cast<const void*>(v.fn), cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmemOptin));
      }
    }
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
  const Variant variant = variant_for(M, dtype_c == B200_F32);
  rc = b200::make_operand_map(&map_a, A, dtype_ab, static_cast<uint64_t>(M), static_cast<uint64_t>(K), static_cast<uint32_t>(variant.am));
  if (rc != B200_OK) return rc;
  rc = b200::make_operand_map(&map_b, B, dtype_ab, static_cast<uint64_t>(N), static_cast<uint64_t>(K), kTileN);
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
  p.stages = variant.stages;
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
  const int smem = gemm::smem_bytes(kTileN, variant.stages, 1, false, variant.am);
  variant.fn<<<grid, gemm::kThreads, smem, s>>>(map_a, map_b, no_scales, no_scales, p);
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

// Outcome of the calls made so far on the current device, read back without allocating.
extern "C" int b200_gemm_splitk_noalloc_status(uint32_t words[4]) {
  B200_REQUIRE(words != nullptr, "gemm_splitk_noalloc_status: words is NULL");
  words[0] = words[1] = words[2] = words[3] = 0;
  int dev = 0;
  B200_CUDA_OK(cudaGetDevice(&dev));
  B200_REQUIRE(dev >= 0 && dev < kMaxDevices, "gemm_splitk_noalloc_status: device index %d not supported", dev);
  uint32_t* status = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_setup_mu);
    if (!g_setup[dev].ready) return B200_OK;  // never called on this device
    status = g_setup[dev].status;
  }
  B200_CUDA_OK(cudaDeviceSynchronize());
  B200_CUDA_OK(cudaMemcpy(words, status, 4 * sizeof(uint32_t), cudaMemcpyDeviceToHost));
  if (words[0] != 0) {
    return b200::fail(B200_ERR_TIMEOUT, "gemm_splitk_noalloc: device wait timed out: code 0x%x cta %u tile %u k-block %u; C of that call was not written",
                      words[0], words[1], words[2], words[3]);
  }
  return B200_OK;
}
