// GEMM half of the aster_b200 C ABI: plan (kernel selection + validation), run, timing loops,
// B packing for the direct-B path, and the L2 flush.
//
// A "plan" plays the role of the reference's compiled artifact + loaded module
// (compile_multitile_gemm / GpuModule, test_102_gemm_python_multitile_lds_cdna3.py:391-414):
// everything that depends only on the problem description is decided once; pointers arrive
// with each run, exactly like the 3-pointer kernarg ABI of the reference kernel (:148-151).
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstring>
#include <mutex>
#include <new>

#include "common.h"
#include "gemm_kernel.cuh"

namespace {

using gemm::Params;

// ---------------------------------------------------------------------------------------------
// cuTensorMapEncodeTiled, resolved through the runtime so that the library has no link-time
// dependency on libcuda (it must load on machines without a driver).
// ---------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    cudaGetLastError();
  });
  return fn;
}

}  // namespace

// Row-major [rows, cols] matrix of `elt_bytes`-wide elements, tiled in boxes of
// box_rows x (128 bytes of columns), written to shared memory with the 128-byte swizzle.
// Out-of-range parts of a box read as zero, which is what makes ragged M, N and K safe.
int b200::make_operand_map(CUtensorMap* map, const void* base, int dtype, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return b200::fail(B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMapDataType dt;
  uint32_t eb;
  switch (dtype) {
    case B200_F16: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; eb = 2; break;
    case B200_BF16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; eb = 2; break;
    default: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; eb = 1; break;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * eb};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(gemm::kRowBytes / eb), box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    return b200::fail(B200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rows=%llu cols=%llu box_rows=%u)",
                      static_cast<int>(r), (unsigned long long)rows, (unsigned long long)cols, box_rows);
  }
  return B200_OK;
}

namespace {

using b200::make_operand_map;

// Packed block scales as a matrix of 32-bit words: one 512-byte row per [128 rows][4 K blocks]
// block, copied whole and unswizzled.
int make_scale_map(CUtensorMap* map, const void* base, uint64_t blocks) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return b200::fail(B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {gemm::kScaleBlockBytes / 4, blocks};
  cuuint64_t strides[1] = {gemm::kScaleBlockBytes};
  cuuint32_t box[2] = {gemm::kScaleBlockBytes / 4, 1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return b200::fail(B200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (%llu scale blocks)", static_cast<int>(r), (unsigned long long)blocks);
  return B200_OK;
}

using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, const Params);

template <int CG>
KernelFn select_kernel_cg(int bn, bool f32) {
  switch (bn) {
    case 32: return f32 ? gemm::gemm_tn_kernel<32, float, CG> : gemm::gemm_tn_kernel<32, __nv_bfloat16, CG>;
    case 64: return f32 ? gemm::gemm_tn_kernel<64, float, CG> : gemm::gemm_tn_kernel<64, __nv_bfloat16, CG>;
    case 128: return f32 ? gemm::gemm_tn_kernel<128, float, CG> : gemm::gemm_tn_kernel<128, __nv_bfloat16, CG>;
    case 256: return f32 ? gemm::gemm_tn_kernel<256, float, CG> : gemm::gemm_tn_kernel<256, __nv_bfloat16, CG>;
    default: return nullptr;
  }
}

// Short-A variants (skinny M): one CTA per tile, 64- or 128-column tiles.
template <int AM>
KernelFn select_kernel_short_a(int bn, bool f32) {
  if (bn == 64) return f32 ? gemm::gemm_tn_kernel<64, float, 1, false, AM> : gemm::gemm_tn_kernel<64, __nv_bfloat16, 1, false, AM>;
  if (bn == 128) return f32 ? gemm::gemm_tn_kernel<128, float, 1, false, AM> : gemm::gemm_tn_kernel<128, __nv_bfloat16, 1, false, AM>;
  return nullptr;
}

KernelFn select_kernel(int bn, int dtype_c, int cta_group, bool mx, int am) {
  const bool f32 = dtype_c == B200_F32 || dtype_c == B200_I32;  // 32-bit outputs share the store path
  if (am == 32) return select_kernel_short_a<32>(bn, f32);
  if (am == 64) return select_kernel_short_a<64>(bn, f32);
  if (mx) {
    if (cta_group == 2) {
      if (bn == 256) return f32 ? gemm::gemm_tn_kernel<256, float, 2, true> : gemm::gemm_tn_kernel<256, __nv_bfloat16, 2, true>;
      return f32 ? gemm::gemm_tn_kernel<128, float, 2, true> : gemm::gemm_tn_kernel<128, __nv_bfloat16, 2, true>;
    }
    if (bn == 256) return f32 ? gemm::gemm_tn_kernel<256, float, 1, true> : gemm::gemm_tn_kernel<256, __nv_bfloat16, 1, true>;
    return f32 ? gemm::gemm_tn_kernel<128, float, 1, true> : gemm::gemm_tn_kernel<128, __nv_bfloat16, 1, true>;
  }
  return cta_group == 2 ? select_kernel_cg<2>(bn, f32) : select_kernel_cg<1>(bn, f32);
}

int elt_bytes(int dtype) {
  switch (dtype) {
    case B200_F16:
    case B200_BF16: return 2;
    case B200_E4M3:
    case B200_E5M2:
    case B200_E5M2_E4M3:
    case B200_E4M3_E5M2:
    case B200_MXE4M3:
    case B200_MXE5M2:
    case B200_I8: return 1;
    case B200_F32:
    case B200_I32: return 4;
    default: return 0;
  }
}

int ceil_div(int64_t a, int64_t b) { return static_cast<int>((a + b - 1) / b); }

bool is_mx(int dtype) { return dtype == B200_MXE4M3 || dtype == B200_MXE5M2; }

bool is_f8(int dtype) { return dtype == B200_E4M3 || dtype == B200_E5M2 || dtype == B200_E5M2_E4M3 || dtype == B200_E4M3_E5M2; }

// tcgen05 instruction descriptor for the plan's operand types and MMA shape.
uint32_t idesc_for(int dtype_ab, uint32_t umma_m, uint32_t umma_n) {
  if (is_mx(dtype_ab)) {
    const uint32_t fmt = dtype_ab == B200_MXE5M2 ? 1u : 0u;
    return sm100::make_idesc_mx(fmt, fmt, umma_m, umma_n);
  }
  uint32_t d_fmt = 1u, a_fmt = 0u, b_fmt = 0u;  // f32 accumulators, f16 / e4m3 inputs
  switch (dtype_ab) {
    case B200_BF16: a_fmt = b_fmt = 1u; break;
    case B200_E5M2: a_fmt = b_fmt = 1u; break;
    case B200_E5M2_E4M3: a_fmt = 1u; break;
    case B200_E4M3_E5M2: b_fmt = 1u; break;
    case B200_I8: d_fmt = 2u; a_fmt = b_fmt = 1u; break;  // signed 8-bit, s32 accumulators
    default: break;
  }
  return sm100::make_idesc(d_fmt, a_fmt, b_fmt, umma_m, umma_n);
}

int mma_kind_for(int dtype_ab) { return dtype_ab == B200_I8 ? sm100::kKindI8 : (is_f8(dtype_ab) ? sm100::kKindF8 : sm100::kKindF16); }

constexpr int kMaxSmemOptin = 232448;  // 227 KB: the sm_100 per-block opt-in limit
constexpr int kDefaultSms = 148;

// Packs B into the shared-memory image of each (n block, k block) tile: BN rows of 128 bytes,
// 16-byte chunk c of row r stored at chunk position c ^ (r % 8) (the 128-byte swizzle), tiles
// laid out n-block-major.  Rows >= N and K positions >= K are zero.  One thread per 16-byte chunk.
// `preshuffled`: the input is shuffle_weight(B) (kittens_helpers.py:90-119), whose flat index
// for logical (n, k) is ((((n/16 * K/32 + k/32) * 4 + (k%16)/4) * 16 + n%16) * 2 + (k%32)/16) * 4 + k%4.
__global__ void __launch_bounds__(256) pack_b_kernel(const uint8_t* __restrict__ b_in, uint8_t* __restrict__ b_out,
                                                     long long N, long long K, int eb, int bn, long long n_blocks,
                                                     long long k_blocks, int preshuffled) {
  const long long chunks_per_tile = static_cast<long long>(bn) * 8;
  const long long total = n_blocks * k_blocks * chunks_per_tile;
  const int elems_per_chunk = 16 / eb;
  const int kb_elems = gemm::kRowBytes / eb;
  for (long long g = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; g < total;
       g += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long tile = g / chunks_per_tile;
    const int in_tile = static_cast<int>(g - tile * chunks_per_tile);
    const int r = in_tile >> 3;
    const int c = in_tile & 7;
    const long long nb = tile / k_blocks;
    const long long kb = tile - nb * k_blocks;
    const long long n = nb * bn + r;
    const long long k0 = kb * kb_elems + static_cast<long long>(c) * elems_per_chunk;
    alignas(16) uint8_t chunk[16];
    for (int e = 0; e < elems_per_chunk; ++e) {
      const long long k = k0 + e;
      for (int byte = 0; byte < eb; ++byte) {
        uint8_t val = 0;
        if (n < N && k < K) {
          long long src;
          if (preshuffled) {
            const long long kbl = K / 32;
            const long long kl = k % 32;
            src = ((((n / 16 * kbl + k / 32) * 4 + (kl % 16) / 4) * 16 + n % 16) * 2 + kl / 16) * 4 + kl % 4;
          } else {
            src = n * K + k;
          }
          val = b_in[src * eb + byte];
        }
        chunk[e * eb + byte] = val;
      }
    }
    uint8_t* dst = b_out + tile * (chunks_per_tile * 16) + static_cast<long long>(r) * 128 + ((c ^ (r & 7)) << 4);
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(chunk);
  }
}

// Row-major E8M0 scales [rows][K/32] -> blocks of [128 rows][4 K blocks] in the order the
// block-scaled kernel streams them ([row block][K stage], row r of a block at byte
// (r % 32) * 16 + (r / 32) * 4).  Positions beyond rows or K/32 get 127 (= 2^0): the operand
// bytes they would scale are zero-filled by the loads.
__global__ void __launch_bounds__(256) pack_mx_scales_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, long long rows,
                                                             long long k_blocks32, long long row_blocks, long long k_stages) {
  const long long total = row_blocks * k_stages * gemm::kScaleBlockBytes;
  for (long long g = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; g < total;
       g += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long blk = g / gemm::kScaleBlockBytes;
    const int in_blk = static_cast<int>(g - blk * gemm::kScaleBlockBytes);
    const long long rb = blk / k_stages;
    const long long ks = blk - rb * k_stages;
    const int r = (in_blk >> 4) + 32 * ((in_blk & 15) >> 2);
    const long long row = rb * 128 + r;
    const long long kb = ks * 4 + (in_blk & 3);
    out[g] = (row < rows && kb < k_blocks32) ? in[row * k_blocks32 + kb] : static_cast<uint8_t>(127);
  }
}

// Streams a buffer larger than the L2 so that the next kernel starts from a cold cache.
struct FlushState {
  void* buf = nullptr;
  size_t bytes = 0;
  int device = -1;
};
FlushState g_flush;
std::mutex g_flush_mu;

}  // namespace

struct b200_gemm_plan {
  b200_gemm_desc desc;
  int bn = 0;
  int cg = 1;         // CTAs per MMA: 1, or 2 for a CTA pair (cluster of two)
  int am = gemm::kBM; // rows of A per stage: 128, or 32 / 64 for skinny M (see gemm::stage_bytes)
  bool mx = false;    // block-scaled 8-bit floats: scales come from b200_gemm_plan_set_mx_scales
  const void* sfa = nullptr;
  const void* sfb = nullptr;
  CUtensorMap map_sfa = {}, map_sfb = {};  // all zero (never dereferenced) unless mx
#ifdef B200_BRINGUP
  unsigned long long* timeline = nullptr;  // see b200_gemm_debug_timeline
#endif
  int stages = 0;
  int split_k = 1;
  int grid = 0;
  int sm_count = kDefaultSms;
  int smem = 0;
  int eb_ab = 2;
  int kb_elems = 64;
  int total_kb = 0;   // K blocks over the whole K (padded to a multiple of split_k)
  int num_kb = 0;     // per split
  int m_blocks = 0, n_blocks = 0;
  int raster_group = 8;
  // Tail split (see gemm::Params): decided from the tile count and the persistent grid.
  int units_cap = kDefaultSms;  // CTAs (pairs) the persistent grid may use
  int tail_tiles = 0, tail_parts = 0, tail_kb0 = 0, tail_kb = 0;
  int64_t tail_ws_bytes = 0;   // flags + partial tiles; 0 = tail split not useful for this plan
  int64_t tail_flag_bytes = 0;
  // The parts of every tile are the CTAs of one cluster and exchange their partial sums through
  // its shared memory (see gemm::Params::cluster_exchange); needs no workspace.
  bool cluster_exchange = false;
  bool cluster_exchange_ok = true;  // cleared when the device cannot co-schedule the clusters
  // Workspaces whose flag area has been zeroed (a pipeline alternates between a few).
  static constexpr int kSeenSlots = 4;
  const void* tail_ws_seen[kSeenSlots] = {};
  int tail_ws_next = 0;
  KernelFn kernel = nullptr;
  bool attr_set = false;
  int attr_device = -1;
  uint32_t* status = nullptr;  // device, 8 words, allocated on first run
  int status_device = -1;
  // Tensor maps are a pure function of (pointer, shape): the last few of each operand are kept, so
  // that a caller rotating over a few buffers (a host pipeline's slots, operand sets) does not
  // re-encode on every launch.
  static constexpr int kMapSlots = 4;
  const void* map_a_ptr[kMapSlots] = {};
  const void* map_b_ptr[kMapSlots] = {};
  CUtensorMap map_a[kMapSlots], map_b[kMapSlots];
  int map_a_next = 0, map_b_next = 0;
};

namespace {

bool direct_b(const b200_gemm_plan* p) { return p->desc.b_layout != B200_B_ROW_MAJOR_NK; }

int64_t packed_b_bytes(const b200_gemm_plan* p) {
  if (!direct_b(p)) return 0;
  return static_cast<int64_t>(p->n_blocks) * p->total_kb * p->bn * gemm::kRowBytes;
}

// Decide whether the last, partly filled round of tiles should be cut along K.  `units` =
// CTAs (pairs) in the persistent grid.  Worth it when the last round would keep at most half
// of the units busy and each K range still has a few K blocks.
void plan_tail_split(b200_gemm_plan* plan) {
  plan->tail_tiles = plan->tail_parts = plan->tail_kb0 = plan->tail_kb = 0;
  plan->tail_ws_bytes = plan->tail_flag_bytes = 0;
  plan->cluster_exchange = false;
  if (plan->split_k > 1 || (plan->desc.reserved[1] & 1) != 0) return;  // reserved[1] bit 0: caller opted out
  if (plan->desc.dtype_ab == B200_I8) return;  // partial tiles are exchanged as fp32; s32 sums stay whole
  const int units = plan->units_cap;
  const int tiles = plan->m_blocks * plan->n_blocks;
  if (units < 2 || tiles < 1) return;
  const int tail = tiles % units;  // tiles < units: every tile is a tail tile
  if (tail == 0) return;
  // Parts: a power of two (each part finishes BN / parts columns, a multiple of 32) that the idle
  // units can host, with no empty part and enough K blocks each to pay for the exchange: it costs
  // 3-5 us (export, fence, flag, read back), a K block of a full-width tile about 0.36 us, so a
  // split that saves fewer than ~12 K blocks per unit makes the launch longer (512^3: 8 K blocks,
  // 9.3 -> 6 us per launch without the split).
  constexpr int kMinKbPerPart = 12;
  int parts = 0;
  for (int cand = 8; cand >= 2; cand /= 2) {
    if (cand > units / tail || plan->bn / cand < 32 || plan->num_kb / cand < kMinKbPerPart) continue;
    const int per = (plan->num_kb + cand - 1) / cand;
    if ((plan->num_kb + per - 1) / per != cand) continue;
    parts = cand;
    break;
  }
  if (parts < 2) return;
  const int tail_kb = (plan->num_kb + parts - 1) / parts;
  plan->tail_tiles = tail;
  plan->tail_parts = parts;
  plan->tail_kb0 = tail_kb;
  plan->tail_kb = tail_kb;
  // One round, one part per CTA (skinny problems: a few column tiles, a long K): the parts of a
  // tile form a cluster and exchange through its shared memory.  The parking area (a 128 x BN
  // fp32 tile) must fit in the stage ring.  reserved[1] bit 2 keeps the exchange in the workspace.
  if (plan->cg == 1 && !plan->mx && plan->cluster_exchange_ok && (plan->desc.reserved[1] & 4) == 0 && tail == tiles &&
      tiles * parts <= units &&
      static_cast<int64_t>(plan->stages) * gemm::stage_bytes(plan->bn, 1, false, plan->am) >= static_cast<int64_t>(gemm::kBM) * plan->bn * 4) {
    plan->cluster_exchange = true;
    return;  // no flags, no partial tiles in global memory
  }
  const int64_t flags = static_cast<int64_t>(tail) * parts * plan->cg * gemm::kEpilogueWarps * sizeof(uint32_t);
  plan->tail_flag_bytes = (flags + 255) / 256 * 256;
  plan->tail_ws_bytes = plan->tail_flag_bytes + static_cast<int64_t>(tail) * parts * (gemm::kBM * plan->cg) * plan->bn * sizeof(float);
}

// Persistent grid: one CTA (pair) per work item up to `units_cap`.
void size_grid(b200_gemm_plan* plan, int units_cap) {
  plan->units_cap = units_cap < 1 ? 1 : units_cap;
  plan_tail_split(plan);
  const int64_t tiles = static_cast<int64_t>(plan->m_blocks) * plan->n_blocks;
  int64_t items = plan->split_k > 1 ? tiles * plan->split_k : tiles;
  if (plan->tail_parts > 1) items = tiles - plan->tail_tiles + static_cast<int64_t>(plan->tail_tiles) * plan->tail_parts;
  const int64_t units = items < plan->units_cap ? items : plan->units_cap;
  plan->grid = static_cast<int>(units) * plan->cg;
}

int64_t workspace_bytes(const b200_gemm_plan* p) {
  if (p->split_k <= 1) return 0;
  return static_cast<int64_t>(p->split_k) * p->desc.M * p->desc.N * 4;
}

int ensure_device_state(b200_gemm_plan* plan, cudaStream_t stream) {
  int dev = 0;
  B200_CUDA_OK(cudaGetDevice(&dev));
  if (!plan->attr_set || plan->attr_device != dev) {
    int cc_major = 0;
    B200_CUDA_OK(cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    if (cc_major != 10) {
      return b200::fail(B200_ERR_NO_DEVICE, "device %d has compute capability %d.x; the GEMM kernels need sm_100", dev, cc_major);
    }
    // The limit, not this plan's own footprint: kernel instances are shared by all plans (and by
    // b200_gemm_splitk_noalloc), and a later plan with a shallower ring must not lower the
    // ceiling under an earlier one with a deeper ring.
    B200_CUDA_OK(cudaFuncSetAttribute(reinterpret_cast<const void*>(plan->kernel),
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmemOptin));
    int sms = kDefaultSms;
    B200_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    plan->sm_count = sms;
    int cap = plan->desc.max_ctas > 0 ? plan->desc.max_ctas : sms;
    int units_cap = cap;
    if (plan->cg == 2) {
      // Persistent pairs: as many clusters of two as can be resident at once.
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(static_cast<unsigned>(sms - sms % 2));
      cfg.blockDim = dim3(gemm::kThreads);
      cfg.dynamicSmemBytes = static_cast<size_t>(plan->smem);
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 2;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, reinterpret_cast<const void*>(plan->kernel), &cfg) != cudaSuccess || clusters < 1) {
        cudaGetLastError();
        clusters = sms / 2;
      }
      units_cap = cap / 2 < 1 ? 1 : cap / 2;
      if (units_cap > clusters) units_cap = clusters;
    }
    size_grid(plan, units_cap);
    if (plan->cluster_exchange) {
      // All clusters of the launch must be resident at once (each CTA waits for its peers).
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(static_cast<unsigned>(plan->grid));
      cfg.blockDim = dim3(gemm::kThreads);
      cfg.dynamicSmemBytes = static_cast<size_t>(plan->smem);
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = static_cast<unsigned>(plan->tail_parts);
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, reinterpret_cast<const void*>(plan->kernel), &cfg) != cudaSuccess ||
          clusters * plan->tail_parts < plan->grid) {
        cudaGetLastError();
        plan->cluster_exchange_ok = false;  // exchange through the workspace instead, when the caller lends one
        size_grid(plan, units_cap);
      }
    }
    for (auto& seen : plan->tail_ws_seen) seen = nullptr;
    plan->attr_set = true;
    plan->attr_device = dev;
    for (int i = 0; i < b200_gemm_plan::kMapSlots; ++i) plan->map_a_ptr[i] = plan->map_b_ptr[i] = nullptr;
  }
  if (plan->status == nullptr || plan->status_device != dev) {
    if (plan->status != nullptr) cudaFree(plan->status);
    plan->status = nullptr;
    B200_CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&plan->status), gemm::kStatusWords * sizeof(uint32_t)));
    // Cleared on the launch stream: ordered before the plan's first kernel there, whatever kind
    // of stream it is (a memset on the legacy default stream would not be ordered against a
    // non-blocking stream and could wipe what that first kernel reports).
    B200_CUDA_OK(cudaMemsetAsync(plan->status, 0, gemm::kStatusWords * sizeof(uint32_t), stream));
    plan->status_device = dev;
  }
  return B200_OK;
}

int check_run_args(const b200_gemm_plan* plan, const void* A, const void* B, const void* C, const float* bias,
                   const void* workspace, size_t workspace_bytes_in) {
  B200_REQUIRE(plan != nullptr, "plan is NULL");
  B200_REQUIRE(A && B && C, "gemm_run: A, B and C must be non-NULL");
  B200_REQUIRE(((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15u) == 0,
               "gemm_run: A, B and C must be 16-byte aligned");
  const bool needs_bias = plan->desc.epilogue == B200_EPI_BIAS_RELU || plan->desc.epilogue == B200_EPI_BIAS;
  B200_REQUIRE(!needs_bias || bias != nullptr, "gemm_run: this plan's epilogue needs a bias vector");
  const int64_t need = workspace_bytes(plan);
  if (need > 0 && (workspace == nullptr || static_cast<int64_t>(workspace_bytes_in) < need)) {
    return b200::fail(B200_ERR_WORKSPACE, "gemm_run: split-K needs a %lld-byte workspace, got %zu", (long long)need,
                      workspace_bytes_in);
  }
  // Partial sums are written and read back as 16-byte vectors.
  B200_REQUIRE(need == 0 || (reinterpret_cast<uintptr_t>(workspace) & 15u) == 0,
               "gemm_run: the split-K workspace must be 16-byte aligned");
  return B200_OK;
}

int launch(b200_gemm_plan* plan, const void* A, const void* B, void* C, const float* bias, const float* scale_a,
           const float* scale_b, void* workspace, size_t workspace_size, cudaStream_t stream) {
  const b200_gemm_desc& d = plan->desc;
  B200_REQUIRE(d.dtype_c != B200_I32 || (scale_a == nullptr && scale_b == nullptr),
               "gemm_run: i32 output carries the integer sums unchanged; scales need f32 or bf16 output");
  B200_REQUIRE(!plan->mx || (plan->sfa != nullptr && plan->sfb != nullptr),
               "gemm_run: a block-scaled plan needs its scales first (b200_gemm_plan_set_mx_scales)");
  int ia = -1, ib = -1;
  for (int i = 0; i < b200_gemm_plan::kMapSlots; ++i) {
    if (plan->map_a_ptr[i] == A) ia = i;
    if (plan->map_b_ptr[i] == B) ib = i;
  }
  if (ia < 0) {
    ia = plan->map_a_next;
    plan->map_a_ptr[ia] = nullptr;
    int rc = make_operand_map(&plan->map_a[ia], A, d.dtype_ab, static_cast<uint64_t>(d.M), static_cast<uint64_t>(d.K), static_cast<uint32_t>(plan->am));  // per CTA
    if (rc != B200_OK) return rc;
    plan->map_a_ptr[ia] = A;
    plan->map_a_next = (ia + 1) % b200_gemm_plan::kMapSlots;
  }
  if (ib < 0) {
    ib = plan->map_b_next;
    plan->map_b_ptr[ib] = nullptr;
    if (direct_b(plan)) {
      plan->map_b[ib] = plan->map_a[ia];  // never dereferenced: packed B is streamed with 1-D bulk copies
    } else {
      int rc = make_operand_map(&plan->map_b[ib], B, d.dtype_ab, static_cast<uint64_t>(d.N), static_cast<uint64_t>(d.K),
                                static_cast<uint32_t>(plan->bn / plan->cg));
      if (rc != B200_OK) return rc;
    }
    plan->map_b_ptr[ib] = B;
    plan->map_b_next = (ib + 1) % b200_gemm_plan::kMapSlots;
  }
  Params p;
  std::memset(&p, 0, sizeof(p));
  p.M = static_cast<int>(d.M);
  p.N = static_cast<int>(d.N);
  p.K = static_cast<int>(d.K);
  p.m_blocks = plan->m_blocks;
  p.n_blocks = plan->n_blocks;
  p.num_tiles = plan->m_blocks * plan->n_blocks;
  p.num_kb = plan->num_kb;
  p.kb_elems = plan->kb_elems;
  p.split_k = plan->split_k;
  p.stages = plan->stages;
  p.raster_group = plan->raster_group;
  p.mma_kind = mma_kind_for(d.dtype_ab);
  p.acc_int = d.dtype_ab == B200_I8 ? (d.dtype_c == B200_I32 ? 2 : 1) : 0;
  p.idesc = idesc_for(d.dtype_ab, static_cast<uint32_t>(gemm::kBM * plan->cg), static_cast<uint32_t>(plan->bn));
  p.relu = (d.epilogue == B200_EPI_BIAS_RELU || d.epilogue == B200_EPI_RELU) ? 1 : 0;
  p.bias_axis = d.bias_axis;
  p.bias = (d.epilogue == B200_EPI_BIAS_RELU || d.epilogue == B200_EPI_BIAS) ? bias : nullptr;
  p.scale_a = scale_a;
  p.scale_b = scale_b;
  p.C = C;
  p.sf_k_stages = ceil_div(d.K, gemm::kRowBytes);
  p.b_packed = direct_b(plan) ? B : nullptr;
  p.workspace = static_cast<float*>(workspace);
  p.status = plan->status;
#ifdef B200_BRINGUP
  p.timeline = plan->timeline;
#endif
  p.static_b = (d.reserved[1] & 2) != 0 ? 1 : 0;
  p.debug_mode = d.reserved[0];
  p.wait_limit_ms = d.reserved[2] > 0 ? static_cast<unsigned>(d.reserved[2]) : 0u;
  if (plan->tail_parts > 1 && plan->cluster_exchange) {
    p.tail_tiles = plan->tail_tiles;
    p.tail_parts = plan->tail_parts;
    p.tail_kb0 = plan->tail_kb0;
    p.tail_kb = plan->tail_kb;
    p.cluster_exchange = 1;
  } else if (plan->tail_parts > 1 && workspace != nullptr && static_cast<int64_t>(workspace_size) >= plan->tail_ws_bytes &&
             (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0) {
    // The caller lent the optional workspace: cut the last round of tiles along K.
    // A launch recorded into a CUDA graph is replayed with the epoch it was recorded with, so
    // the flags it left would read as "written" to its own next replay: every recorded launch
    // therefore clears the flags first (a memset node per replay), and forgets the workspace,
    // so that the next launch outside a graph clears what the replays leave behind.
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    B200_CUDA_OK(cudaStreamIsCapturing(stream, &capturing));
    int seen = -1;
    for (int i = 0; i < b200_gemm_plan::kSeenSlots; ++i) {
      if (plan->tail_ws_seen[i] == workspace) seen = i;
    }
    if (capturing != cudaStreamCaptureStatusNone || seen < 0) {
      B200_CUDA_OK(cudaMemsetAsync(workspace, 0, static_cast<size_t>(plan->tail_flag_bytes), stream));
      if (capturing != cudaStreamCaptureStatusNone) {
        if (seen >= 0) plan->tail_ws_seen[seen] = nullptr;
      } else {
        plan->tail_ws_seen[plan->tail_ws_next] = workspace;
        plan->tail_ws_next = (plan->tail_ws_next + 1) % b200_gemm_plan::kSeenSlots;
      }
    }
    p.tail_tiles = plan->tail_tiles;
    p.tail_parts = plan->tail_parts;
    p.tail_kb0 = plan->tail_kb0;
    p.tail_kb = plan->tail_kb;
    p.tail_flags = static_cast<uint32_t*>(workspace);
    p.tail_ws = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + plan->tail_flag_bytes);
    // Epochs are unique across the plans of the process: a workspace that two plans take turns
    // with never holds a flag that a later launch of the other plan could mistake for its own.
    static std::atomic<uint32_t> next_epoch{0};
    p.epoch = ++next_epoch;
    if (p.epoch == 0) p.epoch = ++next_epoch;  // 0 is the cleared state of a flag
  }
  {
    // Programmatic stream serialisation: this launch may begin its prologue (barrier set-up,
    // TMEM allocation, descriptor prefetch) while the previous kernel of the stream drains; the
    // kernel waits for that kernel's completion before it touches global memory.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(plan->grid));
    cfg.blockDim = dim3(gemm::kThreads);
    cfg.dynamicSmemBytes = static_cast<size_t>(plan->smem);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    unsigned n_attr = 0;
    if (plan->cg == 2 || p.cluster_exchange != 0) {
      attr[n_attr].id = cudaLaunchAttributeClusterDimension;
      attr[n_attr].val.clusterDim.x = plan->cg == 2 ? 2u : static_cast<unsigned>(plan->tail_parts);
      attr[n_attr].val.clusterDim.y = 1;
      attr[n_attr].val.clusterDim.z = 1;
      ++n_attr;
    }
    if ((d.reserved[0] & 16) == 0) {
      attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
      ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    B200_CUDA_OK(cudaLaunchKernelEx(&cfg, plan->kernel, plan->map_a[ia], plan->map_b[ib], plan->map_sfa, plan->map_sfb, p));
  }
  b200::count_launch();
  B200_CUDA_OK(cudaGetLastError());
  if (plan->split_k > 1) {
    const size_t vecs = static_cast<size_t>(d.M) * d.N / 4 + 1;
    size_t blocks = (vecs + 255) / 256;
    const size_t cap = static_cast<size_t>(plan->sm_count) * 8;
    if (blocks > cap) blocks = cap;
    if (d.dtype_c == B200_F32) {
      gemm::splitk_reduce_kernel<float><<<static_cast<int>(blocks), 256, 0, stream>>>(p);
    } else {
      gemm::splitk_reduce_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, stream>>>(p);
    }
    b200::count_launch();
    B200_CUDA_OK(cudaGetLastError());
  }
  return B200_OK;
}

}  // namespace

extern "C" {

int b200_gemm_plan_create(const b200_gemm_desc* desc, b200_gemm_plan** out) {
  B200_REQUIRE(desc != nullptr && out != nullptr, "gemm_plan_create: NULL argument");
  *out = nullptr;
  const b200_gemm_desc& d = *desc;
  B200_REQUIRE(d.M >= 1 && d.N >= 1 && d.K >= 1, "gemm_plan_create: M, N, K must be >= 1 (got %lld, %lld, %lld)",
               (long long)d.M, (long long)d.N, (long long)d.K);
  B200_REQUIRE(d.M < (1ll << 31) - 256 && d.N < (1ll << 31) - 256 && d.K < (1ll << 31) - 256,
               "gemm_plan_create: each of M, N, K must be below 2^31");
  const bool mx = is_mx(d.dtype_ab);
  B200_REQUIRE(d.dtype_ab == B200_F16 || d.dtype_ab == B200_BF16 || is_f8(d.dtype_ab) || d.dtype_ab == B200_I8 || mx,
               "gemm_plan_create: dtype_ab=%d is not f16, bf16, e4m3, e5m2 (or a mix of the two), i8 or a block-scaled fp8", d.dtype_ab);
  if (mx) {
    B200_REQUIRE(d.K % 32 == 0, "gemm_plan_create: block-scaled inputs need K %% 32 == 0 (one scale per 32 elements), got K=%lld", (long long)d.K);
    B200_REQUIRE(d.b_layout == B200_B_ROW_MAJOR_NK, "gemm_plan_create: block-scaled inputs take row-major B");
    B200_REQUIRE(d.tile_n == 0 || d.tile_n == 128 || d.tile_n == 256, "gemm_plan_create: block-scaled inputs use tile_n=128 or 256 (got %d)", d.tile_n);
  }
  B200_REQUIRE(d.dtype_c == B200_F32 || d.dtype_c == B200_BF16 || d.dtype_c == B200_I32,
               "gemm_plan_create: dtype_c=%d is not f32, bf16 or i32", d.dtype_c);
  B200_REQUIRE(d.dtype_c != B200_I32 || d.dtype_ab == B200_I8, "gemm_plan_create: i32 output needs i8 inputs");
  B200_REQUIRE(d.dtype_c != B200_I32 || d.epilogue == B200_EPI_NONE,
               "gemm_plan_create: i32 output carries the integer sums unchanged; bias, ReLU and scales need f32 or bf16 output");
  B200_REQUIRE(d.dtype_ab != B200_I8 || d.split_k <= 1,
               "gemm_plan_create: i8 inputs do not split K (split_k=%d): integer sums are not exchanged as fp32", d.split_k);
  B200_REQUIRE(d.b_layout >= B200_B_ROW_MAJOR_NK && d.b_layout <= B200_B_PACKED, "gemm_plan_create: bad b_layout %d", d.b_layout);
  B200_REQUIRE(d.epilogue >= B200_EPI_NONE && d.epilogue <= B200_EPI_RELU, "gemm_plan_create: bad epilogue %d", d.epilogue);
  B200_REQUIRE(d.bias_axis == B200_BIAS_AXIS_N || d.bias_axis == B200_BIAS_AXIS_M, "gemm_plan_create: bad bias_axis %d", d.bias_axis);
  const int eb = elt_bytes(d.dtype_ab);
  // TMA needs 16-byte multiples for the row pitch of A and B.
  B200_REQUIRE((d.K * eb) % 16 == 0, "gemm_plan_create: K=%lld gives a %lld-byte row pitch; it must be a multiple of 16 bytes",
               (long long)d.K, (long long)(d.K * eb));
  if (d.b_layout == B200_B_REF_PRESHUFFLED) {
    // Preconditions of the reference's shuffle_weight (kittens_helpers.py:107-108).
    B200_REQUIRE(d.N % 16 == 0 && d.K % 32 == 0, "gemm_plan_create: preshuffled B needs N %% 16 == 0 and K %% 32 == 0");
  }
  B200_REQUIRE(d.tile_m == 0 || d.tile_m == gemm::kBM || d.tile_m == 2 * gemm::kBM,
               "gemm_plan_create: tile_m=%d unsupported (128, or 256 for a CTA pair)", d.tile_m);
  B200_REQUIRE(d.tile_n == 0 || d.tile_n == 32 || d.tile_n == 64 || d.tile_n == 128 || d.tile_n == 256,
               "gemm_plan_create: tile_n=%d unsupported (32, 64, 128, 256)", d.tile_n);
  const int kb_elems = gemm::kRowBytes / eb;
  B200_REQUIRE(d.tile_k == 0 || d.tile_k == kb_elems, "gemm_plan_create: tile_k=%d unsupported (%d for this dtype)", d.tile_k, kb_elems);
  B200_REQUIRE(d.cta_group >= 0 && d.cta_group <= 2, "gemm_plan_create: cta_group=%d unsupported (1 or 2)", d.cta_group);
  B200_REQUIRE(!(d.cta_group == 2 && d.tile_m == gemm::kBM) && !(d.cta_group == 1 && d.tile_m == 2 * gemm::kBM),
               "gemm_plan_create: tile_m=%d contradicts cta_group=%d (128 rows per CTA)", d.tile_m, d.cta_group);
  B200_REQUIRE(!(d.b_layout != B200_B_ROW_MAJOR_NK && (d.cta_group == 2 || d.tile_m == 2 * gemm::kBM)),
               "gemm_plan_create: the direct-B path runs with cta_group=1");
  B200_REQUIRE(!((d.cta_group == 2 || d.tile_m == 2 * gemm::kBM) && d.tile_n == 32),
               "gemm_plan_create: a CTA pair needs tile_n >= 64");
  B200_REQUIRE(d.stages >= 0 && d.stages <= gemm::kMaxStages, "gemm_plan_create: stages=%d outside [0,%d]", d.stages, gemm::kMaxStages);
  B200_REQUIRE(d.split_k >= -1 && d.split_k <= 64, "gemm_plan_create: split_k=%d outside [-1,64]", d.split_k);
  B200_REQUIRE(d.max_ctas >= 0 && d.raster_group >= 0, "gemm_plan_create: max_ctas and raster_group must be >= 0");
#ifndef B200_BRINGUP
  B200_REQUIRE((d.reserved[0] & ~(8 | 16)) == 0,
               "gemm_plan_create: reserved[0]=%d asks for a work-skipping bring-up mode; those exist only in a library built with -DB200_BRINGUP",
               d.reserved[0]);
#endif

  b200_gemm_plan* plan = new (std::nothrow) b200_gemm_plan();
  if (plan == nullptr) return b200::fail(B200_ERR_INVALID, "gemm_plan_create: out of host memory");
  plan->desc = d;
  plan->desc.label[sizeof(plan->desc.label) - 1] = 0;
  plan->eb_ab = eb;
  plan->kb_elems = kb_elems;
  const int k_blocks = ceil_div(d.K, kb_elems);

  // CTA pair or single CTA.  A pair stages half of the B tile per SM, which leaves room for a
  // deeper ring; it needs at least one full 256-row tile to pay off and row-major B.
  int cg = d.cta_group != 0 ? d.cta_group : (d.tile_m == 2 * gemm::kBM ? 2 : (d.tile_m == gemm::kBM ? 1 : 0));
  // Short K and few tiles (512^3: 8 K blocks): the launch is a latency chain -- start-up, a few
  // stages, one epilogue -- which more and smaller CTAs shorten (one CTA per 128 x 32 tile:
  // 6.7 us per launch against 7.9 us for pairs on 256 x 64 tiles).
  const bool short_k = k_blocks <= 16;
  if (cg == 0) {
    cg = (d.b_layout == B200_B_ROW_MAJOR_NK && d.M >= 2 * gemm::kBM && d.tile_n != 32) ? 2 : 1;
    if (cg == 2 && short_k && !mx && d.tile_n == 0 &&
        static_cast<int64_t>(ceil_div(d.M, gemm::kBM)) * ceil_div(d.N, 32) <= kDefaultSms) {  // 128 x 32 tiles still fit one round
      cg = 1;
    }
    // A pair pays a cluster round trip per tile (accumulator hand-over, commit to both CTAs).
    // With at most 8 K blocks per tile that outweighs the shared B traffic it saves (8192 x 8192 x
    // 512: 66 us with single CTAs, 76 us with pairs), and so it does when all 128 x 256 tiles run
    // in one round on more than half of the SMs, up to 64 K blocks (2048^3: 16.3 against 17.0 us;
    // at 128 K blocks the pair's deeper ring and halved B traffic win: 512 x 8192 x 8192 56 against 74 us).
    const int64_t wide_tiles = static_cast<int64_t>(ceil_div(d.M, gemm::kBM)) * ceil_div(d.N, 256);
    if (cg == 2 && !mx && (k_blocks <= 8 || (k_blocks <= 64 && wide_tiles > kDefaultSms / 2 && wide_tiles <= kDefaultSms))) cg = 1;
  }
  plan->cg = cg;
  plan->mx = mx;
  plan->m_blocks = ceil_div(d.M, gemm::kBM * cg);

  // Tile width: the widest tile whose tile count still fills the machine; wide tiles halve the
  // shared-memory traffic per flop, narrow ones keep more SMs busy on small problems.
  int bn = d.tile_n;
  if (bn == 0 && mx) {
    // 256 columns unless that leaves SMs without a tile: a 128-column tile is bound by shared-memory reads.
    bn = (static_cast<int64_t>(plan->m_blocks) * ceil_div(d.N, 256) >= kDefaultSms / cg) ? 256 : 128;
  }
  if (bn == 0) {
    const int units = kDefaultSms / cg;  // CTAs or pairs that run at once
    if (cg == 1 && short_k && static_cast<int64_t>(plan->m_blocks) * ceil_div(d.N, 32) <= units) {
      bn = 32;  // the latency case above
    } else {
      // Estimated launch time in microseconds, from measured constants: a K block of a
      // 256-column tile takes 0.36 us (512 tensor-pipe cycles at the clock the power cap leaves);
      // a 128-column tile runs at 0.75 of that rate and a 128 x 64 x 16 MMA still occupies the
      // pipe for ~100 cycles, so narrower tiles cost 0.66 and 0.78 of a wide one per K block;
      // HBM streams 6.2 TB/s; the partial-sum exchange of a tail split costs ~4 us and a tile's
      // epilogue 2.6 us per 256 columns; every tile adds about 0.5 us of hand-over.  A last
      // partial round counts 1/parts when the tail split can cut it.
      static const struct {
        int bn;
        double cost;
      } kWidths[] = {{256, 1.0}, {128, 0.66}, {64, 0.78}};
      const double hbm_us = (static_cast<double>(d.M + d.N) * d.K * eb + static_cast<double>(d.M) * d.N * elt_bytes(d.dtype_c)) / 6.2e6;
      double best = 0.0;
      for (const auto& w : kWidths) {
        const int64_t tiles = static_cast<int64_t>(plan->m_blocks) * ceil_div(d.N, w.bn);
        const int64_t tail = tiles % units;
        double rounds = static_cast<double>(tiles / units);
        int parts = 1;
        if (tail != 0) {
          for (int cand = 8; cand >= 2; cand /= 2) {
            if (cand <= units / tail && w.bn / cand >= 32 && k_blocks / cand >= 12) {
              parts = cand;
              break;
            }
          }
          rounds += 1.0 / parts;
        }
        const double compute_us = rounds * (k_blocks * 0.36 * w.cost + 0.5);  // 0.5 us of fixed cost per tile
        const double t = (compute_us > hbm_us ? compute_us : hbm_us) + (parts > 1 ? 4.0 : 0.0) + 2.6 * w.bn / 256.0;
        if (bn == 0 || t < best - 1e-9) {
          bn = w.bn;
          best = t;
        }
      }
    }
    while (bn > (cg == 2 ? 64 : 32) && bn / 2 >= d.N) bn /= 2;
  }
  plan->bn = bn;
  plan->n_blocks = ceil_div(d.N, bn);

  int split = d.split_k <= 1 ? 1 : d.split_k;
  if (d.split_k == -1 && d.dtype_ab != B200_I8) {  // integer sums never split
    // Skinny problems: too few tiles to occupy the SMs, so cut K until they do, keeping at
    // least four K blocks per partition.
    const int64_t tiles = static_cast<int64_t>(plan->m_blocks) * plan->n_blocks;
    while (tiles * split * 2 <= kDefaultSms && k_blocks / (split * 2) >= 4 && split < 64) split *= 2;
  }
  if (split > k_blocks) split = k_blocks;
  plan->split_k = split;
  plan->num_kb = ceil_div(k_blocks, split);
  plan->total_kb = plan->num_kb * split;

  // Skinny M (at most 64 rows, one CTA per tile): stage only 32 or 64 rows of A, so that the
  // ring holds more of B, the operand that such a problem streams from HBM.  tile_m = 128
  // asks for full A stages.
  int am = gemm::kBM;
  if (cg == 1 && !mx && d.tile_m == 0 && d.M <= 64 && (bn == 64 || bn == 128)) am = d.M <= 32 ? 32 : 64;
  plan->am = am;
  // Full-A stages never profit from more than 8 slots.  Short-A stages belong to problems that
  // stream B from HBM, and a stream of 16 KB copies is fastest with about 100 KB per SM on request
  // (a copy-only probe over 128 SMs: 6.9 / 7.1 / 6.5 TB/s with 64 / 96 / 160 KB in flight; the
  // M = 16, N = K = 8192 launch: 27.1 / 27.5 / 27.9 us with 6 / 10 / 11 slots): 112 KB of B tiles.
  const int b_stage_bytes = bn / cg * gemm::kRowBytes;
  const int short_a_cap = std::max(4, std::min(gemm::kMaxStages, (112 * 1024 + b_stage_bytes - 1) / b_stage_bytes));
  const int stage_cap = am < gemm::kBM ? short_a_cap : 8;
  const int max_stages = (kMaxSmemOptin - gemm::kBarrierBytes - 1024 - gemm::a_overrun_bytes(bn, cg, mx, am)) / gemm::stage_bytes(bn, cg, mx, am);
  int stages = d.stages > 0 ? d.stages : (max_stages < stage_cap ? max_stages : stage_cap);
  if (stages > max_stages) {
    delete plan;
    return b200::fail(B200_ERR_INVALID, "gemm_plan_create: %d stages of %d bytes exceed the %d-byte shared memory limit", stages,
                      gemm::stage_bytes(bn, cg, mx, am), kMaxSmemOptin);
  }
  plan->stages = stages;
  plan->smem = gemm::smem_bytes(bn, stages, cg, mx, am);
  // Two resident CTAs would both ask for TMEM; keep the footprint above half the SM's shared
  // memory whenever two allocations (2 * tmem_columns) would not fit in the 512 columns.
  if (2 * gemm::tmem_columns(bn, mx) > 512 && plan->smem <= kMaxSmemOptin / 2) plan->smem = kMaxSmemOptin / 2 + 1024;
  // Tiles are walked in groups of `raster_group` m-blocks, m fastest: a group's rows of A stay in
  // the L2 while B streams past once per group.  Groups whose A rows add up to about 32 MiB
  // measured fastest on every configured problem (4096^3: 16 pair rows, 8192^3: 8, K = 2048: 32,
  // fp8 8192^3: 16 -- +2 to 4 % over a fixed 8, DRAM reads of 4096^3 107 -> 76 MB); larger groups
  // fall out of the L2 (8192^3 with 32: -11 %).
  if (d.raster_group > 0) {
    plan->raster_group = d.raster_group;
  } else {
    const int64_t block_bytes = static_cast<int64_t>(gemm::kBM) * cg * d.K * eb;
    int64_t g = (int64_t{32} << 20) / (block_bytes > 0 ? block_bytes : 1);
    if (g > plan->m_blocks) g = plan->m_blocks;
    plan->raster_group = g < 1 ? 1 : static_cast<int>(g);
  }
  plan->kernel = select_kernel(bn, d.dtype_c, cg, mx, am);
  const int cap = d.max_ctas > 0 ? d.max_ctas : kDefaultSms;
  size_grid(plan, cg == 2 ? (cap / 2 < 1 ? 1 : cap / 2) : cap);
  *out = plan;
  return B200_OK;
}

int b200_gemm_plan_destroy(b200_gemm_plan* plan) {
  if (plan == nullptr) return B200_OK;
  if (plan->status != nullptr) cudaFree(plan->status);
  cudaGetLastError();
  delete plan;
  return B200_OK;
}

int b200_gemm_plan_resources(const b200_gemm_plan* plan, b200_gemm_resources* out) {
  B200_REQUIRE(plan != nullptr && out != nullptr, "gemm_plan_resources: NULL argument");
  std::memset(out, 0, sizeof(*out));
  out->tile_m = gemm::kBM * plan->cg;
  out->tile_n = plan->bn;
  out->tile_k = plan->kb_elems;
  out->stages = plan->stages;
  out->cta_group = plan->cg;
  out->split_k = plan->split_k;
  out->grid_ctas = plan->grid;
  out->block_threads = gemm::kThreads;
  out->smem_bytes = plan->smem;
  out->tmem_columns = gemm::tmem_columns(plan->bn, plan->mx);
  out->ctas_per_sm = plan->smem > kMaxSmemOptin / 2 ? 1 : 2;
  out->num_tiles = static_cast<int64_t>(plan->m_blocks) * plan->n_blocks;
  out->workspace_bytes = workspace_bytes(plan);
  out->packed_b_bytes = packed_b_bytes(plan);
  out->optional_workspace_bytes = plan->tail_ws_bytes;
  out->tail_tiles = plan->tail_tiles;
  out->tail_parts = plan->tail_parts;
  out->tail_exchange = plan->tail_parts > 1 ? (plan->cluster_exchange ? 2 : 1) : 0;
  // Registers per thread come from the loaded function; without a device this stays -1.
  out->regs_per_thread = -1;
  cudaFuncAttributes fa;
  if (cudaFuncGetAttributes(&fa, reinterpret_cast<const void*>(plan->kernel)) == cudaSuccess) {
    out->regs_per_thread = fa.numRegs;
  }
  cudaGetLastError();
  return B200_OK;
}

int b200_pack_b(const b200_gemm_plan* plan, const void* b_in, void* b_packed, void* stream) {
  B200_REQUIRE(plan != nullptr && b_in != nullptr && b_packed != nullptr, "pack_b: NULL argument");
  B200_REQUIRE(direct_b(plan), "pack_b: the plan's b_layout is row-major; nothing to pack");
  B200_REQUIRE((reinterpret_cast<uintptr_t>(b_packed) & 15u) == 0, "pack_b: output must be 16-byte aligned");
  const long long total = static_cast<long long>(plan->n_blocks) * plan->total_kb * plan->bn * 8;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  pack_b_kernel<<<static_cast<int>(blocks), 256, 0, b200::as_stream(stream)>>>(
      static_cast<const uint8_t*>(b_in), static_cast<uint8_t*>(b_packed), plan->desc.N, plan->desc.K, plan->eb_ab, plan->bn,
      plan->n_blocks, plan->total_kb, plan->desc.b_layout == B200_B_REF_PRESHUFFLED ? 1 : 0);
  b200::count_launch();
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}

#ifdef B200_BRINGUP
int b200_gemm_debug_timeline(b200_gemm_plan* plan, void* device_buffer) {
  B200_REQUIRE(plan != nullptr, "gemm_debug_timeline: plan is NULL");
  B200_REQUIRE((reinterpret_cast<uintptr_t>(device_buffer) & 7u) == 0, "gemm_debug_timeline: buffer must be 8-byte aligned");
  plan->timeline = static_cast<unsigned long long*>(device_buffer);
  return B200_OK;
}
#endif

int b200_mx_scales_bytes(int64_t rows, int64_t K, size_t* bytes) {
  B200_REQUIRE(bytes != nullptr, "mx_scales_bytes: bytes is NULL");
  B200_REQUIRE(rows >= 1 && K >= 32 && K % 32 == 0, "mx_scales_bytes: rows must be >= 1 and K a positive multiple of 32");
  *bytes = static_cast<size_t>(ceil_div(rows, 128)) * ceil_div(K, gemm::kRowBytes) * gemm::kScaleBlockBytes;
  return B200_OK;
}

int b200_pack_mx_scales(const void* scales_in, void* scales_packed, int64_t rows, int64_t K, void* stream) {
  B200_REQUIRE(scales_in != nullptr && scales_packed != nullptr, "pack_mx_scales: NULL argument");
  B200_REQUIRE(rows >= 1 && K >= 32 && K % 32 == 0, "pack_mx_scales: rows must be >= 1 and K a positive multiple of 32");
  B200_REQUIRE((reinterpret_cast<uintptr_t>(scales_packed) & 15u) == 0, "pack_mx_scales: output must be 16-byte aligned");
  const long long row_blocks = ceil_div(rows, 128), k_stages = ceil_div(K, gemm::kRowBytes);
  long long blocks = (row_blocks * k_stages * gemm::kScaleBlockBytes + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  pack_mx_scales_kernel<<<static_cast<int>(blocks), 256, 0, b200::as_stream(stream)>>>(
      static_cast<const uint8_t*>(scales_in), static_cast<uint8_t*>(scales_packed), rows, K / 32, row_blocks, k_stages);
  b200::count_launch();
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}

int b200_gemm_plan_set_mx_scales(b200_gemm_plan* plan, const void* scales_a_packed, const void* scales_b_packed) {
  B200_REQUIRE(plan != nullptr, "gemm_plan_set_mx_scales: plan is NULL");
  B200_REQUIRE(plan->mx, "gemm_plan_set_mx_scales: the plan's dtype_ab is not block-scaled");
  B200_REQUIRE(scales_a_packed != nullptr && scales_b_packed != nullptr, "gemm_plan_set_mx_scales: NULL scales");
  B200_REQUIRE(((reinterpret_cast<uintptr_t>(scales_a_packed) | reinterpret_cast<uintptr_t>(scales_b_packed)) & 15u) == 0,
               "gemm_plan_set_mx_scales: packed scales must be 16-byte aligned");
  const uint64_t k_stages = static_cast<uint64_t>(ceil_div(plan->desc.K, gemm::kRowBytes));
  int rc = make_scale_map(&plan->map_sfa, scales_a_packed, static_cast<uint64_t>(ceil_div(plan->desc.M, 128)) * k_stages);
  if (rc != B200_OK) return rc;
  rc = make_scale_map(&plan->map_sfb, scales_b_packed, static_cast<uint64_t>(ceil_div(plan->desc.N, 128)) * k_stages);
  if (rc != B200_OK) return rc;
  plan->sfa = scales_a_packed;
  plan->sfb = scales_b_packed;
  return B200_OK;
}

int b200_gemm_run(b200_gemm_plan* plan, const void* A, const void* B, void* C, const float* bias, const float* scale_a,
                  const float* scale_b, void* workspace, size_t workspace_bytes_in, void* stream) {
  int rc = check_run_args(plan, A, B, C, bias, workspace, workspace_bytes_in);
  if (rc != B200_OK) return rc;
  rc = ensure_device_state(plan, b200::as_stream(stream));
  if (rc != B200_OK) return rc;
  return launch(plan, A, B, C, bias, scale_a, scale_b, workspace, workspace_bytes_in, b200::as_stream(stream));
}

int b200_gemm_time(b200_gemm_plan* plan, const void* A, const void* B, void* C, const float* bias, const float* scale_a,
                   const float* scale_b, void* workspace, size_t workspace_bytes_in, int iters, int flush_l2,
                   float* times_ms) {
  B200_REQUIRE(iters >= 1 && times_ms != nullptr, "gemm_time: iters must be >= 1 and times_ms non-NULL");
  int rc = check_run_args(plan, A, B, C, bias, workspace, workspace_bytes_in);
  if (rc != B200_OK) return rc;
  rc = ensure_device_state(plan, nullptr);
  if (rc != B200_OK) return rc;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  B200_CUDA_OK(cudaEventCreate(&e0));
  B200_CUDA_OK(cudaEventCreate(&e1));
  for (int it = 0; it < iters && rc == B200_OK; ++it) {
    if (flush_l2) rc = b200_flush_l2(nullptr);
    if (rc != B200_OK) break;
    cudaEventRecord(e0, nullptr);
    rc = launch(plan, A, B, C, bias, scale_a, scale_b, workspace, workspace_bytes_in, nullptr);
    cudaEventRecord(e1, nullptr);
    cudaError_t e = cudaEventSynchronize(e1);
    if (rc == B200_OK && e != cudaSuccess) rc = b200::fail(B200_ERR_CUDA, "gemm_time: %s", cudaGetErrorString(e));
    if (rc == B200_OK) cudaEventElapsedTime(&times_ms[it], e0, e1);
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  return rc;
}

int b200_gemm_time_batch(b200_gemm_plan* plan, const void* A, const void* B, void* C, const float* bias,
                         const float* scale_a, const float* scale_b, void* workspace, size_t workspace_bytes_in, int iters,
                         float* total_ms) {
  B200_REQUIRE(iters >= 1 && total_ms != nullptr, "gemm_time_batch: iters must be >= 1 and total_ms non-NULL");
  int rc = check_run_args(plan, A, B, C, bias, workspace, workspace_bytes_in);
  if (rc != B200_OK) return rc;
  rc = ensure_device_state(plan, nullptr);
  if (rc != B200_OK) return rc;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  B200_CUDA_OK(cudaEventCreate(&e0));
  B200_CUDA_OK(cudaEventCreate(&e1));
  cudaEventRecord(e0, nullptr);
  for (int it = 0; it < iters && rc == B200_OK; ++it) rc = launch(plan, A, B, C, bias, scale_a, scale_b, workspace, workspace_bytes_in, nullptr);
  cudaEventRecord(e1, nullptr);
  cudaError_t e = cudaEventSynchronize(e1);
  if (rc == B200_OK && e != cudaSuccess) rc = b200::fail(B200_ERR_CUDA, "gemm_time_batch: %s", cudaGetErrorString(e));
  if (rc == B200_OK) cudaEventElapsedTime(total_ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  return rc;
}

int b200_status_read(b200_gemm_plan* plan, uint32_t words[4]) {
  B200_REQUIRE(plan != nullptr && words != nullptr, "status_read: NULL argument");
  words[0] = words[1] = words[2] = words[3] = 0;
  if (plan->status == nullptr) return B200_OK;  // never launched
  B200_CUDA_OK(cudaDeviceSynchronize());
  B200_CUDA_OK(cudaMemcpy(words, plan->status, 4 * sizeof(uint32_t), cudaMemcpyDeviceToHost));
  if (words[0] != 0) {
    B200_CUDA_OK(cudaMemset(plan->status, 0, 4 * sizeof(uint32_t)));
    return b200::fail(B200_ERR_TIMEOUT, "device wait timed out: code 0x%x cta %u tile %u k-block %u", words[0], words[1], words[2],
                      words[3]);
  }
  return B200_OK;
}

int b200_gemm_last_sm_mhz(b200_gemm_plan* plan, float* mhz) {
  B200_REQUIRE(plan != nullptr && mhz != nullptr, "gemm_last_sm_mhz: NULL argument");
  *mhz = 0.0f;
  if (plan->status == nullptr) return B200_OK;
  B200_CUDA_OK(cudaDeviceSynchronize());
  uint32_t w[8];
  B200_CUDA_OK(cudaMemcpy(w, plan->status, sizeof(w), cudaMemcpyDeviceToHost));
  const double cycles = static_cast<double>((static_cast<uint64_t>(w[5]) << 32) | w[4]);
  const double ns = static_cast<double>((static_cast<uint64_t>(w[7]) << 32) | w[6]);
  if (ns > 0) *mhz = static_cast<float>(cycles / ns * 1000.0);
  return B200_OK;
}

int b200_gemm_clock_totals(b200_gemm_plan* plan, uint64_t* sm_cycles, uint64_t* nanoseconds, uint64_t* launches) {
  B200_REQUIRE(plan != nullptr && sm_cycles != nullptr && nanoseconds != nullptr && launches != nullptr, "gemm_clock_totals: NULL argument");
  *sm_cycles = *nanoseconds = *launches = 0;
  if (plan->status == nullptr) return B200_OK;
  B200_CUDA_OK(cudaDeviceSynchronize());
  uint32_t w[gemm::kStatusWords];
  B200_CUDA_OK(cudaMemcpy(w, plan->status, sizeof(w), cudaMemcpyDeviceToHost));
  *sm_cycles = (static_cast<uint64_t>(w[9]) << 32) | w[8];
  *nanoseconds = (static_cast<uint64_t>(w[11]) << 32) | w[10];
  *launches = w[12];
  return B200_OK;
}

int b200_flush_l2(void* stream) {
  std::lock_guard<std::mutex> lock(g_flush_mu);
  int dev = 0;
  B200_CUDA_OK(cudaGetDevice(&dev));
  if (g_flush.buf == nullptr || g_flush.device != dev) {
    if (g_flush.buf != nullptr) cudaFree(g_flush.buf);
    g_flush.buf = nullptr;
    int l2 = 0;
    B200_CUDA_OK(cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev));
    g_flush.bytes = static_cast<size_t>(l2) * 2;
    if (g_flush.bytes < (256u << 20)) g_flush.bytes = 256u << 20;
    B200_CUDA_OK(cudaMalloc(&g_flush.buf, g_flush.bytes));
    g_flush.device = dev;
  }
  B200_CUDA_OK(cudaMemsetAsync(g_flush.buf, 0, g_flush.bytes, b200::as_stream(stream)));
  return B200_OK;
}

}  // extern "C"
