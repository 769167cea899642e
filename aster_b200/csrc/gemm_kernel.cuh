// Persistent, warp-specialised tcgen05 GEMM for sm_100a:  C[M,N] = epilogue(A[M,K] . B[N,K]^T).
//
// This is the B200 counterpart of the reference's scheduled MFMA GEMM kernel
// (contrib/kittens/test/test_102_gemm_python_multitile_lds_cdna3.py:75-350): where that kernel
// stages 16x64-byte tiles through XOR-swizzled LDS with cooperative global loads and issues
// v_mfma_f32_16x16x16_f16 per wave, this one stages 128-byte-swizzled operand tiles in shared
// memory with TMA and issues tcgen05.mma from a single thread with the accumulator in tensor
// memory.  The software pipeline the reference builds with per-operation stage numbers
// (kittens_helpers.py:137-157) becomes an mbarrier ring of `stages` shared-memory slots.
//
// CTA = 192 threads:
//   warp 0     producer: waits empty[s], arms full[s] with the stage's byte count, issues the
//              TMA loads of the A tile (BM x 128 B) and the B tile (BN x 128 B)
//   warp 1     MMA issuer: owns the TMEM allocation; waits full[s], issues 4 tcgen05.mma per
//              stage (each consumes 32 bytes of K), commits to empty[s]; after the last K block
//              of a tile commits to acc_full[a]
//   warps 2-5  epilogue: wait acc_full[a], read the accumulator with tcgen05.ld (warp w owns
//              TMEM lanes 32*(w%4)..+31 = 32 rows of the tile), apply scale/bias/ReLU/cast,
//              store to C, arrive on acc_empty[a]
// The accumulator is double buffered in TMEM (2 x BN columns) so the epilogue of tile i
// overlaps the main loop of tile i+1.  Tiles are dealt round-robin to the persistent CTAs in
// an order that keeps concurrently running CTAs on neighbouring rows/columns (L2 reuse).
//
// Every wait is bounded: after kWaitTimeoutNs it records a code in the status words, raises
// the CTA's abort flag and every role falls through to the common teardown, which drains
// outstanding copies and MMAs (bounded again), frees TMEM and returns.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdint>

#include "ptx_sm100.cuh"

namespace gemm {

constexpr int kBM = 128;             // rows per CTA tile = TMEM lanes
constexpr int kRowBytes = 128;       // bytes of K per stage row (one swizzle span)
constexpr int kMmasPerStage = 4;     // 128 B / 32 B consumed per tcgen05.mma
constexpr int kMaxStages = 8;
constexpr int kThreads = 192;
constexpr int kEpilogueWarps = 4;
constexpr unsigned long long kWaitTimeoutNs = 2000000000ull;  // 2 s
constexpr unsigned long long kDrainTimeoutNs = 20000000ull;   // 20 ms

// Status codes (status[0]); status[1] = blockIdx.x, status[2] = tile, status[3] = k block.
enum : uint32_t {
  kStatusOk = 0,
  kStatusProducerEmptyWait = 0x10,
  kStatusMmaFullWait = 0x20,
  kStatusMmaAccEmptyWait = 0x21,
  kStatusEpilogueAccFullWait = 0x30,
};

struct Params {
  int M, N, K;
  int m_blocks, n_blocks;
  int num_tiles;       // m_blocks * n_blocks
  int num_kb;          // K blocks per tile (per split)
  int kb_elems;        // elements of K per stage (128 B / element size)
  int split_k;         // >= 1; work item = (tile, split)
  int stages;
  int raster_group;    // m-blocks per rasterisation group
  uint32_t idesc;
  int kind_f8;
  int relu;
  int bias_axis;       // 0 = per column (N), 1 = per row (M)
  const float* bias;   // may be null
  const float* scale_a;
  const float* scale_b;
  void* C;
  const void* b_packed;  // non-null: B comes as packed tile images, streamed with 1-D bulk copies
  float* workspace;      // split-K partial sums [split][M][N] fp32
  uint32_t* status;
};

__host__ __device__ constexpr int stage_bytes(int bn) { return (kBM + bn) * kRowBytes; }
// Barrier block that follows the stage ring: full[8], empty[8], acc_full[2], acc_empty[2],
// drain, TMEM base slot, abort flag.
constexpr int kBarrierBytes = 256;
__host__ __device__ constexpr int smem_bytes(int bn, int stages) { return stages * stage_bytes(bn) + kBarrierBytes + 1024; }
__host__ __device__ constexpr int tmem_columns(int bn) { return 2 * bn < 32 ? 32 : 2 * bn; }  // bn is a power of two

struct Waiter {
  volatile uint32_t* abort_flag;
  uint32_t* status;

  // Spin on an mbarrier phase with a time limit.  Returns false when the CTA is aborting.
  __device__ __forceinline__ bool wait(uint32_t bar, uint32_t parity, uint32_t code, int tile, int kb,
                                       unsigned long long limit_ns = kWaitTimeoutNs) const {
    if (sm100::mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = sm100::globaltimer_ns();
#pragma unroll 1
    for (uint32_t spin = 1;; ++spin) {
      if (sm100::mbar_try_wait(bar, parity)) return true;
      if ((spin & 63u) == 0u) {
        if (*abort_flag != 0u) return false;
        if (sm100::globaltimer_ns() - t0 > limit_ns) {
          if (code != 0u && atomicCAS(status, 0u, code) == 0u) {
            status[1] = blockIdx.x;
            status[2] = static_cast<uint32_t>(tile);
            status[3] = static_cast<uint32_t>(kb);
          }
          *abort_flag = 1u;
          return false;
        }
      }
    }
  }
};

// Work item -> (m block, n block).  Groups of `raster_group` m-blocks are walked m-fastest so
// that the ~148 tiles in flight share a few A row panels and B row panels in L2.
__device__ __forceinline__ void tile_coords(const Params& p, int tile, int& m_blk, int& n_blk) {
  const int group_span = p.raster_group * p.n_blocks;
  const int group = tile / group_span;
  const int first_m = group * p.raster_group;
  const int rows = min(p.raster_group, p.m_blocks - first_m);
  const int in_group = tile - group * group_span;
  m_blk = first_m + in_group % rows;
  n_blk = in_group / rows;
}

template <typename OutT>
struct OutVec;
template <>
struct OutVec<float> {
  static constexpr int kPerVec = 4;  // elements per 16-byte store
};
template <>
struct OutVec<__nv_bfloat16> {
  static constexpr int kPerVec = 8;
};

// Store 32 consecutive outputs of one row.  `vec_ok`: the row segment is 16-byte aligned and
// entirely inside the matrix.
template <typename OutT>
__device__ __forceinline__ void store_row32(OutT* dst, const float (&x)[32], bool vec_ok, int valid) {
  if (vec_ok) {
    if constexpr (sizeof(OutT) == 4) {
      float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
      for (int j = 0; j < 8; ++j) d4[j] = make_float4(x[4 * j], x[4 * j + 1], x[4 * j + 2], x[4 * j + 3]);
    } else {
      uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t w[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          __nv_bfloat162 h = __floats2bfloat162_rn(x[8 * j + 2 * t], x[8 * j + 2 * t + 1]);
          w[t] = *reinterpret_cast<uint32_t*>(&h);
        }
        d4[j] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (j < valid) {
        if constexpr (sizeof(OutT) == 4) {
          dst[j] = x[j];
        } else {
          dst[j] = __float2bfloat16_rn(x[j]);
        }
      }
    }
  }
}

template <int BN, typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const Params p) {
#if defined(__CUDA_ARCH_FEAT_SM100_ALL)
  using namespace sm100;
  static_assert(BN == 32 || BN == 64 || BN == 128 || BN == 256, "unsupported tile width");
  constexpr uint32_t kABytes = kBM * kRowBytes;
  constexpr uint32_t kBBytes = BN * kRowBytes;
  constexpr uint32_t kStageBytes = kABytes + kBBytes;
  constexpr uint32_t kTmemCols = tmem_columns(BN);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_raw_u32 = smem_u32(smem_raw);
  const uint32_t smem_base = (smem_raw_u32 + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
  const uint32_t bar_base = smem_base + static_cast<uint32_t>(p.stages) * kStageBytes;
  uint8_t* bar_ptr = smem_raw + (bar_base - smem_raw_u32);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 64u + 8u * s; };
  auto acc_full_bar = [&](int a) { return bar_base + 128u + 8u * a; };
  auto acc_empty_bar = [&](int a) { return bar_base + 144u + 8u * a; };
  const uint32_t drain_bar = bar_base + 160u;
  const uint32_t tmem_slot = bar_base + 168u;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(bar_ptr + 168);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bar_ptr + 172);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const Waiter waiter{abort_flag, p.status};
  const int num_items = p.num_tiles * p.split_k;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), kEpilogueWarps);
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0u;
    fence_barrier_init();
    fence_proxy_async_smem();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) tmem_alloc<1>(tmem_slot, kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    // ------------------------------- producer -------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
        const int tile = item / p.split_k;
        const int split = item - tile * p.split_k;
        int m_blk, n_blk;
        tile_coords(p, tile, m_blk, n_blk);
        const int kb0 = split * p.num_kb;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!waiter.wait(empty_bar(stage), phase ^ 1u, kStatusProducerEmptyWait, tile, kb)) {
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_base + stage * kStageBytes;
          const uint32_t b_dst = a_dst + kABytes;
          mbar_arrive_expect_tx(full_bar(stage), kStageBytes);
          tma_load_2d(a_dst, &tmap_a, full_bar(stage), (kb0 + kb) * p.kb_elems, m_blk * kBM);
          if (p.b_packed != nullptr) {
            const size_t blk = static_cast<size_t>(n_blk) * (static_cast<size_t>(p.num_kb) * p.split_k) + (kb0 + kb);
            bulk_load_1d(b_dst, static_cast<const uint8_t*>(p.b_packed) + blk * kBBytes, kBBytes, full_bar(stage));
          } else {
            tma_load_2d(b_dst, &tmap_b, full_bar(stage), (kb0 + kb) * p.kb_elems, n_blk * BN);
          }
          ++issued;
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // Aborting: let the copies already issued land before the CTA may exit.
        for (int s = 0; s < p.stages; ++s) {
          if (issued > s) {
            const long long last = (issued - 1) - ((issued - 1 - s) % p.stages);  // last issue into slot s
            waiter.wait(full_bar(s), static_cast<uint32_t>((last / p.stages) & 1), 0u, 0, 0, kDrainTimeoutNs);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
        const int tile = item / p.split_k;
        if (!waiter.wait(acc_empty_bar(acc), acc_phase ^ 1u, kStatusMmaAccEmptyWait, tile, 0)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!waiter.wait(full_bar(stage), phase, kStatusMmaFullWait, tile, kb)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_src = smem_base + stage * kStageBytes;
          const uint64_t desc_a = make_smem_desc_sw128(a_src);
          const uint64_t desc_b = make_smem_desc_sw128(a_src + kABytes);
#pragma unroll
          for (int k = 0; k < kMmasPerStage; ++k) {
            // +32 bytes of K per instruction = +2 in the descriptor's 16-byte address units.
            umma_ss<1>(tmem_d, desc_a + 2u * k, desc_b + 2u * k, p.idesc, (kb | k) != 0 ? 1u : 0u, p.kind_f8 != 0);
          }
          umma_commit<1>(empty_bar(stage));
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit<1>(acc_full_bar(acc));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (!ok) {
        // Aborting: wait for the MMAs already issued before TMEM and shared memory go away.
        umma_commit<1>(drain_bar);
        waiter.wait(drain_bar, 0u, 0u, 0, 0, kDrainTimeoutNs);
      }
    }
  } else {
    // ------------------------------- epilogue -------------------------------
    const int quarter = warp & 3;  // TMEM lanes this warp may read
    const int row_in_tile = quarter * 32 + lane;
    float alpha = 1.0f;
    if (p.scale_a != nullptr) alpha *= __ldg(p.scale_a);
    if (p.scale_b != nullptr) alpha *= __ldg(p.scale_b);
    OutT* const C = static_cast<OutT*>(p.C);
    const bool n_vec_ok = (p.N % OutVec<OutT>::kPerVec) == 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
      const int tile = item / p.split_k;
      const int split = item - tile * p.split_k;
      int m_blk, n_blk;
      tile_coords(p, tile, m_blk, n_blk);
      if (!waiter.wait(acc_full_bar(acc), acc_phase, kStatusEpilogueAccFullWait, tile, 0)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int row = m_blk * kBM + row_in_tile;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN);
      float bias_row = 0.0f;
      if (p.bias != nullptr && p.bias_axis == 1 && row_ok) bias_row = __ldg(p.bias + row);
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(taddr + static_cast<uint32_t>(c), v);
        tmem_ld_wait();
        const int col0 = n_blk * BN + c;
        if (col0 >= p.N) continue;  // warp-uniform
        const int valid = min(32, p.N - col0);
        float x[32];
        if (p.split_k > 1) {
          // Partial sums go to the workspace untouched; the reduction applies the epilogue.
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(v[j]);
          if (row_ok) {
            float* wdst = p.workspace + (static_cast<size_t>(split) * p.M + row) * p.N + col0;
            store_row32<float>(wdst, x, (p.N % 4) == 0 && valid == 32, valid);
          }
          continue;
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(v[j]) * alpha;
        if (p.bias != nullptr) {
          if (p.bias_axis == 0) {
#pragma unroll
            for (int j = 0; j < 32; ++j) x[j] += (j < valid) ? __ldg(p.bias + col0 + j) : 0.0f;
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) x[j] += bias_row;
          }
        }
        if (p.relu) {
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] = fmaxf(x[j], 0.0f);
        }
        if (row_ok) store_row32<OutT>(C + static_cast<size_t>(row) * p.N + col0, x, n_vec_ok && valid == 32, valid);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(acc));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // ------------------------------- teardown -------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, kTmemCols);
  }
#endif
}

// Split-K reduction + epilogue: C = epilogue(sum_s workspace[s]).  HBM-bound, 16-byte accesses.
template <typename OutT>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const Params p) {
  const float* ws = p.workspace;
  OutT* C = static_cast<OutT*>(p.C);
  float alpha = 1.0f;
  if (p.scale_a != nullptr) alpha *= __ldg(p.scale_a);
  if (p.scale_b != nullptr) alpha *= __ldg(p.scale_b);
  const size_t mn = static_cast<size_t>(p.M) * p.N;
  const size_t gsz = static_cast<size_t>(gridDim.x) * blockDim.x;
  if ((p.N % 4) == 0) {
    const size_t nvec = mn / 4;
    for (size_t v = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec; v += gsz) {
      float4 acc = __ldcs(reinterpret_cast<const float4*>(ws) + v);
      for (int s = 1; s < p.split_k; ++s) {
        const float4 t = __ldcs(reinterpret_cast<const float4*>(ws + s * mn) + v);
        acc.x += t.x;
        acc.y += t.y;
        acc.z += t.z;
        acc.w += t.w;
      }
      const size_t e = v * 4;
      const int row = static_cast<int>(e / p.N);
      const int col = static_cast<int>(e - static_cast<size_t>(row) * p.N);
      float x[4] = {acc.x * alpha, acc.y * alpha, acc.z * alpha, acc.w * alpha};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (p.bias != nullptr) x[j] += __ldg(p.bias + (p.bias_axis == 0 ? col + j : row));
        if (p.relu) x[j] = fmaxf(x[j], 0.0f);
      }
      if constexpr (sizeof(OutT) == 4) {
        reinterpret_cast<float4*>(C)[v] = make_float4(x[0], x[1], x[2], x[3]);
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(x[0], x[1]);
        __nv_bfloat162 hi = __floats2bfloat162_rn(x[2], x[3]);
        uint2 w = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        reinterpret_cast<uint2*>(C)[v] = w;
      }
    }
  } else {
    for (size_t e = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < mn; e += gsz) {
      float acc = ws[e];
      for (int s = 1; s < p.split_k; ++s) acc += ws[s * mn + e];
      const int row = static_cast<int>(e / p.N);
      const int col = static_cast<int>(e - static_cast<size_t>(row) * p.N);
      float x = acc * alpha;
      if (p.bias != nullptr) x += __ldg(p.bias + (p.bias_axis == 0 ? col : row));
      if (p.relu) x = fmaxf(x, 0.0f);
      if constexpr (sizeof(OutT) == 4) {
        C[e] = x;
      } else {
        C[e] = __float2bfloat16_rn(x);
      }
    }
  }
}

}  // namespace gemm
