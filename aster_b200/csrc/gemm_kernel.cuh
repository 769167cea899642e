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
constexpr int kMaxStages = 16;
constexpr int kThreads = 192;
constexpr int kEpilogueWarps = 4;
constexpr unsigned long long kWaitTimeoutNs = 2000000000ull;  // 2 s
constexpr unsigned long long kDrainTimeoutNs = 20000000ull;   // 20 ms

// Status codes (status[0]); status[1] = blockIdx.x, status[2] = tile, status[3] = k block.
// status[4..5] = SM cycles and status[6..7] = nanoseconds that CTA 0 spent in the kernel (the
// SM clock actually seen by the launch is their ratio); status[8..9], [10..11] and [12] = the
// same two quantities and the launch count summed over all launches (kStatusWords words in all).
constexpr int kStatusWords = 16;
enum : uint32_t {
  kStatusOk = 0,
  kStatusProducerEmptyWait = 0x10,
  kStatusMmaFullWait = 0x20,
  kStatusMmaAccEmptyWait = 0x21,
  kStatusEpilogueAccFullWait = 0x30,
  kStatusTailFlagWait = 0x31,
  kStatusClusterExchangeWait = 0x32,
};

struct Params {
  int M, N, K;
  int m_blocks, n_blocks;  // tiles along M (128 rows, or 256 for a CTA pair) and N
  int num_tiles;       // m_blocks * n_blocks
  int num_kb;          // K blocks per tile (per split)
  int kb_elems;        // elements of K per stage (128 B / element size)
  int split_k;         // >= 1; work item = (tile, split)
  int stages;
  int raster_group;    // m-blocks per rasterisation group
  uint32_t idesc;
  int mma_kind;        // sm100::MmaKind
  int acc_int;         // s32 accumulators (8-bit integer inputs): 1 = convert to float for the epilogue, 2 = store as they are
  int relu;
  int bias_axis;       // 0 = per column (N), 1 = per row (M)
  const float* bias;   // may be null
  const float* scale_a;
  const float* scale_b;
  void* C;
  // Block-scaled kernels: the E8M0 scales of A and B come in blocks of [128 rows][4 K blocks]
  // (row r of a block at byte (r % 32) * 16 + (r / 32) * 4), ordered [row block][K stage] with
  // sf_k_stages = ceil(K / 128) blocks per row block; the kernel's two scale tensor maps see
  // each array as one 512-byte row per block.
  int sf_k_stages;
  const void* b_packed;  // non-null: B comes as packed tile images, streamed with 1-D bulk copies
  float* workspace;      // split-K partial sums [split][M][N] fp32
  uint32_t* status;
  // Tail split: when the last round of tiles would leave most units idle, each of the
  // `tail_tiles` last tiles is cut into `tail_parts` K ranges handled by different units; each
  // part then finishes 1/tail_parts of the tile's columns, adding the other parts' fp32 partial
  // sums for that slice (exchanged through `tail_ws`, announced through `tail_flags` = epoch).
  // tail_parts <= 1: off.
  int tail_tiles;
  int tail_parts;
  int tail_kb0;           // K blocks of part 0 (equal to tail_kb)
  int tail_kb;            // K blocks of every other part
  float* tail_ws;         // [tail_tiles][tail_parts][tile rows][BN] fp32, a part writes only the other parts' slices
  uint32_t* tail_flags;   // [tail_tiles][tail_parts][CG][4 epilogue warps]
  uint32_t epoch;         // changes every launch; a flag equal to it means "written in this launch"
  // Non-zero: every tile is a tail tile, every CTA has exactly one part, and the `tail_parts`
  // parts of a tile are the CTAs of one cluster (one CTA per MMA), so the partial sums are
  // exchanged through the cluster's shared memory: each CTA parks its partial sums for the other
  // parts' column slices in its own stage ring (idle once its last MMA has completed), signals
  // the peers' barriers and reads its own slice out of the peers' shared memory.  No workspace,
  // no flags in global memory.
  int cluster_exchange;
  // Bit 3 (8): fault injection for the wait-limit test -- the producer never hands a stage over,
  // so the consumers' bounded waits must expire.  Bit 4 (16, host only): launch without
  // programmatic stream serialisation.  The other bits exist only in bring-up builds
  // (-DB200_BRINGUP) and make the kernel skip work, i.e. return garbage: bits 0-1: 1 = producer
  // signals without copying, 2 = MMA warp commits without multiplying; bit 2: skip the tail-split
  // exchange; bit 5: the epilogue computes but does not store C; bit 6: 16-byte stores only; bit 7: no
  // wait for the previous kernel of the stream.
  int debug_mode;
  unsigned wait_limit_ms;  // limit of every bounded wait; 0 = default
  // Non-zero: nothing that precedes a launch in its stream writes B (a weight matrix), so the
  // producer may request the first ring of B tiles before the previous kernel has completed.
  int static_b;
#ifdef B200_BRINGUP
  // Bring-up aid: when non-null, every CTA writes global-timer readings (ns) of its milestones to
  // timeline[blockIdx.x * 16 + slot]: 0 entry, 1 prologue done, 2 previous kernel complete,
  // 3 first copy issued, 4 first stage landed, 5 last MMA committed, 6 last accumulator ready,
  // 7 last epilogue done, 8 exit, 9..15 last MMA of the CTA's first seven work items committed
  // (slot 12 is then overwritten with the SM cycles of the last item's epilogue).  A stamp costs
  // about a microsecond (the global timer is slow to read): intervals between stamps of one
  // thread include that.
  unsigned long long* timeline;
#endif
};

#ifdef B200_BRINGUP
constexpr bool kBringup = true;
__device__ __forceinline__ void stamp(const Params& p, int slot) {
  if (p.timeline != nullptr) p.timeline[static_cast<size_t>(blockIdx.x) * 16 + slot] = sm100::globaltimer_ns();
}
#else
constexpr bool kBringup = false;
__device__ __forceinline__ void stamp(const Params&, int) {}
#endif
// True when a bring-up build was asked for one of the work-skipping modes in `bits`.
__device__ __forceinline__ bool bringup_mode(const Params& p, int bits) { return kBringup && (p.debug_mode & bits) != 0; }

// Block-scaled (MX) stages carry the E8M0 scales of their 128 elements of K behind the operand
// tiles: one 512-byte block for the 128 rows of A and one per 128 rows of B, padded so that
// the next stage stays 1024-byte aligned.
constexpr int kScaleBlockBytes = 512;  // 128 rows x 4 K blocks of 32
__host__ __device__ constexpr int scale_stage_bytes(int bn) { return (kScaleBlockBytes * (1 + bn / 128) + 1023) / 1024 * 1024; }
// `am` = rows of A that a stage holds: 128, or 32 / 64 for skinny problems (M <= am), whose
// stages then spend their bytes on B.  The MMA still reads 128 rows from the stage's start; the
// rows beyond `am` are whatever follows in shared memory and only reach accumulator rows that no
// one reads (rows >= M are never loaded from TMEM or stored).
__host__ __device__ constexpr int stage_bytes(int bn, int cg = 1, bool mx = false, int am = kBM) {
  return (am + bn / cg) * kRowBytes + (mx ? scale_stage_bytes(bn) : 0);
}
// Barrier block that follows the stage ring (and, for am < 128, the slack that the last stage's
// 128-row A read runs into): full[16], empty[16], acc_full[2], acc_empty[2], drain, TMEM base
// slot, abort flag, and one barrier per epilogue warp for the cluster exchange.
constexpr int kBarrierBytes = 384;
// Bytes behind the last stage that the MMA's 128-row read of a short A tile still touches: the
// read covers 16 KB from the stage's start, i.e. the stage's own B tile first, and only runs past
// the stage when A and B together are shorter than that (32 rows of A with a 64-column tile).
__host__ __device__ constexpr int a_overrun_bytes(int bn, int cg = 1, bool mx = false, int am = kBM) {
  return kBM * kRowBytes > stage_bytes(bn, cg, mx, am) ? kBM * kRowBytes - stage_bytes(bn, cg, mx, am) : 0;
}
__host__ __device__ constexpr int smem_bytes(int bn, int stages, int cg = 1, bool mx = false, int am = kBM) {
  return stages * stage_bytes(bn, cg, mx, am) + a_overrun_bytes(bn, cg, mx, am) + kBarrierBytes + 1024;
}
// Two accumulators of bn columns; a block-scaled kernel adds two sets of 16 scale columns.
constexpr int kScaleTmemCols = 16;
__host__ __device__ constexpr int tmem_columns(int bn, bool mx = false) {  // bn is a power of two
  return mx ? 512 : (2 * bn < 32 ? 32 : 2 * bn);
}

// Has more than `limit` ns passed since `t0`?  A single reading of the global timer is not
// trusted: a reading that looks like an expiry is confirmed by a second one, and a start stamp
// that lies in the future (a torn or stepped timer value) is replaced, so that one bad reading
// cannot turn into a spurious timeout.
__device__ __forceinline__ bool wait_expired(unsigned long long& t0, unsigned long long limit) {
  const unsigned long long now = sm100::globaltimer_ns();
  if (now < t0) {
    t0 = now;
    return false;
  }
  if (now - t0 <= limit) return false;
  const unsigned long long again = sm100::globaltimer_ns();
  return again >= now && again - t0 > limit;
}

struct Waiter {
  volatile uint32_t* abort_flag;
  uint32_t* status;
  unsigned long long limit_ns;

  // Wait for an mbarrier phase with a time limit.  Returns false when the CTA is aborting.
  // The first poll is inline; only a miss pays for the bookkeeping of the bounded spin.
  __device__ __forceinline__ bool wait(uint32_t bar, uint32_t parity, uint32_t code, int tile, int kb,
                                       unsigned long long limit = 0) const {
    if (sm100::mbar_try_wait(bar, parity)) return true;
    return wait_slow(bar, parity, code, tile, kb, limit != 0 ? limit : limit_ns);
  }

  // Wait of a whole warp that can afford some wake-up latency (the epilogue, which has a whole
  // main loop of slack): lane 0 polls with a sleep between polls, the other lanes idle at the
  // shuffle.  128 threads spinning on a barrier for the length of a main loop burn power that
  // the tensor pipe could use -- the kernel runs against the board's power limit.
  // kClusterScope: the arrivals come from other CTAs of the cluster (acquire at cluster scope).
  template <bool kClusterScope = false>
  __device__ __forceinline__ bool wait_relaxed(uint32_t bar, uint32_t parity, uint32_t code, int tile, unsigned sleep_ns) const {
    auto poll = [&]() { return kClusterScope ? sm100::mbar_try_wait_cluster(bar, parity) : sm100::mbar_try_wait(bar, parity); };
    int ok = 1;
    if ((threadIdx.x & 31) == 0 && !poll()) {
      unsigned long long t0 = sm100::globaltimer_ns();
#pragma unroll 1
      for (uint32_t spin = 1;; ++spin) {
        __nanosleep(sleep_ns);
        if (poll()) break;
        if ((spin & 15u) == 0u) {
          if (*abort_flag != 0u) {
            ok = 0;
            break;
          }
          if (wait_expired(t0, limit_ns)) {
            if (atomicCAS(status, 0u, code) == 0u) {
              status[1] = blockIdx.x;
              status[2] = static_cast<uint32_t>(tile);
              status[3] = 0u;
            }
            *abort_flag = 1u;
            ok = 0;
            break;
          }
        }
      }
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    __syncwarp();  // the other lanes' reads come after lane 0's acquire (the warp barrier orders memory among its lanes)
    return ok != 0;
  }

  __device__ __noinline__ bool wait_slow(uint32_t bar, uint32_t parity, uint32_t code, int tile, int kb,
                                         unsigned long long limit) const {
    unsigned long long t0 = sm100::globaltimer_ns();
#pragma unroll 1
    for (uint32_t spin = 1;; ++spin) {
      if (sm100::mbar_try_wait(bar, parity)) return true;
      if ((spin & 63u) == 0u) {
        if (*abort_flag != 0u) return false;
        if (wait_expired(t0, limit)) {
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

// Bounded wait of a whole warp for a global-memory flag written by another CTA of the same
// launch.  Only lane 0 polls (with a short sleep between polls): dozens of warps hammering the
// same L2 line delay the very store they are waiting for.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t want, const Waiter& waiter, int tile) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0 && sm100::ld_acquire_gpu(flag) != want) {
    unsigned long long t0 = sm100::globaltimer_ns();
#pragma unroll 1
    for (uint32_t spin = 1;; ++spin) {
      __nanosleep(64);
      if (sm100::ld_acquire_gpu(flag) == want) break;
      if ((spin & 63u) == 0u) {
        if (*waiter.abort_flag != 0u) {
          ok = 0;
          break;
        }
        if (wait_expired(t0, waiter.limit_ns)) {
          if (atomicCAS(waiter.status, 0u, static_cast<uint32_t>(kStatusTailFlagWait)) == 0u) {
            waiter.status[1] = blockIdx.x;
            waiter.status[2] = static_cast<uint32_t>(tile);
            waiter.status[3] = 0u;
          }
          *waiter.abort_flag = 1u;
          ok = 0;
          break;
        }
      }
    }
  }
  ok = __shfl_sync(0xffffffffu, ok, 0);
  __syncwarp();  // the other lanes' reads of the partial tile come after lane 0's acquire (the warp barrier orders memory among its lanes)
  return ok != 0;
}

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

// One unit of work for a CTA (pair): a tile, a K range of it, and what to do with the result.
struct WorkItem {
  int tile;
  int kb0;    // first K block
  int nkb;    // K blocks to accumulate
  int split;  // split-K partition (results go to the split-K workspace), 0 otherwise
  int part;   // tail split: -1 = whole tile, 0 = owner, > 0 = contributor
  int tail_index;  // index of the tile among the tail tiles
};

__device__ __forceinline__ int num_work_items(const Params& p) {
  if (p.split_k > 1) return p.num_tiles * p.split_k;
  return p.tail_parts > 1 ? p.num_tiles - p.tail_tiles + p.tail_tiles * p.tail_parts : p.num_tiles;
}

__device__ __forceinline__ WorkItem decode_item(const Params& p, int item) {
  WorkItem w;
  w.split = 0;
  w.part = -1;
  w.tail_index = 0;
  if (p.split_k > 1) {
    w.tile = item / p.split_k;
    w.split = item - w.tile * p.split_k;
    w.kb0 = w.split * p.num_kb;
    w.nkb = p.num_kb;
    return w;
  }
  // The split tiles come FIRST: their parts start together on neighbouring units, and the
  // exchange of partial sums (flags, L2 round trips) then runs in the epilogue warps while the
  // units' MMA warps are already on their next, whole tiles.  Scheduled last, the same exchange
  // sat exposed at the end of the launch.
  const int tail_items = p.tail_parts > 1 ? p.tail_tiles * p.tail_parts : 0;
  const int whole = p.num_tiles - (p.tail_parts > 1 ? p.tail_tiles : 0);
  if (item >= tail_items) {
    w.tile = item - tail_items;
    w.kb0 = 0;
    w.nkb = p.num_kb;
    return w;
  }
  const int t = item;
  w.tail_index = t / p.tail_parts;
  w.part = t - w.tail_index * p.tail_parts;
  w.tile = whole + w.tail_index;
  if (w.part == 0) {
    w.kb0 = 0;
    w.nkb = p.tail_kb0;
  } else {
    w.kb0 = p.tail_kb0 + (w.part - 1) * p.tail_kb;
    w.nkb = min(p.tail_kb, p.num_kb - w.kb0);
  }
  return w;
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
// entirely inside the matrix; `wide_ok`: it is 32-byte aligned as well.
template <typename OutT>
__device__ __forceinline__ void store_row32(OutT* dst, const float (&x)[32], bool vec_ok, int valid, bool wide_ok = false) {
  if (vec_ok) {
    if constexpr (sizeof(OutT) == 4) {
      if (wide_ok) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          sm100::st_global_v8(dst + 8 * j, __float_as_uint(x[8 * j]), __float_as_uint(x[8 * j + 1]), __float_as_uint(x[8 * j + 2]),
                              __float_as_uint(x[8 * j + 3]), __float_as_uint(x[8 * j + 4]), __float_as_uint(x[8 * j + 5]),
                              __float_as_uint(x[8 * j + 6]), __float_as_uint(x[8 * j + 7]));
        }
      } else {
        float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
        for (int j = 0; j < 8; ++j) d4[j] = make_float4(x[4 * j], x[4 * j + 1], x[4 * j + 2], x[4 * j + 3]);
      }
    } else {
      uint32_t w[16];
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * t], x[2 * t + 1]);
        w[t] = *reinterpret_cast<uint32_t*>(&h);
      }
      if (wide_ok) {
        sm100::st_global_v8(dst, w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]);
        sm100::st_global_v8(dst + 16, w[8], w[9], w[10], w[11], w[12], w[13], w[14], w[15]);
      } else {
        uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
        for (int j = 0; j < 4; ++j) d4[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
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

// CG = 1: one CTA owns a 128 x BN tile.  CG = 2: a CTA pair (cluster of two) owns a 256 x BN
// tile; CTA r of the pair stages rows [128 r, 128 r + 128) of the A tile and rows
// [BN/2 r, BN/2 r + BN/2) of the B tile, the leader (r = 0) issues tcgen05.mma.cta_group::2
// for both, and each CTA ends up with its 128 rows x BN columns of the accumulator in its own
// tensor memory.  The pair halves the B bytes each SM must stage per flop, which buys deeper
// rings in the same shared memory.  In the pair, full[] lives in the leader and counts the
// bytes of both CTAs' copies; empty[] and acc_full[] exist in both CTAs and the leader's
// commits arrive on each; acc_empty[] lives in the leader and collects both CTAs' epilogues.
template <int BN, typename OutT, int CG, bool MX = false, int AM = kBM>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb, const Params p) {
#if defined(__CUDA_ARCH_FEAT_SM100_ALL)
  using namespace sm100;
  static_assert(BN == 32 || BN == 64 || BN == 128 || BN == 256, "unsupported tile width");
  static_assert(CG == 1 || CG == 2, "one CTA or a CTA pair");
  constexpr uint32_t kBRows = BN / CG;  // B rows staged by this CTA
  static_assert(AM == kBM || (CG == 1 && !MX && (AM == 32 || AM == 64)), "short A stages: one CTA, plain operands, 32 or 64 rows");
  constexpr uint32_t kABytes = AM * kRowBytes;
  constexpr uint32_t kBBytes = kBRows * kRowBytes;
  constexpr uint32_t kStageBytes = stage_bytes(BN, CG, MX, AM);
  constexpr uint32_t kLoadBytes = kABytes + kBBytes + (MX ? kScaleBlockBytes * (1 + BN / 128) : 0);  // bytes one CTA copies per stage
  constexpr uint32_t kTmemCols = tmem_columns(BN, MX);
  // Block-scaled tiles of 256 columns keep a single accumulator: two of them would fill the
  // 512 TMEM columns and leave none for the scales (the epilogue then does not overlap the next
  // main loop, which costs less than the shared-memory bound of a 128-column tile).
  constexpr int kAccBufs = (MX && BN == 256) ? 1 : 2;
  static_assert(!MX || BN == 128 || BN == 256, "block-scaled tiles are 128 or 256 columns wide");
  static_assert(!MX || kAccBufs * BN + 2 * kScaleTmemCols <= 512, "accumulators and scales share the 512 columns");
  constexpr int kTileM = kBM * CG;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_raw_u32 = smem_u32(smem_raw);
  const uint32_t smem_base = (smem_raw_u32 + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
  const uint32_t bar_base = smem_base + static_cast<uint32_t>(p.stages) * kStageBytes + a_overrun_bytes(BN, CG, MX, AM);
  uint8_t* bar_ptr = smem_raw + (bar_base - smem_raw_u32);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 128u + 8u * s; };
  auto acc_full_bar = [&](int a) { return bar_base + 256u + 8u * a; };
  auto acc_empty_bar = [&](int a) { return bar_base + 272u + 8u * a; };
  auto xchg_bar = [&](int q) { return bar_base + 320u + 8u * q; };
  const uint32_t drain_bar = bar_base + 288u;
  const uint32_t tmem_slot = bar_base + 296u;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(bar_ptr + 296);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bar_ptr + 300);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  long long t_cycles = 0;
  unsigned long long t_ns = 0;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    t_cycles = clock64();
    t_ns = globaltimer_ns();
  }
  if (threadIdx.x == 0) stamp(p, 0);
  const Waiter waiter{abort_flag, p.status, p.wait_limit_ms != 0 ? p.wait_limit_ms * 1000000ull : kWaitTimeoutNs};
  const int num_items = num_work_items(p);
  const uint32_t cta_rank = CG == 2 ? cluster_ctarank() : 0u;  // position in the pair
  const bool leader = cta_rank == 0u;
  const int first_item = static_cast<int>(blockIdx.x) / CG;    // one work item per CTA (pair) at a time
  const int item_stride = static_cast<int>(gridDim.x) / CG;

  // B tile of ring slot `stg` for K block `kb_abs` (called by the producer's elected lane).
  auto issue_b = [&](int stg, int n_blk_, int b_row_, int kb_abs) {
    const uint32_t b_dst = smem_base + stg * kStageBytes + kABytes;
    const int k_elem = kb_abs * p.kb_elems;
    if constexpr (CG == 1) {
      if (p.b_packed != nullptr) {
        const size_t blk = static_cast<size_t>(n_blk_) * (static_cast<size_t>(p.num_kb) * p.split_k) + kb_abs;
        bulk_load_1d(b_dst, static_cast<const uint8_t*>(p.b_packed) + blk * kBBytes, kBBytes, full_bar(stg));
      } else {
        tma_load_2d(b_dst, &tmap_b, full_bar(stg), k_elem, b_row_);
      }
    } else {
      tma_load_2d_pair(b_dst, &tmap_b, map_to_cta(full_bar(stg), 0u), k_elem, b_row_);
    }
  };
  // Arm the slot's barrier with the bytes of all copies of the stage (both CTAs' in a pair,
  // where every copy completes on the leader's barrier).
  auto arm = [&](int stg) {
    if constexpr (CG == 1) {
      mbar_arrive_expect_tx(full_bar(stg), kLoadBytes);
    } else {
      if (leader) mbar_arrive_expect_tx(full_bar(stg), 2u * kLoadBytes);
    }
  };
  // Static B (a weight matrix that nothing earlier in the stream writes): the producer warp
  // requests the first ring of B tiles before the previous kernel of the stream has completed;
  // everything else (A, scales, all writes) comes after griddep_wait.  Returns the slots armed.
  auto request_first_ring = [&]() -> int {
    int n = 0;
    if ((p.debug_mode & 8) == 0 && !bringup_mode(p, 3) && first_item < num_items) {
      const WorkItem w = decode_item(p, first_item);
      int m_blk, n_blk;
      tile_coords(p, w.tile, m_blk, n_blk);
      const int b_row = n_blk * BN + static_cast<int>(cta_rank * kBRows);
      n = min(p.stages, w.nkb);
      if (elect_one()) {
        stamp(p, 3);
        for (int kb = 0; kb < n; ++kb) {
          arm(kb);
          issue_b(kb, n_blk, b_row, w.kb0 + kb);
        }
      }
      __syncwarp();
    }
    return n;
  };
  int pre = 0;  // ring slots whose B tile is already on its way when the producer loop starts

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), kEpilogueWarps * CG);
    }
    mbar_init(drain_bar, 1);
    if constexpr (CG == 1) {
      if (p.cluster_exchange != 0) {
        for (int q = 0; q < kEpilogueWarps; ++q) mbar_init(xchg_bar(q), static_cast<uint32_t>(p.tail_parts - 1));  // the same warp of every other part
      }
    }
    *abort_flag = 0u;
    fence_barrier_init();
    fence_proxy_async_smem();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
    if constexpr (MX) {
      prefetch_tensormap(&tmap_sfa);
      prefetch_tensormap(&tmap_sfb);
    }
  }
  if constexpr (CG == 1) {
    // One CTA per tile: the full[] barriers are this CTA's own, so the request can go out right
    // behind their initialisation (same warp), ahead of the TMEM allocation and the barriers below.
    if (warp == 0 && p.static_b != 0) {
      __syncwarp();
      pre = request_first_ring();
    }
  }
  if (warp == 1) tmem_alloc<CG>(tmem_slot, kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  // the peers' barriers exist before anyone signals them
  if constexpr (CG == 2) {
    cluster_sync_all();
  } else {
    if (p.cluster_exchange != 0) cluster_sync_all();
  }
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;
  // Everything above touched only this CTA's shared and tensor memory.  From here on global
  // memory is read and written, so the previous kernel of the stream must be complete; the next
  // one may already set itself up behind this one (it waits at this same point).
  if (threadIdx.x == 0) stamp(p, 1);
  griddep_launch_dependents();
  if (bringup_mode(p, 128)) {
    // measures what the dependence on the previous kernel costs; only valid when nothing in the stream writes A, B or reads C
  } else if (CG == 1 || warp != 0 || p.static_b == 0) griddep_wait();  // the producer of a static-B pair plan waits after its early B requests
  if (threadIdx.x == 32) stamp(p, 2);

  if (warp == 0) {
    // ------------------------------- producer -------------------------------
    // The whole warp walks the loop (every lane polls the barrier); one elected lane issues.
    if constexpr (CG == 2) {
      if (p.static_b != 0) {
        pre = request_first_ring();  // the follower's copies complete on the leader's barriers: only after the cluster barrier
        griddep_wait();
      }
    }
    int stage = 0;
    uint32_t phase = 0;
    long long issued = 0;
    bool ok = true;
    for (int item = first_item; ok && item < num_items; item += item_stride) {
      const WorkItem w = decode_item(p, item);
      const int tile = w.tile;
      int m_blk, n_blk;
      tile_coords(p, tile, m_blk, n_blk);
      const int kb0 = w.kb0;
      const int a_row = m_blk * kTileM + static_cast<int>(cta_rank) * kBM;
      const int b_row = n_blk * BN + static_cast<int>(cta_rank * kBRows);
      for (int kb = 0; kb < w.nkb; ++kb) {
        if (!waiter.wait(empty_bar(stage), phase ^ 1u, kStatusProducerEmptyWait, tile, kb)) {
          ok = false;
          break;
        }
        const bool b_requested = item == first_item && kb < pre;  // armed and B on its way since before the wait
        if (elect_one()) {
          if (issued == 0 && pre == 0) stamp(p, 3);
          const uint32_t a_dst = smem_base + stage * kStageBytes;
          const uint32_t b_dst = a_dst + kABytes;
          const int k_elem = (kb0 + kb) * p.kb_elems;
          // Block-scaled stages: scale blocks behind the operand tiles.  Every CTA takes the block
          // of its own 128 rows of A and the blocks of all BN columns of B.  K stages beyond the
          // data (split-K padding) carry zero-filled operands, so any scale will do there.
          [[maybe_unused]] const uint32_t sf_dst = b_dst + kBBytes;
          [[maybe_unused]] const int ks = min(kb0 + kb, p.sf_k_stages - 1);
          [[maybe_unused]] const int sfa_blk = m_blk * CG + static_cast<int>(cta_rank);
          [[maybe_unused]] const int sfb_blk = n_blk * (BN / 128);
          if (p.debug_mode & 8) {
            // injected fault: the stage is never handed over, so the consumer's wait must run out
          } else if (kBringup && (p.debug_mode & 3) == 1) {
            if (leader) mbar_arrive(full_bar(stage));
          } else if constexpr (CG == 1) {
            if (!b_requested) arm(stage);
            if constexpr (MX) {
              tma_load_2d(sf_dst, &tmap_sfa, full_bar(stage), 0, sfa_blk * p.sf_k_stages + ks);
#pragma unroll
              for (int q = 0; q < BN / 128; ++q) {
                tma_load_2d(sf_dst + (1 + q) * kScaleBlockBytes, &tmap_sfb, full_bar(stage), 0, (sfb_blk + q) * p.sf_k_stages + ks);
              }
            }
            tma_load_2d(a_dst, &tmap_a, full_bar(stage), k_elem, a_row);
            if (!b_requested) issue_b(stage, n_blk, b_row, kb0 + kb);
          } else {
            // Both CTAs' copies complete on the leader's barrier, which the leader arms with
            // the byte count of the pair.
            const uint32_t leader_full = map_to_cta(full_bar(stage), 0u);
            if (!b_requested) arm(stage);
            if constexpr (MX) {
              tma_load_2d_pair(sf_dst, &tmap_sfa, leader_full, 0, sfa_blk * p.sf_k_stages + ks);
#pragma unroll
              for (int q = 0; q < BN / 128; ++q) {
                tma_load_2d_pair(sf_dst + (1 + q) * kScaleBlockBytes, &tmap_sfb, leader_full, 0, (sfb_blk + q) * p.sf_k_stages + ks);
              }
            }
            tma_load_2d_pair(a_dst, &tmap_a, leader_full, k_elem, a_row);
            if (!b_requested) issue_b(stage, n_blk, b_row, kb0 + kb);
          }
        }
        __syncwarp();
        ++issued;
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    if (!ok && leader) {
      // Aborting: let the copies already issued land before the CTA may exit.
      for (int s = 0; s < p.stages; ++s) {
        if (issued > s) {
          const long long last = (issued - 1) - ((issued - 1 - s) % p.stages);  // last issue into slot s
          waiter.wait(full_bar(s), static_cast<uint32_t>((last / p.stages) & 1), 0u, 0, 0, kDrainTimeoutNs);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader CTA only) -------------------------------
    if (leader) {
      // Everything the per-stage path needs is kept in registers and advanced incrementally:
      // the issuing thread's own instruction latency between two stages is on the critical path.
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      const uint32_t desc_hi = smem_desc_hi_sw128();
      const uint32_t a_lo0 = smem_desc_lo(smem_base);
      const uint32_t b_off = kABytes >> 4;
      uint32_t a_lo = a_lo0;
      uint32_t full_addr = full_bar(0);
      uint32_t empty_addr = empty_bar(0);
      const uint32_t peer_delta = CG == 2 ? map_to_cta(bar_base, 1u) - bar_base : 0u;  // same offset in the peer CTA
      const bool do_mma = !(kBringup && (p.debug_mode & 3) == 2);
      const int mma_kind = p.mma_kind;
      const uint32_t idesc = p.idesc;
      [[maybe_unused]] uint32_t sf_set = 0;
      const int stages = p.stages;
      bool first_stage = true;
      for (int item = first_item; ok && item < num_items; item += item_stride) {
        const WorkItem w = decode_item(p, item);
        const int tile = w.tile;
        const int num_kb = w.nkb;
        if (!waiter.wait(acc_empty_bar(acc), acc_phase ^ 1u, kStatusMmaAccEmptyWait, tile, 0)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!waiter.wait(full_addr, phase, kStatusMmaFullWait, tile, kb)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (first_stage) {
            first_stage = false;
            if (lane == 0) stamp(p, 4);
          }
          if (elect_one()) {
            if constexpr (MX) {
              // Scales of this stage: shared memory -> TMEM (alternating column sets), then the
              // four block-scaled MMAs; tcgen05 operations of one thread execute in order.
              const uint32_t sf_smem = smem_base + static_cast<uint32_t>(stage) * kStageBytes + kABytes + kBBytes;
              const uint32_t sf_tmem = tmem_base + static_cast<uint32_t>(kAccBufs * BN) + sf_set * kScaleTmemCols;  // behind the accumulators
              if (do_mma) umma_mx_stage<CG, BN / 128>(tmem_d, a_lo, a_lo + b_off, desc_hi, idesc, kb != 0 ? 1u : 0u, sf_tmem, smem_desc_lo_scales(sf_smem));
            } else {
              if (do_mma) umma_stage<CG>(tmem_d, a_lo, a_lo + b_off, desc_hi, idesc, kb != 0 ? 1u : 0u, mma_kind);
            }
            umma_commit<CG>(empty_addr);
            if constexpr (CG == 2) umma_commit<CG>(empty_addr + peer_delta);
          }
          __syncwarp();
          if constexpr (MX) sf_set ^= 1u;
          ++stage;
          a_lo += kStageBytes >> 4;
          full_addr += 8u;
          empty_addr += 8u;
          if (stage == stages) {
            stage = 0;
            phase ^= 1u;
            a_lo = a_lo0;
            full_addr = full_bar(0);
            empty_addr = empty_bar(0);
          }
        }
        if (!ok) break;
        if (elect_one()) {
          umma_commit<CG>(acc_full_bar(acc));
          if constexpr (CG == 2) umma_commit<CG>(acc_full_bar(acc) + peer_delta);
        }
        __syncwarp();
        if (lane == 0) {
          stamp(p, 5);  // overwritten per item: the last one stays
          const int nth = (item - first_item) / item_stride;
          if (nth < 7) stamp(p, 9 + nth);  // commit time of this CTA's first seven work items
        }
        acc = (acc + 1) % kAccBufs;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (!ok) {
        // Aborting: wait for the MMAs already issued before TMEM and shared memory go away.
        if (elect_one()) umma_commit<CG>(drain_bar);
        __syncwarp();
        waiter.wait(drain_bar, 0u, 0u, 0, 0, kDrainTimeoutNs);
      }
    }
  } else {
    // ------------------------------- epilogue -------------------------------
    const int quarter = warp & 3;  // TMEM lanes this warp may read
    // One warp per lane quarter.  (Two warps per quarter, each taking half of the columns, made
    // every launch slower: the tail of a launch is bound by the rate of store requests, not by
    // the number of epilogue chains, and the extra warps cost registers and power.)
    constexpr int c_begin = 0;
    constexpr int c_end = BN;
    const int row_in_tile = static_cast<int>(cta_rank) * kBM + quarter * 32 + lane;
    float alpha = 1.0f;
    if (p.scale_a != nullptr) alpha *= __ldg(p.scale_a);
    if (p.scale_b != nullptr) alpha *= __ldg(p.scale_b);
    OutT* const C = static_cast<OutT*>(p.C);
    const bool n_vec_ok = (p.N % OutVec<OutT>::kPerVec) == 0;
    const bool bias_vec_ok = (reinterpret_cast<uintptr_t>(p.bias) & 15u) == 0;  // chunks start at multiples of 32 columns
    // 32-byte stores: every row segment starts on a 32-byte boundary (chunks start at multiples of 32 columns)
    const bool n_wide_ok = (p.N % (2 * OutVec<OutT>::kPerVec)) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 31u) == 0 && !bringup_mode(p, 64);
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int item = first_item; ok && item < num_items; item += item_stride) {
      const WorkItem w = decode_item(p, item);
      const int tile = w.tile;
      const int split = w.split;
      int m_blk, n_blk;
      tile_coords(p, tile, m_blk, n_blk);
      // A CTA with a single work item has no later main loop for this wait to hide behind: poll
      // tightly there (the launch ends with this epilogue); otherwise sleep between polls.
      if (!waiter.wait_relaxed(acc_full_bar(acc), acc_phase, kStatusEpilogueAccFullWait, tile, num_items <= item_stride ? 20u : 256u)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      if (warp == 2 && lane == 0) stamp(p, 6);  // overwritten per item: the last one stays
      [[maybe_unused]] long long epi_c0 = 0;
      if constexpr (kBringup) epi_c0 = clock64();
      const int row = m_blk * kTileM + row_in_tile;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN);
      float bias_row = 0.0f;
      if (p.bias != nullptr && p.bias_axis == 1 && row_ok) bias_row = __ldg(p.bias + row);
      // Tail split: partial tiles travel in "register image" order -- for each 32-column chunk,
      // float4 j of lane l sits at [warp slab][chunk][j][l] -- because the contributor and the
      // owner use the same lane <-> (row, column) mapping.  Every exchange access is therefore a
      // fully coalesced 512-byte warp access; a row-major exchange was 8x slower end to end.
      const size_t tail_tile_elems = static_cast<size_t>(kTileM) * BN;
      const int flag_lane = static_cast<int>(cta_rank) * 4 + quarter;  // one flag per epilogue warp
      const size_t warp_slab = static_cast<size_t>(static_cast<int>(cta_rank) * 4 + quarter) * (32u * BN);  // floats per lane quarter = 32 rows x BN
      // A warp whose 32 rows all lie beyond M has nothing to read, exchange or store.
      const bool slab_ok = (m_blk * kTileM + static_cast<int>(cta_rank) * kBM + quarter * 32) < p.M;
      const bool exchange = !bringup_mode(p, 4) && slab_ok;
      // Tail split: the parts of a tile (equal K ranges on different units) each finish one
      // slice of its columns.  A part first exports its partial sums for the *other* parts'
      // slices, raises its flag, waits for the others' flags and then adds their partial sums
      // to its own slice -- a reduce-scatter among the parts.  Every unit exchanges and
      // finishes 1/parts of the tile, where a single owner used to read and finish all of it.
      const bool tail_item = w.part >= 0;
      int lo = c_begin, hi = slab_ok ? c_end : c_begin;  // the columns this warp finishes
      const size_t part_stride4 = tail_tile_elems / 4;   // float4 per partial tile
      float4* const tile_regions = reinterpret_cast<float4*>(p.tail_ws + static_cast<size_t>(w.tail_index) * p.tail_parts * tail_tile_elems + warp_slab) + lane;
      uint32_t* const tile_flags = p.tail_flags + static_cast<size_t>(w.tail_index) * p.tail_parts * (CG * 4) + flag_lane;
      // Cluster exchange: this lane's float4 column of this warp's slab in the CTA's own parking
      // area, the start of the (by now idle) stage ring; same "register image" order.
      bool via_cluster = false;
      if constexpr (CG == 1) via_cluster = p.cluster_exchange != 0;
      const uint32_t park = smem_base + static_cast<uint32_t>(quarter) * (32u * BN * 4u) + static_cast<uint32_t>(lane) * 16u;
      // float4 j of chunk c of part q's partial sums for this lane.
      auto partial = [&](int q, int c, int j) -> float4 {
        if (via_cluster) return ld_shared_cluster_f4(map_to_cta(park, static_cast<uint32_t>(q)) + static_cast<uint32_t>(c * 8 + j * 32) * 16u);
        return __ldcg(tile_regions + static_cast<size_t>(q) * part_stride4 + static_cast<size_t>(c) * 8u + j * 32);
      };
      if (tail_item) {
        const int slice = BN / p.tail_parts;  // a multiple of 32 (the plan sees to it)
        lo = w.part * slice;
        hi = slab_ok ? lo + slice : lo;
        if (exchange && via_cluster) {
          // The accumulator is complete, so every stage of the ring has been consumed and nothing
          // more is on its way into it (one work item per CTA): park the other parts' slices there.
#pragma unroll 1
          for (int c = 0; c < BN; c += 32) {
            if ((c >= lo && c < lo + slice) || n_blk * BN + c >= p.N) continue;  // own slice, or beyond the matrix
            uint32_t v[32];
            tmem_ld_32x32b_x32(taddr + static_cast<uint32_t>(c), v);
            tmem_ld_wait();
            const uint32_t dst = park + static_cast<uint32_t>(c) * 128u;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              st_shared_f4(dst + j * 512u, __uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]),
                           __uint_as_float(v[4 * j + 3]));
            }
          }
          // Publish to the same warp of every other part (release at cluster scope, cumulative over
          // what the warp barrier made lane 0 observe), then wait for theirs.
          __syncwarp();
          if (lane == 0) {
            for (int q = 0; q < p.tail_parts; ++q) {
              if (q != w.part) mbar_arrive_remote(map_to_cta(xchg_bar(quarter), static_cast<uint32_t>(q)));
            }
          }
          if (!waiter.template wait_relaxed<true>(xchg_bar(quarter), 0u, kStatusClusterExchangeWait, tile, 32u)) {
            ok = false;
            break;
          }
        } else if (exchange) {
          float4* const mine = tile_regions + static_cast<size_t>(w.part) * part_stride4;
#pragma unroll 1
          for (int c = 0; c < BN; c += 32) {
            if ((c >= lo && c < lo + slice) || n_blk * BN + c >= p.N) continue;  // own slice, or beyond the matrix
            uint32_t v[32];
            tmem_ld_32x32b_x32(taddr + static_cast<uint32_t>(c), v);
            tmem_ld_wait();
            float4* wdst = mine + static_cast<size_t>(c) * 8u;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              wdst[j * 32] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]),
                                         __uint_as_float(v[4 * j + 3]));
            }
          }
          // Publish: the warp barrier orders every lane's stores before lane 0's release of the
          // flag the other parts poll (a release is cumulative over what its thread has observed).
          __syncwarp();
          if (lane == 0) st_release_gpu(tile_flags + static_cast<size_t>(w.part) * (CG * 4), p.epoch);
          for (int q = 0; q < p.tail_parts; ++q) {
            if (q == w.part) continue;
            if (!wait_flag(tile_flags + static_cast<size_t>(q) * (CG * 4), p.epoch, waiter, tile)) {
              ok = false;
              break;
            }
          }
          if (!ok) break;
        }
      }
      // This lane's float4 column of the first other part's partial tile; its first chunk is loaded now.
      const int first_other = w.part == 0 ? 1 : 0;
      float4 ahead[8];
      if (tail_item && exchange && lo < hi) {
#pragma unroll
        for (int j = 0; j < 8; ++j) ahead[j] = partial(first_other, lo, j);
      }
      // Whole tiles of a floating-point product (no K split of any kind, at least 64 columns) take
      // a leaner path: 64 columns per TMEM load and wait, i.e. two independent conversion and
      // store chains per iteration and half the loop trips.  An epilogue warp is a serial chain
      // on one scheduler; this is the cheap way to give it instruction-level parallelism.
      if constexpr (BN >= 64) {
        if (!tail_item && p.split_k <= 1 && p.acc_int == 0 && !bringup_mode(p, 64)) {
#pragma unroll 1
          for (int c = 0; c < (slab_ok ? BN : 0); c += 64) {
            uint32_t v[64];
            tmem_ld_32x32b_x64(taddr + static_cast<uint32_t>(c), v);
            tmem_ld_wait();
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int col0 = n_blk * BN + c + 32 * h;
              if (col0 >= p.N) continue;  // warp-uniform
              const int valid = min(32, p.N - col0);
              float x[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(v[32 * h + j]);
              if (alpha != 1.0f) {
#pragma unroll
                for (int j = 0; j < 32; ++j) x[j] *= alpha;
              }
              if (p.bias != nullptr) {
                if (p.bias_axis == 0) {
                  if (valid == 32 && bias_vec_ok) {
                    const float4* b4 = reinterpret_cast<const float4*>(p.bias + col0);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                      const float4 t = __ldg(b4 + j);
                      x[4 * j] += t.x;
                      x[4 * j + 1] += t.y;
                      x[4 * j + 2] += t.z;
                      x[4 * j + 3] += t.w;
                    }
                  } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) x[j] += (j < valid) ? __ldg(p.bias + col0 + j) : 0.0f;
                  }
                } else {
#pragma unroll
                  for (int j = 0; j < 32; ++j) x[j] += bias_row;
                }
              }
              if (p.relu) {
#pragma unroll
                for (int j = 0; j < 32; ++j) x[j] = fmaxf(x[j], 0.0f);
              }
              if (row_ok && !bringup_mode(p, 32)) {
                store_row32<OutT>(C + static_cast<size_t>(row) * p.N + col0, x, n_vec_ok && valid == 32, valid, n_wide_ok);
              }
            }
          }
          lo = hi;  // nothing left for the general loop below
        }
      }
      // One 32-column chunk of this warp's rows per iteration.  (Keeping the next chunk's TMEM
      // load in flight during the current one was tried twice: with two 32-column register sets
      // the compiler spills, which is not an option for registers that an asynchronous load is
      // still writing; with two 16-column sets it fits, but a tile's epilogue only went from 3.9
      // to 3.6 us -- the time is in issuing the conversion and store instructions, not in the
      // TMEM load latency.)
#pragma unroll 1
      for (int c = lo; c < hi; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(taddr + static_cast<uint32_t>(c), v);
        tmem_ld_wait();
        float x[32];
        if (p.acc_int == 1) {
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] = static_cast<float>(static_cast<int>(v[j]));
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(v[j]);
        }
        const int col0 = n_blk * BN + c;
        if (col0 >= p.N) continue;  // warp-uniform
        const int valid = min(32, p.N - col0);
        if (p.split_k > 1) {
          // Partial sums go to the workspace untouched; the reduction applies the epilogue.
          if (row_ok) {
            float* wdst = p.workspace + (static_cast<size_t>(split) * p.M + row) * p.N + col0;
            store_row32<float>(wdst, x, (p.N % 4) == 0 && valid == 32, valid);
          }
          continue;
        }
        if (p.acc_int == 2) {
          // Integer sums (never part of a K split: the plan refuses it) are moved, not converted:
          // C receives the s32 words bit for bit.
          if (row_ok) store_row32<OutT>(C + static_cast<size_t>(row) * p.N + col0, x, n_vec_ok && valid == 32, valid);
          continue;
        }
        if (tail_item && exchange) {
          // The first other part's chunk was fetched one iteration ahead (`ahead`); further
          // parts, if any, are read in place, in increasing part order.
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            x[4 * j] += ahead[j].x;
            x[4 * j + 1] += ahead[j].y;
            x[4 * j + 2] += ahead[j].z;
            x[4 * j + 3] += ahead[j].w;
          }
          if (c + 32 < hi) {
#pragma unroll
            for (int j = 0; j < 8; ++j) ahead[j] = partial(first_other, c + 32, j);
          }
          for (int q = first_other + 1; q < p.tail_parts; ++q) {
            if (q == w.part) continue;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 t = partial(q, c, j);
              x[4 * j] += t.x;
              x[4 * j + 1] += t.y;
              x[4 * j + 2] += t.z;
              x[4 * j + 3] += t.w;
            }
          }
          // This chunk of the other parts' partial sums has been consumed and nobody reads it again:
          // drop its lines from the L2 instead of letting them be written back to DRAM on eviction.
          // (Every j covers 512 contiguous bytes of the warp: four 128-byte lines, one per eighth lane.)
          if (!via_cluster && (lane & 7) == 0) {
            for (int q = 0; q < p.tail_parts; ++q) {
              if (q == w.part) continue;
              const float4* base = tile_regions + static_cast<size_t>(q) * part_stride4 + static_cast<size_t>(c) * 8u;
#pragma unroll
              for (int j = 0; j < 8; ++j) discard_l2_line(base + j * 32);
            }
          }
        }
        if (alpha != 1.0f) {  // warp-uniform; the plain product skips 32 multiplies per chunk
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] *= alpha;
        }
        if (p.bias != nullptr) {
          if (p.bias_axis == 0) {
            if (valid == 32 && bias_vec_ok) {
              // every lane needs the same 32 bias values: eight 16-byte loads instead of 32 scalar ones
              const float4* b4 = reinterpret_cast<const float4*>(p.bias + col0);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float4 t = __ldg(b4 + j);
                x[4 * j] += t.x;
                x[4 * j + 1] += t.y;
                x[4 * j + 2] += t.z;
                x[4 * j + 3] += t.w;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) x[j] += (j < valid) ? __ldg(p.bias + col0 + j) : 0.0f;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) x[j] += bias_row;
          }
        }
        if (p.relu) {
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] = fmaxf(x[j], 0.0f);
        }
        if (row_ok && !bringup_mode(p, 32)) {
          store_row32<OutT>(C + static_cast<size_t>(row) * p.N + col0, x, n_vec_ok && valid == 32, valid, n_wide_ok);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (CG == 1) {
          mbar_arrive(acc_empty_bar(acc));
        } else {
          mbar_arrive_remote(map_to_cta(acc_empty_bar(acc), 0u));
        }
      }
      acc = (acc + 1) % kAccBufs;
      if (acc == 0) acc_phase ^= 1u;
      if (warp == 2 && lane == 0) {
        stamp(p, 7);  // overwritten per item: the last one stays
#ifdef B200_BRINGUP
        if (p.timeline != nullptr) p.timeline[static_cast<size_t>(blockIdx.x) * 16 + 12] = static_cast<unsigned long long>(clock64() - epi_c0);
#endif
      }
    }
  }

  // ------------------------------- teardown -------------------------------
  tc_fence_before_sync();
  __syncthreads();
  // no CTA leaves while another of its cluster may still signal it or read its shared memory
  if constexpr (CG == 2) {
    cluster_sync_all();
  } else {
    if (p.cluster_exchange != 0) cluster_sync_all();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<CG>(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0) stamp(p, 8);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    const unsigned long long cyc = static_cast<unsigned long long>(clock64() - t_cycles);
    const unsigned long long ns = globaltimer_ns() - t_ns;
    p.status[4] = static_cast<uint32_t>(cyc);
    p.status[5] = static_cast<uint32_t>(cyc >> 32);
    p.status[6] = static_cast<uint32_t>(ns);
    p.status[7] = static_cast<uint32_t>(ns >> 32);
    // Running totals over all launches that used these status words: the host takes differences
    // around a timed region and gets the average SM clock of exactly the launches it timed.
    atomicAdd(reinterpret_cast<unsigned long long*>(p.status + 8), cyc);
    atomicAdd(reinterpret_cast<unsigned long long*>(p.status + 10), ns);
    atomicAdd(p.status + 12, 1u);
  }
#endif
}

// Split-K reduction + epilogue: C = epilogue(sum_s workspace[s]).  HBM-bound, 16-byte accesses.
template <typename OutT>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const Params p) {
  // A main kernel whose bounded wait gave up did not write all of its partial sums: leave C alone
  // rather than reduce whatever an earlier launch left in the workspace.
  if (*reinterpret_cast<const volatile uint32_t*>(p.status) != kStatusOk) return;
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
