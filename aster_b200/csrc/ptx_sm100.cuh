// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the GEMM kernels use:
// mbarrier, TMA (cp.async.bulk[.tensor]), tcgen05 (TMEM allocation, MMA, commit, load) and the
// shared-memory / instruction descriptors tcgen05.mma consumes.  Device code only.
#pragma once

#include <cstdint>

namespace sm100 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// True in exactly one lane of a fully converged warp (the same lane every time).  Code that
// issues TMA or tcgen05 instructions from one thread runs its loops warp-uniformly and guards
// only the issue with this, so the compiler sees a converged warp around the instruction.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "elect.sync _|p, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---------------------------------------------------------------------------------------------
// global-memory flags between CTAs of one launch
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Drop a 128-byte line from the L2 without writing it back (its contents become undefined):
// for exchange data that has been consumed and must not cost a DRAM write when it is evicted.
__device__ __forceinline__ void discard_l2_line(const void* p) {
  asm volatile("discard.global.L2 [%0], 128;" ::"l"(p) : "memory");
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// shared::cluster address of the location at this CTA's shared-memory address `local_addr`
// inside CTA `cta_rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t cta_rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(cta_rank));
  return remote;
}
// Arrive on a barrier given by a shared::cluster address (this CTA's or a peer's).
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Cluster-wide barrier over all threads of all CTAs (release/acquire).
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// One poll with acquire semantics at cluster scope: a true answer makes visible what the
// arriving threads of OTHER CTAs of the cluster wrote to shared memory before they arrived with
// mbar_arrive_remote (release.cluster).
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// 16-byte store to this CTA's shared memory and 16-byte load from the shared memory of any CTA
// of the cluster (address from map_to_cta): the partial-sum exchange between the CTAs that
// share a tile's K range.
__device__ __forceinline__ void st_shared_f4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ float4 ld_shared_cluster_f4(uint32_t cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(cluster_addr) : "memory");
  return v;
}
// One poll of the barrier's phase (the hardware may park the thread briefly before answering).
// A longer suspend hint or single-lane polling was measured slower: the wake-up latency lands
// on the critical path of the MMA issue loop.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// ---------------------------------------------------------------------------------------------
// TMA
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
// 2-D tiled load; c0 is the innermost (contiguous) coordinate and c0 * element size must be a
// multiple of 16 bytes.  Completion is signalled as transaction bytes on `bar`.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const void* tmap, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_dst),
      "l"(tmap), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
// Same, for a CTA pair: `bar` may name the barrier of the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const void* tmap, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_dst),
      "l"(tmap), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
// 1-D bulk copy global -> shared; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_load_1d(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_dst),
               "l"(gsrc), "r"(bytes), "r"(bar)
               : "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05: tensor memory and MMA
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Whole-warp calls.  `ncols` is a power of two in [32, 512]; the base address is written to
// the shared-memory word at `smem_slot`.
template <int CTA_GROUP>
__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t ncols) {
  if constexpr (CTA_GROUP == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  } else {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
}
template <int CTA_GROUP>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (CTA_GROUP == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
  } else {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
  }
}

// Operand kinds of tcgen05.mma used here: 16-bit floats (instruction K = 16), 8-bit floats and
// 8-bit integers (K = 32: always 32 bytes of K per instruction).
enum MmaKind : int { kKindF16 = 0, kKindF8 = 1, kKindI8 = 2 };

// The four MMAs of one pipeline stage in a single instruction sequence: D (+)= A_k . B_k^T for
// the four 32-byte K slices of a 128-byte-swizzled stage.  `a_lo` / `b_lo` are the low words of
// the operands' shared-memory descriptors (start address >> 4 | LBO), `desc_hi` their common
// high word; each slice advances the low word by 2 (32 bytes).  `accumulate_first` = 0 makes
// the first MMA overwrite D.  Kept as one asm block so that nothing but two adds and two moves
// separates consecutive tcgen05.mma: the issuing thread's instruction latency between MMAs is
// what starves the tensor pipe otherwise.
#define B200_MMA_STAGE_ASM(GROUP, KIND)                                                         \
  asm volatile(                                                                                 \
      "{\n"                                                                                     \
      ".reg .pred p, q;\n"                                                                      \
      ".reg .b64 da, db;\n"                                                                     \
      ".reg .b32 la, lb;\n"                                                                     \
      "setp.ne.b32 p, %5, 0;\n"                                                                 \
      "setp.eq.b32 q, 0, 0;\n"                                                                  \
      "mov.b64 da, {%1, %3};\n"                                                                 \
      "mov.b64 db, {%2, %3};\n"                                                                 \
      "tcgen05.mma.cta_group::" GROUP ".kind::" KIND " [%0], da, db, %4, p;\n"                  \
      "add.u32 la, %1, 2;\n"                                                                    \
      "add.u32 lb, %2, 2;\n"                                                                    \
      "mov.b64 da, {la, %3};\n"                                                                 \
      "mov.b64 db, {lb, %3};\n"                                                                 \
      "tcgen05.mma.cta_group::" GROUP ".kind::" KIND " [%0], da, db, %4, q;\n"                  \
      "add.u32 la, %1, 4;\n"                                                                    \
      "add.u32 lb, %2, 4;\n"                                                                    \
      "mov.b64 da, {la, %3};\n"                                                                 \
      "mov.b64 db, {lb, %3};\n"                                                                 \
      "tcgen05.mma.cta_group::" GROUP ".kind::" KIND " [%0], da, db, %4, q;\n"                  \
      "add.u32 la, %1, 6;\n"                                                                    \
      "add.u32 lb, %2, 6;\n"                                                                    \
      "mov.b64 da, {la, %3};\n"                                                                 \
      "mov.b64 db, {lb, %3};\n"                                                                 \
      "tcgen05.mma.cta_group::" GROUP ".kind::" KIND " [%0], da, db, %4, q;\n"                  \
      "}\n" ::"r"(tmem_d),                                                                      \
      "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate_first)                     \
      : "memory")

template <int CTA_GROUP>
__device__ __forceinline__ void umma_stage(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc,
                                           uint32_t accumulate_first, int kind) {
  if constexpr (CTA_GROUP == 1) {
    if (kind == kKindF8) {
      B200_MMA_STAGE_ASM("1", "f8f6f4");
    } else if (kind == kKindI8) {
      B200_MMA_STAGE_ASM("1", "i8");
    } else {
      B200_MMA_STAGE_ASM("1", "f16");
    }
  } else {
    if (kind == kKindF8) {
      B200_MMA_STAGE_ASM("2", "f8f6f4");
    } else if (kind == kKindI8) {
      B200_MMA_STAGE_ASM("2", "i8");
    } else {
      B200_MMA_STAGE_ASM("2", "f16");
    }
  }
}
#undef B200_MMA_STAGE_ASM

// Shared-memory matrix descriptor for a K-major operand tile whose rows are 128 bytes long and
// stored with the 128-byte swizzle (the image TMA writes with CU_TENSOR_MAP_SWIZZLE_128B).
//   bits  0-13  start address >> 4          bits 16-29  leading byte offset >> 4 (1: unused here)
//   bits 32-45  stride byte offset >> 4 (8 rows * 128 B = 1024 -> 64)
//   bits 46-47  descriptor version (1 on sm_100)         bits 61-63  layout (2 = SWIZZLE_128B)
// The tile base must be 1024-byte aligned; stepping along K inside the 128-byte row adds the
// byte offset >> 4 to the start-address field.
// The descriptor is handled as its low and high 32-bit words (the high word does not depend on
// the address).
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t smem_addr) { return ((smem_addr >> 4) & 0x3FFFu) | (1u << 16); }
__device__ __forceinline__ constexpr uint32_t smem_desc_hi_sw128() { return (1024u >> 4) | (1u << 14) | (2u << 29); }

// Make `bar` (a shared::cluster address) complete one arrival once every tcgen05 operation
// previously issued by this thread has finished.
template <int CTA_GROUP>
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  if constexpr (CTA_GROUP == 1) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
  } else {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
  }
}

// Instruction descriptor, both operands K-major.
//   bits 4-5 D format (1 = f32, 2 = s32)   bits 7-9 A format   bits 10-12 B format
//   bits 17-22 N >> 3                      bits 24-28 M >> 4
// Formats: kind::f16 0 = f16, 1 = bf16; kind::f8f6f4 0 = e4m3, 1 = e5m2; kind::i8 0 = u8, 1 = s8.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t d_format, uint32_t a_format, uint32_t b_format, uint32_t umma_m,
                                                  uint32_t umma_n) {
  return (d_format << 4) | (a_format << 7) | (b_format << 10) | ((umma_n >> 3) << 17) | ((umma_m >> 4) << 24);
}

// 32-byte global store (sm_100): half as many store requests as two 16-byte stores, which is
// what bounds an epilogue whose lanes each write their own row.
__device__ __forceinline__ void st_global_v8(void* ptr, uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t e, uint32_t f,
                                             uint32_t g, uint32_t h) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "r"(a), "r"(b), "r"(c), "r"(d), "r"(e),
               "r"(f), "r"(g), "r"(h)
               : "memory");
}

// Programmatic dependent launch.  `griddep_launch_dependents` lets the next kernel of the stream
// (if it was launched with programmatic stream serialisation) start its own prologue while this
// grid is still running; `griddep_wait` blocks until every grid this one depends on has finished
// and its memory is visible.  Both do nothing in a kernel launched the ordinary way.
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- block-scaled 8-bit floats (kind::mxf8f6f4): one E8M0 scale per 32 elements of K ----
// Instruction descriptor of the block-scaled kinds (accumulators are always f32):
//   bits 4-5 scale id of B   bits 7-9 A format   bits 10-12 B format   bits 17-22 N >> 3
//   bit 23 scale format (1 = E8M0)   bits 24-28 M >> 4   bits 29-30 scale id of A
// A scale id selects one byte of the 32-bit scale column: the scales of four consecutive
// K blocks of 32 share a column, so the four MMAs of a 128-byte stage use ids 0..3.
__host__ __device__ constexpr uint32_t make_idesc_mx(uint32_t a_format, uint32_t b_format, uint32_t umma_m, uint32_t umma_n) {
  return (a_format << 7) | (b_format << 10) | ((umma_n >> 3) << 17) | (1u << 23) | ((umma_m >> 4) << 24);
}

// One block-scaled pipeline stage in a single instruction sequence: the scale blocks of the
// stage (one for A, NB for B, 512 bytes apart in shared memory starting at the block that
// `sf_lo` describes) go to TMEM columns sf_tmem (A) and sf_tmem + 4 .. (B), then the four MMAs
// of the 128-byte stage follow with scale ids 0..3.  As in umma_stage, keeping the sequence in
// one asm block keeps the issuing thread's own latency off the tensor pipe's critical path.
// Shared-memory descriptor of a scale block (low / high word): 32 rows of 16 bytes, rows
// contiguous (no swizzle, groups of 8 rows 128 bytes apart).  tcgen05.cp.32x128b.warpx4 copies
// such a block into four TMEM columns (row i -> lane i of each of the four 32-lane quarters).
__device__ __forceinline__ constexpr uint32_t smem_desc_hi_scales() { return (128u >> 4) | (1u << 14); }
__device__ __forceinline__ uint32_t smem_desc_lo_scales(uint32_t smem_addr) { return ((smem_addr >> 4) & 0x3FFFu) | (1u << 16); }

#define B200_MX_MMA(GROUP, J)                                                                   \
  "add.u32 la, %1, " #J "*2;\n"                                                                 \
  "add.u32 lb, %2, " #J "*2;\n"                                                                 \
  "add.u32 id, %4, " #J "*0x20000010;\n"                                                        \
  "mov.b64 da, {la, %3};\n"                                                                     \
  "mov.b64 db, {lb, %3};\n"                                                                     \
  "tcgen05.mma.cta_group::" GROUP ".kind::mxf8f6f4.block_scale [%0], da, db, id, [%6], [tb], q;\n"

#define B200_MX_STAGE_ASM(GROUP)                                                                \
  asm volatile(                                                                                 \
      "{\n"                                                                                     \
      ".reg .pred p, q;\n"                                                                      \
      ".reg .b64 da, db, sd;\n"                                                                 \
      ".reg .b32 la, lb, id, ls, tb, tc;\n"                                                     \
      "setp.ne.b32 p, %5, 0;\n"                                                                 \
      "mov.b64 sd, {%7, %8};\n"                                                                 \
      "tcgen05.cp.cta_group::" GROUP ".32x128b.warpx4 [%6], sd;\n"                              \
      "add.u32 ls, %7, 32;\n"                                                                   \
      "add.u32 tb, %6, 4;\n"                                                                    \
      "mov.b64 sd, {ls, %8};\n"                                                                 \
      "tcgen05.cp.cta_group::" GROUP ".32x128b.warpx4 [tb], sd;\n"                              \
      "setp.eq.b32 q, %9, 2;\n"                                                                 \
      "add.u32 ls, %7, 64;\n"                                                                   \
      "add.u32 tc, %6, 8;\n"                                                                    \
      "mov.b64 sd, {ls, %8};\n"                                                                 \
      "@q tcgen05.cp.cta_group::" GROUP ".32x128b.warpx4 [tc], sd;\n"                           \
      "setp.eq.b32 q, 0, 0;\n"                                                                  \
      "mov.b64 da, {%1, %3};\n"                                                                 \
      "mov.b64 db, {%2, %3};\n"                                                                 \
      "tcgen05.mma.cta_group::" GROUP ".kind::mxf8f6f4.block_scale [%0], da, db, %4, [%6], [tb], p;\n" \
      B200_MX_MMA(GROUP, 1) B200_MX_MMA(GROUP, 2) B200_MX_MMA(GROUP, 3) "}\n" ::"r"(tmem_d),     \
      "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate_first), "r"(sf_tmem), "r"(sf_lo), "r"(sf_hi), "r"(NB)   \
      : "memory")

// CTA_GROUP = 2: issued by the leader of a CTA pair; each tcgen05.cp then copies from the same
// shared-memory offset of both CTAs into each CTA's own TMEM (every CTA holds the scales of its
// own 128 rows of A and of all columns of the B tile).
template <int CTA_GROUP, int NB>
__device__ __forceinline__ void umma_mx_stage(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc,
                                              uint32_t accumulate_first, uint32_t sf_tmem, uint32_t sf_lo) {
  static_assert(NB == 1 || NB == 2, "one or two 128-row scale blocks of B");
  constexpr uint32_t sf_hi = smem_desc_hi_scales();
  if constexpr (CTA_GROUP == 1) {
    B200_MX_STAGE_ASM("1");
  } else {
    B200_MX_STAGE_ASM("2");
  }
}
#undef B200_MX_STAGE_ASM
#undef B200_MX_MMA

// Load 32 consecutive fp32 columns of this thread's TMEM lane (warp w may touch lanes
// 32*(w%4) .. 32*(w%4)+31; thread i of the warp reads lane base+i).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
// Same for 64 columns (two calls' worth of data behind one wait).
__device__ __forceinline__ void tmem_ld_32x32b_x64(uint32_t taddr, uint32_t (&v)[64]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
      "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
      "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31]), "=r"(v[32]),
        "=r"(v[33]), "=r"(v[34]), "=r"(v[35]), "=r"(v[36]), "=r"(v[37]), "=r"(v[38]), "=r"(v[39]), "=r"(v[40]),
        "=r"(v[41]), "=r"(v[42]), "=r"(v[43]), "=r"(v[44]), "=r"(v[45]), "=r"(v[46]), "=r"(v[47]), "=r"(v[48]),
        "=r"(v[49]), "=r"(v[50]), "=r"(v[51]), "=r"(v[52]), "=r"(v[53]), "=r"(v[54]), "=r"(v[55]), "=r"(v[56]),
        "=r"(v[57]), "=r"(v[58]), "=r"(v[59]), "=r"(v[60]), "=r"(v[61]), "=r"(v[62]), "=r"(v[63])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace sm100
