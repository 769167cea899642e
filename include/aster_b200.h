/*
 * aster_b200 C ABI: the drop-in boundary for ASTER's GEMM hot path on NVIDIA B200 (sm_100a).
 *
 * Every entry point is extern "C", takes plain pointers and sizes, returns an int status
 * (0 = B200_OK) and never throws.  The text of the most recent failure on the calling thread
 * is available from b200_last_error().  Device pointers are raw CUDA device addresses; a
 * `stream` argument is a cudaStream_t passed as void* (NULL = the legacy default stream, which
 * is what the reference runtime launches on: python/aster/execution/core.py:562-597).
 *
 * Each group cites the reference interface it stands in for (paths are relative to the
 * iree-org/aster source tree).
 */
#ifndef ASTER_B200_H_
#define ASTER_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------------ */
/* Status codes                                                                               */
/* ------------------------------------------------------------------------------------------ */
enum {
  B200_OK = 0,
  B200_ERR_INVALID = 1,     /* bad argument: shape, alignment, enum value, NULL pointer        */
  B200_ERR_CUDA = 2,        /* a CUDA runtime/driver call failed; see b200_last_error()         */
  B200_ERR_UNSUPPORTED = 3, /* valid request that this build or device cannot serve            */
  B200_ERR_TIMEOUT = 4,     /* a bounded device-side wait gave up; see b200_status_read()       */
  B200_ERR_NO_DEVICE = 5,   /* no CUDA device / not an sm_100 part                              */
  B200_ERR_WORKSPACE = 6    /* caller-provided workspace is missing or too small               */
};

/* Thread-local message of the last failing call ("" if none).  Mirrors the reference's
 * "HIP error at file:line - msg" runtime_error text (python/lib/RuntimeModule.cpp:126-134). */
const char* b200_last_error(void);
const char* b200_version(void);

/* ------------------------------------------------------------------------------------------ */
/* Runtime: stands in for the nanobind `hip_*` functions of python/lib/RuntimeModule.cpp       */
/* ------------------------------------------------------------------------------------------ */

typedef struct b200_props {
  char name[128];
  int32_t cc_major, cc_minor;
  int32_t sm_count;
  int32_t max_smem_per_block_optin; /* bytes */
  int32_t smem_per_sm;              /* bytes */
  int32_t regs_per_sm;
  int32_t l2_bytes;
  int32_t sm_clock_khz;
  int32_t mem_clock_khz;
  int32_t mem_bus_bits;
  int64_t total_mem_bytes;
} b200_props;

int b200_init(int device);                        /* hip_init                RuntimeModule.cpp:143 */
int b200_device_count(int* count);                /* hip_get_device_count    :336 */
int b200_set_device(int device);                  /* hip_set_device          :343 */
int b200_get_device(int* device);                 /* hip_get_device          :353 */
int b200_device_props(int device, b200_props* p); /* hip_get_device_props    :169 */
/* PCI bus id ("0000:3b:00.0") of a device, to find the same GPU through NVML. */
int b200_device_pci_bus_id(int device, char* buf, int len);
int b200_clear_last_error(void);                  /* hip_clear_last_error    :164 */
int b200_device_synchronize(void);                /* hip_device_synchronize  :302 */
/* hip_device_reset (:348) has no safe meaning on a shared GPU: always B200_ERR_UNSUPPORTED. */
int b200_device_reset(void);

int b200_malloc(void** dptr, size_t bytes);                         /* hip_malloc :307 */
int b200_free(void* dptr);                                          /* hip_free   :314 */
int b200_memcpy_h2d(void* dst, const void* src, size_t bytes);      /* hip_memcpy_host_to_device   :321 */
int b200_memcpy_d2h(void* dst, const void* src, size_t bytes);      /* hip_memcpy_device_to_host   :326 */
int b200_memcpy_d2d(void* dst, const void* src, size_t bytes);      /* hip_memcpy_device_to_device :331 */
int b200_memset(void* dst, int value, size_t bytes);
/* Pinned host memory, for end-to-end timing with host buffers. */
int b200_host_alloc(void** hptr, size_t bytes);
int b200_host_free(void* hptr);
int b200_memcpy_h2d_async(void* dst, const void* src, size_t bytes, void* stream);
int b200_memcpy_d2h_async(void* dst, const void* src, size_t bytes, void* stream);

int b200_event_create(void** event);                                /* hip_event_create       :360 */
int b200_event_destroy(void* event);                                /* hip_event_destroy      :367 */
int b200_event_record(void* event, void* stream);                   /* hip_event_record       :376 */
int b200_event_synchronize(void* event);                            /* hip_event_synchronize  :382 */
int b200_event_elapsed_ms(void* start, void* stop, float* ms);      /* hip_event_elapsed_time :388 */
int b200_stream_create(void** stream);                              /* hip_stream_create      :397 */
int b200_stream_destroy(void* stream);                              /* hip_stream_destroy     :404 */
int b200_stream_synchronize(void* stream);                          /* hip_stream_synchronize :413 */

/* Evict the L2 by streaming a private buffer larger than the L2 (allocated on first use on the
 * current device).  Stands in for FlushLLC (python/aster/execution/flush_llc.py:25-204). */
int b200_flush_l2(void* stream);

/* ------------------------------------------------------------------------------------------ */
/* GEMM  C[M,N] = A[M,K] . B[N,K]^T, fp32 accumulation                                         */
/* Stands in for compile_multitile_gemm + GpuModule (the "plan") and execute_multitile_hsaco   */
/* (the "run"): contrib/kittens/test/test_102_gemm_python_multitile_lds_cdna3.py:391-436.      */
/* ------------------------------------------------------------------------------------------ */

enum {
  B200_F16 = 0, B200_BF16 = 1, B200_E4M3 = 2, B200_F32 = 3,
  /* Further operand types of the reference's MFMA list (include/aster/Dialect/AMDGCN/IR/
   * Instructions/MMA.td:138-375 bf8 and fp8/bf8 mixes, :636-727 i8 with i32 accumulators). */
  B200_E5M2 = 4,      /* OCP e5m2 ("bf8") for A and B                                          */
  B200_I8 = 5,        /* signed 8-bit integers, 32-bit integer accumulation                    */
  B200_I32 = 6,       /* dtype_c only, with B200_I8 inputs: the integer sums, unchanged        */
  B200_E5M2_E4M3 = 7, /* A e5m2, B e4m3                                                        */
  B200_E4M3_E5M2 = 8, /* A e4m3, B e5m2                                                        */
  /* Block-scaled fp8 ("MX"): every 32 consecutive elements of a row of A or B along K share
   * one E8M0 scale (a power of two, stored as the biased exponent byte; 127 = 1.0), applied
   * inside the tensor core.  The B200 form of the reference's v_mfma_scale_f32_16x16x128_f8f6f4
   * (include/aster/Dialect/AMDGCN/IR/Instructions/MMA.td; test/integration/
   * test_mfma_f8f6f4_e2e.py:39-95).  Scales are attached with b200_gemm_plan_set_mx_scales. */
  B200_MXE4M3 = 9,
  B200_MXE5M2 = 10
};
/* Layout of the B operand handed to b200_pack_b / b200_gemm_run. */
enum {
  B200_B_ROW_MAJOR_NK = 0,    /* B[N,K], K contiguous (reference OperandPath.LDS)                 */
  B200_B_REF_PRESHUFFLED = 1, /* shuffle_weight(B): contrib/kittens/test/kittens_helpers.py:90-119 */
  B200_B_PACKED = 2           /* row-major B that b200_pack_b turns into this plan's packed tiles  */
};
enum { B200_EPI_NONE = 0, B200_EPI_BIAS_RELU = 1, B200_EPI_BIAS = 2, B200_EPI_RELU = 3 };
enum { B200_BIAS_AXIS_N = 0, B200_BIAS_AXIS_M = 1 };

typedef struct b200_gemm_desc {
  int64_t M, N, K;
  int32_t dtype_ab;  /* B200_F16 | B200_BF16 | B200_E4M3 | B200_E5M2 | the two mixes | B200_I8   */
  int32_t dtype_c;   /* B200_F32 | B200_BF16 | B200_I32 (i8 inputs, no epilogue, no scales)     */
  int32_t b_layout;  /* B200_B_*                                                                */
  int32_t epilogue;  /* B200_EPI_*                                                              */
  int32_t bias_axis; /* B200_BIAS_AXIS_*                                                        */
  int32_t tile_m;    /* CTA tile rows: 128 (one CTA) or 256 (CTA pair); 0 = choose.  With 0 and
                      * M <= 64 a stage holds only 32 or 64 rows of A (more ring slots for B);
                      * 128 asks for full A stages                                              */
  int32_t tile_n;    /* CTA tile columns: 64, 128 or 256; 0 = choose                            */
  int32_t tile_k;    /* elements per pipeline stage along K; 0 = 128 bytes' worth               */
  int32_t stages;    /* shared-memory ring depth (<= 16); 0 = as many as fit, up to 8; with short
                      * A stages as many as keep 112 KB of B tiles on request (7 of 16 KB)      */
  int32_t cta_group; /* 1 or 2 CTAs per MMA; 0 = choose                                         */
  int32_t split_k;   /* K partitions reduced through an fp32 workspace; 0/1 = none, -1 = choose */
  int32_t max_ctas;  /* persistent grid size cap; 0 = number of SMs                             */
  int32_t raster_group; /* m-blocks per rasterisation group; 0 = choose                         */
  int32_t reserved[3];  /* [0] 0 = normal; 8 = fault injection for tests of the wait limit: the producer
                         * never hands a stage over, so the consumers' bounded waits expire; 16 = launch
                         * without programmatic stream serialisation (other bits are refused unless the
                         * library was built with -DB200_BRINGUP), [1] bit 0 = never use the tail split,
                         * bit 1 = B is static: nothing enqueued before a launch in its stream writes
                         * B (a weight matrix), so the kernel may request its first B tiles while the
                         * previous kernel of the stream is still finishing, bit 2 = a tail split
                         * exchanges through the workspace even where a cluster could, [2] limit of the
                         * device-side waits in ms (0 = 2000) */
  char label[256];   /* provenance only: the reference label string (gemm_config.py:678-701)    */
} b200_gemm_desc;

typedef struct b200_gemm_resources {
  int32_t tile_m, tile_n, tile_k, stages, cta_group, split_k;
  int32_t grid_ctas, block_threads;
  int32_t smem_bytes;     /* dynamic shared memory per CTA                                      */
  int32_t tmem_columns;   /* tensor-memory columns allocated per CTA                            */
  int32_t regs_per_thread;
  int32_t ctas_per_sm;
  int64_t num_tiles;
  int64_t workspace_bytes; /* required size of the run-time workspace (0 if none)               */
  int64_t packed_b_bytes;  /* size of the packed B buffer (0 for row-major plans)               */
  /* Tail split: when the tile count leaves the last round of the persistent grid mostly idle,
   * a caller that lends a 256-byte aligned workspace of at least optional_workspace_bytes lets
   * the last tail_tiles tiles be cut into tail_parts K ranges on otherwise idle SMs (partials
   * meet in the workspace, fixed summation order).  0 = not useful for this plan.  Without the
   * workspace the plan runs whole tiles only.  Launches that use one workspace must be ordered
   * (one stream); plans may take turns with it. */
  int64_t optional_workspace_bytes;
  int32_t tail_tiles, tail_parts;
  /* How the parts of a cut tile meet: 0 = no tail split, 1 = through the lent workspace,
   * 2 = through the shared memory of a thread-block cluster (skinny problems whose tiles all fit
   * in one round: the parts of a tile are the CTAs of one cluster; needs no workspace and is
   * always on; reserved[1] bit 2 of the description asks for the workspace form instead). */
  int32_t tail_exchange;
  int32_t reserved0;
} b200_gemm_resources;

typedef struct b200_gemm_plan b200_gemm_plan;

/* Validate the description (divisibility, alignment, enum values) and select a kernel
 * instance.  Never undefined behaviour on bad input: returns B200_ERR_INVALID. */
int b200_gemm_plan_create(const b200_gemm_desc* desc, b200_gemm_plan** plan);
int b200_gemm_plan_destroy(b200_gemm_plan* plan);
/* What the selected kernel needs; feeds the harness's post-compile resource filter
 * (contrib/kittens/test/bench/bench_search.py:454-476). */
int b200_gemm_plan_resources(const b200_gemm_plan* plan, b200_gemm_resources* out);

/* Convert B from the plan's declared caller layout (REF_PRESHUFFLED or PACKED = row-major
 * input) into the packed tile image the direct-B kernel streams.  Runs once, outside the
 * timed region, like the reference's host-side shuffle (bench_harness.py:567-574). */
int b200_pack_b(const b200_gemm_plan* plan, const void* b_in, void* b_packed, void* stream);

/* One launch.  A: [M,K] row-major.  B: [N,K] row-major, or the packed buffer for direct-B
 * plans.  C: [M,N] row-major, fully overwritten.  bias: fp32, length N (or M), may be NULL
 * when the epilogue has no bias.  scale_a / scale_b: device pointers to one fp32 each
 * (per-tensor dequantisation scales), NULL = 1.0.  workspace: device scratch of at least
 * resources.workspace_bytes, 16-byte aligned (may be NULL when that is 0); a workspace of at least
 * resources.optional_workspace_bytes additionally enables the tail split.
 * `stream` may be recording a CUDA graph (create the plan beforehand: that allocates); the
 * addresses are baked into the recorded launch, and a recorded tail-split launch carries a
 * small memset node that clears its ready flags on every replay. */
int b200_gemm_run(b200_gemm_plan* plan, const void* A, const void* B, void* C,
                  const float* bias, const float* scale_a, const float* scale_b,
                  void* workspace, size_t workspace_bytes, void* stream);

/* The reference's timing loop done natively (python/aster/execution/core.py:698-703): for
 * each of `iters` iterations [optional L2 flush] event, launch, event, synchronise.
 * times_ms receives `iters` floats. */
int b200_gemm_time(b200_gemm_plan* plan, const void* A, const void* B, void* C,
                   const float* bias, const float* scale_a, const float* scale_b,
                   void* workspace, size_t workspace_bytes, int iters, int flush_l2,
                   float* times_ms);
/* Same, but one event pair around `iters` back-to-back launches; *total_ms is their sum. */
int b200_gemm_time_batch(b200_gemm_plan* plan, const void* A, const void* B, void* C,
                         const float* bias, const float* scale_a, const float* scale_b,
                         void* workspace, size_t workspace_bytes, int iters, float* total_ms);

/* Device-side status words of the last launch of this plan (synchronises the device).
 * words[0] = 0 when every bounded wait completed; otherwise a code naming the wait that gave
 * up (role, barrier, tile).  Returns B200_ERR_TIMEOUT when words[0] != 0. */
int b200_status_read(b200_gemm_plan* plan, uint32_t words[4]);
/* SM clock (MHz) that the plan's last launch actually ran at: cycles over nanoseconds that
 * CTA 0 spent in the kernel (synchronises the device).  0 if the plan was never launched.
 * Per-launch tracing in the spirit of the reference's s_memtime cycle counters (README.md:273). */
int b200_gemm_last_sm_mhz(b200_gemm_plan* plan, float* mhz);
/* The same two counters summed over every launch of the plan so far, with the number of
 * launches (synchronises the device).  Differences taken around a timed region give the average
 * SM clock of exactly the launches that were timed: cycles / nanoseconds * 1000 = MHz.  (A burst
 * of launches starts at a high clock and sinks towards what the power cap allows, so the last
 * launch alone reads lower than the burst's average.) */
int b200_gemm_clock_totals(b200_gemm_plan* plan, uint64_t* sm_cycles, uint64_t* nanoseconds, uint64_t* launches);
/* Number of kernel launches issued by this library on the calling process so far. */
int b200_launch_count(int64_t* count);

/* Split-K GEMM that allocates nothing: C[M,N] = A[M,K] . B[N,K]^T with the fp32 partial sums
 * kept in a 16 MiB scratch array built into the library image instead of a caller workspace.
 * (No counterpart in the reference; it exists for hosts that cannot call cudaMalloc at GEMM
 * time: all device memory already belongs to their own pool, or an allocation's device-wide
 * synchronisation is not acceptable on their path.)
 *  - A, B, C: device pointers, 16-byte aligned, row-major, K contiguous in A and B.
 *  - dtype_ab: B200_F16 | B200_BF16 | B200_E4M3; dtype_c: B200_F32 | B200_BF16; no epilogue.
 *  - split_k in [1, 64] partitions of K (clamped to the number of 128-byte K blocks).
 *  - Limit: split_k * M * N * 4 bytes <= 16 MiB, else B200_ERR_WORKSPACE (use b200_gemm_run
 *    with your own workspace for larger problems).
 *  - The scratch is shared by all calls on a device and keeps the last call's contents; calls
 *    that overlap on the GPU race on it, so order them on one stream.
 *  - The first call on each device does a one-time host-side set-up (address lookup of the
 *    built-in array, kernel attributes); make it before any stream capture begins.
 * Calls no cudaMalloc / cudaFree and no allocating library routine. */
int b200_gemm_splitk_noalloc(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                             int32_t dtype_ab, int32_t dtype_c, int32_t split_k, void* stream);
/* Did the b200_gemm_splitk_noalloc calls made so far on the current device complete?  (They
 * have no plan to pass to b200_status_read; like them, this has no counterpart in the reference
 * and allocates nothing.)  Synchronises the device and copies back the status words of the
 * most recent call: words[0] = 0 when every bounded device-side wait completed, else a code
 * naming the wait that gave up, and the return value is B200_ERR_TIMEOUT; the C of such a call
 * is left unwritten (its reduction is skipped). */
int b200_gemm_splitk_noalloc_status(uint32_t words[4]);

/* ------------------------------------------------------------------------------------------ */
/* Bandwidth kernels                                                                          */
/* ------------------------------------------------------------------------------------------ */

/* c[i] = a[i] + b[i]; examples/03_vector_add/kernel.mlir:49-89 (int32, wrapping add). */
int b200_vector_add_i32(const int32_t* a, const int32_t* b, int32_t* c, size_t n, void* stream);
int b200_vector_add_f32(const float* a, const float* b, float* c, size_t n, void* stream);
/* dst[M,N] = src[M,N], fp32 row-major, N % 4 == 0; elements outside MxN are not touched.
 * `depth` (1..8) = 16-byte loads in flight per thread, `num_ctas` = grid size over which the
 * chunks are dealt (0 = one CTA per chunk, at most 512 per SM, which is the fastest).
 * examples/06_copy_layout/copy_2d_padded.py:34-151. */
int b200_copy_2d_padded_f32(const float* src, float* dst, int64_t M, int64_t N, int depth,
                            int num_ctas, void* stream);
/* out[i] = max(a[i] + b[i], 0); examples/07_simple_fusion/simple_fusion.py:62-144. */
int b200_add_relu_f32(const float* a, const float* b, float* out, size_t n, void* stream);

/* ---- block-scaled fp8 (dtype_ab = B200_MXE4M3 | B200_MXE5M2) -----------------------------
 * C = (A * 2^(sa-127)) . (B * 2^(sb-127))^T with sa[M][K/32], sb[N][K/32] bytes.  K % 32 == 0;
 * row-major B; tile_n 128 or 256.  The kernel streams the scales in blocks of
 * [128 rows][4 K blocks]; b200_pack_mx_scales turns row-major scales (device memory,
 * [rows][K/32] bytes) into that order (device memory of b200_mx_scales_bytes bytes, 16-byte
 * aligned).  b200_gemm_plan_set_mx_scales attaches the packed scales of A and B to a plan;
 * b200_gemm_run / _time then run it like any other plan (scale_a / scale_b stay available as
 * per-tensor factors). */
int b200_mx_scales_bytes(int64_t rows, int64_t K, size_t* bytes);
int b200_pack_mx_scales(const void* scales_in, void* scales_packed, int64_t rows, int64_t K, void* stream);
int b200_gemm_plan_set_mx_scales(b200_gemm_plan* plan, const void* scales_a_packed, const void* scales_b_packed);

/* ---- optional: gather row shards of C onto every GPU (NCCL over NVLink) ------------------
 * No counterpart in the reference, whose multi-GPU support is fan-out of whole configurations
 * over worker processes (contrib/kittens/test/bench/bench_harness.py:1013-1053).  One process
 * drives `ndev` GPUs; each GPU computes the rows [rank*M/ndev, (rank+1)*M/ndev) of C with its
 * own plan, and these calls put all of C on every GPU.  NCCL is opened at run time (the
 * soname libnccl.so.2, or the file ASTER_B200_NCCL_LIB names), the way the reference opens
 * its HIP runtime (python/lib/RuntimeModule.cpp:38-116); without it every call returns
 * B200_ERR_UNSUPPORTED.  The GEMM itself never needs these. */
typedef struct b200_comm b200_comm;
int b200_nccl_version(int* version);
/* devs == NULL means devices 0..ndev-1.  The calling thread's current device is restored. */
int b200_nccl_init_all(int ndev, const int* devs, b200_comm** comm);
int b200_nccl_destroy(b200_comm* comm);
/* Rank `rank` contributes `bytes_per_rank` bytes at c_shard and receives ndev*bytes_per_rank
 * bytes at c_full (both on that rank's GPU; c_shard may be its own slot inside c_full, and no
 * other overlap is accepted).  `stream` belongs to that rank's GPU.  A thread that issues the
 * call for more than one rank must bracket the calls with b200_nccl_group_start/_end, or use
 * b200_allgather_rows_all, which checks every rank's arguments before it hands any to NCCL. */
int b200_nccl_group_start(void);
int b200_nccl_group_end(void);
int b200_allgather_rows(b200_comm* comm, int rank, const void* c_shard, void* c_full,
                        size_t bytes_per_rank, void* stream);
/* All ranks at once: arrays of ndev pointers (streams may be NULL: each GPU's default stream). */
int b200_allgather_rows_all(b200_comm* comm, const void* const* c_shards, void* const* c_fulls,
                            size_t bytes_per_rank, void* const* streams);

#ifdef __cplusplus
}
#endif
#endif /* ASTER_B200_H_ */
