// HBM-bound kernels of the hot path: vector_add, copy_2d_padded, add_relu.
//
// All three move 32 bytes per thread per access when the pointers allow it (256-bit loads and
// stores, sm_100; one warp touches 1 KB contiguous) and 16 bytes otherwise, keep several
// independent loads in flight per thread, and walk their chunks grid-stride.  The 32-byte form
// halves the memory instructions and requests: copy_2d_padded 5.91 -> 6.18 TB/s on a B200.  The
// grid is one CTA per chunk up to kCtasPerSm per SM, far more than are resident (8 per SM): a CTA
// that has stored its chunk makes room for a fresh one whose loads go out at once, where a
// resident CTA looping over its chunks alternates between loading and storing.  Measured on
// copy_2d_padded 16384 x 16380 with 8 / 16 / 32 / 64 / 128 / 256 CTAs per SM: 6.16 / 6.51 / 6.64 /
// 6.73 / 6.79 / 6.82 TB/s (a device-to-device cudaMemcpy: 6.54); vector_add over 2^28 elements
// with 8 / 32 / 128 / 512: 6.59 / 6.85 / 6.95 / 7.01 TB/s.  Loads bypass L1
// allocation (`ld.global.nc.L1::no_allocate`) and stores are streaming (`st.global.cs`): every
// byte is touched exactly once, so caching it would only evict useful lines.
//
// Algorithmic bytes per element: vector_add / add_relu 12 (two 4-byte reads, one write);
// copy 8.
#include "common.h"

#include <cstdlib>

namespace {

constexpr int kThreads = 256;
constexpr int kCtasPerSm = 512;  // cap of the grid; beyond it the CTAs loop

template <typename V>
__device__ __forceinline__ V ld_stream(const V* p) {
  static_assert(sizeof(V) == 16, "16-byte vectors only");
  int4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return *reinterpret_cast<V*>(&r);
}

template <typename V>
__device__ __forceinline__ void st_stream(V* p, V v) {
  static_assert(sizeof(V) == 16, "16-byte vectors only");
  int4 r = *reinterpret_cast<int4*>(&v);
  asm volatile("st.global.cs.v4.s32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(r.x), "r"(r.y), "r"(r.z), "r"(r.w)
               : "memory");
}

// 32-byte accesses (sm_100): half the load/store instructions and requests of the 16-byte walk.
struct alignas(32) Vec32 {
  uint32_t w[8];
};
__device__ __forceinline__ Vec32 ld_stream32(const Vec32* p) {
  Vec32 r;
  asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3]), "=r"(r.w[4]), "=r"(r.w[5]), "=r"(r.w[6]), "=r"(r.w[7])
               : "l"(p));
  return r;
}
__device__ __forceinline__ void st_stream32(Vec32* p, const Vec32& v) {
  asm volatile("st.global.cs.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]),
               "r"(v.w[4]), "r"(v.w[5]), "r"(v.w[6]), "r"(v.w[7])
               : "memory");
}

struct AddI32 {
  using T = int32_t;
  using V = int4;
  // Wrapping add, like v_add_u32 in the reference kernel.
  static __device__ __forceinline__ T op(T a, T b) {
    return static_cast<T>(static_cast<uint32_t>(a) + static_cast<uint32_t>(b));
  }
};
struct AddF32 {
  using T = float;
  using V = float4;
  static __device__ __forceinline__ T op(T a, T b) { return __fadd_rn(a, b); }
};
struct AddReluF32 {
  using T = float;
  using V = float4;
  // v_add_f32 then v_max_f32 with 0 (examples/07_simple_fusion/pin-fusion-asm.mlir:34-62).
  static __device__ __forceinline__ T op(T a, T b) { return fmaxf(__fadd_rn(a, b), 0.0f); }
};

template <typename Op>
__device__ __forceinline__ typename Op::V apply4(typename Op::V a, typename Op::V b) {
  typename Op::V c;
  c.x = Op::op(a.x, b.x);
  c.y = Op::op(a.y, b.y);
  c.z = Op::op(a.z, b.z);
  c.w = Op::op(a.w, b.w);
  return c;
}

// Elementwise c = op(a, b) over n elements.  `UNROLL` 16-byte vectors per input per thread are
// loaded before any is consumed.  Requires 16-byte aligned pointers; the last n % 4 elements
// are handled by the first threads of the grid.
template <typename Op, int UNROLL>
__global__ void __launch_bounds__(kThreads) elementwise_vec_kernel(const typename Op::T* __restrict__ a,
                                                                  const typename Op::T* __restrict__ b,
                                                                  typename Op::T* __restrict__ c, size_t n) {
  using V = typename Op::V;
  const size_t nvec = n / 4;
  const V* av = reinterpret_cast<const V*>(a);
  const V* bv = reinterpret_cast<const V*>(b);
  V* cv = reinterpret_cast<V*>(c);
  const size_t chunk = static_cast<size_t>(kThreads) * UNROLL;
  const size_t nchunks = nvec / chunk;
  for (size_t ch = blockIdx.x; ch < nchunks; ch += gridDim.x) {
    const size_t base = ch * chunk + threadIdx.x;
    V ra[UNROLL], rb[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) ra[u] = ld_stream(av + base + u * kThreads);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) rb[u] = ld_stream(bv + base + u * kThreads);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) st_stream(cv + base + u * kThreads, apply4<Op>(ra[u], rb[u]));
  }
  // Vector remainder (fewer than one chunk) and scalar tail.
  const size_t gtid = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x;
  const size_t gsz = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t v = nchunks * chunk + gtid; v < nvec; v += gsz) st_stream(cv + v, apply4<Op>(ld_stream(av + v), ld_stream(bv + v)));
  for (size_t i = nvec * 4 + gtid; i < n; i += gsz) c[i] = Op::op(a[i], b[i]);
}

template <typename T>
__device__ __forceinline__ T from_bits(uint32_t w);
template <>
__device__ __forceinline__ int32_t from_bits<int32_t>(uint32_t w) { return static_cast<int32_t>(w); }
template <>
__device__ __forceinline__ float from_bits<float>(uint32_t w) { return __uint_as_float(w); }
__device__ __forceinline__ uint32_t to_bits(int32_t x) { return static_cast<uint32_t>(x); }
__device__ __forceinline__ uint32_t to_bits(float x) { return __float_as_uint(x); }

template <typename Op>
__device__ __forceinline__ Vec32 apply8(const Vec32& a, const Vec32& b) {
  Vec32 c;
#pragma unroll
  for (int j = 0; j < 8; ++j) c.w[j] = to_bits(Op::op(from_bits<typename Op::T>(a.w[j]), from_bits<typename Op::T>(b.w[j])));
  return c;
}

// The same over 32-byte vectors (all pointers 32-byte aligned): half the memory instructions.
template <typename Op, int UNROLL>
__global__ void __launch_bounds__(kThreads) elementwise_wide_kernel(const typename Op::T* __restrict__ a,
                                                                   const typename Op::T* __restrict__ b,
                                                                   typename Op::T* __restrict__ c, size_t n) {
  const size_t nvec = n / 8;
  const Vec32* av = reinterpret_cast<const Vec32*>(a);
  const Vec32* bv = reinterpret_cast<const Vec32*>(b);
  Vec32* cv = reinterpret_cast<Vec32*>(c);
  const size_t chunk = static_cast<size_t>(kThreads) * UNROLL;
  const size_t nchunks = nvec / chunk;
  for (size_t ch = blockIdx.x; ch < nchunks; ch += gridDim.x) {
    const size_t base = ch * chunk + threadIdx.x;
    Vec32 ra[UNROLL], rb[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) ra[u] = ld_stream32(av + base + u * kThreads);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) rb[u] = ld_stream32(bv + base + u * kThreads);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) st_stream32(cv + base + u * kThreads, apply8<Op>(ra[u], rb[u]));
  }
  const size_t gtid = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x;
  const size_t gsz = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t v = nchunks * chunk + gtid; v < nvec; v += gsz) st_stream32(cv + v, apply8<Op>(ld_stream32(av + v), ld_stream32(bv + v)));
  for (size_t i = nvec * 8 + gtid; i < n; i += gsz) c[i] = Op::op(a[i], b[i]);
}

// Fallback for pointers that are not 16-byte aligned: 4-byte accesses, still coalesced.
template <typename Op>
__global__ void __launch_bounds__(kThreads) elementwise_scalar_kernel(const typename Op::T* __restrict__ a,
                                                                     const typename Op::T* __restrict__ b,
                                                                     typename Op::T* __restrict__ c, size_t n) {
  const size_t gsz = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += gsz) c[i] = Op::op(a[i], b[i]);
}

int sm_count() {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms > 0 ? sms : 148;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename Op>
int launch_elementwise(const typename Op::T* a, const typename Op::T* b, typename Op::T* c, size_t n, void* stream,
                       const char* what) {
  if (n == 0) return B200_OK;
  B200_REQUIRE(a && b && c, "%s: NULL pointer", what);
  constexpr int UNROLL = 4;
  const size_t per_cta = static_cast<size_t>(kThreads) * UNROLL * 4;
  size_t want = (n + per_cta - 1) / per_cta;
  const size_t cap = static_cast<size_t>(sm_count()) * kCtasPerSm;
  const int grid = static_cast<int>(want < cap ? (want ? want : 1) : cap);
  const bool aligned32 = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 31u) == 0;
  if (aligned32) {
    elementwise_wide_kernel<Op, UNROLL / 2><<<grid, kThreads, 0, b200::as_stream(stream)>>>(a, b, c, n);
  } else if (aligned16(a) && aligned16(b) && aligned16(c)) {
    elementwise_vec_kernel<Op, UNROLL><<<grid, kThreads, 0, b200::as_stream(stream)>>>(a, b, c, n);
  } else {
    elementwise_scalar_kernel<Op><<<grid, kThreads, 0, b200::as_stream(stream)>>>(a, b, c, n);
  }
  b200::count_launch();
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}

// dst[r, c] = src[r, c] for r < M, c < N; both row-major with pitch N, N % 4 == 0.
//
// The reference tiles the M x N iteration space into (row, 256-column tile) items, pads the
// last column tile and relies on buffer descriptors to drop the lanes that fall outside
// (examples/06_copy_layout/copy_2d_padded.py:46-69).  With rows packed back to back and N a
// multiple of 4, the matrix is one run of M*N/4 16-byte vectors, none of which straddles a row
// or leaves the matrix, so this kernel walks that run directly: no padded lanes, no per-item
// division, and the tail of one row coalesces with the head of the next.  Elements outside
// M x N are never addressed, which is the contract the reference's sentinel check tests.
// DEPTH = 16-byte loads each thread has in flight before its first store: the reference's
// `depth` software-pipelining knob (:71-96).  Chunks of kThreads * DEPTH vectors are dealt
// round-robin to the CTAs, like the reference deals items (:74-76); `num_ctas` = 0 launches one
// CTA per chunk up to the grid cap.
template <int DEPTH>
__global__ void __launch_bounds__(kThreads) copy_2d_padded_kernel(const float4* __restrict__ src, float4* __restrict__ dst,
                                                                 size_t nvec) {
  const size_t chunk = static_cast<size_t>(kThreads) * DEPTH;
  const size_t nchunks = nvec / chunk;
  for (size_t ch = blockIdx.x; ch < nchunks; ch += gridDim.x) {
    const size_t base = ch * chunk + threadIdx.x;
    float4 v[DEPTH];
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) v[d] = ld_stream(src + base + d * kThreads);
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) st_stream(dst + base + d * kThreads, v[d]);
  }
  const size_t gsz = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t i = nchunks * chunk + static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < nvec; i += gsz)
    st_stream(dst + i, ld_stream(src + i));
}

// Same walk as copy_2d_padded_kernel over 32-byte vectors (both pointers 32-byte aligned); the
// 16-byte remainder, if any, is copied by the caller's tail launch of the 16-byte kernel.
template <int DEPTH>
__global__ void __launch_bounds__(kThreads) copy_2d_padded_wide_kernel(const Vec32* __restrict__ src, Vec32* __restrict__ dst, size_t nvec) {
  const size_t chunk = static_cast<size_t>(kThreads) * DEPTH;
  const size_t nchunks = nvec / chunk;
  for (size_t ch = blockIdx.x; ch < nchunks; ch += gridDim.x) {
    const size_t base = ch * chunk + threadIdx.x;
    Vec32 v[DEPTH];
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) v[d] = ld_stream32(src + base + d * kThreads);
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) st_stream32(dst + base + d * kThreads, v[d]);
  }
  const size_t gsz = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t i = nchunks * chunk + static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < nvec; i += gsz)
    st_stream32(dst + i, ld_stream32(src + i));
}

}  // namespace

extern "C" {

int b200_vector_add_i32(const int32_t* a, const int32_t* b, int32_t* c, size_t n, void* stream) {
  return launch_elementwise<AddI32>(a, b, c, n, stream, "vector_add_i32");
}

int b200_vector_add_f32(const float* a, const float* b, float* c, size_t n, void* stream) {
  return launch_elementwise<AddF32>(a, b, c, n, stream, "vector_add_f32");
}

int b200_add_relu_f32(const float* a, const float* b, float* out, size_t n, void* stream) {
  return launch_elementwise<AddReluF32>(a, b, out, n, stream, "add_relu_f32");
}

int b200_copy_2d_padded_f32(const float* src, float* dst, int64_t M, int64_t N, int depth, int num_ctas,
                            void* stream) {
  B200_REQUIRE(M >= 0 && N >= 0, "copy_2d_padded: negative extent %lld x %lld", (long long)M, (long long)N);
  // Same precondition as the reference: a 16-byte access must not straddle the end of a row.
  B200_REQUIRE(N % 4 == 0, "copy_2d_padded: N=%lld must be a multiple of 4", (long long)N);
  B200_REQUIRE(depth >= 1 && depth <= 8, "copy_2d_padded: depth=%d outside [1,8]", depth);
  B200_REQUIRE(num_ctas >= 0, "copy_2d_padded: num_ctas=%d is negative", num_ctas);
  if (M == 0 || N == 0) return B200_OK;
  B200_REQUIRE(src && dst, "copy_2d_padded: NULL pointer");
  B200_REQUIRE(aligned16(src) && aligned16(dst), "copy_2d_padded: pointers must be 16-byte aligned");
  const size_t nvec = static_cast<size_t>(M) * static_cast<size_t>(N) / 4;
  // Round depth up to the instantiated pipeline depths {1,2,4,8}.
  int d = 1;
  while (d < depth) d *= 2;
  const size_t per_cta = static_cast<size_t>(kThreads) * d;
  const size_t want = (nvec + per_cta - 1) / per_cta;
  const size_t cap = num_ctas > 0 ? static_cast<size_t>(num_ctas) : static_cast<size_t>(sm_count()) * kCtasPerSm;
  const int grid = static_cast<int>(want < cap ? want : cap);
  cudaStream_t s = b200::as_stream(stream);
  const float4* s4 = reinterpret_cast<const float4*>(src);
  float4* d4 = reinterpret_cast<float4*>(dst);
  if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 31u) == 0 && nvec >= 2) {
    // 32-byte walk over the even part; an odd last 16-byte vector is copied by a one-CTA launch below.
    const size_t nwide = nvec / 2;
    const Vec32* s8 = reinterpret_cast<const Vec32*>(src);
    Vec32* d8 = reinterpret_cast<Vec32*>(dst);
    const int dw = d > 4 ? 4 : d;  // bytes in flight per thread as for the 16-byte walk of twice the depth
    const size_t want_w = (nwide + static_cast<size_t>(kThreads) * dw - 1) / (static_cast<size_t>(kThreads) * dw);
    const int grid_w = static_cast<int>(want_w < cap ? want_w : cap);
    switch (dw) {
      case 1: copy_2d_padded_wide_kernel<1><<<grid_w, kThreads, 0, s>>>(s8, d8, nwide); break;
      case 2: copy_2d_padded_wide_kernel<2><<<grid_w, kThreads, 0, s>>>(s8, d8, nwide); break;
      default: copy_2d_padded_wide_kernel<4><<<grid_w, kThreads, 0, s>>>(s8, d8, nwide); break;
    }
    b200::count_launch();
    B200_CUDA_OK(cudaGetLastError());
    if (nvec % 2 != 0) {
      copy_2d_padded_kernel<1><<<1, kThreads, 0, s>>>(s4 + (nvec - 1), d4 + (nvec - 1), 1);
      b200::count_launch();
      B200_CUDA_OK(cudaGetLastError());
    }
    return B200_OK;
  }
  switch (d) {
    case 1: copy_2d_padded_kernel<1><<<grid, kThreads, 0, s>>>(s4, d4, nvec); break;
    case 2: copy_2d_padded_kernel<2><<<grid, kThreads, 0, s>>>(s4, d4, nvec); break;
    case 4: copy_2d_padded_kernel<4><<<grid, kThreads, 0, s>>>(s4, d4, nvec); break;
    default: copy_2d_padded_kernel<8><<<grid, kThreads, 0, s>>>(s4, d4, nvec); break;
  }
  b200::count_launch();
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}

}  // extern "C"
