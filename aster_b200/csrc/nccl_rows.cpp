// Optional multi-GPU part of the aster_b200 C ABI: one process drives several GPUs and gathers
// the row shards of C onto every GPU with NCCL over NVLink.
//
// The reference has no collective (its multi-GPU support is config-level fan-out over worker
// processes, contrib/kittens/test/bench/bench_harness.py:1013-1053); this exists for callers
// that shard M across GPUs and then want the whole C everywhere.  NCCL is not linked: it is
// opened at run time, like the reference opens its HIP runtime
// (python/lib/RuntimeModule.cpp:38-116), so the library loads on machines without NCCL and
// every call here reports B200_ERR_UNSUPPORTED instead.
#include "common.h"

#include <dlfcn.h>

#include <cstdlib>
#include <mutex>
#include <vector>

namespace {

using ncclComm_t = void*;
constexpr int kNcclInt8 = 0;  // ncclInt8 / ncclChar in nccl.h

struct NcclApi {
  void* handle = nullptr;
  int (*CommInitAll)(ncclComm_t*, int, const int*) = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  int (*GetVersion)(int*) = nullptr;
  char why[256] = {0};
};

NcclApi g_nccl;
std::once_flag g_nccl_once;

template <typename F>
bool bind(void* h, const char* name, F& fn) {
  fn = reinterpret_cast<F>(dlsym(h, name));
  return fn != nullptr;
}

void load_nccl() {
  // ASTER_B200_NCCL_LIB names the library explicitly; otherwise the soname is resolved the
  // usual way, which also finds a copy that the process (e.g. PyTorch) has already loaded.
  const char* names[] = {std::getenv("ASTER_B200_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
  for (const char* n : names) {
    if (n == nullptr || n[0] == 0) continue;
    g_nccl.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (g_nccl.handle != nullptr) break;
    snprintf(g_nccl.why, sizeof(g_nccl.why), "%s", dlerror());
  }
  if (g_nccl.handle == nullptr) return;
  void* h = g_nccl.handle;
  bool ok = bind(h, "ncclCommInitAll", g_nccl.CommInitAll) && bind(h, "ncclCommDestroy", g_nccl.CommDestroy) &&
            bind(h, "ncclGroupStart", g_nccl.GroupStart) && bind(h, "ncclGroupEnd", g_nccl.GroupEnd) &&
            bind(h, "ncclAllGather", g_nccl.AllGather) && bind(h, "ncclGetErrorString", g_nccl.GetErrorString) &&
            bind(h, "ncclGetVersion", g_nccl.GetVersion);
  if (!ok) {
    snprintf(g_nccl.why, sizeof(g_nccl.why), "NCCL library lacks a required symbol");
    dlclose(h);
    g_nccl.handle = nullptr;
  }
}

int need_nccl() {
  std::call_once(g_nccl_once, load_nccl);
  if (g_nccl.handle == nullptr) {
    return b200::fail(B200_ERR_UNSUPPORTED, "NCCL runtime not available - %s", g_nccl.why);
  }
  return B200_OK;
}

}  // namespace

#define B200_NCCL_OK(expr)                                                                          \
  do {                                                                                              \
    int _r = (expr);                                                                                \
    if (_r != 0) {                                                                                  \
      return b200::fail(B200_ERR_CUDA, "NCCL error at %s:%d - %s (%s)", __FILE__, __LINE__,         \
                        g_nccl.GetErrorString(_r), #expr);                                          \
    }                                                                                               \
  } while (0)

struct b200_comm {
  std::vector<int> devices;
  std::vector<ncclComm_t> comms;
};

extern "C" {

int b200_nccl_version(int* version) {
  B200_REQUIRE(version != nullptr, "version is NULL");
  if (int rc = need_nccl()) return rc;
  B200_NCCL_OK(g_nccl.GetVersion(version));
  return B200_OK;
}

int b200_nccl_init_all(int ndev, const int* devs, b200_comm** out) {
  B200_REQUIRE(out != nullptr, "out is NULL");
  *out = nullptr;
  B200_REQUIRE(ndev >= 1 && ndev <= 64, "ndev %d out of range [1,64]", ndev);
  if (int rc = need_nccl()) return rc;
  int visible = 0;
  B200_CUDA_OK(cudaGetDeviceCount(&visible));
  auto* c = new b200_comm;
  for (int i = 0; i < ndev; ++i) {
    int d = devs ? devs[i] : i;
    bool dup = false;
    for (int seen : c->devices) dup = dup || seen == d;
    if (d < 0 || d >= visible || dup) {
      delete c;
      return b200::fail(B200_ERR_INVALID, "device list entry %d = %d is out of range [0,%d) or repeated", i, d, visible);
    }
    c->devices.push_back(d);
  }
  c->comms.assign(ndev, nullptr);
  int prev = 0;
  cudaGetDevice(&prev);
  int r = g_nccl.CommInitAll(c->comms.data(), ndev, c->devices.data());
  cudaSetDevice(prev);
  if (r != 0) {
    delete c;
    return b200::fail(B200_ERR_CUDA, "NCCL error in ncclCommInitAll - %s", g_nccl.GetErrorString(r));
  }
  *out = c;
  return B200_OK;
}

int b200_nccl_destroy(b200_comm* comm) {
  if (comm == nullptr) return B200_OK;
  if (int rc = need_nccl()) return rc;
  int first_err = 0;
  for (ncclComm_t c : comm->comms) {
    if (c == nullptr) continue;
    int r = g_nccl.CommDestroy(c);
    if (r != 0 && first_err == 0) first_err = r;
  }
  delete comm;
  if (first_err != 0) return b200::fail(B200_ERR_CUDA, "NCCL error in ncclCommDestroy - %s", g_nccl.GetErrorString(first_err));
  return B200_OK;
}

int b200_nccl_group_start(void) {
  if (int rc = need_nccl()) return rc;
  B200_NCCL_OK(g_nccl.GroupStart());
  return B200_OK;
}

int b200_nccl_group_end(void) {
  if (int rc = need_nccl()) return rc;
  B200_NCCL_OK(g_nccl.GroupEnd());
  return B200_OK;
}

// Argument checks shared by the two gather calls.  They run before anything is handed to NCCL:
// a collective that only some ranks joined would leave the others' kernels waiting.
static int check_gather_args(const b200_comm* comm, int rank, const void* c_shard, const void* c_full, size_t bytes_per_rank) {
  B200_REQUIRE(rank >= 0 && rank < (int)comm->comms.size(), "rank %d out of range [0,%zu)", rank, comm->comms.size());
  B200_REQUIRE(c_shard != nullptr && c_full != nullptr, "c_shard / c_full is NULL (rank %d)", rank);
  // NCCL takes the in-place form only when the shard already sits in its slot of c_full; any
  // other overlap is an error there, so refuse it here with a readable message.
  const char* s = static_cast<const char*>(c_shard);
  const char* f = static_cast<const char*>(c_full);
  const char* slot = f + (size_t)rank * bytes_per_rank;
  bool overlaps = s < f + comm->comms.size() * bytes_per_rank && f < s + bytes_per_rank;
  B200_REQUIRE(!overlaps || s == slot, "c_shard overlaps c_full outside rank %d's own slot", rank);
  return B200_OK;
}

int b200_allgather_rows(b200_comm* comm, int rank, const void* c_shard, void* c_full, size_t bytes_per_rank, void* stream) {
  B200_REQUIRE(comm != nullptr, "comm is NULL");
  if (int rc = need_nccl()) return rc;
  if (int rc = check_gather_args(comm, rank, c_shard, c_full, bytes_per_rank)) return rc;
  if (bytes_per_rank == 0) return B200_OK;
  B200_NCCL_OK(g_nccl.AllGather(c_shard, c_full, bytes_per_rank, kNcclInt8, comm->comms[rank], b200::as_stream(stream)));
  return B200_OK;
}

int b200_allgather_rows_all(b200_comm* comm, const void* const* c_shards, void* const* c_fulls, size_t bytes_per_rank,
                            void* const* streams) {
  B200_REQUIRE(comm != nullptr && c_shards != nullptr && c_fulls != nullptr, "comm / c_shards / c_fulls is NULL");
  if (int rc = need_nccl()) return rc;
  const int n = (int)comm->comms.size();
  for (int r = 0; r < n; ++r) {
    if (int rc = check_gather_args(comm, r, c_shards[r], c_fulls[r], bytes_per_rank)) return rc;
  }
  if (bytes_per_rank == 0) return B200_OK;
  B200_NCCL_OK(g_nccl.GroupStart());
  int first_err = 0;
  for (int r = 0; r < n; ++r) {
    int e = g_nccl.AllGather(c_shards[r], c_fulls[r], bytes_per_rank, kNcclInt8, comm->comms[r],
                             b200::as_stream(streams ? streams[r] : nullptr));
    if (e != 0 && first_err == 0) first_err = e;
  }
  int end = g_nccl.GroupEnd();
  if (first_err != 0) return b200::fail(B200_ERR_CUDA, "NCCL error in ncclAllGather - %s", g_nccl.GetErrorString(first_err));
  if (end != 0) return b200::fail(B200_ERR_CUDA, "NCCL error in ncclGroupEnd - %s", g_nccl.GetErrorString(end));
  return B200_OK;
}

}  // extern "C"
