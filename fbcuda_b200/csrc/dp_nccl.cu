// Communicator for the data-parallel accGradParameters: batch shards on different GPUs (one
// process per GPU), weights replicated, the weight gradient summed over NCCL.
//
// Has no counterpart in the reference (it has no multi-GPU code at all); what is summed is the
// result of its accGradParameters (fbfft/FFTIteratedConvolution.cuh:409-524) over the shards.
//
// NCCL is bound at run time (dlopen of libnccl.so.2 on the first communicator call), so the
// transforms and single-GPU passes carry no dependency on it; inside a process that already
// loaded an NCCL (e.g. through torch) that copy is the one found.  The communicator is created
// non-blocking, which is what makes the initialisation time limit possible: every NCCL call that
// answers "in progress" is polled until it settles or the limit runs out, and a communicator
// whose limit ran out is aborted, never left half-built.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <thread>

#include "../../include/fbfft_b200.h"
#include "common.cuh"
#include "dp_comm.h"

namespace fbfft_b200 {

namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

NcclApi& api() {
  static NcclApi a;
  static std::once_flag once;
  std::call_once(once, [] {
    for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
      a.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
      if (a.handle) break;
    }
    if (!a.handle) return;
    bool all = true;
    auto sym = [&](const char* n) {
      void* p = dlsym(a.handle, n);
      if (!p) all = false;
      return p;
    };
    a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(sym("ncclGetUniqueId"));
    a.CommInitRankConfig = reinterpret_cast<decltype(a.CommInitRankConfig)>(sym("ncclCommInitRankConfig"));
    a.CommGetAsyncError = reinterpret_cast<decltype(a.CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
    a.CommAbort = reinterpret_cast<decltype(a.CommAbort)>(sym("ncclCommAbort"));
    a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(sym("ncclCommDestroy"));
    a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(sym("ncclAllReduce"));
    a.ReduceScatter = reinterpret_cast<decltype(a.ReduceScatter)>(sym("ncclReduceScatter"));
    a.AllGather = reinterpret_cast<decltype(a.AllGather)>(sym("ncclAllGather"));
    a.GroupStart = reinterpret_cast<decltype(a.GroupStart)>(sym("ncclGroupStart"));
    a.GroupEnd = reinterpret_cast<decltype(a.GroupEnd)>(sym("ncclGroupEnd"));
    a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(sym("ncclGetErrorString"));
    a.ok = all;
  });
  return a;
}

int fail(int code, const char* msg) {
  set_last_error(msg);
  return code;
}

int fail_nccl(const char* what, ncclResult_t r) {
  char buf[240];
  std::snprintf(buf, sizeof(buf), "%s: NCCL error %d (%s)", what, (int)r, api().GetErrorString ? api().GetErrorString(r) : "?");
  return fail(kCudaError, buf);
}

}  // namespace

struct Comm {
  ncclComm_t nccl = nullptr;
  int rank = 0, world = 1;
  int timeout_ms = 0;
};

// Polls a non-blocking communicator until the pending call settled; aborts nothing by itself.
static ncclResult_t settle(Comm* c, ncclResult_t r, int timeout_ms) {
  if (r != ncclInProgress) return r;
  const auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    ncclResult_t state = ncclSuccess;
    const ncclResult_t q = api().CommGetAsyncError(c->nccl, &state);
    if (q != ncclSuccess) return q;
    if (state != ncclInProgress) return state;
    if (std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count() > timeout_ms)
      return ncclInProgress;
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

int comm_rank(const Comm* c) { return c->rank; }
int comm_world(const Comm* c) { return c->world; }

int comm_all_reduce(Comm* c, float* buf, size_t count, cudaStream_t s) {
  const ncclResult_t r = settle(c, api().AllReduce(buf, buf, count, ncclFloat, ncclSum, c->nccl, s), c->timeout_ms);
  return r == ncclSuccess ? kSuccess : fail_nccl("all-reduce of the weight gradient", r);
}

// `rows` in-place reduce-scatters issued as one group: row i covers world * count floats starting at
// base + i * row_stride, of which this rank keeps those at rank * count
int comm_reduce_scatter_rows(Comm* c, float* base, int rows, size_t row_stride, size_t count, cudaStream_t s) {
  ncclResult_t r = api().GroupStart();
  if (r != ncclSuccess) return fail_nccl("group start", r);
  for (int i = 0; i < rows && (r == ncclSuccess || r == ncclInProgress); ++i) {
    float* row = base + (size_t)i * row_stride;
    r = api().ReduceScatter(row, row + (size_t)c->rank * count, count, ncclFloat, ncclSum, c->nccl, s);
  }
  const ncclResult_t e = settle(c, api().GroupEnd(), c->timeout_ms);
  if (r != ncclSuccess && r != ncclInProgress) return fail_nccl("reduce-scatter of the weight-gradient spectrum", r);
  return e == ncclSuccess ? kSuccess : fail_nccl("reduce-scatter of the weight-gradient spectrum", e);
}

// in place: this rank's `count` floats already sit at base + rank * count
int comm_all_gather(Comm* c, float* base, size_t count, cudaStream_t s) {
  const ncclResult_t r =
      settle(c, api().AllGather(base + (size_t)c->rank * count, base, count, ncclFloat, c->nccl, s), c->timeout_ms);
  return r == ncclSuccess ? kSuccess : fail_nccl("all-gather of the weight gradient", r);
}

}  // namespace fbfft_b200

using namespace fbfft_b200;

extern "C" {

int fbfft_b200_comm_unique_id(void* id_out) {
  if (!id_out) return fail(kUnsupportedDimension, "comm_unique_id: null output");
  if (!api().ok) return fail(kCudaError, "comm_unique_id: libnccl.so.2 could not be loaded");
  static_assert(sizeof(ncclUniqueId) == FBFFT_B200_UNIQUE_ID_BYTES, "unique id size");
  ncclUniqueId id;
  const ncclResult_t r = api().GetUniqueId(&id);
  if (r != ncclSuccess) return fail_nccl("comm_unique_id", r);
  std::memcpy(id_out, &id, sizeof(id));
  return kSuccess;
}

int fbfft_b200_comm_init(const void* unique_id, int rank, int world, int timeout_ms, fbfft_b200_comm** out) {
  if (out) *out = nullptr;
  if (!unique_id || !out) return fail(kUnsupportedDimension, "comm_init: null argument");
  if (world < 1 || rank < 0 || rank >= world) return fail(kUnsupportedDimension, "comm_init: need 0 <= rank < world");
  if (timeout_ms <= 0) return fail(kUnsupportedDimension, "comm_init: the time limit must be positive (milliseconds)");
  if (!api().ok) return fail(kCudaError, "comm_init: libnccl.so.2 could not be loaded");
  ncclUniqueId id;
  std::memcpy(&id, unique_id, sizeof(id));
  ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
  cfg.blocking = 0;
  // FBFFT_B200_NCCL_MAX_CTAS caps the blocks NCCL's kernels use, so that they fit on the SMs a caller
  // keeps free of the persistent contraction (fbfft_b200_set_contraction_reserved_sms)
  if (const char* e = std::getenv("FBFFT_B200_NCCL_MAX_CTAS")) {
    const int v = std::atoi(e);
    if (v >= 1 && v <= 64) cfg.maxCTAs = v;
  }
  Comm* c = new Comm;
  c->rank = rank, c->world = world, c->timeout_ms = timeout_ms;
  ncclResult_t r = api().CommInitRankConfig(&c->nccl, world, id, rank, &cfg);
  if (r == ncclInProgress && c->nccl) r = settle(c, r, timeout_ms);
  if (r != ncclSuccess) {
    const bool timed_out = r == ncclInProgress;
    if (c->nccl) api().CommAbort(c->nccl);
    delete c;
    if (timed_out) return fail(kCudaError, "comm_init: the other ranks did not join within the time limit; communicator aborted");
    return fail_nccl("comm_init", r);
  }
  *out = reinterpret_cast<fbfft_b200_comm*>(c);
  return kSuccess;
}

int fbfft_b200_comm_info(const fbfft_b200_comm* comm, int* rank, int* world) {
  if (!comm) return fail(kUnsupportedDimension, "comm_info: null communicator");
  const Comm* c = reinterpret_cast<const Comm*>(comm);
  if (rank) *rank = c->rank;
  if (world) *world = c->world;
  return kSuccess;
}

int fbfft_b200_comm_destroy(fbfft_b200_comm* comm) {
  if (!comm) return fail(kUnsupportedDimension, "comm_destroy: null communicator");
  Comm* c = reinterpret_cast<Comm*>(comm);
  ncclResult_t r = ncclSuccess;
  if (c->nccl) r = settle(c, api().CommDestroy(c->nccl), c->timeout_ms);
  delete c;
  return r == ncclSuccess ? kSuccess : fail_nccl("comm_destroy", r);
}

int fbfft_b200_dp_shard(long long total, int world, int rank, long long* lo, long long* count) {
  if (total < 0 || world < 1 || rank < 0 || rank >= world || !lo || !count)
    return fail(kUnsupportedDimension, "dp_shard: need total >= 0, 0 <= rank < world and two outputs");
  const long long base = total / world, extra = total % world;
  *lo = rank * base + (rank < extra ? rank : extra);
  *count = base + (rank < extra ? 1 : 0);
  return kSuccess;
}

}  // extern "C"
