// Data-parallel gradient mean over NCCL (NVLink / NVSwitch): the device-side replacement of grad's
// host-memory `Replicas.averageGrads` (src/nn/replicas.zig:57-91).  NCCL is resolved at run time with
// dlopen, the way grad resolves libcuda and cuDNN (src/gpu/dynlib.zig:28-60), so the library carries no
// link-time dependency on it.  The reduction is ONE in-place ncclAllReduce(ncclAvg) over the flat gradient
// vector (the reference sums the replicas' vectors and multiplies by 1/N, replicas.zig:73-80; for the replica
// counts in use, powers of two, scaling before or after the sum gives the same bits); every rank ends with
// identical bits because an NCCL allreduce delivers the same result to all ranks.
//
// Failure handling follows `Replicas.stop` releasing the waiters (replicas.zig:36-53) in the form a device
// collective allows: the communicator is created non-blocking, every NCCL call that answers "in progress" is
// polled with ncclCommGetAsyncError against a host deadline, and when the deadline passes (a replica that never
// joined, a peer that died) the communicator is aborted -- which also ends a collective already running on the
// device -- and the call returns GB_ERR_TIMEOUT instead of waiting for ever.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <thread>

#include "../../include/gradb200.h"

namespace {

struct NcclApi {
  ncclResult_t (*ncclGetUniqueId)(ncclUniqueId*);
  ncclResult_t (*ncclCommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*);
  ncclResult_t (*ncclCommGetAsyncError)(ncclComm_t, ncclResult_t*);
  ncclResult_t (*ncclAllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
  ncclResult_t (*ncclCommAbort)(ncclComm_t);
  ncclResult_t (*ncclCommDestroy)(ncclComm_t);
  bool ok = false;
};

// GB_NCCL_LIBRARY names the library to load instead of libnccl.so.2 (a particular NCCL build; the tests point it
// at a stand-in whose calls never complete, to drive the deadline path without a GPU).
NcclApi& nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* lib = nullptr;
    if (const char* named = getenv("GB_NCCL_LIBRARY")) {
      lib = dlopen(named, RTLD_NOW | RTLD_GLOBAL);
    } else {
      for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
        lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
        if (lib) break;
      }
    }
    if (!lib) return;
    api.ncclGetUniqueId = (decltype(api.ncclGetUniqueId))dlsym(lib, "ncclGetUniqueId");
    api.ncclCommInitRankConfig = (decltype(api.ncclCommInitRankConfig))dlsym(lib, "ncclCommInitRankConfig");
    api.ncclCommGetAsyncError = (decltype(api.ncclCommGetAsyncError))dlsym(lib, "ncclCommGetAsyncError");
    api.ncclAllReduce = (decltype(api.ncclAllReduce))dlsym(lib, "ncclAllReduce");
    api.ncclCommAbort = (decltype(api.ncclCommAbort))dlsym(lib, "ncclCommAbort");
    api.ncclCommDestroy = (decltype(api.ncclCommDestroy))dlsym(lib, "ncclCommDestroy");
    api.ok = api.ncclGetUniqueId && api.ncclCommInitRankConfig && api.ncclCommGetAsyncError && api.ncclAllReduce && api.ncclCommAbort &&
             api.ncclCommDestroy;
  });
  return api;
}

using Clock = std::chrono::steady_clock;

uint32_t default_timeout_ms() {
  static const uint32_t ms = [] {
    const char* v = getenv("GB_COMM_TIMEOUT_MS");
    return v ? (uint32_t)std::max(1, atoi(v)) : 60000u;
  }();
  return ms;
}

}  // namespace

struct gb_comm {
  ncclComm_t comm = nullptr;
  int nranks = 1, rank = 0, device = 0;
  uint32_t timeout_ms = 60000;
  bool aborted = false;
};

namespace {

void abort_comm(gb_comm* c) {
  c->aborted = true;
  if (c->comm) {
    nccl().ncclCommAbort(c->comm);
    c->comm = nullptr;
  }
}

// Polls the communicator until the call that answered `first` has settled; aborts it when the deadline passes.
int settle(gb_comm* c, ncclResult_t first) {
  ncclResult_t state = first;
  const auto start = Clock::now();
  const auto deadline = start + std::chrono::milliseconds(c->timeout_ms);
  while (state == ncclInProgress) {
    const auto now = Clock::now();
    if (now > deadline) {
      abort_comm(c);
      return GB_ERR_TIMEOUT;
    }
    // an enqueue settles within microseconds: poll without sleeping at first, so that back-to-back collectives are
    // not spaced by the poll interval; back off once the wait is clearly a wait for a peer
    if (now - start > std::chrono::microseconds(500)) std::this_thread::sleep_for(std::chrono::microseconds(50));
    if (nccl().ncclCommGetAsyncError(c->comm, &state) != ncclSuccess) state = ncclInternalError;
  }
  if (state != ncclSuccess) {
    abort_comm(c);
    return GB_ERR_NCCL;
  }
  return GB_OK;
}

}  // namespace

extern "C" {

int gb_comm_unique_id(void* out128) {
  if (!out128) return GB_ERR_INVALID;
  if (!nccl().ok) return GB_ERR_NCCL;
  ncclUniqueId id;
  if (nccl().ncclGetUniqueId(&id) != ncclSuccess) return GB_ERR_NCCL;
  static_assert(sizeof(id) == 128, "the id travels as 128 bytes");
  std::memcpy(out128, &id, sizeof(id));
  return GB_OK;
}

int gb_comm_create(int nranks, int rank, const void* unique_id128, int device_ordinal, gb_comm** out) {
  if (!out || nranks < 1 || rank < 0 || rank >= nranks) return GB_ERR_INVALID;
  *out = nullptr;
  gb_comm* c = new gb_comm();
  c->nranks = nranks;
  c->rank = rank;
  c->device = device_ordinal;
  c->timeout_ms = default_timeout_ms();
  if (nranks > 1) {
    if (!unique_id128) { delete c; return GB_ERR_INVALID; }
    if (!nccl().ok) { delete c; return GB_ERR_NCCL; }
    // a negative ordinal keeps the caller's current device
    if (device_ordinal >= 0 && cudaSetDevice(device_ordinal) != cudaSuccess) { delete c; return GB_ERR_CUDA; }
    ncclUniqueId id;
    std::memcpy(&id, unique_id128, sizeof(id));
    ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
    config.blocking = 0;
    const ncclResult_t r = nccl().ncclCommInitRankConfig(&c->comm, nranks, id, rank, &config);
    if (r != ncclSuccess && r != ncclInProgress) { delete c; return GB_ERR_NCCL; }
    const int rc = settle(c, ncclInProgress);   // the communicator is usable once its state reads ncclSuccess
    if (rc != GB_OK) { delete c; return rc; }
  }
  *out = c;
  return GB_OK;
}

int gb_comm_set_timeout(gb_comm* comm, uint32_t timeout_ms) {
  if (!comm || timeout_ms == 0) return GB_ERR_INVALID;
  comm->timeout_ms = timeout_ms;
  return GB_OK;
}

int gb_allreduce_mean(gb_comm* comm, void* stream, float* grads, size_t count) {
  if (!comm || (!grads && count != 0)) return GB_ERR_INVALID;
  if (comm->aborted) return GB_ERR_NCCL;          // error.Stopped in the reference (replicas.zig:41-43)
  if (comm->nranks == 1 || count == 0) return GB_OK;   // a single replica returns at once (replicas.zig:58)
  const ncclResult_t r = nccl().ncclAllReduce(grads, grads, count, ncclFloat32, ncclAvg, comm->comm, (cudaStream_t)stream);
  if (r != ncclSuccess && r != ncclInProgress) {
    abort_comm(comm);
    return GB_ERR_NCCL;
  }
  return settle(comm, r);   // returns once the collective is enqueued on `stream`, not when it has run
}

int gb_comm_finish(gb_comm* comm, void* stream) {
  if (!comm) return GB_ERR_INVALID;
  if (comm->aborted) return GB_ERR_NCCL;
  const auto deadline = Clock::now() + std::chrono::milliseconds(comm->timeout_ms);
  for (;;) {
    const cudaError_t q = cudaStreamQuery((cudaStream_t)stream);
    if (q == cudaSuccess) return GB_OK;
    if (q != cudaErrorNotReady) return GB_ERR_CUDA;
    if (comm->comm) {
      ncclResult_t state = ncclSuccess;
      if (nccl().ncclCommGetAsyncError(comm->comm, &state) != ncclSuccess || (state != ncclSuccess && state != ncclInProgress)) {
        abort_comm(comm);
        return GB_ERR_NCCL;
      }
    }
    if (Clock::now() > deadline) {
      abort_comm(comm);   // ends the collective that is still waiting for a peer on the device
      return GB_ERR_TIMEOUT;
    }
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

int gb_comm_abort(gb_comm* comm) {
  if (!comm) return GB_ERR_INVALID;
  abort_comm(comm);
  return GB_OK;
}

void gb_comm_destroy(gb_comm* comm) {
  if (!comm) return;
  if (comm->comm) nccl().ncclCommDestroy(comm->comm);
  delete comm;
}

}  // extern "C"
