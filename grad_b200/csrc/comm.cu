// Data-parallel gradient mean over NCCL (NVLink / NVSwitch): the device-side replacement of grad's
// host-memory `Replicas.averageGrads` (src/nn/replicas.zig:57-91).  NCCL is resolved at run time with
// dlopen, the way grad resolves libcuda and cuDNN (src/gpu/dynlib.zig:28-60), so the library carries no
// link-time dependency on it.  The reduction is an in-place ncclSum followed by one scale kernel: the
// reference sums, then multiplies by 1/N (replicas.zig:73-80); every rank ends with identical bits because
// an NCCL allreduce delivers the same result to all ranks.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstring>
#include <mutex>

#include "../../include/gradb200.h"

namespace {

struct NcclUniqueId {
  char internal[128];
};
typedef void* NcclComm;

struct NcclApi {
  int (*ncclGetUniqueId)(NcclUniqueId*);
  int (*ncclCommInitRank)(NcclComm*, int, NcclUniqueId, int);
  int (*ncclAllReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t);
  int (*ncclCommAbort)(NcclComm);
  int (*ncclCommDestroy)(NcclComm);
  bool ok = false;
};

NcclApi& nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* lib = nullptr;
    for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
      lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
      if (lib) break;
    }
    if (!lib) return;
    api.ncclGetUniqueId = (decltype(api.ncclGetUniqueId))dlsym(lib, "ncclGetUniqueId");
    api.ncclCommInitRank = (decltype(api.ncclCommInitRank))dlsym(lib, "ncclCommInitRank");
    api.ncclAllReduce = (decltype(api.ncclAllReduce))dlsym(lib, "ncclAllReduce");
    api.ncclCommAbort = (decltype(api.ncclCommAbort))dlsym(lib, "ncclCommAbort");
    api.ncclCommDestroy = (decltype(api.ncclCommDestroy))dlsym(lib, "ncclCommDestroy");
    api.ok = api.ncclGetUniqueId && api.ncclCommInitRank && api.ncclAllReduce && api.ncclCommAbort && api.ncclCommDestroy;
  });
  return api;
}

constexpr int kNcclFloat32 = 7;   // ncclFloat
constexpr int kNcclSum = 0;       // ncclSum

__global__ void scale_kernel(float* v, size_t n, float scale) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) v[i] *= scale;
}

}  // namespace

struct gb_comm {
  NcclComm comm = nullptr;
  int nranks = 1, rank = 0, device = 0;
  bool aborted = false;
};

extern "C" {

int gb_comm_unique_id(void* out128) {
  if (!out128) return GB_ERR_INVALID;
  if (!nccl().ok) return GB_ERR_NCCL;
  NcclUniqueId id;
  if (nccl().ncclGetUniqueId(&id) != 0) return GB_ERR_NCCL;
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
  if (nranks > 1) {
    if (!unique_id128) { delete c; return GB_ERR_INVALID; }
    if (!nccl().ok) { delete c; return GB_ERR_NCCL; }
    if (cudaSetDevice(device_ordinal) != cudaSuccess) { delete c; return GB_ERR_CUDA; }
    NcclUniqueId id;
    std::memcpy(&id, unique_id128, sizeof(id));
    if (nccl().ncclCommInitRank(&c->comm, nranks, id, rank) != 0) { delete c; return GB_ERR_NCCL; }
  }
  *out = c;
  return GB_OK;
}

int gb_allreduce_mean(gb_comm* comm, void* stream, float* grads, size_t count) {
  if (!comm || (!grads && count != 0)) return GB_ERR_INVALID;
  if (comm->aborted) return GB_ERR_NCCL;          // error.Stopped in the reference (replicas.zig:41-43)
  if (comm->nranks == 1 || count == 0) return GB_OK;   // a single replica returns at once (replicas.zig:58)
  if (nccl().ncclAllReduce(grads, grads, count, kNcclFloat32, kNcclSum, comm->comm, (cudaStream_t)stream) != 0) return GB_ERR_NCCL;
  const unsigned blocks = (unsigned)((count + 1023) / 1024 < 1184 ? (count + 1023) / 1024 : 1184);
  scale_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(grads, count, 1.0f / (float)comm->nranks);
  return cudaGetLastError() == cudaSuccess ? GB_OK : GB_ERR_CUDA;
}

int gb_comm_abort(gb_comm* comm) {
  if (!comm) return GB_ERR_INVALID;
  comm->aborted = true;
  if (comm->comm) {
    nccl().ncclCommAbort(comm->comm);
    comm->comm = nullptr;
  }
  return GB_OK;
}

void gb_comm_destroy(gb_comm* comm) {
  if (!comm) return;
  if (comm->comm) nccl().ncclCommDestroy(comm->comm);
  delete comm;
}

}  // extern "C"
