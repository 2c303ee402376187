// NCCL plumbing of the multi-GPU path: one communicator per context over the
// GPUs of one node, used for the all-gather of the dense operand (x or B)
// that precedes the local kernel of a row shard.  Not a reference feature (the
// reference is single GPU).  NCCL is bound at run time with dlopen so that the
// library itself has no link-time dependency on it; a process that already
// loaded NCCL (PyTorch does) shares that copy.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstdio>
#include <cstring>

#include "../../include/sparsewave_b200.h"
#include "swb_kernels.h"

namespace {

// The parts of nccl.h this file needs (NCCL 2.x ABI).
struct NcclUniqueId { char internal[128]; };
using NcclComm = void *;
constexpr int kNcclFloat32 = 7, kNcclUint8 = 1;
struct NcclApi {
  int (*GetUniqueId)(NcclUniqueId *) = nullptr;
  int (*CommInitRank)(NcclComm *, int, NcclUniqueId, int) = nullptr;
  int (*CommDestroy)(NcclComm) = nullptr;
  int (*AllGather)(const void *, void *, size_t, int, NcclComm, cudaStream_t) = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
  bool ok = false;
};

NcclApi &nccl() {
  static NcclApi api;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (h) {
      api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
      api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
      api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
      api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(h, "ncclAllGather"));
      api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
      api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather && api.GetErrorString;
    }
  }
  return api;
}

int comm_fail(swb_context *ctx, int status, const char *what, const char *detail) {
  char buf[512];
  snprintf(buf, sizeof buf, "%s: %s", what, detail);
  swb::set_context_error(ctx, buf);
  return status;
}

}  // namespace

extern "C" {

int swb_comm_unique_id(uint8_t id[128]) {
  if (!id) {
    swb::set_thread_error("unique id buffer is NULL");
    return SWB_ERR_INVALID_ARGUMENT;
  }
  NcclApi &api = nccl();
  if (!api.ok) {
    swb::set_thread_error("NCCL (libnccl.so.2) could not be loaded");
    return SWB_ERR_UNSUPPORTED;
  }
  NcclUniqueId u;
  int r = api.GetUniqueId(&u);
  if (r != 0) {
    swb::set_thread_error(api.GetErrorString(r));
    return SWB_ERR_CUDA;
  }
  memcpy(id, u.internal, 128);
  return SWB_OK;
}

int swb_comm_init(swb_context *ctx, const uint8_t id[128], int n_ranks, int rank) {
  if (!ctx) {
    swb::set_thread_error("context is NULL");
    return SWB_ERR_INVALID_ARGUMENT;
  }
  if (!id || n_ranks < 1 || rank < 0 || rank >= n_ranks)
    return comm_fail(ctx, SWB_ERR_INVALID_ARGUMENT, "comm init", "bad unique id, rank or rank count");
  NcclApi &api = nccl();
  if (!api.ok) return comm_fail(ctx, SWB_ERR_UNSUPPORTED, "comm init", "NCCL (libnccl.so.2) could not be loaded");
  if (swb::context_comm(ctx)) return comm_fail(ctx, SWB_ERR_INVALID_ARGUMENT, "comm init", "the context already has a communicator");
  cudaError_t e = cudaSetDevice(swb::context_device(ctx));
  if (e != cudaSuccess) return comm_fail(ctx, SWB_ERR_CUDA, "cudaSetDevice", cudaGetErrorString(e));
  NcclUniqueId u;
  memcpy(u.internal, id, 128);
  NcclComm comm = nullptr;
  int r = api.CommInitRank(&comm, n_ranks, u, rank);
  if (r != 0) return comm_fail(ctx, SWB_ERR_CUDA, "ncclCommInitRank", api.GetErrorString(r));
  swb::set_context_comm(ctx, comm, n_ranks, rank);
  return SWB_OK;
}

int swb_comm_allgather(swb_context *ctx, const void *send, void *recv, int64_t bytes_per_rank, swb_stream stream) {
  if (!ctx) {
    swb::set_thread_error("context is NULL");
    return SWB_ERR_INVALID_ARGUMENT;
  }
  NcclComm comm = swb::context_comm(ctx);
  if (!comm) return comm_fail(ctx, SWB_ERR_INVALID_ARGUMENT, "all-gather", "the context has no communicator (swb_comm_init)");
  if (bytes_per_rank < 0 || (bytes_per_rank > 0 && (!send || !recv)))
    return comm_fail(ctx, SWB_ERR_INVALID_ARGUMENT, "all-gather", "bad buffer or size");
  if (bytes_per_rank == 0) return SWB_OK;
  cudaError_t e = cudaSetDevice(swb::context_device(ctx));
  if (e != cudaSuccess) return comm_fail(ctx, SWB_ERR_CUDA, "cudaSetDevice", cudaGetErrorString(e));
  NcclApi &api = nccl();
  int r;
  if (bytes_per_rank % 4 == 0)
    r = api.AllGather(send, recv, (size_t)(bytes_per_rank / 4), kNcclFloat32, comm, static_cast<cudaStream_t>(stream));
  else
    r = api.AllGather(send, recv, (size_t)bytes_per_rank, kNcclUint8, comm, static_cast<cudaStream_t>(stream));
  if (r != 0) return comm_fail(ctx, SWB_ERR_CUDA, "ncclAllGather", api.GetErrorString(r));
  return SWB_OK;
}

void swb_comm_destroy(swb_context *ctx) {
  if (!ctx) return;
  NcclComm comm = swb::context_comm(ctx);
  if (comm && nccl().ok) nccl().CommDestroy(comm);
  swb::set_context_comm(ctx, nullptr, 1, 0);
}

}  // extern "C"
