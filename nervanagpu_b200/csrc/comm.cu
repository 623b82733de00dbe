// Weight-gradient all-reduce across the GPUs of one NVSwitch box. The reference is single-GPU
// (nervanagpu/nervanagpu.py:491, stream None, no collective anywhere); data parallelism over the
// minibatch dimension N is an addition: fprop/bprop need no exchange, update_conv and the dW GEMMs
// sum their fp32 results over ranks. One process per GPU; NCCL is loaded at run time so that the
// single-GPU paths carry no dependency on it.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <mutex>

#include "../../include/nervana_b200.h"
#include "host.h"

namespace ngb {
namespace {

struct NcclApi {
  ncclResult_t (*getUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*commInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*commDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*commAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*allReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*commGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  const char* (*getErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

NcclApi& nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return;
    api.getUniqueId = reinterpret_cast<decltype(api.getUniqueId)>(dlsym(h, "ncclGetUniqueId"));
    api.commInitRank = reinterpret_cast<decltype(api.commInitRank)>(dlsym(h, "ncclCommInitRank"));
    api.commDestroy = reinterpret_cast<decltype(api.commDestroy)>(dlsym(h, "ncclCommDestroy"));
    api.commAbort = reinterpret_cast<decltype(api.commAbort)>(dlsym(h, "ncclCommAbort"));
    api.allReduce = reinterpret_cast<decltype(api.allReduce)>(dlsym(h, "ncclAllReduce"));
    api.commGetAsyncError = reinterpret_cast<decltype(api.commGetAsyncError)>(dlsym(h, "ncclCommGetAsyncError"));
    api.getErrorString = reinterpret_cast<decltype(api.getErrorString)>(dlsym(h, "ncclGetErrorString"));
    api.ok = api.getUniqueId && api.commInitRank && api.commDestroy && api.allReduce && api.getErrorString;
  });
  return api;
}

int nccl_fail(ncclResult_t r, const char* what) {
  return fail(NG_ERR_NCCL, "NCCL error %d (%s) in %s", static_cast<int>(r), nccl().getErrorString(r), what);
}

}  // namespace
}  // namespace ngb

using namespace ngb;

extern "C" {

int ng_comm_unique_id_bytes(void) { return static_cast<int>(sizeof(ncclUniqueId)); }

int ng_comm_unique_id(void* id_out) {
  if (!id_out) return fail(NG_ERR_INVALID_ARG, "id_out is null");
  NcclApi& api = nccl();
  if (!api.ok) return fail(NG_ERR_NCCL, "libnccl.so.2 could not be loaded");
  ncclUniqueId id;
  ncclResult_t r = api.getUniqueId(&id);
  if (r != ncclSuccess) return nccl_fail(r, "ncclGetUniqueId");
  memcpy(id_out, &id, sizeof(id));
  return NG_OK;
}

int ng_comm_init(void** comm, int nranks, int rank, const void* id_bytes) {
  if (!comm || !id_bytes) return fail(NG_ERR_INVALID_ARG, "null argument");
  if (nranks < 1 || rank < 0 || rank >= nranks) return fail(NG_ERR_INVALID_ARG, "bad rank %d of %d", rank, nranks);
  NcclApi& api = nccl();
  if (!api.ok) return fail(NG_ERR_NCCL, "libnccl.so.2 could not be loaded");
  if (!current_ctx()) return NG_ERR_CUDA;
  ncclUniqueId id;
  memcpy(&id, id_bytes, sizeof(id));
  ncclComm_t c;
  ncclResult_t r = api.commInitRank(&c, nranks, id, rank);
  if (r != ncclSuccess) return nccl_fail(r, "ncclCommInitRank");
  *comm = c;
  return NG_OK;
}

int ng_comm_allreduce_f32(void* comm, void* buf, size_t count, void* stream) {
  if (!comm || !buf) return fail(NG_ERR_INVALID_ARG, "null argument");
  NcclApi& api = nccl();
  ncclResult_t r = api.allReduce(buf, buf, count, ncclFloat32, ncclSum, static_cast<ncclComm_t>(comm),
                                 static_cast<cudaStream_t>(stream));
  if (r != ncclSuccess) return nccl_fail(r, "ncclAllReduce");
  return NG_OK;
}

int ng_comm_async_error(void* comm) {
  if (!comm) return fail(NG_ERR_INVALID_ARG, "null communicator");
  NcclApi& api = nccl();
  if (!api.commGetAsyncError) return NG_OK;
  ncclResult_t st = ncclSuccess;
  ncclResult_t r = api.commGetAsyncError(static_cast<ncclComm_t>(comm), &st);
  if (r != ncclSuccess) return nccl_fail(r, "ncclCommGetAsyncError");
  if (st != ncclSuccess && st != ncclInProgress) return nccl_fail(st, "asynchronous communicator error");
  return NG_OK;
}

int ng_comm_destroy(void* comm) {
  if (!comm) return NG_OK;
  NcclApi& api = nccl();
  ncclResult_t r = api.commDestroy(static_cast<ncclComm_t>(comm));
  if (r != ncclSuccess) return nccl_fail(r, "ncclCommDestroy");
  return NG_OK;
}

}  // extern "C"
