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
#include "common.cuh"
#include "host.h"
#include "status.h"

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

// ------------------------------------------------------------------------------------------
// Gradient sum over peer memory, fused with the SGD step.
// The last buckets of a step's gradients are small (AlexNet conv1: 93 KB) and nothing follows
// them in the step, so what they cost is latency: an NCCL all-reduce plus an element-wise kernel
// take 26 us on two GPUs and more on eight. This kernel does both in one launch per GPU. Every
// GPU has mapped the others' buffers (CUDA IPC): it stores its slice of the gradient into its own
// slot of every peer's staging area (plain stores over NVLink, nobody waits for them), fences,
// raises its flag in every peer's control block, then waits for the peers' flags in its own
// memory, sums the slots in rank order (the same bits on every GPU), stores the sum and applies
// w += lr * sum. Nothing is ever polled across NVLink. Blocks are independent: block b of every
// GPU handles the same slice and waits only for block b of the others. Every wait has a time
// limit, after which the block records NG_DEV_TIMEOUT_PEER in the device status word and returns.
// Launch k (counted per block, on every GPU alike) uses staging half k & 1; a GPU stores into a
// peer's half only after that peer has reported launch k - 2 done.
constexpr int kPeerMax = 8;
constexpr int kPeerBlocks = 64;
constexpr int kPeerThreads = 512;
constexpr size_t kPeerStageBytes = size_t(4) << 20;      // per slot: the largest slice summed this way

struct PeerCtl {                                  // in front of the staging area, one per GPU
  unsigned ready[2][kPeerMax][kPeerBlocks];       // [half][source rank][block]: launch whose slot is complete
  unsigned done[kPeerMax][kPeerBlocks];           // [reader rank][block]: last launch that rank has finished reading
  unsigned step[kPeerBlocks];                     // launches so far (private to the owner)
};
constexpr size_t kPeerCtlBytes = 8192;
static_assert(sizeof(PeerCtl) <= kPeerCtlBytes, "control block");

struct PeerArgs {
  uint8_t* base[kPeerMax];             // every rank's buffer (control block + staging slots); [rank] is local
  int nranks, rank;
};

struct PeerGroup {
  PeerArgs args;
  void* own = nullptr;
  void* opened[kPeerMax] = {};
  int device = -1;
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 ld_fresh_f4(const float4* p) {   // never from a stale L1 line
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint8_t* peer_slot(uint8_t* base, int nranks, int half, int src) {
  return base + kPeerCtlBytes + (static_cast<size_t>(half) * nranks + src) * kPeerStageBytes;
}
// one thread waits until *flag >= want (flags only grow, in this GPU's own memory); false after limit_ns
__device__ bool peer_wait(const unsigned* flag, unsigned want, uint64_t limit_ns) {
  uint64_t t0 = 0;
  for (unsigned it = 1;; ++it) {
    if (static_cast<int>(ld_acquire_sys(flag) - want) >= 0) return true;
    if ((it & 0x3f) == 0) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) return false;
    }
  }
}

__global__ void __launch_bounds__(kPeerThreads) peer_sum_sgd_kernel(PeerArgs a, float* __restrict__ grad,
                                                                   __half* __restrict__ w, long long count, float lr,
                                                                   int* status, unsigned long long limit_ns) {
  __shared__ int ok_s;
  const int b = blockIdx.x, me = a.rank, nr = a.nranks;
  PeerCtl* mine = reinterpret_cast<PeerCtl*>(a.base[me]);
  const unsigned k = mine->step[b] + 1;     // (read by every thread before thread 0 writes it back below)
  const int half = static_cast<int>(k & 1u);
  // this block's slice: whole float4 groups, the ragged tail in the last block
  const long long groups = count / 4;
  const long long per = (groups + gridDim.x - 1) / gridDim.x;
  const long long g0 = b * per, g1 = min(groups, g0 + per);
  const bool tail = b == gridDim.x - 1 && (count & 3) != 0;
  __syncthreads();
  if (threadIdx.x == 0) {
    mine->step[b] = k;
    ok_s = 1;
  }
  __syncthreads();
  // the peers' halves are free once they have reported the launch before last done
  if (threadIdx.x < nr && static_cast<int>(threadIdx.x) != me && k >= 2) {
    if (!peer_wait(&mine->done[threadIdx.x][b], k - 2, limit_ns)) {
      atomicCAS(status, 0, NG_DEV_TIMEOUT_PEER);
      ok_s = 0;
    }
  }
  __syncthreads();
  if (!ok_s) return;     // (a peer is stuck: nothing is stored anywhere)
  // my slice into my slot of every peer's staging area
  for (int r = 0; r < nr; ++r) {
    if (r == me) continue;
    float* dst = reinterpret_cast<float*>(peer_slot(a.base[r], nr, half, me));
    for (long long g = g0 + threadIdx.x; g < g1; g += blockDim.x)
      reinterpret_cast<float4*>(dst)[g] = reinterpret_cast<const float4*>(grad)[g];
    if (tail)
      for (long long i = groups * 4 + threadIdx.x; i < count; i += blockDim.x) dst[i] = grad[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < nr && static_cast<int>(threadIdx.x) != me)
    st_release_sys(&reinterpret_cast<PeerCtl*>(a.base[threadIdx.x])->ready[half][me][b], k);
  if (threadIdx.x < nr && static_cast<int>(threadIdx.x) != me) {
    if (!peer_wait(&mine->ready[half][threadIdx.x][b], k, limit_ns)) {
      atomicCAS(status, 0, NG_DEV_TIMEOUT_PEER);
      ok_s = 0;
    }
  }
  __syncthreads();
  if (!ok_s) return;     // (a peer did not arrive: the gradient and the weights stay as they are)
  // sum in rank order, store the sum, step the weights: w = RN16(w + sum * lr), the two
  // operations rounded separately as the generated element-wise kernel does
  for (long long g = g0 + threadIdx.x; g < g1; g += blockDim.x) {
    float4 s = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int r = 0; r < nr; ++r) {
      const float4 v = r == me ? reinterpret_cast<const float4*>(grad)[g]
                               : ld_fresh_f4(reinterpret_cast<const float4*>(peer_slot(a.base[me], nr, half, r)) + g);
      s.x = __fadd_rn(s.x, v.x); s.y = __fadd_rn(s.y, v.y); s.z = __fadd_rn(s.z, v.z); s.w = __fadd_rn(s.w, v.w);
    }
    reinterpret_cast<float4*>(grad)[g] = s;
    if (w) {
      __half2* wp = reinterpret_cast<__half2*>(w) + 2 * g;
      const float2 w0 = __half22float2(wp[0]), w1 = __half22float2(wp[1]);
      wp[0] = __floats2half2_rn(__fadd_rn(w0.x, __fmul_rn(s.x, lr)), __fadd_rn(w0.y, __fmul_rn(s.y, lr)));
      wp[1] = __floats2half2_rn(__fadd_rn(w1.x, __fmul_rn(s.z, lr)), __fadd_rn(w1.y, __fmul_rn(s.w, lr)));
    }
  }
  if (tail)
    for (long long i = groups * 4 + threadIdx.x; i < count; i += blockDim.x) {
      float s = 0.0f;
      for (int r = 0; r < nr; ++r) {
        const volatile float* sp = reinterpret_cast<const volatile float*>(peer_slot(a.base[me], nr, half, r));
        s = __fadd_rn(s, r == me ? grad[i] : sp[i]);
      }
      grad[i] = s;
      if (w) w[i] = __float2half_rn(__fadd_rn(__half2float(w[i]), __fmul_rn(s, lr)));
    }
  __syncthreads();
  // tell every peer that its slot in this half has been read
  if (threadIdx.x < nr && static_cast<int>(threadIdx.x) != me)
    st_release_sys(&reinterpret_cast<PeerCtl*>(a.base[threadIdx.x])->done[me][b], k);
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

int ng_peer_handle_bytes(void) { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }

size_t ng_peer_max_bytes(void) { return kPeerStageBytes; }

int ng_peer_create(void** group, int nranks, int rank, void* handle_out) {
  if (!group || !handle_out) return fail(NG_ERR_INVALID_ARG, "null argument");
  if (nranks < 1 || nranks > kPeerMax || rank < 0 || rank >= nranks)
    return fail(NG_ERR_INVALID_ARG, "bad rank %d of %d (at most %d GPUs)", rank, nranks, kPeerMax);
  DeviceCtx* c = current_ctx();
  if (!c) return NG_ERR_CUDA;
  PeerGroup* g = new PeerGroup();
  g->device = c->device;
  g->args.nranks = nranks;
  g->args.rank = rank;
  const size_t bytes = kPeerCtlBytes + 2 * static_cast<size_t>(nranks) * kPeerStageBytes;
  cudaError_t e = cudaMalloc(&g->own, bytes);
  if (e == cudaSuccess) e = cudaMemset(g->own, 0, bytes);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, g->own);
  if (e != cudaSuccess) {
    if (g->own) cudaFree(g->own);
    delete g;
    return cuda_fail(e, "peer staging buffer");
  }
  memcpy(handle_out, &h, sizeof(h));
  g->args.base[rank] = static_cast<uint8_t*>(g->own);
  *group = g;
  return NG_OK;
}

int ng_peer_connect(void* group, const void* handles) {
  PeerGroup* g = static_cast<PeerGroup*>(group);
  if (!g || !handles) return fail(NG_ERR_INVALID_ARG, "null argument");
  for (int r = 0; r < g->args.nranks; ++r) {
    if (r == g->args.rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, static_cast<const uint8_t*>(handles) + r * sizeof(h), sizeof(h));
    void* p = nullptr;
    NG_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    g->opened[r] = p;
    g->args.base[r] = static_cast<uint8_t*>(p);
  }
  return NG_OK;
}

int ng_peer_sum_sgd_f32(void* group, void* grad, void* weights_f16, size_t count, float lr, void* stream) {
  PeerGroup* g = static_cast<PeerGroup*>(group);
  if (!g || !grad) return fail(NG_ERR_INVALID_ARG, "null argument");
  if (count * sizeof(float) > kPeerStageBytes)
    return fail(NG_ERR_TOO_LARGE, "%zu floats exceed the peer staging buffer (%zu bytes)", count, kPeerStageBytes);
  if ((reinterpret_cast<uintptr_t>(grad) & 15u) || (reinterpret_cast<uintptr_t>(weights_f16) & 7u))
    return fail(NG_ERR_INVALID_ARG, "gradient / weight slices must start on 16 / 8 byte boundaries");
  DeviceCtx* c = current_ctx();
  if (!c) return NG_ERR_CUDA;
  for (int r = 0; r < g->args.nranks; ++r)
    if (!g->args.base[r]) return fail(NG_ERR_INVALID_ARG, "peer group is not connected");
  if (count == 0) return NG_OK;
  peer_sum_sgd_kernel<<<kPeerBlocks, kPeerThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      g->args, static_cast<float*>(grad), static_cast<__half*>(weights_f16), static_cast<long long>(count), lr,
      c->status, c->wait_limit_ns);
  NG_CHECK_LAUNCH();
  return NG_OK;
}

int ng_peer_destroy(void* group) {
  PeerGroup* g = static_cast<PeerGroup*>(group);
  if (!g) return NG_OK;
  cudaDeviceSynchronize();
  for (int r = 0; r < g->args.nranks; ++r)
    if (g->opened[r]) cudaIpcCloseMemHandle(g->opened[r]);
  if (g->own) cudaFree(g->own);
  delete g;
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
