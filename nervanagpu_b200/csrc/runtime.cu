// Runtime services of the C-ABI: device selection, memory, copies, memsets, streams, events,
// error strings. They stand in for the PyCUDA calls the reference's host code makes
// (nervanagpu/nervanagpu.py:133,145,298-311,712-729,1333-1350; nervanagpu/layers.py:775-778).
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>

#include "../../include/nervana_b200.h"
#include "host.h"

namespace ngb {

static thread_local std::string g_last_error;

int fail(int code, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(NG_ERR_CUDA, "CUDA error %d (%s) in %s", static_cast<int>(e), cudaGetErrorString(e), what);
}

static Tuning g_tuning;
Tuning& tuning_mutable() { return const_cast<Tuning&>(tuning()); }

const Tuning& tuning() {
  Tuning& t = g_tuning;
  static std::once_flag once;
  std::call_once(once, [] {
    Tuning& t = g_tuning;
    auto num = [](const char* name, int unset) {
      const char* v = getenv(name);
      return v && *v ? atoi(v) : unset;
    };
    t.tile_rows = num("NG_TILE_ROWS", 0);
    t.tile_cols = num("NG_TILE_COLS", 0);
    t.kb_rows = num("NG_KB_ROWS", 0);
    t.reduce_lanes = num("NG_REDUCE_LANES", 0);
    t.update_groups = num("NG_UPDATE_GROUPS", 0);
    t.update_stack = num("NG_UPDATE_STACK", 0);
    t.update_min_stages = num("NG_UPDATE_MIN_STAGES", 0);
    t.merge_boxes = num("NG_MERGE_BOXES", -1);
    t.split_tail = num("NG_SPLIT_TAIL", -1);
    t.lean_kernels = num("NG_LEAN_KERNELS", -1);
    t.update_swap = num("NG_UPDATE_SWAP", -1);
    t.pair_mma = num("NG_PAIR_MMA", -1);
    t.chan_block = num("NG_CHAN_BLOCK", -1);
    t.space_to_depth = num("NG_SPACE_TO_DEPTH", -1);
    t.dependent_launch = num("NG_DEPENDENT_LAUNCH", -1);
    t.max_ctas = num("NG_MAX_CTAS", 0);
    t.conv_splits = num("NG_CONV_SPLITS", -1);
    t.max_stages = num("NG_MAX_STAGES", 0);
    t.feed_bytes_per_ns = num("NG_FEED_BYTES_PER_NS", 0);
  });
  return t;
}

static std::atomic<unsigned long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
static std::atomic<unsigned long long> g_fallback_launches{0};
void count_fallback_launch() { g_fallback_launches.fetch_add(1, std::memory_order_relaxed); }

static std::mutex g_ctx_mutex;
static DeviceCtx g_ctx[64];

DeviceCtx* current_ctx() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    cuda_fail(e, "cudaGetDevice");
    return nullptr;
  }
  if (dev < 0 || dev >= 64) {
    fail(NG_ERR_INVALID_ARG, "device index %d out of range", dev);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_ctx_mutex);
  DeviceCtx* c = &g_ctx[dev];
  if (c->device == dev) return c;
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, dev);
  if (e != cudaSuccess) {
    cuda_fail(e, "cudaGetDeviceProperties");
    return nullptr;
  }
  if (prop.major != 10) {
    fail(NG_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library contains sm_100a code only", dev, prop.major,
         prop.minor);
    return nullptr;
  }
  e = cudaMalloc(&c->status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(c->status, 0, sizeof(int));
  if (e != cudaSuccess) {
    cuda_fail(e, "status word allocation");
    return nullptr;
  }
  c->sm_count = prop.multiProcessorCount;
  c->device = dev;
  return c;
}

// grows one scratch buffer to at least `bytes`
static int grow_scratch(DeviceCtx* c, DeviceCtx::Scratch& s, size_t bytes) {
  if (bytes > s.bytes) {
    if (c->capturing) {
      return fail(NG_ERR_UNSUPPORTED,
                  "the workspace would have to grow during a capture: run the sequence once before recording it");
    }
    // growing: earlier launches may still read the old buffer, and so does every replay of a
    // recorded sequence that was recorded with it
    NG_CUDA(cudaDeviceSynchronize());
    if (s.ptr) {
      if (c->live_graphs > 0) c->retired.push_back(s.ptr);
      else NG_CUDA(cudaFree(s.ptr));
    }
    s.ptr = nullptr;
    s.bytes = 0;
    size_t want = bytes + (bytes >> 2);
    want = (want + (1u << 20) - 1) & ~((size_t(1) << 20) - 1);
    NG_CUDA(cudaMalloc(&s.ptr, want));
    s.bytes = want;
  }
  return NG_OK;
}

int ensure_workspace(DeviceCtx* c, cudaStream_t stream, size_t bytes) {
  // one scratch buffer per stream: calls queued on different streams may run at the same time
  DeviceCtx::Scratch& s = c->scratch[stream];
  const int rc = grow_scratch(c, s, bytes);
  if (rc != NG_OK) return rc;
  c->ws = s.ptr;
  c->ws_bytes = s.bytes;
  return NG_OK;
}

int ensure_aux(DeviceCtx* c, cudaStream_t stream, size_t bytes, void** ptr) {
  DeviceCtx::Scratch& s = c->aux[stream];
  const int rc = grow_scratch(c, s, bytes);
  if (rc != NG_OK) return rc;
  *ptr = s.ptr;
  return NG_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tensor_map(CUtensorMap* out, const void* base, const uint64_t dims[5], const uint64_t strides_bytes[4],
                    const uint32_t box[5], int elem_bytes) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return fail(NG_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available from the driver");
  cuuint64_t gdim[5], gstr[4];
  cuuint32_t bdim[5], estr[5];
  for (int i = 0; i < 5; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estr[i] = 1;
  }
  for (int i = 0; i < 4; ++i) gstr[i] = strides_bytes[i];
  const uint32_t inner_bytes = box[0] * elem_bytes;
  CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_NONE;
  if (inner_bytes == 128) sw = CU_TENSOR_MAP_SWIZZLE_128B;
  else if (inner_bytes == 64) sw = CU_TENSOR_MAP_SWIZZLE_64B;
  else if (inner_bytes == 32) sw = CU_TENSOR_MAP_SWIZZLE_32B;
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(out, dt, 5, const_cast<void*>(base), gdim, gstr, bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(NG_ERR_CUDA,
                "cuTensorMapEncodeTiled failed (%d): base=%p dims=(%llu,%llu,%llu,%llu,%llu) strides=(%llu,%llu,%llu,%llu) "
                "box=(%u,%u,%u,%u,%u)",
                static_cast<int>(r), base, (unsigned long long)dims[0], (unsigned long long)dims[1],
                (unsigned long long)dims[2], (unsigned long long)dims[3], (unsigned long long)dims[4],
                (unsigned long long)strides_bytes[0], (unsigned long long)strides_bytes[1],
                (unsigned long long)strides_bytes[2], (unsigned long long)strides_bytes[3], box[0], box[1], box[2],
                box[3], box[4]);
  return NG_OK;
}

}  // namespace ngb

using namespace ngb;

namespace {
template <typename T>
__global__ void fill_kernel(T* dst, T value, size_t count) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < count;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    dst[i] = value;
}
template <typename T>
int fill(void* dst, T value, size_t count, void* stream) {
  if (count == 0) return NG_OK;
  DeviceCtx* c = current_ctx();
  if (!c) return NG_ERR_CUDA;
  const int threads = 256;
  size_t blocks = (count + threads - 1) / threads;
  const size_t cap = static_cast<size_t>(c->sm_count) * 16;
  if (blocks > cap) blocks = cap;
  fill_kernel<T><<<static_cast<unsigned>(blocks), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<T*>(dst), value, count);
  NG_CHECK_LAUNCH();
  return NG_OK;
}
}  // namespace

extern "C" {

const char* ng_last_error(void) { return g_last_error.c_str(); }

int ng_init(int device) {
  NG_CUDA(cudaSetDevice(device));
  return current_ctx() ? NG_OK : NG_ERR_CUDA;
}

int ng_device_count(int* count) {
  if (!count) return fail(NG_ERR_INVALID_ARG, "count is null");
  NG_CUDA(cudaGetDeviceCount(count));
  return NG_OK;
}

int ng_sm_count(int* count) {
  if (!count) return fail(NG_ERR_INVALID_ARG, "count is null");
  DeviceCtx* c = current_ctx();
  if (!c) return NG_ERR_CUDA;
  *count = c->sm_count;
  return NG_OK;
}

int ng_malloc(void** ptr, size_t bytes) {
  if (!ptr) return fail(NG_ERR_INVALID_ARG, "ptr is null");
  NG_CUDA(cudaMalloc(ptr, bytes ? bytes : 1));
  return NG_OK;
}

int ng_free(void* ptr) {
  if (ptr) NG_CUDA(cudaFree(ptr));
  return NG_OK;
}

int ng_host_alloc(void** ptr, size_t bytes) {
  if (!ptr) return fail(NG_ERR_INVALID_ARG, "ptr is null");
  NG_CUDA(cudaHostAlloc(ptr, bytes ? bytes : 1, cudaHostAllocDefault));
  return NG_OK;
}

int ng_host_free(void* ptr) {
  if (ptr) NG_CUDA(cudaFreeHost(ptr));
  return NG_OK;
}

int ng_mem_info(size_t* free_bytes, size_t* total_bytes) {
  NG_CUDA(cudaMemGetInfo(free_bytes, total_bytes));
  return NG_OK;
}

int ng_memcpy_h2d_async(void* dst, const void* src, size_t bytes, void* stream) {
  NG_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
  return NG_OK;
}

int ng_memcpy_d2h_async(void* dst, const void* src, size_t bytes, void* stream) {
  NG_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
  return NG_OK;
}

int ng_memcpy_d2d_async(void* dst, const void* src, size_t bytes, void* stream) {
  NG_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
  return NG_OK;
}

int ng_memset_d8_async(void* dst, unsigned char value, size_t count, void* stream) {
  NG_CUDA(cudaMemsetAsync(dst, value, count, static_cast<cudaStream_t>(stream)));
  return NG_OK;
}


int ng_memset_d16_async(void* dst, unsigned short value, size_t count, void* stream) {
  if (value == 0) return ng_memset_d8_async(dst, 0, count * 2, stream);
  return fill<unsigned short>(dst, value, count, stream);
}

int ng_memset_d32_async(void* dst, unsigned int value, size_t count, void* stream) {
  if (value == 0) return ng_memset_d8_async(dst, 0, count * 4, stream);
  return fill<unsigned int>(dst, value, count, stream);
}

int ng_stream_create(void** stream) {
  cudaStream_t s;
  NG_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *stream = s;
  return NG_OK;
}

int ng_stream_destroy(void* stream) {
  NG_CUDA(cudaStreamDestroy(static_cast<cudaStream_t>(stream)));
  return NG_OK;
}

int ng_stream_sync(void* stream) {
  NG_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  return NG_OK;
}

int ng_stream_wait_event(void* stream, void* event) {
  NG_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(event), 0));
  return NG_OK;
}

int ng_event_create(void** event) {
  cudaEvent_t e;
  NG_CUDA(cudaEventCreate(&e));
  *event = e;
  return NG_OK;
}

int ng_event_destroy(void* event) {
  NG_CUDA(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
  return NG_OK;
}

int ng_event_record(void* event, void* stream) {
  NG_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)));
  return NG_OK;
}

int ng_event_sync(void* event) {
  NG_CUDA(cudaEventSynchronize(static_cast<cudaEvent_t>(event)));
  return NG_OK;
}

int ng_event_elapsed_ms(void* start, void* end, float* ms) {
  NG_CUDA(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(end)));
  return NG_OK;
}

int ng_device_status(int* code) {
  DeviceCtx* c = current_ctx();
  if (!c) return NG_ERR_CUDA;
  int v = 0;
  NG_CUDA(cudaMemcpy(&v, c->status, sizeof(int), cudaMemcpyDeviceToHost));
  if (code) *code = v;
  if (v != 0) cudaMemset(c->status, 0, sizeof(int));
  // kernels launched by ng_hgemm_static_scratch report through a status word of their own
  int vs = 0;
  const int rc = static_scratch_status(c->device, &vs);
  if (rc != NG_OK) return rc;
  if (v == 0) v = vs;
  if (code) *code = v;
  if (v != 0) return fail(NG_ERR_TIMEOUT, "a kernel gave up a bounded wait (site %d)", v);
  return NG_OK;
}

int ng_launch_count(unsigned long long* count) {
  if (!count) return fail(NG_ERR_INVALID_ARG, "count is null");
  *count = g_launches.load(std::memory_order_relaxed);
  return NG_OK;
}

int ng_tune(const char* name, int value) {
  if (!name) return fail(NG_ERR_INVALID_ARG, "name is null");
  Tuning& t = tuning_mutable();
  struct Field { const char* name; int* slot; };
  const Field fields[] = {
      {"tile_rows", &t.tile_rows}, {"tile_cols", &t.tile_cols}, {"kb_rows", &t.kb_rows},
      {"reduce_lanes", &t.reduce_lanes}, {"update_groups", &t.update_groups}, {"update_stack", &t.update_stack},
      {"update_min_stages", &t.update_min_stages}, {"max_ctas", &t.max_ctas}, {"conv_splits", &t.conv_splits},
      {"max_stages", &t.max_stages}, {"feed_bytes_per_ns", &t.feed_bytes_per_ns}, {"merge_boxes", &t.merge_boxes}, {"split_tail", &t.split_tail},
      {"lean_kernels", &t.lean_kernels}, {"update_swap", &t.update_swap}, {"pair_mma", &t.pair_mma}, {"chan_block", &t.chan_block}, {"space_to_depth", &t.space_to_depth}, {"dependent_launch", &t.dependent_launch}};
  for (const Field& f : fields)
    if (strcmp(f.name, name) == 0) {
      *f.slot = value;
      return NG_OK;
    }
  return fail(NG_ERR_INVALID_ARG, "unknown tuning field '%s'", name);
}

int ng_fallback_launch_count(unsigned long long* count) {
  if (!count) return fail(NG_ERR_INVALID_ARG, "count is null");
  *count = g_fallback_launches.load(std::memory_order_relaxed);
  return NG_OK;
}

int ng_sync(void) {
  NG_CUDA(cudaDeviceSynchronize());
  return ng_device_status(nullptr);
}

// ---- replaying a recorded sequence of calls (CUDA graphs) ---------------------------------
// Between ng_graph_capture_begin and ng_graph_capture_end every call of this library on `stream`
// is recorded instead of run. The recording keeps the pointers, shapes, scalars and random
// offsets of the calls; replaying it costs one launch on the host.
struct NgGraph {
  cudaGraphExec_t exec = nullptr;
  DeviceCtx* ctx = nullptr;
  unsigned long long kernels = 0;   // kernel launches one replay stands for
};

int ng_graph_capture_begin(void* stream) {
  DeviceCtx* c = current_ctx();
  if (!c) return NG_ERR_CUDA;
  if (!stream) return fail(NG_ERR_INVALID_ARG, "capture needs a stream of its own, not the default stream");
  if (c->capturing) return fail(NG_ERR_INVALID_ARG, "a capture is already open");
  NG_CUDA(cudaStreamBeginCapture(static_cast<cudaStream_t>(stream), cudaStreamCaptureModeThreadLocal));
  c->capturing = true;
  c->capture_launches0 = g_launches.load(std::memory_order_relaxed);
  return NG_OK;
}

int ng_graph_capture_end(void* stream, void** graph_out) {
  DeviceCtx* c = current_ctx();
  if (!c) return NG_ERR_CUDA;
  if (!c->capturing) return fail(NG_ERR_INVALID_ARG, "no capture is open");
  c->capturing = false;
  cudaGraph_t graph = nullptr;
  NG_CUDA(cudaStreamEndCapture(static_cast<cudaStream_t>(stream), &graph));
  if (!graph_out) {
    cudaGraphDestroy(graph);
    return fail(NG_ERR_INVALID_ARG, "graph_out is null");
  }
  NgGraph* g = new NgGraph;
  cudaError_t e = cudaGraphInstantiate(&g->exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) {
    delete g;
    return cuda_fail(e, "cudaGraphInstantiate");
  }
  const unsigned long long now = g_launches.load(std::memory_order_relaxed);
  g->kernels = now - c->capture_launches0;
  g->ctx = c;
  ++c->live_graphs;
  // the recorded launches did not run
  g_launches.fetch_sub(g->kernels, std::memory_order_relaxed);
  *graph_out = g;
  return NG_OK;
}

int ng_graph_launch(void* graph, void* stream) {
  NgGraph* g = static_cast<NgGraph*>(graph);
  if (!g || !g->exec) return fail(NG_ERR_INVALID_ARG, "graph is null");
  NG_CUDA(cudaGraphLaunch(g->exec, static_cast<cudaStream_t>(stream)));
  g_launches.fetch_add(g->kernels, std::memory_order_relaxed);
  return NG_OK;
}

int ng_graph_destroy(void* graph) {
  NgGraph* g = static_cast<NgGraph*>(graph);
  if (!g) return NG_OK;
  if (g->exec) NG_CUDA(cudaGraphExecDestroy(g->exec));
  if (g->ctx && --g->ctx->live_graphs == 0) {
    // scratch buffers that recordings were still pointing at
    for (void* ptr : g->ctx->retired) cudaFree(ptr);
    g->ctx->retired.clear();
  }
  delete g;
  return NG_OK;
}

}  // extern "C"
