/*
 * libnervana_b200.so -- C ABI of the B200 (sm_100a) compute core behind the nervanagpu API.
 *
 * Every entry point takes plain pointers and sizes and returns an int status (0 = NG_OK,
 * negative = error; ng_last_error() gives the message of the last failure on this thread).
 * Device pointers are caller-owned; the library owns only its per-device workspace, loaded
 * element-wise modules and communicators. Launches are asynchronous on the given stream
 * (NULL = default stream); nothing synchronises except the calls that say so.
 *
 * Each declaration names the piece of the reference (VisionSystemsInc/nervanagpu) it replaces.
 */
#ifndef NERVANA_B200_H_
#define NERVANA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes (mirrors csrc/status.h) ------------------------------------------------ */
#define NG_OK 0
#define NG_ERR_INVALID_ARG (-1)
#define NG_ERR_UNSUPPORTED (-2)
#define NG_ERR_CUDA (-3)
#define NG_ERR_NVRTC (-4)
#define NG_ERR_NCCL (-5)
#define NG_ERR_TIMEOUT (-6)
#define NG_ERR_NOT_INITIALIZED (-7)
#define NG_ERR_TOO_LARGE (-8)

/* ---- runtime services ------------------------------------------------------------------
 * Replace the PyCUDA calls of the reference host code: pycuda.autoinit / Context
 * (README.md:67, nervanagpu/layers.py:775-778), drv.mem_alloc, memcpy_{htod,dtoh,dtod}_async,
 * memset_d{8,16,32}_async (nervanagpu/nervanagpu.py:133,145,298-311,716), drv.Event
 * (nervanagpu/nervanagpu.py:712,727-729,1348-1350). */
const char* ng_last_error(void);
int ng_init(int device);
int ng_device_count(int* count);
int ng_sm_count(int* count);
int ng_malloc(void** ptr, size_t bytes);
int ng_free(void* ptr);
int ng_host_alloc(void** ptr, size_t bytes);   /* pinned host memory */
int ng_host_free(void* ptr);
int ng_mem_info(size_t* free_bytes, size_t* total_bytes);
int ng_memcpy_h2d_async(void* dst, const void* src, size_t bytes, void* stream);
int ng_memcpy_d2h_async(void* dst, const void* src, size_t bytes, void* stream);
int ng_memcpy_d2d_async(void* dst, const void* src, size_t bytes, void* stream);
int ng_memset_d8_async(void* dst, unsigned char value, size_t count, void* stream);
int ng_memset_d16_async(void* dst, unsigned short value, size_t count, void* stream);
int ng_memset_d32_async(void* dst, unsigned int value, size_t count, void* stream);
int ng_stream_create(void** stream);
int ng_stream_destroy(void* stream);
int ng_stream_sync(void* stream);
int ng_stream_wait_event(void* stream, void* event);
int ng_event_create(void** event);
int ng_event_destroy(void* event);
int ng_event_record(void* event, void* stream);
int ng_event_sync(void* event);
int ng_event_elapsed_ms(void* start, void* end, float* ms);
/* Synchronise the device, then report (and clear) the device status words: NG_ERR_TIMEOUT if a
 * kernel abandoned one of its bounded waits (kernels of ng_hgemm_static_scratch included). */
int ng_sync(void);
int ng_device_status(int* code);
/* Every wait inside the kernels is bounded (2 s by default): a kernel whose wait runs out records
 * the site, unwinds and returns; ng_sync / ng_device_status then report NG_ERR_TIMEOUT and the
 * context stays usable. ng_set_wait_limit_ns changes the bound for later launches on the current
 * device (0 = default). ng_test_wait_expires launches one thread that waits, for at most
 * limit_ns (<= 100 ms), on a barrier nothing arrives at, so that tests can see the error path
 * work; waited_ns (device memory, may be NULL) receives how long it waited. Neither has a
 * counterpart in the reference, whose kernels do not wait on anything. */
int ng_set_wait_limit_ns(unsigned long long limit_ns);
int ng_test_wait_expires(unsigned long long limit_ns, unsigned long long* waited_ns, void* stream);
/* Number of kernels this library has launched so far in this process (its own kernels and the
 * generated element-wise ones; memcpy / memset / NCCL calls are not counted). */
int ng_launch_count(unsigned long long* count);
/* Tuning aids of the tensor-core engine (tile shape, partitions, CTA pairs ...), as the NG_*
 * environment variables set them at start-up; `name` is the variable's name without the NG_
 * prefix, in lower case ("pair_mma", "tile_rows", ...). For tests and measurements: results do
 * not depend on them beyond fp32 summation order. No counterpart in the reference. */
int ng_tune(const char* name, int value);
/* Number of GEMM / convolution calls so far that ran on the plain CUDA-core fall-back kernels
 * (operands TMA cannot address, strided layers with fewer than 64 images) instead of the
 * tensor-core engine. A benchmark that claims the tensor-core path checks that this stays 0. */
int ng_fallback_launch_count(unsigned long long* count);

/* Record-and-replay of a sequence of calls (a CUDA graph). The reference drives every kernel
 * with its own pycuda launch (nervanagpu/nervanagpu.py:642-734, 959-1105) and has nothing like
 * this; it exists because a training step of ~40 short kernels is otherwise bound by the host.
 * Between begin and end, the library's calls on `stream` (not the default stream) are recorded,
 * not run; the sequence must have run once before, so that scratch memory has its final size and
 * generated kernels are compiled. A replay repeats the recorded pointers, scalars and random
 * offsets; ng_launch_count counts the kernels of every replay. A recording also keeps the
 * library's scratch pointers of its calls: if a later, larger call on the same stream makes the
 * scratch grow, the old buffer stays allocated until the last recording is destroyed
 * (ng_graph_destroy), so replays stay valid. */
int ng_graph_capture_begin(void* stream);
int ng_graph_capture_end(void* stream, void** graph);
int ng_graph_launch(void* graph, void* stream);
int ng_graph_destroy(void* graph);

/* ---- GEMM --------------------------------------------------------------------------------
 * C[m x n] = relu?(alpha * op(A) * op(B)) + beta * C, row-major, fp16 storage, fp32 accumulate.
 * a_t: A is stored k x m; b_t: B is stored n x k; leading dimensions in elements.
 * sr_bits: 0 = round to nearest even, 1..10 = stochastic rounding keeping that many mantissa
 * bits, random bits from Philox4x32-10 keyed by `seed`, stream position `rng_offset`.
 * Replaces hgemm_{nn,nt,tn}[_vec]_{128x128,128x64,128x32,32x128} launched by NervanaGPU.dot
 * (nervanagpu/nervanagpu.py:959-1105; kernels/sass/hgemm_common_128x128.sass). */
int ng_hgemm(const void* A, const void* B, void* C, int a_t, int b_t, int m, int n, int k, int lda, int ldb, int ldc,
             float alpha, float beta, int relu, int sr_bits, unsigned long long seed, unsigned int rng_offset,
             void* stream);
/* Same contract, always on the SIMT kernel that serves operands TMA cannot address. */
int ng_hgemm_simt(const void* A, const void* B, void* C, int a_t, int b_t, int m, int n, int k, int lda, int ldb,
                  int ldc, float alpha, float beta, int relu, int sr_bits, unsigned long long seed,
                  unsigned int rng_offset, void* stream);
/* NervanaGPU.batched_dot (nervanagpu/nervanagpu.py:820-957): batch_grid independent products
 * (strides ldaz/ldbz/ldcz, 0 = operand shared), or batch_loops products summed into one C. */
int ng_hgemm_batched(const void* A, const void* B, void* C, int a_t, int b_t, int m, int n, int k, int lda, int ldb,
                     int ldc, float alpha, float beta, int relu, int sr_bits, unsigned long long seed,
                     unsigned int rng_offset, int batch_grid, int batch_loops, long long ldaz, long long ldbz,
                     long long ldcz, void* stream);

/* ng_hgemm for callers that must not allocate device memory. It has no counterpart in the
 * reference. Same arguments and result contract as ng_hgemm, restricted to operands TMA can
 * address (16-byte aligned, leading dimensions multiples of 8), computed as a split-K product
 * (when k > 64; a single 64-wide block of k is stored directly) whose fp32 partial tiles live in
 * a fixed device array inside the library instead of the cudaMalloc'ed workspace ng_hgemm grows
 * on demand. The call makes no cudaMalloc / cudaFree and calls no allocating routine.
 *   - limit: 2 * m * n * 4 bytes must fit in NG_STATIC_SCRATCH_BYTES, else NG_ERR_TOO_LARGE;
 *   - the array costs NG_STATIC_SCRATCH_BYTES of memory on every GPU that loads the library;
 *   - the first call on each device looks up the array's device address (and sets a function
 *     attribute); make that first call outside any stream capture;
 *   - all calls share the one array: calls that can overlap on the GPU (different streams or
 *     threads) race on it; issue them on one stream or serialise them yourself. Nothing in the
 *     array has to start at zero: every call overwrites the part it later reads;
 *   - its kernels' bounded waits report through a status word in the same fixed memory:
 *     ng_sync / ng_device_status include it, and ng_static_scratch_status reads (and clears) it
 *     alone, without allocating anything (it copies four bytes and so waits for the device). */
#define NG_STATIC_SCRATCH_BYTES (16u << 20)
int ng_hgemm_static_scratch(const void* A, const void* B, void* C, int a_t, int b_t, int m, int n, int k, int lda,
                            int ldb, int ldc, float alpha, float beta, int relu, int sr_bits,
                            unsigned long long seed, unsigned int rng_offset, void* stream);
int ng_static_scratch_status(int* code);

/* ---- convolution ---------------------------------------------------------------------------
 * Activations are (C,D,H,W,N), filters (C,T,R,S,K), outputs (K,M,P,Q,N), all fp16, N innermost.
 * The descriptor carries what ConvLayer stores (nervanagpu/layers.py:281-313); output
 * dimensions are M,P,Q = ceil((X - f + 1 + 2*pad) / stride) (nervanagpu/layers.py:297-301).
 * N and K must be multiples of 8 (nervanagpu/layers.py:291-292). */
typedef struct ng_conv_desc {
  int N, C, K;
  int D, H, W;
  int T, R, S;
  int pad_d, pad_h, pad_w;
  int str_d, str_h, str_w;
} ng_conv_desc;

/* Kernel family selector, for tests and benchmarks. AUTO picks the tensor-core path whenever
 * the shape allows it; the others fail with NG_ERR_UNSUPPORTED rather than switch silently. */
#define NG_PATH_AUTO 0
#define NG_PATH_TENSOR 1   /* tcgen05 implicit GEMM fed by TMA */
#define NG_PATH_SIMT 2     /* plain CUDA-core kernel, any legal shape */
#define NG_PATH_IM2COL 3   /* update only: im2col buffer + tensor-core GEMM */

int ng_conv_output_dims(const ng_conv_desc* desc, int* M, int* P, int* Q);
/* O = RN16(relu?(alpha * conv(I, F))). Replaces hconv_fprop_K64_N64 via NervanaGPU.fprop_conv
 * (nervanagpu/nervanagpu.py:642-650,671-734). */
int ng_conv_fprop(const ng_conv_desc* desc, const void* I, const void* F, void* O, float alpha, int relu, int path,
                  void* stream);
/* gradI = RN16(alpha * conv_transpose(E, F)). Replaces hconv_bprop_C64_N64 / hconv_bprop_C32_N64
 * and their dimShuffle / transpose + zero-fill pre-passes (nervanagpu/nervanagpu.py:652-659,685-693). */
int ng_conv_bprop(const ng_conv_desc* desc, const void* F, const void* E, void* gradI, float alpha, int path,
                  void* stream);
/* gradF = alpha * sum over (m,p,q,n) of I patches x E; gradF is fp32 (out_f32 = 1, what ConvLayer
 * uses, nervanagpu/layers.py:289) or fp16. Replaces hconv_updat_C128_K64 / _K128, their zero-fill
 * and fp32_convert passes (nervanagpu/nervanagpu.py:661-669,695-698,715-724). The summation
 * order is fixed (split partials in library workspace, then one ordered reduction), unlike the
 * reference's atomics. */
int ng_conv_update(const ng_conv_desc* desc, const void* I, const void* E, void* gradF, int out_f32, float alpha,
                   int path, void* stream);

/* ---- pooling -------------------------------------------------------------------------------
 * Max pooling over windows (J,T,R,S) of (C,D,H,W); what PoolLayer stores
 * (nervanagpu/layers.py:542-584). K,M,P,Q = ceil((X - f + 1 + 2*pad) / stride). */
typedef struct ng_pool_desc {
  int N, C;
  int D, H, W;
  int J, T, R, S;
  int pad_j, pad_d, pad_h, pad_w;
  int str_j, str_d, str_h, str_w;
} ng_pool_desc;

int ng_pool_output_dims(const ng_pool_desc* desc, int* K, int* M, int* P, int* Q);
/* dtype_bytes: 2 = fp16 (hpool_max), 4 = fp32 (spool_max). Replaces the mode-0 launch of
 * NervanaGPU._execute_pool (nervanagpu/nervanagpu.py:773-778,789-818). */
int ng_pool_fprop(const ng_pool_desc* desc, int dtype_bytes, const void* I, void* O, void* stream);
/* gradI[argmax of each window] += E, every other element 0 (no zero-fill pass needed). Replaces
 * the mode-1 launch and the B.fill(0) before it (nervanagpu/nervanagpu.py:780-787,811). */
int ng_pool_bprop(const ng_pool_desc* desc, int dtype_bytes, const void* I, const void* E, void* gradI, void* stream);
/* The same followed by the ReLU mask of the layer below, gradI *= (I > 0), in one pass: a window
 * whose maximum is not positive passes no error on. Equal, bit for bit, to ng_pool_bprop and then
 * the element-wise mask the reference's layers apply as a separate kernel (Layer.bprop_relu,
 * nervanagpu/layers.py:87-96), because only a window's maximum receives error at all. */
int ng_pool_bprop_relu(const ng_pool_desc* desc, int dtype_bytes, const void* I, const void* E, void* gradI,
                       void* stream);
/* The pooling ops the reference declares besides max (PoolLayer(op=...), nervanagpu/layers.py:542-552):
 * op 0 = max (the two entries above), 1 = avg, 2 = l2. The reference defines avg and l2 only in
 * numpy (benchmarks/pool_test.py:141-146: mean / root of the sum of squares over all J*T*R*S window
 * positions, positions outside the tensor counting as zeros) and launches its max kernel for every
 * op (nervanagpu/nervanagpu.py:797); here they run on the device. Their backward passes are the
 * derivatives of those definitions: gradI += E / (J*T*R*S), and gradI += E * I / O (0 where O is 0). */
int ng_pool_fprop_op(const ng_pool_desc* desc, int op, int dtype_bytes, const void* I, void* O, void* stream);
int ng_pool_bprop_op(const ng_pool_desc* desc, int op, int dtype_bytes, const void* I, const void* E, void* gradI,
                     void* stream);
/* Forward pass that records each window's argmax (one byte per output element) in a buffer of the
 * caller, and backward pass from that record, which then reads neither the input nor recomputes
 * any window. The reference's backward kernel rescans every window (hpool_max.sass mode 1,
 * launched at nervanagpu/nervanagpu.py:780-787); a training step that keeps the record between
 * its forward and backward pass saves that scan. ng_pool_argmax_bytes gives the buffer size, or 0
 * for shapes without this path (then use ng_pool_fprop / ng_pool_bprop). relu_mask as in
 * ng_pool_bprop_relu. Results equal ng_pool_fprop / ng_pool_bprop / ng_pool_bprop_relu bit for bit. */
int ng_pool_argmax_bytes(const ng_pool_desc* desc, int dtype_bytes, size_t* bytes);
int ng_pool_fprop_argmax(const ng_pool_desc* desc, int dtype_bytes, const void* I, void* O, void* argmax, void* stream);
int ng_pool_bprop_argmax(const ng_pool_desc* desc, int dtype_bytes, const void* argmax, const void* E, void* gradI,
                         int relu_mask, void* stream);

/* ---- generated element-wise kernels -----------------------------------------------------------
 * Replace pycuda.compiler.SourceModule / Function.prepare / prepared_async_call for the CUDA-C
 * source emitted by the float_ew compiler (nervanagpu/float_ew.py:1030-1035,1314). `args` is an
 * array of pointers to the argument values, in kernel-parameter order. */
int ng_ew_compile(const char* source, const char* kernel_name, int fast_math, void** handle);
/* Compile only (no device needed): checks that generated source builds for sm_100a. */
int ng_ew_compile_only(const char* source, int fast_math);
const char* ng_ew_compile_log(void);
int ng_ew_launch(void* handle, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned by, unsigned bz,
                 unsigned shared_bytes, void** args, void* stream);
int ng_ew_release(void* handle);

/* ---- multi-GPU (one process per GPU) ------------------------------------------------------------
 * No counterpart in the single-GPU reference (nervanagpu/nervanagpu.py:491); used to sum the
 * fp32 weight gradients of update_conv / dW GEMMs over the ranks that share a minibatch. */
int ng_comm_unique_id_bytes(void);
int ng_comm_unique_id(void* id_out);
int ng_comm_init(void** comm, int nranks, int rank, const void* id_bytes);
int ng_comm_allreduce_f32(void* comm, void* buf, size_t count, void* stream);
int ng_comm_async_error(void* comm);
int ng_comm_destroy(void* comm);

/* Gradient sum over peer memory fused with the SGD step, for slices of at most ng_peer_max_bytes():
 * grad[i] = sum over the GPUs of grad[i] (in rank order, the same bits everywhere), then, when
 * weights_f16 is not null, w[i] = RN16(w[i] + lr * grad[i]). One process per GPU on one NVLink box:
 * ng_peer_create allocates this GPU's staging buffer and returns its CUDA IPC handle
 * (ng_peer_handle_bytes() bytes), the host exchanges the handles of all ranks (in rank order) and passes
 * them to ng_peer_connect; every rank then calls ng_peer_sum_sgd_f32 with the same counts in the same order.
 * Waits on peers are bounded (ng_set_wait_limit_ns); a rank that gives up reports through ng_device_status.
 * Cites no reference interface: the reference is single-GPU (nervanagpu/nervanagpu.py:491). */
int ng_peer_handle_bytes(void);
size_t ng_peer_max_bytes(void);
int ng_peer_create(void** group, int nranks, int rank, void* handle_out);
int ng_peer_connect(void* group, const void* handles);
int ng_peer_sum_sgd_f32(void* group, void* grad, void* weights_f16, size_t count, float lr, void* stream);
int ng_peer_destroy(void* group);

/* ---- the reference's own C interface ---------------------------------------------------------
 * Same names and signatures as nervanagpu/kernels/C_interface/nervana_c_api.h:31-128 (bool
 * result, message on stderr). CUstream is passed as void* here; the ABI is identical.
 * hgemm is served by ng_hgemm; the fp32 sgemm entry points report failure. */
#ifndef NERVANA_B200_NO_LEGACY_DECLS
#ifdef __cplusplus
#define NG_BOOL bool
#else
#include <stdbool.h>
#define NG_BOOL bool
#endif
NG_BOOL nervana_loadKernels(const char* const base_path);
NG_BOOL nervana_unloadKernels(void);
size_t nervana_randStateSizeBytes(void);
NG_BOOL nervana_hgemm(short* A, short* B, short* C, NG_BOOL a_t, NG_BOOL b_t, int m, int n, int k, int lda, int ldb,
                      int ldc, float alpha, float beta, unsigned int* rand_state, NG_BOOL stochastic_round,
                      NG_BOOL apply_relu, void* stream, int grid);
NG_BOOL nervana_hgemm_colmajor(short* A, short* B, short* C, NG_BOOL a_t, NG_BOOL b_t, int m, int n, int k, int lda,
                               int ldb, int ldc, float alpha, float beta, unsigned int* rand_state,
                               NG_BOOL stochastic_round, NG_BOOL apply_relu, void* stream, int grid);
NG_BOOL nervana_sgemm(float* A, float* B, float* C, NG_BOOL a_t, NG_BOOL b_t, int m, int n, int k, int lda, int ldb,
                      int ldc, float alpha, float beta, unsigned int* rand_state, NG_BOOL stochastic_round,
                      NG_BOOL apply_relu, void* stream, int grid);
NG_BOOL nervana_sgemm_colmajor(float* A, float* B, float* C, NG_BOOL a_t, NG_BOOL b_t, int m, int n, int k, int lda,
                               int ldb, int ldc, float alpha, float beta, unsigned int* rand_state,
                               NG_BOOL stochastic_round, NG_BOOL apply_relu, void* stream, int grid);
#endif

#ifdef __cplusplus
}
#endif

#endif /* NERVANA_B200_H_ */
