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
/* Synchronise the device, then report (and clear) the device status word: NG_ERR_TIMEOUT if a
 * kernel abandoned one of its bounded waits. */
int ng_sync(void);
int ng_device_status(int* code);

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

#ifdef __cplusplus
}
#endif

#endif /* NERVANA_B200_H_ */
