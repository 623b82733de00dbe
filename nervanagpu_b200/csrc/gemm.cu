// ng.dot on the device: C = relu?(alpha * op(A) * op(B)) + beta * C, fp16 in, fp32 accumulate,
// fp16 out with round-to-nearest-even or stochastic rounding.
// Mirrors NervanaGPU.dot / batched_dot (nervanagpu/nervanagpu.py:820-1105) and the C interface
// nervana_hgemm (nervanagpu/kernels/C_interface/nervana_c_api.h:31-128).
//
// Shapes whose operands TMA can address (16-byte aligned base, leading dimensions that are
// multiples of 8 elements) run on the tcgen05 engine; anything else runs on a plain SIMT
// kernel so that every legal call of the reference API still executes on the GPU.
#include <algorithm>

#include "../../include/nervana_b200.h"
#include "epilogue.cuh"
#include "host.h"

namespace ngb {

namespace {

// ------------------------------------------------------------------------------------------
// SIMT fallback: 64x64 tile per CTA, 4x4 outputs per thread, arbitrary strides.
// ------------------------------------------------------------------------------------------
struct SimtGemmArgs {
  const __half* A;
  const __half* B;
  void* C;
  int a_t, b_t;
  int m, n, k;
  long long lda, ldb, ldc;
  long long az, bz, cz;   // batch strides (elements)
  int loops;              // batches accumulated into one output
  long long alz, blz;     // strides between accumulated batches
  int out_f32;
  EpiArgs ea;
};

__global__ void __launch_bounds__(256) gemm_simt_kernel(SimtGemmArgs g) {
  __shared__ float sA[16][64 + 1];
  __shared__ float sB[16][64 + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const int z = blockIdx.z;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int l = 0; l < g.loops; ++l) {
    const __half* A = g.A + z * g.az + l * g.alz;
    const __half* B = g.B + z * g.bz + l * g.blz;
    for (int k0 = 0; k0 < g.k; k0 += 16) {
      for (int i = threadIdx.x; i < 16 * 64; i += 256) {
        int kk, mm;
        if (g.a_t) { mm = i & 63; kk = i >> 6; } else { kk = i & 15; mm = i >> 4; }
        const int gm = m0 + mm, gk = k0 + kk;
        float v = 0.0f;
        if (gm < g.m && gk < g.k) v = __half2float(g.a_t ? A[gk * g.lda + gm] : A[gm * g.lda + gk]);
        sA[kk][mm] = v;
      }
      for (int i = threadIdx.x; i < 16 * 64; i += 256) {
        int kk, nn;
        if (g.b_t) { kk = i & 15; nn = i >> 4; } else { nn = i & 63; kk = i >> 6; }
        const int gn = n0 + nn, gk = k0 + kk;
        float v = 0.0f;
        if (gn < g.n && gk < g.k) v = __half2float(g.b_t ? B[gn * g.ldb + gk] : B[gk * g.ldb + gn]);
        sB[kk][nn] = v;
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < 16; ++kk) {
        float a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = sA[kk][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = sB[kk][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
      __syncthreads();
    }
  }
  for (int i = 0; i < 4; ++i) {
    const int row = m0 + ty * 4 + i;
    if (row >= g.m) continue;
    for (int j = 0; j < 4; ++j) {
      const int col = n0 + tx * 4 + j;
      if (col >= g.n) continue;
      const long long off = z * g.cz + row * g.ldc + col;
      float c = epi_scale(g.ea, acc[i][j]);
      if (g.out_f32) {
        float* out = static_cast<float*>(g.C) + off;
        if (g.ea.beta != 0.0f) c = fmaf(g.ea.beta, *out, c);
        *out = c;
      } else {
        __half* out = static_cast<__half*>(g.C) + off;
        if (g.ea.beta != 0.0f) c = fmaf(g.ea.beta, __half2float(*out), c);
        if (g.ea.sr_bits) {
          const unsigned long long lin = (static_cast<unsigned long long>(z) * g.m + row) * g.n + col;
          uint32_t rnd[8];
          sr_bits8(g.ea, lin >> 3, rnd);
          *out = f2h_sr(c, rnd[lin & 7ull], g.ea.sr_bits);
        } else {
          *out = f2h_rn(c);
        }
      }
    }
  }
}

bool tma_ok(const void* p, long long ld) {
  return (reinterpret_cast<uintptr_t>(p) & 15u) == 0 && (ld & 7) == 0;
}

}  // namespace

int run_gemm(const GemmCall& g, cudaStream_t stream) {
  if (!g.A || !g.B || !g.C) return fail(NG_ERR_INVALID_ARG, "null operand");
  if (g.m <= 0 || g.n <= 0 || g.k <= 0) return fail(NG_ERR_INVALID_ARG, "m, n, k must be positive");
  if (g.a_t && g.b_t) return fail(NG_ERR_UNSUPPORTED, "op 'tt' is not supported");
  if (g.sr_bits < 0 || g.sr_bits > 10) return fail(NG_ERR_INVALID_ARG, "stochastic rounding keeps 1..10 mantissa bits");
  const long long min_lda = g.a_t ? g.m : g.k, min_ldb = g.b_t ? g.k : g.n;
  if (g.lda < min_lda || g.ldb < min_ldb || g.ldc < g.n) return fail(NG_ERR_INVALID_ARG, "leading dimension too small");
  DeviceCtx* c = current_ctx();
  if (!c) return NG_ERR_CUDA;

  EpiArgs ea;
  ea.alpha = g.alpha; ea.beta = g.beta; ea.relu = g.relu; ea.sr_bits = g.sr_bits;
  ea.seed_lo = static_cast<uint32_t>(g.seed); ea.seed_hi = static_cast<uint32_t>(g.seed >> 32);
  ea.rng_offset = g.rng_offset;

  const bool batched_ok = g.loops == 1 && (g.az % 8 == 0) && (g.bz % 8 == 0);
  const bool use_tc = !g.force_simt && tma_ok(g.A, g.lda) && tma_ok(g.B, g.ldb) && batched_ok;
  if (!use_tc) {
    SimtGemmArgs s;
    s.A = static_cast<const __half*>(g.A); s.B = static_cast<const __half*>(g.B); s.C = g.C;
    s.a_t = g.a_t; s.b_t = g.b_t; s.m = g.m; s.n = g.n; s.k = g.k;
    s.lda = g.lda; s.ldb = g.ldb; s.ldc = g.ldc;
    s.az = g.az; s.bz = g.bz; s.cz = g.cz; s.loops = g.loops; s.alz = g.alz; s.blz = g.blz;
    s.out_f32 = g.out_f32; s.ea = ea;
    dim3 grid((g.n + 63) / 64, (g.m + 63) / 64, g.batch);
    count_fallback_launch();
    gemm_simt_kernel<<<grid, 256, 0, stream>>>(s);
    NG_CHECK_LAUNCH();
    return NG_OK;
  }

  TcParams p = {};
  p.mode = TC_GEMM;
  p.block_n = g.n <= 64 ? 64 : (g.n <= 128 ? 128 : 256);
  p.M = g.m; p.N = g.n;
  p.tiles_n = (g.n + p.block_n - 1) / p.block_n;
  p.nz = g.batch;
  p.num_kb = (g.k + kChunk - 1) / kChunk;
  tc_pick_tile_rows(c, p, static_cast<long long>(p.tiles_n) * p.nz, p.num_kb);
  // Two or more row tiles and 128 or 256 columns: CTA pairs (a 256-row tile over two SMs, each of
  // which loads half of the B columns).
  if (tuning().pair_mma == 1 && g.m > kTileM && p.block_n >= 128) {
    p.pair = 1;
    p.m_halves = 1;
    p.tiles_m = (g.m + 2 * kTileM - 1) / (2 * kTileM);
  }
  const int bn_cta = p.pair ? p.block_n / 2 : p.block_n;
  TcOperandLayout lay;
  lay.a_mn_major = g.a_t ? 1 : 0;   // stored k x m: m contiguous
  lay.b_mn_major = g.b_t ? 0 : 1;   // stored k x n: n contiguous
  lay.kb_rows = kChunk;
  // an operand whose contiguous dimension is m (or n), a multiple of 64: the map gets the 64-wide
  // chunk number as a dimension of its own, and one box brings a 128-row half (a column tile)
  const bool merge_off = tuning().merge_boxes == 0;
  lay.a_merge = !merge_off && g.a_t && g.m % kChunk == 0;
  lay.b_merge_static = !merge_off && !g.b_t && g.n % kChunk == 0 && bn_cta >= 2 * kChunk;
  tc_fill_mma(p, lay);
  p.a_zmul = g.az != 0; p.b_zmul = g.bz != 0;
  p.C = g.C; p.Cold = g.beta != 0.0f ? g.C : nullptr;
  p.ldc = g.ldc; p.c_zstride = g.cz;
  p.alpha = g.alpha; p.beta = g.beta; p.relu = g.relu; p.sr_bits = g.sr_bits; p.out_f32 = g.out_f32;
  const int esz = g.out_f32 ? 4 : 2;
  const int vec_elems = 16 / esz;
  p.vec_ok = (reinterpret_cast<uintptr_t>(g.C) & 15u) == 0 && g.ldc % vec_elems == 0 && g.cz % vec_elems == 0;
  p.seed_lo = ea.seed_lo; p.seed_hi = ea.seed_hi; p.rng_offset = g.rng_offset;
  p.splits = choose_splits(c, static_cast<long long>(p.tiles_m) * p.tiles_n * p.nz, p.num_kb,
                           static_cast<long long>(g.m) * g.n * g.batch);

  // Tensor maps. Dimension 0 is the contiguous one; dimension 2 walks the batch.
  CUtensorMap mapA, mapB;
  {
    uint64_t dims[5] = {1, 1, 1, 1, 1};
    uint64_t str[4] = {16, 16, 16, 16};
    uint32_t box[5] = {kChunk, 1, 1, 1, 1};
    if (g.a_t) { dims[0] = g.m; dims[1] = g.k; box[1] = kChunk; }
    else       { dims[0] = g.k; dims[1] = g.m; box[1] = kTileM * p.m_halves; }
    dims[2] = g.az != 0 ? g.batch : 1;
    str[0] = static_cast<uint64_t>(g.lda) * 2;
    str[1] = g.az != 0 ? static_cast<uint64_t>(g.az) * 2 : str[0] * dims[1];
    str[2] = str[1] * dims[2];
    str[3] = str[2];
    if (lay.a_merge) {   // (m_lo, k, m_hi, batch)
      dims[0] = kChunk; dims[1] = g.k; dims[2] = g.m / kChunk; dims[3] = g.az != 0 ? g.batch : 1;
      str[0] = static_cast<uint64_t>(g.lda) * 2; str[1] = 128;
      str[2] = g.az != 0 ? static_cast<uint64_t>(g.az) * 2 : str[0] * dims[1];
      str[3] = str[2] * dims[3];
      box[1] = kChunk; box[2] = 2;
    }
    int rc = make_tensor_map(&mapA, g.A, dims, str, box);
    if (rc != NG_OK) return rc;
  }
  {
    uint64_t dims[5] = {1, 1, 1, 1, 1};
    uint64_t str[4] = {16, 16, 16, 16};
    uint32_t box[5] = {kChunk, 1, 1, 1, 1};
    if (g.b_t) { dims[0] = g.k; dims[1] = g.n; box[1] = bn_cta; }
    else       { dims[0] = g.n; dims[1] = g.k; box[1] = kChunk; }
    dims[2] = g.bz != 0 ? g.batch : 1;
    str[0] = static_cast<uint64_t>(g.ldb) * 2;
    str[1] = g.bz != 0 ? static_cast<uint64_t>(g.bz) * 2 : str[0] * dims[1];
    str[2] = str[1] * dims[2];
    str[3] = str[2];
    if (lay.b_merge_static) {   // (n_lo, k, n_hi, batch)
      dims[0] = kChunk; dims[1] = g.k; dims[2] = g.n / kChunk; dims[3] = g.bz != 0 ? g.batch : 1;
      str[0] = static_cast<uint64_t>(g.ldb) * 2; str[1] = 128;
      str[2] = g.bz != 0 ? static_cast<uint64_t>(g.bz) * 2 : str[0] * dims[1];
      str[3] = str[2] * dims[3];
      box[1] = kChunk; box[2] = bn_cta / kChunk;
    }
    int rc = make_tensor_map(&mapB, g.B, dims, str, box);
    if (rc != NG_OK) return rc;
  }
  return tc_launch(c, mapA, mapB, p, stream);
}

}  // namespace ngb

using namespace ngb;

extern "C" {

int ng_hgemm(const void* A, const void* B, void* C, int a_t, int b_t, int m, int n, int k, int lda, int ldb, int ldc,
             float alpha, float beta, int relu, int sr_bits, unsigned long long seed, unsigned int rng_offset,
             void* stream) {
  GemmCall g = {};
  g.A = A; g.B = B; g.C = C; g.a_t = a_t; g.b_t = b_t; g.m = m; g.n = n; g.k = k;
  g.lda = lda; g.ldb = ldb; g.ldc = ldc; g.alpha = alpha; g.beta = beta; g.relu = relu; g.sr_bits = sr_bits;
  g.seed = seed; g.rng_offset = rng_offset; g.batch = 1; g.loops = 1;
  return run_gemm(g, static_cast<cudaStream_t>(stream));
}

int ng_hgemm_simt(const void* A, const void* B, void* C, int a_t, int b_t, int m, int n, int k, int lda, int ldb,
                  int ldc, float alpha, float beta, int relu, int sr_bits, unsigned long long seed,
                  unsigned int rng_offset, void* stream) {
  GemmCall g = {};
  g.A = A; g.B = B; g.C = C; g.a_t = a_t; g.b_t = b_t; g.m = m; g.n = n; g.k = k;
  g.lda = lda; g.ldb = ldb; g.ldc = ldc; g.alpha = alpha; g.beta = beta; g.relu = relu; g.sr_bits = sr_bits;
  g.seed = seed; g.rng_offset = rng_offset; g.batch = 1; g.loops = 1; g.force_simt = 1;
  return run_gemm(g, static_cast<cudaStream_t>(stream));
}

int ng_hgemm_batched(const void* A, const void* B, void* C, int a_t, int b_t, int m, int n, int k, int lda, int ldb,
                     int ldc, float alpha, float beta, int relu, int sr_bits, unsigned long long seed,
                     unsigned int rng_offset, int batch_grid, int batch_loops, long long ldaz, long long ldbz,
                     long long ldcz, void* stream) {
  if (batch_grid < 1 || batch_loops < 1) return fail(NG_ERR_INVALID_ARG, "batch counts must be >= 1");
  GemmCall g = {};
  g.A = A; g.B = B; g.C = C; g.a_t = a_t; g.b_t = b_t; g.m = m; g.n = n; g.k = k;
  g.lda = lda; g.ldb = ldb; g.ldc = ldc; g.alpha = alpha; g.beta = beta; g.relu = relu; g.sr_bits = sr_bits;
  g.seed = seed; g.rng_offset = rng_offset;
  g.batch = batch_grid; g.loops = batch_loops;
  if (batch_grid > 1) { g.az = ldaz; g.bz = ldbz; g.cz = ldcz; }
  else { g.alz = ldaz; g.blz = ldbz; }
  return run_gemm(g, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
