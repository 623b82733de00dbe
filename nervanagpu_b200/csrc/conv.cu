// Convolution passes on CDHWN activations / CTRSK filters / KMPQN outputs (fp16 storage).
//   fprop :  O = RN16(relu?(alpha * F (*) I))          nervanagpu/nervanagpu.py:642-650
//   bprop :  dI = RN16(alpha * F^T (*)^T E)             nervanagpu/nervanagpu.py:652-659
//   update:  dF = alpha * sum_{m,p,q,n} Ipatch * E^T    nervanagpu/nervanagpu.py:661-669
// Dimensions follow ConvLayer (nervanagpu/layers.py:281-325): M,P,Q = ceil((X - f + 1 + 2 pad)/stride).
//
// Fast path: the tcgen05 implicit-GEMM engine, fed straight from the activation tensors by TMA
// (padding = out-of-bounds zero fill, no im2col buffer, no filter shuffle):
//   fprop   D[K x MPQN]   = F[crs][k]^T (MN-major A)  *  I patches (MN-major B)
//   bprop   D[C x DHWN]   = F[c][k] per tap (K-major A)  *  E pixels reached through the tap (MN-major B)
//   update  D[C x K]/tap  = I pixels under the tap (K-major A)  *  E (K-major B), reduction over (m,p,q,n)
// A 64-element chunk of the pixel space is either 64 images of one pixel (N % 64 == 0) or, when
// the W stride is 1, 64 consecutive elements of the flattened (x, n) dimension of one image row
// (several pixels of a small minibatch, e.g. the shard of a minibatch that is split over GPUs).
// Image rows that are not a multiple of 64 elements are padded to whole chunks: the last chunk of
// a row runs past its end, where TMA zero-fills (or, between rows of the input, reads pixels
// whose products land in columns that are never stored).
// Small-C weight updates run as im2col + tensor-core GEMM; shapes neither path can address run
// on plain SIMT kernels so that every legal call still executes on the GPU.
#include <algorithm>

#include "../../include/nervana_b200.h"
#include "epilogue.cuh"
#include "host.h"

namespace ngb {

namespace {

struct Geo {
  int N, C, K, D, H, W, T, R, S, M, P, Q;
  int pad_d, pad_h, pad_w, str_d, str_h, str_w;
  __host__ __device__ long long sizeI() const { return 1ll * C * D * H * W * N; }
  __host__ __device__ long long sizeF() const { return 1ll * C * T * R * S * K; }
  __host__ __device__ long long sizeO() const { return 1ll * K * M * P * Q * N; }
};

int out_dim(int x, int f, int pad, int str) {
  // ceil((x - f + 1 + 2 pad) / str), as nervanagpu/layers.py:297-301
  const int num = x - f + 1 + 2 * pad;
  return (num + str - 1) / str;
}

int make_geo(const ng_conv_desc* d, Geo& g) {
  if (!d) return fail(NG_ERR_INVALID_ARG, "conv descriptor is null");
  g.N = d->N; g.C = d->C; g.K = d->K; g.D = d->D; g.H = d->H; g.W = d->W; g.T = d->T; g.R = d->R; g.S = d->S;
  g.pad_d = d->pad_d; g.pad_h = d->pad_h; g.pad_w = d->pad_w;
  g.str_d = d->str_d; g.str_h = d->str_h; g.str_w = d->str_w;
  if (g.N < 1 || g.C < 1 || g.K < 1 || g.D < 1 || g.H < 1 || g.W < 1 || g.T < 1 || g.R < 1 || g.S < 1 ||
      g.str_d < 1 || g.str_h < 1 || g.str_w < 1 || g.pad_d < 0 || g.pad_h < 0 || g.pad_w < 0)
    return fail(NG_ERR_INVALID_ARG, "conv descriptor has a non-positive dimension");
  if (g.N % 8 != 0) return fail(NG_ERR_INVALID_ARG, "N dim must be multiple of 8");
  if (g.K % 8 != 0) return fail(NG_ERR_INVALID_ARG, "K dim must be multiple of 8");
  g.M = out_dim(g.D, g.T, g.pad_d, g.str_d);
  g.P = out_dim(g.H, g.R, g.pad_h, g.str_h);
  g.Q = out_dim(g.W, g.S, g.pad_w, g.str_w);
  if (g.M < 1 || g.P < 1 || g.Q < 1) return fail(NG_ERR_INVALID_ARG, "filter larger than padded input");
  if (g.sizeI() > 0x7fffffffll * 8 || g.sizeO() > 0x7fffffffll * 8) return fail(NG_ERR_TOO_LARGE, "tensor too large");
  return NG_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// chunking of a (m,p,q,n)-like pixel space with innermost extents (xdim, N)
enum ChunkMode { CH_NONE = 0, CH_PIXEL = 1, CH_FLAT = 2 };
ChunkMode pick_chunk_mode(int N, int str_w) {
  if (N % kChunk == 0) return CH_PIXEL;
  if (str_w == 1) return CH_FLAT;
  return CH_NONE;
}
// chunks per image row of `xdim` pixels
int row_chunks(int N, int xdim, ChunkMode mode) {
  return mode == CH_FLAT ? static_cast<int>((1ll * xdim * N + kChunk - 1) / kChunk) : xdim * (N / kChunk);
}
// Columns of the GEMM view of a (rows, xdim, N) pixel space, and (flattened mode with ragged
// rows) the mapping of its padded columns to memory.
long long pixel_columns(TcParams& p, long long rows, int xdim, int N, ChunkMode mode) {
  const int cpr = row_chunks(N, xdim, mode);
  if (mode == CH_FLAT && (1ll * xdim * N) % kChunk != 0) {
    p.c_row_chunks = cpr;
    p.c_row_len = xdim * N;
  }
  return rows * cpr * kChunk;
}

// tensor map over an activation tensor (chan, z, y, x, n) seen as (n | x*n, x | 1, y, z, chan)
// (`blocked`: the tensor is the (z, y, chan, x, n) copy made by chan_block, see there)
int act_map(CUtensorMap* m, const void* base, int chan, int Z, int Y, int X, int N, ChunkMode mode, uint32_t box_chan,
            bool blocked = false) {
  uint64_t dims[5], str[4];
  const uint64_t xn = 1ull * X * N * 2;
  if (mode == CH_PIXEL) {
    dims[0] = N; dims[1] = X; str[0] = 1ull * N * 2;
  } else {
    dims[0] = 1ull * X * N; dims[1] = 1; str[0] = xn;
  }
  dims[2] = Y; dims[3] = Z; dims[4] = chan;
  if (blocked) {
    str[1] = xn * chan; str[2] = xn * chan * Y; str[3] = xn;
  } else {
    str[1] = xn; str[2] = xn * Y; str[3] = xn * Y * Z;
  }
  const uint32_t box[5] = {kChunk, 1, 1, 1, box_chan};
  return make_tensor_map(m, base, dims, str, box);
}

// ---- channel planes further apart than a page -------------------------------------------------
// A TMA box of an activation tensor is [channels][64 elements]: one 128-byte row per channel, the
// rows one channel plane (z * y * x * n elements) apart. When a plane is larger than a 2 MB page
// every row of every box lies in another page, and the loads run at less than half their rate:
// with planes of 1.8 MB the 3-D layer 64 -> 64, 3x3x3, 56x56, N = 32 runs at 620 TFLOP/s, with
// planes of 2.0 MB at 390, of 3.2 MB at 280, whatever the tensor's total size, and with 16
// instead of 64 filters (a quarter of the output) in the same time. The remedy is one pass over
// the tensor before the product: a copy in (z, y, chan, x, n) order, whose channel rows are one
// image row (x * n elements) apart, so that a box spans a few hundred KB. The product reads the
// copy through a tensor map with the same dimensions and other strides; nothing in the kernel
// changes. The copy costs one read and one write of the tensor; every tap of the filter reads
// it again, so it pays from a few taps on.
constexpr long long kPlaneBytesBlocked = 1900000;   // between the last fast (1.81 MB) and first slow (2.01 MB) plane
bool wants_chan_block(int Z, int Y, int X, int N, int taps) {
  if (tuning().chan_block == 0) return false;
  const long long row = 2ll * X * N;
  if (row % 16 != 0) return false;
  if (tuning().chan_block == 2) return true;   // (tests: every shape)
  return taps >= 4 && row * Y * Z > kPlaneBytesBlocked;
}
size_t chan_block_bytes(int chan, int Z, int Y, int X, int N) {
  return (static_cast<size_t>(2) * chan * Z * Y * X * N + 255) & ~size_t(255);
}
// dst[(zy * chan + c)][row] = src[(c * zy_count + zy)][row], rows of `rowv` 16-byte vectors; one warp per row
__global__ void chan_block_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int chan, long long zy_count,
                                  int rowv) {
  const long long r = blockIdx.x * static_cast<long long>(blockDim.y) + threadIdx.y;
  if (r >= zy_count * chan) return;
  const long long zy = r / chan;
  const int c = static_cast<int>(r - zy * chan);
  const uint4* s = src + (c * zy_count + zy) * rowv;
  uint4* d = dst + r * rowv;
  int v = threadIdx.x;
  for (; v + 96 < rowv; v += 128) {   // four loads in flight per lane
    const uint4 a = s[v], b = s[v + 32], e = s[v + 64], f = s[v + 96];
    d[v] = a; d[v + 32] = b; d[v + 64] = e; d[v + 96] = f;
  }
  for (; v < rowv; v += 32) d[v] = s[v];
}
int chan_block(DeviceCtx* c, cudaStream_t stream, const void* src, void* dst, int chan, int Z, int Y, int X, int N) {
  const long long rows = 1ll * chan * Z * Y;
  const long long blocks = (rows + 7) / 8;
  if (blocks > 0x7fffffffll) return fail(NG_ERR_TOO_LARGE, "tensor too large for the channel-blocked copy");
  (void)c;
  chan_block_kernel<<<static_cast<unsigned>(blocks), dim3(32, 8), 0, stream>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), chan, 1ll * Z * Y, X * N / 8);
  NG_CHECK_LAUNCH();
  return NG_OK;
}
// Room for the copies behind the split-K partials of the product `p` (whose tiling and number of
// partitions are final): `n` copies of the given sizes, returned as pointers into the workspace.
int chan_block_room(DeviceCtx* c, cudaStream_t stream, const TcParams& p, const size_t* bytes, void** ptrs, int n) {
  const int nz_out = p.nz_out < 1 ? p.nz : p.nz_out;
  size_t off = p.splits > 1 ? static_cast<size_t>(p.splits) * nz_out * p.M * p.N * sizeof(float) : 0;
  off = (off + 255) & ~size_t(255);
  size_t total = off;
  for (int i = 0; i < n; ++i) total += bytes[i];
  const int rc = ensure_workspace(c, stream, total);
  if (rc != NG_OK) return rc;
  for (int i = 0; i < n; ++i) {
    ptrs[i] = reinterpret_cast<uint8_t*>(c->ws) + off;
    off += bytes[i];
  }
  return NG_OK;
}

// Tensor map over an activation tensor whose box is a whole column tile of `nb` 64-wide chunks
// that lie in one image row: (n, chan, x, y, z) with a box of nb pixels when a pixel is one chunk
// (N = 64), else (n_lo, chan, n_hi, x, y) for 2-D data. The box lands in shared memory chunk by
// chunk, each [box_chan rows][64], as the per-chunk boxes of act_map would. Returns the value for
// TcParams::b_merge, 0 when the shape has no such map.
int act_map_merged(CUtensorMap* m, const void* base, int chan, int Z, int Y, int X, int N, uint32_t box_chan, int nb,
                   bool blocked = false) {
  if (tuning().merge_boxes == 0 || N % kChunk != 0 || nb < 2) return 0;
  const int cpi = N / kChunk;
  const uint64_t xn = 1ull * X * N * 2;
  const uint64_t chan_str = blocked ? xn : xn * Y * Z, y_str = blocked ? xn * chan : xn;
  uint64_t dims[5], str[4];
  uint32_t box[5];
  if (cpi == 1) {
    dims[0] = N; dims[1] = chan; dims[2] = X; dims[3] = Y; dims[4] = Z;
    str[0] = chan_str; str[1] = 1ull * N * 2; str[2] = y_str; str[3] = y_str * Y;
    box[0] = kChunk; box[1] = box_chan; box[2] = nb; box[3] = 1; box[4] = 1;
    return make_tensor_map(m, base, dims, str, box) == NG_OK ? 1 : 0;
  }
  if (Z != 1 || (nb % cpi != 0 && cpi % nb != 0)) return 0;
  dims[0] = kChunk; dims[1] = chan; dims[2] = cpi; dims[3] = X; dims[4] = Y;
  str[0] = chan_str; str[1] = 128; str[2] = 1ull * N * 2; str[3] = y_str;
  box[0] = kChunk; box[1] = box_chan; box[2] = std::min(cpi, nb); box[3] = std::max(1, nb / cpi); box[4] = 1;
  return make_tensor_map(m, base, dims, str, box) == NG_OK ? 2 : 0;
}

// filter (C, TRS, K) with K a multiple of 64, seen as (k_lo, c, k_hi, trs): a box of two chunks of
// 64 filters lands as [chunk][box_c rows][64]
int filter_map_merged(CUtensorMap* m, const void* base, const Geo& g, uint32_t box_c) {
  const int RST = g.T * g.R * g.S;
  uint64_t dims[5] = {kChunk, static_cast<uint64_t>(g.C), static_cast<uint64_t>(g.K / kChunk),
                      static_cast<uint64_t>(RST), 1};
  uint64_t str[4];
  str[0] = 1ull * g.K * 2 * RST; str[1] = 128; str[2] = 1ull * g.K * 2; str[3] = str[0] * g.C;
  const uint32_t box[5] = {kChunk, box_c, 2, 1, 1};
  return make_tensor_map(m, base, dims, str, box);
}

// tensor map over the filter (C, TRS, K) seen as (k, trs, c)
int filter_map(CUtensorMap* m, const void* base, const Geo& g, uint32_t box_c) {
  const int RST = g.T * g.R * g.S;
  uint64_t dims[5] = {static_cast<uint64_t>(g.K), static_cast<uint64_t>(RST), static_cast<uint64_t>(g.C), 1, 1};
  uint64_t str[4];
  str[0] = 1ull * g.K * 2; str[1] = str[0] * RST; str[2] = str[1] * g.C; str[3] = str[2];
  const uint32_t box[5] = {kChunk, 1, box_c, 1, 1};
  return make_tensor_map(m, base, dims, str, box);
}

void fill_taps(TcParams& p, const Geo& g, ChunkMode mode) {
  p.RS = g.R * g.S; p.S = g.S; p.R = g.R;
  p.tap_w = 1; p.tap_h = 1;
  p.pad_d = g.pad_d; p.pad_h = g.pad_h; p.pad_w = g.pad_w;
  p.str_d = g.str_d; p.str_h = g.str_h; p.str_w = g.str_w;
  p.inner_tap = mode == CH_FLAT ? g.N : 0;
  p.x_tap = mode == CH_FLAT ? 0 : 1;
}

void fill_decode(TcParams& p, int N, int X, int Y, int Z, ChunkMode mode) {
  p.dec_cpi = mode == CH_FLAT ? row_chunks(N, X, mode) : N / kChunk;
  p.dec_q = mode == CH_FLAT ? 1 : X;
  p.dec_p = Y;
  p.dec_m = Z;
}

int pick_kb_rows(int C) {
  const int force = tuning().kb_rows;
  if (force >= 16 && force <= 64 && force % 16 == 0) return force;
  int best = 64, best_pad = ((C + 63) / 64) * 64;
  for (int r : {48, 32, 16}) {
    const int pad = ((C + r - 1) / r) * r;
    if (pad < best_pad) { best = r; best_pad = pad; }
  }
  return best;
}

// ------------------------------------------------------------------------------------------
// SIMT fall-backs (one thread per output element, fp32 accumulation)
// ------------------------------------------------------------------------------------------
__global__ void conv_fprop_simt(Geo g, const __half* __restrict__ I, const __half* __restrict__ F, __half* O,
                                float alpha, int relu) {
  const long long total = g.sizeO();
  for (long long i = blockIdx.x * 1ll * blockDim.x + threadIdx.x; i < total; i += 1ll * gridDim.x * blockDim.x) {
    long long r = i;
    const int n = r % g.N; r /= g.N;
    const int q = r % g.Q; r /= g.Q;
    const int p = r % g.P; r /= g.P;
    const int m = r % g.M; r /= g.M;
    const int k = static_cast<int>(r);
    float acc = 0.0f;
    for (int c = 0; c < g.C; ++c)
      for (int t = 0; t < g.T; ++t) {
        const int z = m * g.str_d - g.pad_d + t;
        if (z < 0 || z >= g.D) continue;
        for (int rr = 0; rr < g.R; ++rr) {
          const int y = p * g.str_h - g.pad_h + rr;
          if (y < 0 || y >= g.H) continue;
          for (int s = 0; s < g.S; ++s) {
            const int x = q * g.str_w - g.pad_w + s;
            if (x < 0 || x >= g.W) continue;
            const float iv = __half2float(I[(((1ll * c * g.D + z) * g.H + y) * g.W + x) * g.N + n]);
            const float fv = __half2float(F[(((1ll * c * g.T + t) * g.R + rr) * g.S + s) * g.K + k]);
            acc = fmaf(iv, fv, acc);
          }
        }
      }
    acc *= alpha;
    if (relu) acc = fmaxf(acc, 0.0f);
    O[i] = __float2half_rn(acc);
  }
}

__global__ void conv_bprop_simt(Geo g, const __half* __restrict__ F, const __half* __restrict__ E, __half* dI,
                                float alpha) {
  const long long total = g.sizeI();
  for (long long i = blockIdx.x * 1ll * blockDim.x + threadIdx.x; i < total; i += 1ll * gridDim.x * blockDim.x) {
    long long r = i;
    const int n = r % g.N; r /= g.N;
    const int x = r % g.W; r /= g.W;
    const int y = r % g.H; r /= g.H;
    const int z = r % g.D; r /= g.D;
    const int c = static_cast<int>(r);
    float acc = 0.0f;
    for (int t = 0; t < g.T; ++t) {
      const int mz = z + g.pad_d - t;
      if (mz < 0 || mz % g.str_d) continue;
      const int m = mz / g.str_d;
      if (m >= g.M) continue;
      for (int rr = 0; rr < g.R; ++rr) {
        const int py = y + g.pad_h - rr;
        if (py < 0 || py % g.str_h) continue;
        const int p = py / g.str_h;
        if (p >= g.P) continue;
        for (int s = 0; s < g.S; ++s) {
          const int qx = x + g.pad_w - s;
          if (qx < 0 || qx % g.str_w) continue;
          const int q = qx / g.str_w;
          if (q >= g.Q) continue;
          const __half* f = F + (((1ll * c * g.T + t) * g.R + rr) * g.S + s) * g.K;
          for (int k = 0; k < g.K; ++k) {
            const float ev = __half2float(E[(((1ll * k * g.M + m) * g.P + p) * g.Q + q) * g.N + n]);
            acc = fmaf(__half2float(f[k]), ev, acc);
          }
        }
      }
    }
    dI[i] = __float2half_rn(acc * alpha);
  }
}

// one warp per filter element: lanes stride over (pixel, n), shuffle reduction
__global__ void conv_update_simt(Geo g, const __half* __restrict__ I, const __half* __restrict__ E, void* dF,
                                 int out_f32, float alpha) {
  const long long total = g.sizeF();
  const int lane = threadIdx.x & 31;
  const long long warp0 = (blockIdx.x * 1ll * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (1ll * gridDim.x * blockDim.x) >> 5;
  for (long long i = warp0; i < total; i += nwarps) {
    long long r = i;
    const int k = r % g.K; r /= g.K;
    const int s = r % g.S; r /= g.S;
    const int rr = r % g.R; r /= g.R;
    const int t = r % g.T; r /= g.T;
    const int c = static_cast<int>(r);
    float acc = 0.0f;
    const long long span = 1ll * g.M * g.P * g.Q * g.N;
    for (long long j = lane; j < span; j += 32) {
      long long rj = j;
      const int n = rj % g.N; rj /= g.N;
      const int q = rj % g.Q; rj /= g.Q;
      const int p = rj % g.P; rj /= g.P;
      const int m = static_cast<int>(rj);
      const int z = m * g.str_d - g.pad_d + t, y = p * g.str_h - g.pad_h + rr, x = q * g.str_w - g.pad_w + s;
      if (z < 0 || z >= g.D || y < 0 || y >= g.H || x < 0 || x >= g.W) continue;
      const float iv = __half2float(I[(((1ll * c * g.D + z) * g.H + y) * g.W + x) * g.N + n]);
      const float ev = __half2float(E[1ll * k * span + j]);
      acc = fmaf(iv, ev, acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
      acc *= alpha;
      if (out_f32) static_cast<float*>(dF)[i] = acc;
      else static_cast<__half*>(dF)[i] = __float2half_rn(acc);
    }
  }
}

// ------------------------------------------------------------------------------------------
// im2col: col[crst][pixel * N + n] = I[c, z, y, x, n] (zero outside the image); 8 images per thread
// ------------------------------------------------------------------------------------------
// grid: x covers the (m, p, q, 8-image lane) positions of one patch row, y = (c, t, r, s) patch row
// (whole blocks of live threads whatever N is: with 16 images an output row is only 110 lanes wide)
__global__ void __launch_bounds__(256) im2col_kernel(Geo g, const __half* __restrict__ I, __half* __restrict__ col) {
  const int n8 = g.N / 8;
  const long long per_row = 1ll * g.M * g.P * g.Q * n8;
  const long long t0 = blockIdx.x * 256ll + threadIdx.x;
  if (t0 >= per_row) return;
  const int nv = static_cast<int>(t0 % n8);
  long long pix = t0 / n8;
  const int q = static_cast<int>(pix % g.Q); pix /= g.Q;
  const int p = static_cast<int>(pix % g.P);
  const int m = static_cast<int>(pix / g.P);
  int r = blockIdx.y;
  const int s = r % g.S; r /= g.S;
  const int rr = r % g.R; r /= g.R;
  const int t = r % g.T;
  const int c = r / g.T;
  const int z = m * g.str_d - g.pad_d + t, y = p * g.str_h - g.pad_h + rr, x = q * g.str_w - g.pad_w + s;
  uint4 v = make_uint4(0, 0, 0, 0);
  if (z >= 0 && z < g.D && y >= 0 && y < g.H && x >= 0 && x < g.W)
    v = *reinterpret_cast<const uint4*>(I + (((1ll * c * g.D + z) * g.H + y) * g.W + x) * g.N + nv * 8);
  reinterpret_cast<uint4*>(col)[blockIdx.y * per_row + t0] = v;
}

dim3 im2col_grid(const Geo& g) {
  const long long per_row = 1ll * g.M * g.P * g.Q * (g.N / 8);
  return dim3(static_cast<unsigned>((per_row + 255) / 256), g.C * g.T * g.R * g.S, 1);
}

int launch_1d(long long total, int threads, const DeviceCtx* c) {
  long long blocks = (total + threads - 1) / threads;
  return static_cast<int>(std::max<long long>(1, std::min<long long>(blocks, c->sm_count * 32ll)));
}

// ------------------------------------------------------------------------------------------
// Few input channels (first layers): tap blocks.
// One TMA box (64 n, bw x, bh y, 1, C) of the input carries the C*bh*bw rows that a block of
// bh x bw filter taps needs for one output pixel, already in the order (c, dy, dx). With
// rows = C*bh*bw a multiple of 16 this is one k-block of `rows` reduction rows, so a 3-channel
// 11x11 stride-4 layer runs as 9 k-blocks of 48 rows (bh = bw = 4) instead of 121 k-blocks of
// 16 rows holding 3 useful ones. The filter is re-packed (zero padded) to the same row order:
//   Fp[row = (c*bh + dy)*bw + dx][tb = (t*nr + r')*ns + s'][k] = F[c][t][r'*bh+dy][s'*bw+dx][k].
// ------------------------------------------------------------------------------------------
struct TapBlock {
  int bw = 0, bh = 0, rows = 0, nr = 0, ns = 0;
  bool ok = false;
};

// Weight update with few input rows per tap: one work item accumulates `acc_groups` taps at once
// (one TMEM accumulator each), so every chunk of the error tensor is fetched once per group of
// taps instead of once per tap. The group is limited by tensor memory (512 columns), by the
// shared-memory ring (at least four stages must remain) and balanced over the slices.
// Taps with at most 64 rows are also stacked along the 128 rows of one accumulator (`acc_taps`
// boxes of a_rows rows each), which halves (or better) the MMAs a tap costs.
void set_update_groups(TcParams& p, int taps, int a_rows) {
  const int cap = tuning().update_groups, cap_t = tuning().update_stack;   // limits on groups / stacking
  int t = std::max(1, std::min(std::min(kTileM / a_rows, 8), taps));
  if (cap_t > 0) t = std::max(1, std::min(t, cap_t));
  const int accs = (taps + t - 1) / t;                    // accumulators the whole filter needs
  int g = std::min(std::min(8, 512 / p.block_n), accs);
  if (cap > 0) g = std::max(1, std::min(g, cap));
  const int ring = 232448 - 1024 - 512 - static_cast<int>(kEpiStageBytes) - kTileM * 128;
  const int min_stages = tuning().update_min_stages > 0 ? std::max(2, tuning().update_min_stages) : 3;
  while (g > 1 && ((g * t * a_rows * 128 + p.block_n * 128) * min_stages > ring || g * t > 24)) --g;
  // the taps (not the accumulators) are spread evenly over the work items: 9 taps on items of at
  // most 6 become 5 + 4, not 6 + 3
  const int nz = (accs + g - 1) / g;
  p.taps_per_z = (taps + nz - 1) / nz;
  p.nz = (taps + p.taps_per_z - 1) / p.taps_per_z;
  p.acc_groups = (p.taps_per_z + t - 1) / t;
  p.acc_taps = t;
  p.pack_rows = a_rows;
  p.nz_out = taps;
}

// Column tile of the weight update (output channels): the smallest multiple of 64 that covers K
// in the fewest tiles, so that K = 192 or 384 does not pay for 256-wide MMAs.
int update_block_n(int K) {
  const int tiles = (K + 255) / 256;
  const int per = (K + tiles - 1) / tiles;
  return (per + 63) / 64 * 64;
}

TapBlock pick_tap_block(const Geo& g) {
  TapBlock best;
  long long best_cost = 0;
  for (int bh = 1; bh <= 16; ++bh)
    for (int bw = 1; bw <= 16; ++bw) {
      const int rows = g.C * bh * bw;
      if (rows % 16 != 0 || rows > 64) continue;
      const int nr = (g.R + bh - 1) / bh, ns = (g.S + bw - 1) / bw;
      // padded reduction length, plus a fixed charge per k-block
      const long long cost = 1ll * nr * ns * (rows + 8);
      if (!best.ok || cost < best_cost) {
        best.bw = bw; best.bh = bh; best.rows = rows; best.nr = nr; best.ns = ns; best.ok = true;
        best_cost = cost;
      }
    }
  return best;
}

__global__ void filter_repack_kernel(Geo g, TapBlock tb, const __half* __restrict__ F, __half* __restrict__ Fp) {
  const int k8 = g.K / 8;
  const int ntb = g.T * tb.nr * tb.ns;
  const long long total = 1ll * tb.rows * ntb * k8;
  for (long long i = blockIdx.x * 1ll * blockDim.x + threadIdx.x; i < total; i += 1ll * gridDim.x * blockDim.x) {
    long long r = i;
    const int kv = r % k8; r /= k8;
    const int b = r % ntb;
    const int row = static_cast<int>(r / ntb);
    const int dx = row % tb.bw, dy = (row / tb.bw) % tb.bh, c = row / (tb.bw * tb.bh);
    const int sp = b % tb.ns, rp = (b / tb.ns) % tb.nr, t = b / (tb.ns * tb.nr);
    const int rr = rp * tb.bh + dy, s = sp * tb.bw + dx;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (rr < g.R && s < g.S)
      v = *reinterpret_cast<const uint4*>(F + ((((1ll * c * g.T + t) * g.R + rr) * g.S + s) * g.K + kv * 8));
    reinterpret_cast<uint4*>(Fp)[i] = v;
  }
}

// gradient in tap-block order Dp[tb][row][k] (fp32) -> gradF[c][t][r][s][k]
__global__ void filter_unpack_kernel(Geo g, TapBlock tb, const float* __restrict__ Dp, void* gradF, int out_f32) {
  const long long total = g.sizeF();
  for (long long i = blockIdx.x * 1ll * blockDim.x + threadIdx.x; i < total; i += 1ll * gridDim.x * blockDim.x) {
    long long r = i;
    const int k = r % g.K; r /= g.K;
    const int s = r % g.S; r /= g.S;
    const int rr = r % g.R; r /= g.R;
    const int t = r % g.T;
    const int c = static_cast<int>(r / g.T);
    const int b = (t * tb.nr + rr / tb.bh) * tb.ns + s / tb.bw;
    const int row = (c * tb.bh + rr % tb.bh) * tb.bw + s % tb.bw;
    const float v = Dp[(1ll * b * tb.rows + row) * g.K + k];
    if (out_f32) static_cast<float*>(gradF)[i] = v;
    else static_cast<__half*>(gradF)[i] = __float2half_rn(v);
  }
}

// input map whose box carries one tap block: (64 n, bw, bh, 1, C)
int act_map_tapblock(CUtensorMap* m, const void* base, const Geo& g, const TapBlock& tb) {
  const uint64_t xn = 1ull * g.W * g.N * 2;
  uint64_t dims[5] = {static_cast<uint64_t>(g.N), static_cast<uint64_t>(g.W), static_cast<uint64_t>(g.H),
                      static_cast<uint64_t>(g.D), static_cast<uint64_t>(g.C)};
  uint64_t str[4] = {1ull * g.N * 2, xn, xn * g.H, xn * g.H * g.D};
  const uint32_t box[5] = {kChunk, static_cast<uint32_t>(tb.bw), static_cast<uint32_t>(tb.bh), 1,
                           static_cast<uint32_t>(g.C)};
  return make_tensor_map(m, base, dims, str, box);
}

int fprop_tapblock(DeviceCtx* c, const Geo& g, const TapBlock& tb, const void* I, const void* F, void* O, float alpha,
                   int relu, cudaStream_t stream) {
  const int ntb = g.T * tb.nr * tb.ns;
  const long long cols = 1ll * g.M * g.P * g.Q * g.N;
  const size_t fp_bytes = static_cast<size_t>(tb.rows) * ntb * g.K * 2;
  int rc = ensure_workspace(c, stream, fp_bytes);
  if (rc != NG_OK) return rc;
  __half* Fp = reinterpret_cast<__half*>(c->ws);
  filter_repack_kernel<<<launch_1d(1ll * tb.rows * ntb * g.K / 8, 256, c), 256, 0, stream>>>(
      g, tb, static_cast<const __half*>(F), Fp);
  NG_CHECK_LAUNCH();
  TcParams p = {};
  p.mode = TC_FPROP;
  p.block_n = 256;
  p.M = g.K; p.N = static_cast<int>(cols);
  p.tiles_n = static_cast<int>((cols + p.block_n - 1) / p.block_n);
  p.nz = 1; p.splits = 1;
  TcOperandLayout lay = {1, 1, tb.rows};
  p.red_chunks = 1;
  p.num_kb = ntb;
  tc_pick_tile_rows(c, p, p.tiles_n, p.num_kb);
  // fewer, larger boxes: the filters of a 128-row half as one box (K a multiple of 64), the two
  // image groups of a pixel as one box (N = 128, 2-D)
  const bool merge_off = tuning().merge_boxes == 0;
  lay.a_merge = !merge_off && g.K % kChunk == 0 && g.K > kChunk;
  lay.a_chunks = (g.K + kChunk - 1) / kChunk;
  lay.b_pair = !merge_off && g.N == 2 * kChunk && g.D == 1;
  tc_fill_mma(p, lay);
  fill_taps(p, g, CH_PIXEL);
  p.R = tb.nr; p.S = tb.ns; p.RS = tb.nr * tb.ns; p.tap_w = tb.bw; p.tap_h = tb.bh;
  fill_decode(p, g.N, g.Q, g.P, g.M, CH_PIXEL);
  p.oob_y = g.H;
  p.C = O; p.Cold = nullptr; p.ldc = cols; p.c_zstride = 0;
  p.alpha = alpha; p.beta = 0.0f; p.relu = relu; p.sr_bits = 0; p.out_f32 = 0; p.vec_ok = 1;
  CUtensorMap mapA, mapB;
  {  // packed filter seen as (k, tap block, row), or as (k_lo, row, k_hi, tap block)
    uint64_t dims[5] = {static_cast<uint64_t>(g.K), static_cast<uint64_t>(ntb), static_cast<uint64_t>(tb.rows), 1, 1};
    uint64_t str[4];
    str[0] = 1ull * g.K * 2; str[1] = str[0] * ntb; str[2] = str[1] * tb.rows; str[3] = str[2];
    uint32_t box[5] = {kChunk, 1, static_cast<uint32_t>(tb.rows), 1, 1};
    if (lay.a_merge) {
      dims[0] = kChunk; dims[1] = tb.rows; dims[2] = g.K / kChunk; dims[3] = ntb;
      str[0] = 1ull * g.K * 2 * ntb; str[1] = 128; str[2] = 1ull * g.K * 2; str[3] = str[0] * tb.rows;
      box[1] = tb.rows; box[2] = 2;
    }
    rc = make_tensor_map(&mapA, Fp, dims, str, box);
    if (rc != NG_OK) return rc;
  }
  if (lay.b_pair) {  // (n_lo, x, y, chan, n_hi): both image groups of a pixel's tap block in one box
    const uint64_t xn = 1ull * g.W * g.N * 2;
    uint64_t dims[5] = {kChunk, static_cast<uint64_t>(g.W), static_cast<uint64_t>(g.H), static_cast<uint64_t>(g.C), 2};
    uint64_t str[4] = {1ull * g.N * 2, xn, xn * g.H, 128};
    const uint32_t box[5] = {kChunk, static_cast<uint32_t>(tb.bw), static_cast<uint32_t>(tb.bh),
                             static_cast<uint32_t>(g.C), 2};
    rc = make_tensor_map(&mapB, I, dims, str, box);
  } else {
    rc = act_map_tapblock(&mapB, I, g, tb);
  }
  if (rc != NG_OK) return rc;
  return tc_launch(c, mapA, mapB, p, stream);
}

// gradient with the filters along the rows, Dt[k][tile][box][row] (fp32; tile stride 256 columns,
// `per` boxes of tb.rows columns per tile) -> gradF[c][t][r][s][k]
__global__ void filter_unpack_t_kernel(Geo g, TapBlock tb, int per, int ld, const float* __restrict__ Dt, void* gradF,
                                       int out_f32) {
  const long long total = g.sizeF();
  for (long long i = blockIdx.x * 1ll * blockDim.x + threadIdx.x; i < total; i += 1ll * gridDim.x * blockDim.x) {
    long long r = i;
    const int k = r % g.K; r /= g.K;
    const int s = r % g.S; r /= g.S;
    const int rr = r % g.R; r /= g.R;
    const int t = r % g.T;
    const int c = static_cast<int>(r / g.T);
    const int b = (t * tb.nr + rr / tb.bh) * tb.ns + s / tb.bw;
    const int row = (c * tb.bh + rr % tb.bh) * tb.bw + s % tb.bw;
    const float v = Dt[1ll * k * ld + (b / per) * 256 + (b % per) * tb.rows + row];
    if (out_f32) static_cast<float*>(gradF)[i] = v;
    else static_cast<__half*>(gradF)[i] = __float2half_rn(v);
  }
}

// Few filters (K <= 128) as well as few channels: the roles of the operands are exchanged, so that
// the 128 MMA rows carry the filters and the 256 MMA columns carry the rows of several tap blocks
// (an MMA with 64 columns costs nearly as much as one with 256). Column tile j owns tap blocks
// [j * per, (j + 1) * per); its B operand is their input boxes stacked, its A operand the error box.
int update_tapblock_swapped(DeviceCtx* c, const Geo& g, const TapBlock& tb, const void* I, const void* E,
                            void* gradF, int out_f32, float alpha, cudaStream_t stream) {
  const int ntb = g.T * tb.nr * tb.ns;
  const long long span = 1ll * g.M * g.P * g.Q * g.N;
  const int per = 256 / tb.rows;
  const int tiles = (ntb + per - 1) / per;
  const int ld = tiles * 256;
  const size_t dt_bytes = static_cast<size_t>(g.K) * ld * 4;
  const size_t dt_off = (kMaxSplits * dt_bytes + 255) & ~size_t(255);
  int rc = ensure_workspace(c, stream, dt_off + dt_bytes);
  if (rc != NG_OK) return rc;
  float* Dt = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(c->ws) + dt_off);
  TcParams p = {};
  p.mode = TC_UPDATE;
  p.swap_ab = 1;
  p.block_n = 256;
  p.M = g.K; p.N = ld;
  p.m_halves = 1; p.tiles_m = 1;
  p.tiles_n = tiles;
  p.nz = 1;
  p.taps_per_z = ntb;
  TcOperandLayout lay = {0, 0, kChunk};
  lay.a_box_rows = std::min(g.K, kTileM);
  lay.b_box_rows = tb.rows;
  lay.b_box_count = per;
  p.num_kb = static_cast<int>(span / kChunk);
  tc_fill_mma(p, lay);
  fill_taps(p, g, CH_PIXEL);
  p.R = tb.nr; p.S = tb.ns; p.RS = tb.nr * tb.ns; p.tap_w = tb.bw; p.tap_h = tb.bh;
  fill_decode(p, g.N, g.Q, g.P, g.M, CH_PIXEL);
  p.oob_y = g.H;
  p.C = Dt; p.Cold = nullptr; p.ldc = ld; p.c_zstride = 0;
  p.alpha = alpha; p.beta = 0.0f; p.relu = 0; p.sr_bits = 0; p.out_f32 = 1; p.vec_ok = 1;
  p.splits = choose_splits(c, p.tiles_n, p.num_kb, 1ll * g.K * ld);
  CUtensorMap mapA, mapB;
  rc = act_map(&mapA, E, g.K, g.M, g.P, g.Q, g.N, CH_PIXEL, lay.a_box_rows);
  if (rc != NG_OK) return rc;
  rc = act_map_tapblock(&mapB, I, g, tb);
  if (rc != NG_OK) return rc;
  rc = tc_launch(c, mapA, mapB, p, stream);
  if (rc != NG_OK) return rc;
  filter_unpack_t_kernel<<<launch_1d(g.sizeF(), 256, c), 256, 0, stream>>>(g, tb, per, ld, Dt, gradF, out_f32);
  NG_CHECK_LAUNCH();
  return NG_OK;
}

int update_tapblock(DeviceCtx* c, const Geo& g, const TapBlock& tb, const void* I, const void* E, void* gradF,
                    int out_f32, float alpha, cudaStream_t stream) {
  const bool swap_ok = tuning().update_swap != 0;
  // (worth it when the tap blocks fill at least half of a 256-column tile)
  if (swap_ok && g.K <= kTileM && g.T * tb.nr * tb.ns * tb.rows >= 128)
    return update_tapblock_swapped(c, g, tb, I, E, gradF, out_f32, alpha, stream);
  const int ntb = g.T * tb.nr * tb.ns;
  const long long span = 1ll * g.M * g.P * g.Q * g.N;
  // workspace: [split-K partials of the engine, at most 32 splits][Dp]
  const size_t dp_bytes = static_cast<size_t>(ntb) * tb.rows * g.K * 4;
  const size_t dp_off = (kMaxSplits * dp_bytes + 255) & ~size_t(255);
  int rc = ensure_workspace(c, stream, dp_off + dp_bytes);
  if (rc != NG_OK) return rc;
  float* Dp = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(c->ws) + dp_off);
  TcParams p = {};
  p.mode = TC_UPDATE;
  p.block_n = update_block_n(g.K);
  p.M = tb.rows; p.N = g.K;
  p.m_halves = 1; p.tiles_m = 1;
  p.tiles_n = (g.K + p.block_n - 1) / p.block_n;
  set_update_groups(p, ntb, tb.rows);
  TcOperandLayout lay = {0, 0, kChunk};
  lay.a_box_rows = tb.rows;
  p.num_kb = static_cast<int>(span / kChunk);
  tc_fill_mma(p, lay);
  fill_taps(p, g, CH_PIXEL);
  p.R = tb.nr; p.S = tb.ns; p.RS = tb.nr * tb.ns; p.tap_w = tb.bw; p.tap_h = tb.bh;
  fill_decode(p, g.N, g.Q, g.P, g.M, CH_PIXEL);
  p.oob_y = g.H;
  p.C = Dp; p.Cold = nullptr; p.ldc = g.K; p.c_zstride = 1ll * tb.rows * g.K;
  p.alpha = alpha; p.beta = 0.0f; p.relu = 0; p.sr_bits = 0; p.out_f32 = 1; p.vec_ok = 1;
  p.splits = choose_splits(c, 1ll * p.tiles_n * p.nz, p.num_kb, 1ll * ntb * tb.rows * g.K);
  CUtensorMap mapA, mapB;
  rc = act_map_tapblock(&mapA, I, g, tb);
  if (rc != NG_OK) return rc;
  rc = act_map(&mapB, E, g.K, g.M, g.P, g.Q, g.N, CH_PIXEL, p.block_n);
  if (rc != NG_OK) return rc;
  rc = tc_launch(c, mapA, mapB, p, stream);
  if (rc != NG_OK) return rc;
  filter_unpack_kernel<<<launch_1d(g.sizeF(), 256, c), 256, 0, stream>>>(g, tb, Dp, gradF, out_f32);
  NG_CHECK_LAUNCH();
  return NG_OK;
}

}  // namespace

}  // namespace ngb

using namespace ngb;

// ------------------------------------------------------------------------------------------
// Strided first layers of a small minibatch: space to depth.
// With fewer than 64 images a chunk holds several pixels, which a strided layer does not read
// from consecutive addresses, and with 3 channels a tap is no k-block. Such a layer (AlexNet
// conv1 on the shard of one of 4 or 8 GPUs) is rewritten as a unit-stride layer over
//   I2[(c, dy, dx)][Y][X][n] = I[c][st * Y + dy - pad_h][st * X + dx - pad_w][n]   (zero outside),
//   F2[(c, dy, dx)][r2][s2][k] = F[c][st * r2 + dy][st * s2 + dx][k]               (zero outside),
// O[k][p][q][n] = sum F2 * I2[..][p + r2][q + s2][n]: C * st * st channels (48 for 3 channels and
// stride 4), ceil(R / st) x ceil(S / st) taps, no padding, which is a shape the flattened-row
// tensor-core path handles at any minibatch. The copies cost a pass over the (small) input; the
// im2col matrix this replaces was R * S / st^2 times larger.
struct SpaceToDepth {
  bool ok = false;
  int st = 1, C2 = 0, H2 = 0, W2 = 0, R2 = 0, S2 = 0;
};
SpaceToDepth pick_space_to_depth(const Geo& g) {
  SpaceToDepth z;
  if (tuning().space_to_depth == 0) return z;
  if (g.D != 1 || g.T != 1 || g.pad_d != 0 || g.str_d != 1 || g.str_h != g.str_w || g.str_w < 2) return z;
  z.st = g.str_w;
  z.C2 = g.C * z.st * z.st;
  z.R2 = (g.R + z.st - 1) / z.st;
  z.S2 = (g.S + z.st - 1) / z.st;
  z.H2 = g.P + z.R2 - 1;
  z.W2 = g.Q + z.S2 - 1;
  z.ok = z.C2 >= 16 && z.C2 <= 4096;
  return z;
}
ng_conv_desc space_to_depth_desc(const Geo& g, const SpaceToDepth& z) {
  ng_conv_desc d = {};
  d.N = g.N; d.C = z.C2; d.K = g.K;
  d.D = 1; d.H = z.H2; d.W = z.W2;
  d.T = 1; d.R = z.R2; d.S = z.S2;
  d.pad_d = d.pad_h = d.pad_w = 0;
  d.str_d = d.str_h = d.str_w = 1;
  return d;
}
// one block row per (channel of I2, Y): the threads walk its X * N / 8 16-byte vectors
__global__ void s2d_input_kernel(Geo g, SpaceToDepth z, const uint4* __restrict__ I, uint4* __restrict__ I2) {
  const int nvec = g.N >> 3;
  const int row = blockIdx.x;                 // c2 * H2 + Y
  const int c2 = row / z.H2, Y = row - c2 * z.H2;
  const int dx = c2 % z.st, dy = (c2 / z.st) % z.st, c = c2 / (z.st * z.st);
  const int y = z.st * Y + dy - g.pad_h;
  const bool row_in = y >= 0 && y < g.H;
  const uint4* src = I + (1ll * c * g.H + (row_in ? y : 0)) * g.W * nvec;
  uint4* dst = I2 + 1ll * row * z.W2 * nvec;
  for (int i = threadIdx.x; i < z.W2 * nvec; i += blockDim.x) {
    const int X = i / nvec, v = i - X * nvec;
    const int x = z.st * X + dx - g.pad_w;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (row_in && x >= 0 && x < g.W) val = __ldg(src + x * nvec + v);
    dst[i] = val;
  }
}
// one 16-byte vector (8 filters) of F2 per thread
__global__ void s2d_filter_kernel(Geo g, SpaceToDepth z, const uint4* __restrict__ F, uint4* __restrict__ F2) {
  const int kvec = g.K >> 3;
  const long long total = 1ll * z.C2 * z.R2 * z.S2 * kvec;
  for (long long i = blockIdx.x * 1ll * blockDim.x + threadIdx.x; i < total; i += 1ll * gridDim.x * blockDim.x) {
    long long r = i;
    const int v = static_cast<int>(r % kvec); r /= kvec;
    const int s2 = static_cast<int>(r % z.S2); r /= z.S2;
    const int r2 = static_cast<int>(r % z.R2);
    const int c2 = static_cast<int>(r / z.R2);
    const int dx = c2 % z.st, dy = (c2 / z.st) % z.st, c = c2 / (z.st * z.st);
    const int rr = z.st * r2 + dy, ss = z.st * s2 + dx;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (rr < g.R && ss < g.S) val = __ldg(F + ((1ll * c * g.R + rr) * g.S + ss) * kvec + v);
    F2[i] = val;
  }
}
// gradF[c][r][s][k] = G2[(c, r % st, s % st)][r / st][s / st][k]
__global__ void s2d_filter_grad_kernel(Geo g, SpaceToDepth z, const float* __restrict__ G2, void* gradF, int out_f32) {
  const long long total = g.sizeF();
  for (long long i = blockIdx.x * 1ll * blockDim.x + threadIdx.x; i < total; i += 1ll * gridDim.x * blockDim.x) {
    long long r = i;
    const int k = static_cast<int>(r % g.K); r /= g.K;
    const int ss = static_cast<int>(r % g.S); r /= g.S;
    const int rr = static_cast<int>(r % g.R);
    const int c = static_cast<int>(r / g.R);
    const int c2 = (c * z.st + rr % z.st) * z.st + ss % z.st;
    const float v = G2[((1ll * c2 * z.R2 + rr / z.st) * z.S2 + ss / z.st) * g.K + k];
    if (out_f32) static_cast<float*>(gradF)[i] = v;
    else static_cast<__half*>(gradF)[i] = __float2half_rn(v);
  }
}
size_t round256(size_t b) { return (b + 255) & ~size_t(255); }

extern "C" {

int ng_conv_output_dims(const ng_conv_desc* d, int* M, int* P, int* Q) {
  Geo g;
  int rc = make_geo(d, g);
  if (rc != NG_OK) return rc;
  if (M) *M = g.M;
  if (P) *P = g.P;
  if (Q) *Q = g.Q;
  return NG_OK;
}

int ng_conv_fprop(const ng_conv_desc* d, const void* I, const void* F, void* O, float alpha, int relu, int path,
                  void* stream_) {
  Geo g;
  int rc = make_geo(d, g);
  if (rc != NG_OK) return rc;
  if (!I || !F || !O) return fail(NG_ERR_INVALID_ARG, "null tensor");
  DeviceCtx* c = current_ctx();
  if (!c) return NG_ERR_CUDA;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const ChunkMode mode = pick_chunk_mode(g.N, g.str_w);
  const bool al = aligned16(I) && aligned16(F) && aligned16(O);
  const bool tc = path != NG_PATH_SIMT && path != NG_PATH_IM2COL && mode != CH_NONE && al;
  if (path == NG_PATH_TENSOR && !tc) return fail(NG_ERR_UNSUPPORTED, "shape not addressable by the tensor-core path");
  if ((path == NG_PATH_AUTO || path == NG_PATH_TENSOR) && g.C < 16 && g.N % kChunk == 0 && al) {
    const TapBlock tb = pick_tap_block(g);
    if (tb.ok) return fprop_tapblock(c, g, tb, I, F, O, alpha, relu, stream);
  }
  if (path == NG_PATH_AUTO && g.C < 16 && g.N % kChunk != 0 && al) {
    const SpaceToDepth z = pick_space_to_depth(g);
    if (z.ok) {
      const size_t i2_bytes = round256(2ull * z.C2 * z.H2 * z.W2 * g.N), f2_bytes = round256(2ull * z.C2 * z.R2 * z.S2 * g.K);
      void* aux = nullptr;
      rc = ensure_aux(c, stream, i2_bytes + f2_bytes, &aux);
      if (rc != NG_OK) return rc;
      uint4* I2 = static_cast<uint4*>(aux);
      uint4* F2 = reinterpret_cast<uint4*>(static_cast<uint8_t*>(aux) + i2_bytes);
      s2d_input_kernel<<<z.C2 * z.H2, 256, 0, stream>>>(g, z, static_cast<const uint4*>(I), I2);
      NG_CHECK_LAUNCH();
      s2d_filter_kernel<<<launch_1d(1ll * z.C2 * z.R2 * z.S2 * (g.K / 8), 256, c), 256, 0, stream>>>(
          g, z, static_cast<const uint4*>(F), F2);
      NG_CHECK_LAUNCH();
      const ng_conv_desc d2 = space_to_depth_desc(g, z);
      return ng_conv_fprop(&d2, I2, F2, O, alpha, relu, NG_PATH_AUTO, stream_);
    }
  }
  {
    // Few input channels where tap blocks do not apply: one tap per k-block would feed the tensor
    // core 3 useful rows out of 16, so gather the patches once and run a dense GEMM over all rows:
    //   O[K x span] = F2d[crst][k]^T * col[crst][span]
    const int RST = g.T * g.R * g.S;
    const long long span = 1ll * g.M * g.P * g.Q * g.N;
    const bool small_c = g.C < 16 && path == NG_PATH_AUTO;
    const bool im2col = (small_c || path == NG_PATH_IM2COL) && al && span <= 0x7fffffffll &&
                        1ll * g.C * RST * span * 2 <= (6ll << 30) && g.C * RST <= 65535;
    if (path == NG_PATH_IM2COL && !im2col) return fail(NG_ERR_UNSUPPORTED, "shape not addressable by the im2col path");
    if (im2col) {
      const size_t col_bytes = static_cast<size_t>(g.C) * RST * span * 2;
      rc = ensure_workspace(c, stream, col_bytes);
      if (rc != NG_OK) return rc;
      __half* col = reinterpret_cast<__half*>(c->ws);
      im2col_kernel<<<im2col_grid(g), 256, 0, stream>>>(g, static_cast<const __half*>(I), col);
      NG_CHECK_LAUNCH();
      GemmCall gc = {};
      gc.A = F; gc.B = col; gc.C = O; gc.a_t = 1; gc.b_t = 0;
      gc.m = g.K; gc.n = static_cast<int>(span); gc.k = g.C * RST;
      gc.lda = g.K; gc.ldb = span; gc.ldc = span;
      gc.alpha = alpha; gc.beta = 0.0f; gc.relu = relu; gc.batch = 1; gc.loops = 1;
      return run_gemm(gc, stream);
    }
  }
  if (!tc) {
    count_fallback_launch();
    conv_fprop_simt<<<launch_1d(g.sizeO(), 256, c), 256, 0, stream>>>(
        g, static_cast<const __half*>(I), static_cast<const __half*>(F), static_cast<__half*>(O), alpha, relu);
    NG_CHECK_LAUNCH();
    return NG_OK;
  }
  const int RST = g.T * g.R * g.S;
  const long long ldo = 1ll * g.M * g.P * g.Q * g.N;
  TcParams p = {};
  p.mode = TC_FPROP;
  const long long cols = pixel_columns(p, 1ll * g.M * g.P, g.Q, g.N, mode);
  if (cols > 0x7fffffffll) return fail(NG_ERR_TOO_LARGE, "output too large");
  p.M = g.K; p.N = static_cast<int>(cols);
  p.nz = 1; p.splits = 1;
  TcOperandLayout lay = {1, 1, pick_kb_rows(g.C)};
  p.red_chunks = (g.C + lay.kb_rows - 1) / lay.kb_rows;
  p.num_kb = RST * p.red_chunks;
  tc_pick_tile(c, p, cols, p.num_kb, lay.kb_rows);
  CUtensorMap mapA, mapB, mapBm;
  // fewer, larger boxes where the shapes allow: the filters of a 128-row half as one box, the
  // pixels of a column tile inside one image row as one box
  const bool merge_off = tuning().merge_boxes == 0;
  lay.a_merge = !merge_off && g.K % kChunk == 0 && g.K > kChunk &&
                filter_map_merged(&mapA, F, g, lay.kb_rows) == NG_OK;
  lay.a_chunks = (g.K + kChunk - 1) / kChunk;
  tc_fill_mma(p, lay);
  fill_taps(p, g, mode);
  fill_decode(p, g.N, g.Q, g.P, g.M, mode);
  p.oob_y = g.H;
  p.C = O; p.Cold = nullptr; p.ldc = ldo; p.c_zstride = 0;
  p.alpha = alpha; p.beta = 0.0f; p.relu = relu; p.sr_bits = 0; p.out_f32 = 0; p.vec_ok = 1;
  if (!lay.a_merge) {
    rc = filter_map(&mapA, F, g, lay.kb_rows);
    if (rc != NG_OK) return rc;
  }
  // few tiles (a small minibatch, e.g. the shard of one GPU): the reduction is split over the SMs too
  p.splits = choose_splits(c, 1ll * p.tiles_m * p.tiles_n, p.num_kb, 1ll * g.K * cols, true);
  const bool blocked = wants_chan_block(g.D, g.H, g.W, g.N, RST);
  if (blocked) {   // large channel planes: the product reads a copy in (z, y, chan, x, n) order
    const size_t bytes = chan_block_bytes(g.C, g.D, g.H, g.W, g.N);
    void* copy = nullptr;
    rc = chan_block_room(c, stream, p, &bytes, &copy, 1);
    if (rc == NG_OK) rc = chan_block(c, stream, I, copy, g.C, g.D, g.H, g.W, g.N);
    if (rc != NG_OK) return rc;
    I = copy;
  }
  rc = act_map(&mapB, I, g.C, g.D, g.H, g.W, g.N, mode, lay.kb_rows, blocked);
  if (rc != NG_OK) return rc;
  if (mode == CH_PIXEL && g.str_w == 1)
    p.b_merge = act_map_merged(&mapBm, I, g.C, g.D, g.H, g.W, g.N, lay.kb_rows, p.block_n / kChunk, blocked);
  return tc_launch(c, mapA, mapB, p, stream, p.b_merge ? &mapBm : nullptr);
}

int ng_conv_bprop(const ng_conv_desc* d, const void* F, const void* E, void* gradI, float alpha, int path,
                  void* stream_) {
  Geo g;
  int rc = make_geo(d, g);
  if (rc != NG_OK) return rc;
  if (!F || !E || !gradI) return fail(NG_ERR_INVALID_ARG, "null tensor");
  DeviceCtx* c = current_ctx();
  if (!c) return NG_ERR_CUDA;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const ChunkMode mode = pick_chunk_mode(g.N, g.str_w);
  // in flattened mode the E row (Q*N) is addressed with the same element offsets as the dI row
  const bool tc = path != NG_PATH_SIMT && mode != CH_NONE && aligned16(F) && aligned16(E) && aligned16(gradI);
  if (path == NG_PATH_TENSOR && !tc) return fail(NG_ERR_UNSUPPORTED, "shape not addressable by the tensor-core path");
  if (!tc) {
    count_fallback_launch();
    conv_bprop_simt<<<launch_1d(g.sizeI(), 256, c), 256, 0, stream>>>(
        g, static_cast<const __half*>(F), static_cast<const __half*>(E), static_cast<__half*>(gradI), alpha);
    NG_CHECK_LAUNCH();
    return NG_OK;
  }
  const int RST = g.T * g.R * g.S;
  const long long ldi = 1ll * g.D * g.H * g.W * g.N;
  TcParams p = {};
  p.mode = TC_BPROP;
  const long long cols = pixel_columns(p, 1ll * g.D * g.H, g.W, g.N, mode);
  if (cols > 0x7fffffffll) return fail(NG_ERR_TOO_LARGE, "output too large");
  p.M = g.C; p.N = static_cast<int>(cols);
  p.nz = 1; p.splits = 1;
  TcOperandLayout lay = {0, 1, kChunk};
  p.red_chunks = (g.K + kChunk - 1) / kChunk;
  p.num_kb = RST * p.red_chunks;
  tc_pick_tile(c, p, cols, p.num_kb, kChunk);
  // fewer input channels than tile rows (one row tile): the filter box carries the real rows only
  const int a_rows = p.tiles_m == 1 ? std::min(kTileM * p.m_halves, (g.C + 7) / 8 * 8) : kTileM * p.m_halves;
  lay.a_box_rows = a_rows;
  tc_fill_mma(p, lay);
  fill_taps(p, g, mode);
  fill_decode(p, g.N, g.W, g.H, g.D, mode);
  p.oob_y = g.P;
  p.C = gradI; p.Cold = nullptr; p.ldc = ldi; p.c_zstride = 0;
  p.alpha = alpha; p.beta = 0.0f; p.relu = 0; p.sr_bits = 0; p.out_f32 = 0; p.vec_ok = 1;
  CUtensorMap mapA, mapB, mapBm;
  rc = filter_map(&mapA, F, g, a_rows);
  if (rc != NG_OK) return rc;
  p.splits = choose_splits(c, 1ll * p.tiles_m * p.tiles_n, p.num_kb, 1ll * g.C * cols, true);
  const bool blocked = wants_chan_block(g.M, g.P, g.Q, g.N, RST);
  if (blocked) {   // large channel planes: the product reads a copy in (z, y, chan, x, n) order
    const size_t bytes = chan_block_bytes(g.K, g.M, g.P, g.Q, g.N);
    void* copy = nullptr;
    rc = chan_block_room(c, stream, p, &bytes, &copy, 1);
    if (rc == NG_OK) rc = chan_block(c, stream, E, copy, g.K, g.M, g.P, g.Q, g.N);
    if (rc != NG_OK) return rc;
    E = copy;
  }
  rc = act_map(&mapB, E, g.K, g.M, g.P, g.Q, g.N, mode, kChunk, blocked);
  if (rc != NG_OK) return rc;
  // the error pixels of a column tile inside one image row as one box
  if (mode == CH_PIXEL && g.str_w == 1)
    p.b_merge = act_map_merged(&mapBm, E, g.K, g.M, g.P, g.Q, g.N, kChunk, p.block_n / kChunk, blocked);
  return tc_launch(c, mapA, mapB, p, stream, p.b_merge ? &mapBm : nullptr);
}

int ng_conv_update(const ng_conv_desc* d, const void* I, const void* E, void* gradF, int out_f32, float alpha,
                   int path, void* stream_) {
  Geo g;
  int rc = make_geo(d, g);
  if (rc != NG_OK) return rc;
  if (!I || !E || !gradF) return fail(NG_ERR_INVALID_ARG, "null tensor");
  DeviceCtx* c = current_ctx();
  if (!c) return NG_ERR_CUDA;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const ChunkMode mode = pick_chunk_mode(g.N, g.str_w);
  const bool al = aligned16(I) && aligned16(E) && aligned16(gradF);
  const int RST = g.T * g.R * g.S;
  const long long span = 1ll * g.M * g.P * g.Q * g.N;
  const bool direct = path != NG_PATH_SIMT && path != NG_PATH_IM2COL && mode != CH_NONE && al &&
                      (g.C >= 16 || path == NG_PATH_TENSOR);
  const bool im2col = !direct && path != NG_PATH_SIMT && path != NG_PATH_TENSOR && al &&
                      1ll * g.C * RST * span * 2 <= (6ll << 30) && g.C * RST <= 65535;
  if (path == NG_PATH_TENSOR && !direct) return fail(NG_ERR_UNSUPPORTED, "shape not addressable by the tensor-core path");
  if (path == NG_PATH_IM2COL && !im2col) return fail(NG_ERR_UNSUPPORTED, "shape not addressable by the im2col path");
  if ((path == NG_PATH_AUTO || path == NG_PATH_TENSOR) && g.C < 16 && g.N % kChunk == 0 && al) {
    const TapBlock tb = pick_tap_block(g);
    if (tb.ok) return update_tapblock(c, g, tb, I, E, gradF, out_f32, alpha, stream);
  }
  if (path == NG_PATH_AUTO && g.C < 16 && g.N % kChunk != 0 && al) {
    const SpaceToDepth z = pick_space_to_depth(g);   // see there
    if (z.ok) {
      const size_t i2_bytes = round256(2ull * z.C2 * z.H2 * z.W2 * g.N), g2_bytes = round256(4ull * z.C2 * z.R2 * z.S2 * g.K);
      void* aux = nullptr;
      rc = ensure_aux(c, stream, i2_bytes + g2_bytes, &aux);
      if (rc != NG_OK) return rc;
      uint4* I2 = static_cast<uint4*>(aux);
      float* G2 = reinterpret_cast<float*>(static_cast<uint8_t*>(aux) + i2_bytes);
      s2d_input_kernel<<<z.C2 * z.H2, 256, 0, stream>>>(g, z, static_cast<const uint4*>(I), I2);
      NG_CHECK_LAUNCH();
      const ng_conv_desc d2 = space_to_depth_desc(g, z);
      rc = ng_conv_update(&d2, I2, E, G2, 1, alpha, NG_PATH_AUTO, stream_);
      if (rc != NG_OK) return rc;
      s2d_filter_grad_kernel<<<launch_1d(g.sizeF(), 256, c), 256, 0, stream>>>(g, z, G2, gradF, out_f32);
      NG_CHECK_LAUNCH();
      return NG_OK;
    }
  }
  if (direct) {
    TcParams p = {};
    p.mode = TC_UPDATE;
    p.block_n = update_block_n(g.K);
    p.M = g.C; p.N = g.K;
    p.tiles_n = (g.K + p.block_n - 1) / p.block_n;
    p.nz = RST;
    TcOperandLayout lay = {0, 0, kChunk};
    // one k-block per chunk of the (m, p, q, n) space; ragged image rows are padded to whole
    // chunks, whose tail TMA zero-fills in the error tensor
    p.num_kb = g.M * g.P * row_chunks(g.N, g.Q, mode);
    // the reduction is split to fill the SMs whatever the tile count, so only the operand
    // traffic argues: assume many column tiles
    tc_pick_tile_rows(c, p, 64ll * p.tiles_n * p.nz, p.num_kb);
    int a_rows = kTileM * p.m_halves;
    if (g.C <= 64) {
      // short A boxes leave room in the ring for several taps per work item
      a_rows = (g.C + 7) / 8 * 8;
      lay.a_box_rows = a_rows;
      set_update_groups(p, RST, a_rows);
    }
    tc_fill_mma(p, lay);
    fill_taps(p, g, mode);
    fill_decode(p, g.N, g.Q, g.P, g.M, mode);
    p.oob_y = g.H;
    p.C = gradF; p.Cold = nullptr; p.ldc = 1ll * RST * g.K; p.c_zstride = g.K;
    p.alpha = alpha; p.beta = 0.0f; p.relu = 0; p.sr_bits = 0; p.out_f32 = out_f32; p.vec_ok = 1;
    p.splits = choose_splits(c, 1ll * p.tiles_m * p.tiles_n * p.nz, p.num_kb, 1ll * g.C * g.K * RST);
    CUtensorMap mapA, mapB;
    // large channel planes: the product reads copies in (z, y, chan, x, n) order
    const bool blocked_i = wants_chan_block(g.D, g.H, g.W, g.N, RST);
    const bool blocked_e = wants_chan_block(g.M, g.P, g.Q, g.N, RST);
    if (blocked_i || blocked_e) {
      const size_t bytes[2] = {blocked_i ? chan_block_bytes(g.C, g.D, g.H, g.W, g.N) : 0,
                               blocked_e ? chan_block_bytes(g.K, g.M, g.P, g.Q, g.N) : 0};
      void* copies[2] = {nullptr, nullptr};
      rc = chan_block_room(c, stream, p, bytes, copies, 2);
      if (rc == NG_OK && blocked_i) rc = chan_block(c, stream, I, copies[0], g.C, g.D, g.H, g.W, g.N);
      if (rc == NG_OK && blocked_e) rc = chan_block(c, stream, E, copies[1], g.K, g.M, g.P, g.Q, g.N);
      if (rc != NG_OK) return rc;
      if (blocked_i) I = copies[0];
      if (blocked_e) E = copies[1];
    }
    rc = act_map(&mapA, I, g.C, g.D, g.H, g.W, g.N, mode, a_rows, blocked_i);
    if (rc != NG_OK) return rc;
    rc = act_map(&mapB, E, g.K, g.M, g.P, g.Q, g.N, mode, p.block_n, blocked_e);
    if (rc != NG_OK) return rc;
    return tc_launch(c, mapA, mapB, p, stream);
  }
  if (im2col) {
    // dF[crst][k] = col[crst][span] * E[k][span]^T  (both K-major: an "nt" GEMM with split-K)
    const size_t col_bytes = static_cast<size_t>(g.C) * RST * span * 2;
    const size_t col_off = ((static_cast<size_t>(kMaxSplits) * g.C * RST * g.K * 4) + 255) & ~size_t(255);  // room for partials
    rc = ensure_workspace(c, stream, col_off + col_bytes);
    if (rc != NG_OK) return rc;
    __half* col = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(c->ws) + col_off);
    const long long total = 1ll * g.C * RST * span / 8;
    (void)total;
    im2col_kernel<<<im2col_grid(g), 256, 0, stream>>>(g, static_cast<const __half*>(I), col);
    NG_CHECK_LAUNCH();
    GemmCall gc = {};
    gc.A = col; gc.B = E; gc.C = gradF; gc.a_t = 0; gc.b_t = 1;
    gc.m = g.C * RST; gc.n = g.K;
    if (span > 0x7fffffffll) return fail(NG_ERR_TOO_LARGE, "reduction too long");
    gc.k = static_cast<int>(span);
    gc.lda = span; gc.ldb = span; gc.ldc = g.K;
    gc.alpha = alpha; gc.beta = 0.0f; gc.batch = 1; gc.loops = 1; gc.out_f32 = out_f32;
    return run_gemm(gc, stream);
  }
  const long long warps = g.sizeF();
  count_fallback_launch();
  conv_update_simt<<<launch_1d(warps * 32, 256, c), 256, 0, stream>>>(
      g, static_cast<const __half*>(I), static_cast<const __half*>(E), gradF, out_f32, alpha);
  NG_CHECK_LAUNCH();
  return NG_OK;
}

}  // extern "C"
