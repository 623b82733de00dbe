// Max pooling over (feature map, depth, height, width) windows J,T,R,S on CDHWN tensors.
// Replaces hpool_max / spool_max (kernels/sass/hpool_max.sass) launched by
// NervanaGPU.fprop_pool / bprop_pool (nervanagpu/nervanagpu.py:773-818); output dimensions as
// PoolLayer (nervanagpu/layers.py:565-569).
//
// Numerics follow the reference kernel: taps are scanned in j,t,r,s order with a strict '>'
// compare so the first maximum wins (hpool_max.sass:264-281), taps outside the tensor are
// skipped, and the backward pass adds E[k,m,p,q,n] to dI at the argmax of window (k,m,p,q).
// Here the backward pass is a gather in two stages: the first records the argmax of every window
// (a scratch array in the library's workspace), the second lets each dI element visit the
// windows that contain it in increasing (k,m,p,q) order and sum, in fp32, the errors of those
// whose argmax it is. Overlapping windows so need neither atomics nor a zero-fill pass and the
// result is deterministic. Windows that do not overlap take one pass. The common 2-D shapes
// (3x3/2, 2x2/2, 3x3/3 without padding) have compile-time specialisations. The innermost
// dimension N is contiguous: each thread owns 8 images (one 16-byte lane) when N % 8 == 0, else 1.
#include <algorithm>
#include <cfloat>
#include <cuda_fp16.h>

#include "../../include/nervana_b200.h"
#include "host.h"

namespace ngb {
namespace {

struct PoolGeo {
  int N, C, D, H, W, J, T, R, S, K, M, P, Q;
  int pad_j, pad_d, pad_h, pad_w, str_j, str_d, str_h, str_w;
};

int pool_out_dim(int x, int f, int pad, int str) { return (x - f + 1 + 2 * pad + str - 1) / str; }

int make_pool_geo(const ng_pool_desc* d, PoolGeo& g) {
  if (!d) return fail(NG_ERR_INVALID_ARG, "pool descriptor is null");
  g.N = d->N; g.C = d->C; g.D = d->D; g.H = d->H; g.W = d->W;
  g.J = d->J; g.T = d->T; g.R = d->R; g.S = d->S;
  g.pad_j = d->pad_j; g.pad_d = d->pad_d; g.pad_h = d->pad_h; g.pad_w = d->pad_w;
  g.str_j = d->str_j; g.str_d = d->str_d; g.str_h = d->str_h; g.str_w = d->str_w;
  if (g.N < 1 || g.C < 1 || g.D < 1 || g.H < 1 || g.W < 1 || g.J < 1 || g.T < 1 || g.R < 1 || g.S < 1 ||
      g.str_j < 1 || g.str_d < 1 || g.str_h < 1 || g.str_w < 1 || g.pad_j < 0 || g.pad_d < 0 || g.pad_h < 0 ||
      g.pad_w < 0)
    return fail(NG_ERR_INVALID_ARG, "pool descriptor has a non-positive dimension");
  g.K = pool_out_dim(g.C, g.J, g.pad_j, g.str_j);
  g.M = pool_out_dim(g.D, g.T, g.pad_d, g.str_d);
  g.P = pool_out_dim(g.H, g.R, g.pad_h, g.str_h);
  g.Q = pool_out_dim(g.W, g.S, g.pad_w, g.str_w);
  if (g.K < 1 || g.M < 1 || g.P < 1 || g.Q < 1) return fail(NG_ERR_INVALID_ARG, "window larger than padded input");
  return NG_OK;
}

template <typename T, int V>
struct Vec;
template <>
struct Vec<__half, 8> {
  uint4 raw;
  __device__ float get(int i) const { return __half2float(reinterpret_cast<const __half*>(&raw)[i]); }
  __device__ void set(int i, float v) { reinterpret_cast<__half*>(&raw)[i] = __float2half_rn(v); }
};
template <>
struct Vec<__half, 1> {
  __half raw;
  __device__ float get(int) const { return __half2float(raw); }
  __device__ void set(int, float v) { raw = __float2half_rn(v); }
};
template <>
struct Vec<float, 4> {
  float4 raw;
  __device__ float get(int i) const { return reinterpret_cast<const float*>(&raw)[i]; }
  __device__ void set(int i, float v) { reinterpret_cast<float*>(&raw)[i] = v; }
};
template <>
struct Vec<float, 1> {
  float raw;
  __device__ float get(int) const { return raw; }
  __device__ void set(int, float v) { raw = v; }
};

// Scan window (k,m,p,q): per image lane the max and the flat (c,z,y,x) index of its first occurrence.
template <typename T, int V>
__device__ __forceinline__ void window_max(const PoolGeo& g, const T* __restrict__ I, int k, int m, int p, int q,
                                           int nv, float (&best)[V], int (&arg)[V]) {
#pragma unroll
  for (int i = 0; i < V; ++i) { best[i] = -FLT_MAX; arg[i] = 0; }
  const int c0 = k * g.str_j - g.pad_j, z0 = m * g.str_d - g.pad_d, y0 = p * g.str_h - g.pad_h,
            x0 = q * g.str_w - g.pad_w;
  for (int j = 0; j < g.J; ++j) {
    const int c = c0 + j;
    if (c < 0 || c >= g.C) continue;
    for (int t = 0; t < g.T; ++t) {
      const int z = z0 + t;
      if (z < 0 || z >= g.D) continue;
      for (int r = 0; r < g.R; ++r) {
        const int y = y0 + r;
        if (y < 0 || y >= g.H) continue;
        for (int s = 0; s < g.S; ++s) {
          const int x = x0 + s;
          if (x < 0 || x >= g.W) continue;
          const int flat = ((c * g.D + z) * g.H + y) * g.W + x;
          const Vec<T, V> v = *reinterpret_cast<const Vec<T, V>*>(I + (1ll * flat * g.N + nv * V));
#pragma unroll
          for (int i = 0; i < V; ++i) {
            const float f = v.get(i);
            if (f > best[i]) { best[i] = f; arg[i] = flat; }
          }
        }
      }
    }
  }
}

// first window index along one axis that can contain coordinate x, and the last
__device__ __forceinline__ void window_range(int x, int pad, int f, int str, int nout, int& lo, int& hi) {
  // windows w with w*str - pad <= x <= w*str - pad + f - 1
  const int a = x + pad - f + 1;
  lo = a <= 0 ? 0 : (a + str - 1) / str;
  hi = min(nout - 1, (x + pad) / str);
}

// O and/or arg_out may be null: the forward pass stores the maxima, the first stage of the
// backward pass stores the flat (c,z,y,x) index of each window's first maximum.
template <typename T, int V>
__global__ void pool_fprop_kernel(PoolGeo g, const T* __restrict__ I, T* __restrict__ O, int* __restrict__ arg_out,
                                  int mask_pos) {
  const int nvec = g.N / V;
  const long long total = 1ll * g.K * g.M * g.P * g.Q * nvec;
  for (long long i = blockIdx.x * 1ll * blockDim.x + threadIdx.x; i < total; i += 1ll * gridDim.x * blockDim.x) {
    long long r = i;
    const int nv = r % nvec; r /= nvec;
    const int q = r % g.Q; r /= g.Q;
    const int p = r % g.P; r /= g.P;
    const int m = r % g.M; r /= g.M;
    const int k = static_cast<int>(r);
    float best[V];
    int arg[V];
    window_max<T, V>(g, I, k, m, p, q, nv, best, arg);
    if (O) {
      Vec<T, V> out;
#pragma unroll
      for (int j = 0; j < V; ++j) out.set(j, best[j]);
      *reinterpret_cast<Vec<T, V>*>(O + i * V) = out;
    }
    if (arg_out) {
#pragma unroll
      for (int j = 0; j < V; ++j) arg_out[i * V + j] = (mask_pos && !(best[j] > 0.0f)) ? -1 : arg[j];
    }
  }
}

// Second stage of the backward pass: every input element sums the errors of the windows whose
// recorded argmax it is, visiting them in increasing (k,m,p,q) order.
template <typename T, int V>
__global__ void pool_gather_kernel(PoolGeo g, const int* __restrict__ arg, const T* __restrict__ E,
                                   T* __restrict__ dI) {
  const int nvec = g.N / V;
  const long long total = 1ll * g.C * g.D * g.H * g.W * nvec;
  for (long long i = blockIdx.x * 1ll * blockDim.x + threadIdx.x; i < total; i += 1ll * gridDim.x * blockDim.x) {
    long long r = i;
    const int nv = r % nvec; r /= nvec;
    const int flat = static_cast<int>(r);
    const int x = r % g.W; r /= g.W;
    const int y = r % g.H; r /= g.H;
    const int z = r % g.D; r /= g.D;
    const int c = static_cast<int>(r);
    int k0, k1, m0, m1, p0, p1, q0, q1;
    window_range(c, g.pad_j, g.J, g.str_j, g.K, k0, k1);
    window_range(z, g.pad_d, g.T, g.str_d, g.M, m0, m1);
    window_range(y, g.pad_h, g.R, g.str_h, g.P, p0, p1);
    window_range(x, g.pad_w, g.S, g.str_w, g.Q, q0, q1);
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.0f;
    for (int k = k0; k <= k1; ++k)
      for (int m = m0; m <= m1; ++m)
        for (int p = p0; p <= p1; ++p)
          for (int q = q0; q <= q1; ++q) {
            const long long o = ((((1ll * k * g.M + m) * g.P + p) * g.Q + q) * g.N) + nv * V;
            const Vec<T, V> e = *reinterpret_cast<const Vec<T, V>*>(E + o);
#pragma unroll
            for (int j = 0; j < V; ++j)
              if (arg[o + j] == flat) acc[j] += e.get(j);
          }
    Vec<T, V> out;
#pragma unroll
    for (int j = 0; j < V; ++j) out.set(j, acc[j]);
    *reinterpret_cast<Vec<T, V>*>(dI + i * V) = out;
  }
}

// ------------------------------------------------------------------------------------------
// Specialised 2-D windows (J = T = 1, no padding, fp16, N % 8 == 0): compile-time R,S and strides,
// grid (x: pixel of the plane and image lane, y: channel): two index divisions per thread.
// ------------------------------------------------------------------------------------------
struct Lanes8 {
  float v[8];
};
__device__ __forceinline__ Lanes8 load8(const __half* p) {
  const uint4 r = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&r);
  Lanes8 o;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    o.v[2 * i] = f.x;
    o.v[2 * i + 1] = f.y;
  }
  return o;
}
__device__ __forceinline__ void store8(__half* p, const float (&v)[8]) {
  uint4 r;
  __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = r;
}

// max and first-argmax (tap id r*S+s) of window (p,q) of channel plane `plane` for 8 images
template <int R, int S, int SH, int SW>
__device__ __forceinline__ void window2d(const __half* __restrict__ plane, int H, int W, int N, int p, int q, int n0,
                                         float (&best)[8], int (&arg)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) { best[i] = -FLT_MAX; arg[i] = 0; }
  // all taps are requested before the first compare, so that R*S loads are in flight per thread
  uint4 raw[R * S];
  bool ok[R * S];
#pragma unroll
  for (int r = 0; r < R; ++r) {
#pragma unroll
    for (int s = 0; s < S; ++s) {
      const int y = p * SH + r, x = q * SW + s;
      ok[r * S + s] = y < H && x < W;
      raw[r * S + s] = make_uint4(0, 0, 0, 0);
      if (ok[r * S + s]) raw[r * S + s] = __ldg(reinterpret_cast<const uint4*>(plane + (static_cast<long long>(y) * W + x) * N + n0));
    }
  }
#pragma unroll
  for (int k = 0; k < R * S; ++k) {
    if (!ok[k]) continue;
    const __half2* h = reinterpret_cast<const __half2*>(&raw[k]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      if (f.x > best[2 * i]) { best[2 * i] = f.x; arg[2 * i] = k; }
      if (f.y > best[2 * i + 1]) { best[2 * i + 1] = f.y; arg[2 * i + 1] = k; }
    }
  }
}

template <int R, int S, int SH, int SW>
__global__ void __launch_bounds__(256) pool2d_fprop_kernel(const __half* __restrict__ I, __half* __restrict__ O,
                                                          uint8_t* __restrict__ arg_out, int H, int W, int N,
                                                          int P, int Q, int mask_pos) {
  // one thread per output pixel and vector of 8 images; x walks (p, q, lane) of one channel plane
  // so that no thread of a block is idle whatever Q is
  const int nvec = N >> 3;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= P * Q * nvec) return;
  const int pq = t / nvec;
  const int n0 = (t - pq * nvec) << 3;
  const int p = pq / Q, q = pq - p * Q;
  const int c = blockIdx.y;
  const __half* plane = I + static_cast<long long>(c) * H * W * N;
  // All taps are requested before the first compare. The compares stay in fp16 (the inputs are
  // fp16, so the order is the same as in fp32) on packed pairs: a mask per pair says which of
  // the two running maxima a tap beats, and maxima and tap numbers are merged under that mask;
  // three instructions per pair and tap instead of converting every value to fp32.
  uint4 raw[R * S];
  bool ok[R * S];
#pragma unroll
  for (int r = 0; r < R; ++r) {
#pragma unroll
    for (int s = 0; s < S; ++s) {
      const int y = p * SH + r, x = q * SW + s;
      ok[r * S + s] = y < H && x < W;
      raw[r * S + s] = make_uint4(0, 0, 0, 0);
      if (ok[r * S + s])
        raw[r * S + s] = __ldg(reinterpret_cast<const uint4*>(plane + (static_cast<long long>(y) * W + x) * N + n0));
    }
  }
  uint32_t best[4], arg[4];   // two fp16 maxima / two 16-bit tap numbers per word
#pragma unroll
  for (int i = 0; i < 4; ++i) { best[i] = 0xfc00fc00u; arg[i] = 0u; }   // -inf, tap 0
#pragma unroll
  for (int k = 0; k < R * S; ++k) {
    if (!ok[k]) continue;
    const uint32_t w[4] = {raw[k].x, raw[k].y, raw[k].z, raw[k].w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t m = __hgt2_mask(*reinterpret_cast<const __half2*>(&w[i]), *reinterpret_cast<const __half2*>(&best[i]));
      best[i] = (w[i] & m) | (best[i] & ~m);
      arg[i] = ((static_cast<uint32_t>(k) * 0x00010001u) & m) | (arg[i] & ~m);
    }
  }
  const long long o = ((static_cast<long long>(c) * P + p) * Q + q) * N + n0;
  if (O) *reinterpret_cast<uint4*>(O + o) = make_uint4(best[0], best[1], best[2], best[3]);
  if (arg_out) {
    // one byte per output: the tap (r*S + s) of the first maximum. mask_pos 1: a window whose
    // maximum is not positive names no tap (its error is dropped); mask_pos 2: such windows are
    // flagged in bit 7 and the backward pass decides whether the flag counts.
    if (mask_pos) {
      const uint32_t zero2 = 0u;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t pos = __hgt2_mask(*reinterpret_cast<const __half2*>(&best[i]), *reinterpret_cast<const __half2*>(&zero2));
        arg[i] = mask_pos == 1 ? ((arg[i] & pos) | (0x00ff00ffu & ~pos)) : (arg[i] | (0x00800080u & ~pos));
      }
    }
    uint2 packed;
    packed.x = __byte_perm(arg[0], arg[1], 0x6420);   // low byte of each 16-bit tap number
    packed.y = __byte_perm(arg[2], arg[3], 0x6420);
    *reinterpret_cast<uint2*>(arg_out + o) = packed;
  }
}

// Backward, second stage: the thread that owns the SH x SW input block (a, b) reads the recorded
// argmax and the error of each overlapping window once and credits the block input it names.
template <int R, int S, int SH, int SW>
__global__ void __launch_bounds__(256) pool2d_gather_kernel(const uint8_t* __restrict__ arg,
                                                           const __half* __restrict__ E,
                                                           __half* __restrict__ dI, int H, int W, int N, int P, int Q,
                                                           int BW, uint32_t byte_and) {
  // byte_and 0x7f7f7f7f drops the "maximum not positive" flag of recorded argmax bytes (no ReLU
  // mask wanted); with 0xffffffff a flagged byte is >= 128 and matches no tap.
  constexpr int WP = (R + SH - 1) / SH, WQ = (S + SW - 1) / SW;
  const int nvec = N >> 3;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  const int BH = (H + SH - 1) / SH;
  if (t >= BH * BW * nvec) return;
  const int ab = t / nvec;
  const int n0 = (t - ab * nvec) << 3;
  const int a = ab / BW, b = ab - a * BW;
  const int c = blockIdx.y;
  float acc[SH][SW][8];
#pragma unroll
  for (int dy = 0; dy < SH; ++dy)
#pragma unroll
    for (int dx = 0; dx < SW; ++dx)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[dy][dx][i] = 0.0f;
  // the records and errors of all overlapping windows are requested before any is used
  uint2 rec[WP * WQ];
  uint4 err[WP * WQ];
  bool live[WP * WQ];
#pragma unroll
  for (int wp = 0; wp < WP; ++wp) {
#pragma unroll
    for (int wq = 0; wq < WQ; ++wq) {
      const int p = a - (WP - 1) + wp, q = b - (WQ - 1) + wq;
      const int w = wp * WQ + wq;
      live[w] = p >= 0 && p < P && q >= 0 && q < Q;
      rec[w] = make_uint2(0xffffffffu, 0xffffffffu);
      err[w] = make_uint4(0, 0, 0, 0);
      if (live[w]) {
        const long long o = ((static_cast<long long>(c) * P + p) * Q + q) * N + n0;
        rec[w] = __ldg(reinterpret_cast<const uint2*>(arg + o));
        err[w] = __ldg(reinterpret_cast<const uint4*>(E + o));
      }
    }
  }
#pragma unroll
  for (int wp = 0; wp < WP; ++wp) {
#pragma unroll
    for (int wq = 0; wq < WQ; ++wq) {
      if (!live[wp * WQ + wq]) continue;
      uint2 pk = rec[wp * WQ + wq];
      pk.x &= byte_and;
      pk.y &= byte_and;
      const int idx[8] = {static_cast<int>(pk.x & 255u), static_cast<int>((pk.x >> 8) & 255u),
                          static_cast<int>((pk.x >> 16) & 255u), static_cast<int>(pk.x >> 24),
                          static_cast<int>(pk.y & 255u), static_cast<int>((pk.y >> 8) & 255u),
                          static_cast<int>((pk.y >> 16) & 255u), static_cast<int>(pk.y >> 24)};
      Lanes8 e;
      {
        const __half2* h = reinterpret_cast<const __half2*>(&err[wp * WQ + wq]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __half22float2(h[i]);
          e.v[2 * i] = f.x;
          e.v[2 * i + 1] = f.y;
        }
      }
#pragma unroll
      for (int dy = 0; dy < SH; ++dy) {
        const int r = (WP - 1 - wp) * SH + dy;     // tap row of block input dy inside window p
        if (r >= R) continue;
#pragma unroll
        for (int dx = 0; dx < SW; ++dx) {
          const int s = (WQ - 1 - wq) * SW + dx;
          if (s >= S) continue;
          const int tap = r * S + s;
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (idx[i] == tap) acc[dy][dx][i] += e.v[i];
        }
      }
    }
  }
#pragma unroll
  for (int dy = 0; dy < SH; ++dy) {
    const int y = a * SH + dy;
    if (y >= H) break;
#pragma unroll
    for (int dx = 0; dx < SW; ++dx) {
      const int x = b * SW + dx;
      if (x >= W) break;
      store8(dI + ((static_cast<long long>(c) * H + y) * W + x) * N + n0, acc[dy][dx]);
    }
  }
}

// Each thread owns the SH x SW block of inputs at block coordinates (a, b). The windows that
// overlap the block are visited in increasing (p, q) order; a window's error goes to the block
// input that is its first maximum. Same sums in the same order as the per-element gather.
template <int R, int S, int SH, int SW>
__global__ void __launch_bounds__(256) pool2d_bprop_kernel(const __half* __restrict__ I, const __half* __restrict__ E,
                                                          __half* __restrict__ dI, int H, int W, int N, int P, int Q,
                                                          int BW, int mask_pos) {
  constexpr int WP = (R + SH - 1) / SH, WQ = (S + SW - 1) / SW;
  const int nvec = N >> 3;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  const int BH = (H + SH - 1) / SH;
  if (t >= BH * BW * nvec) return;
  const int ab = t / nvec;
  const int n0 = (t - ab * nvec) << 3;
  const int a = ab / BW, b = ab - a * BW;
  const int c = blockIdx.y;
  const __half* plane = I + static_cast<long long>(c) * H * W * N;
  float acc[SH][SW][8];
#pragma unroll
  for (int dy = 0; dy < SH; ++dy)
#pragma unroll
    for (int dx = 0; dx < SW; ++dx)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[dy][dx][i] = 0.0f;
#pragma unroll
  for (int wp = 0; wp < WP; ++wp) {
    const int p = a - (WP - 1) + wp;
    if (p < 0 || p >= P) continue;
#pragma unroll
    for (int wq = 0; wq < WQ; ++wq) {
      const int q = b - (WQ - 1) + wq;
      if (q < 0 || q >= Q) continue;
      float best[8];
      int arg[8];
      window2d<R, S, SH, SW>(plane, H, W, N, p, q, n0, best, arg);
      if (mask_pos) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (!(best[i] > 0.0f)) arg[i] = 255;
      }
      const Lanes8 e = load8(E + ((static_cast<long long>(c) * P + p) * Q + q) * N + n0);
#pragma unroll
      for (int dy = 0; dy < SH; ++dy) {
        constexpr int dummy = 0;
        (void)dummy;
        const int r = (WP - 1 - wp) * SH + dy;   // tap row of block input dy inside window p
        if (r >= R) continue;
#pragma unroll
        for (int dx = 0; dx < SW; ++dx) {
          const int s = (WQ - 1 - wq) * SW + dx;
          if (s >= S) continue;
          const int tap = r * S + s;
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (arg[i] == tap) acc[dy][dx][i] += e.v[i];
        }
      }
    }
  }
#pragma unroll
  for (int dy = 0; dy < SH; ++dy) {
    const int y = a * SH + dy;
    if (y >= H) break;
#pragma unroll
    for (int dx = 0; dx < SW; ++dx) {
      const int x = b * SW + dx;
      if (x >= W) break;
      store8(dI + ((static_cast<long long>(c) * H + y) * W + x) * N + n0, acc[dy][dx]);
    }
  }
}

template <int R, int S, int SH, int SW>
int launch_pool2d(const PoolGeo& g, const void* I, const void* EO, void* out, int mode, int* arg_ws,
                  cudaStream_t stream) {
  const int nvec = g.N / 8;
  dim3 fgrid((g.P * g.Q * nvec + 255) / 256, g.C);
  if (mode == 0) {
    pool2d_fprop_kernel<R, S, SH, SW><<<fgrid, 256, 0, stream>>>(
        static_cast<const __half*>(I), static_cast<__half*>(const_cast<void*>(EO)), nullptr, g.H, g.W, g.N, g.P, g.Q, 0);
    NG_CHECK_LAUNCH();
  } else if (mode == 3) {
    // forward pass that also records each window's argmax (bit 7: maximum not positive) in the
    // caller's buffer, for a later backward pass that then need not look at the input again
    pool2d_fprop_kernel<R, S, SH, SW><<<fgrid, 256, 0, stream>>>(
        static_cast<const __half*>(I), static_cast<__half*>(const_cast<void*>(EO)), reinterpret_cast<uint8_t*>(arg_ws),
        g.H, g.W, g.N, g.P, g.Q, 2);
    NG_CHECK_LAUNCH();
  } else if (mode == 4 || mode == 5) {
    // backward pass from a recorded argmax; mode 5 also applies the ReLU mask of the layer below
    const int BH = (g.H + SH - 1) / SH, BW = (g.W + SW - 1) / SW;
    dim3 grid((BH * BW * nvec + 255) / 256, g.C);
    pool2d_gather_kernel<R, S, SH, SW><<<grid, 256, 0, stream>>>(
        reinterpret_cast<const uint8_t*>(arg_ws), static_cast<const __half*>(EO), static_cast<__half*>(out), g.H, g.W,
        g.N, g.P, g.Q, BW, mode == 5 ? 0xffffffffu : 0x7f7f7f7fu);
    NG_CHECK_LAUNCH();
  } else if (R <= SH && S <= SW) {
    // windows do not overlap: one pass, each block of inputs sees at most one window
    const int BH = (g.H + SH - 1) / SH, BW = (g.W + SW - 1) / SW;
    dim3 grid((BH * BW * nvec + 255) / 256, g.C);
    pool2d_bprop_kernel<R, S, SH, SW><<<grid, 256, 0, stream>>>(
        static_cast<const __half*>(I), static_cast<const __half*>(EO), static_cast<__half*>(out), g.H, g.W, g.N, g.P,
        g.Q, BW, mode == 2);
    NG_CHECK_LAUNCH();
  } else {
    uint8_t* arg8 = reinterpret_cast<uint8_t*>(arg_ws);
    pool2d_fprop_kernel<R, S, SH, SW><<<fgrid, 256, 0, stream>>>(static_cast<const __half*>(I), nullptr, arg8, g.H,
                                                                g.W, g.N, g.P, g.Q, mode == 2);
    NG_CHECK_LAUNCH();
    const int BH = (g.H + SH - 1) / SH, BW = (g.W + SW - 1) / SW;
    dim3 grid((BH * BW * nvec + 255) / 256, g.C);
    pool2d_gather_kernel<R, S, SH, SW><<<grid, 256, 0, stream>>>(arg8, static_cast<const __half*>(EO),
                                                                 static_cast<__half*>(out), g.H, g.W, g.N, g.P, g.Q, BW,
                                                                 0xffffffffu);
    NG_CHECK_LAUNCH();
  }
  return NG_OK;
}

// returns NG_OK when a specialised kernel ran, 1 when the generic path must be used
int try_pool2d(const PoolGeo& g, const void* I, const void* EO, void* out, int mode, int* arg_ws,
               cudaStream_t stream) {
  const bool plain = g.J == 1 && g.T == 1 && g.D == 1 && g.str_j == 1 && g.str_d == 1 && g.pad_j == 0 &&
                     g.pad_d == 0 && g.pad_h == 0 && g.pad_w == 0 && g.N % 8 == 0 && g.C <= 65535 && g.H <= 65535 &&
                     (reinterpret_cast<uintptr_t>(I) & 15u) == 0 && (reinterpret_cast<uintptr_t>(EO) & 15u) == 0 &&
                     (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
  if (!plain) return 1;
  if (g.R == 3 && g.S == 3 && g.str_h == 2 && g.str_w == 2) return launch_pool2d<3, 3, 2, 2>(g, I, EO, out, mode, arg_ws, stream);
  if (g.R == 2 && g.S == 2 && g.str_h == 2 && g.str_w == 2) return launch_pool2d<2, 2, 2, 2>(g, I, EO, out, mode, arg_ws, stream);
  if (g.R == 3 && g.S == 3 && g.str_h == 3 && g.str_w == 3) return launch_pool2d<3, 3, 3, 3>(g, I, EO, out, mode, arg_ws, stream);
  return 1;
}

int grid_for(long long total, const DeviceCtx* c) {
  const long long blocks = (total + 255) / 256;
  return static_cast<int>(std::max<long long>(1, std::min<long long>(blocks, c->sm_count * 32ll)));
}

// Backward pass when the windows tile the input exactly (no padding, stride == window and the
// extents divisible, in all four pooled dimensions): one thread per window and vector of images
// reads the window once, finds its first maximum and writes every input of the window (the error
// at the maximum, zero elsewhere). One pass, no scratch, each byte moved once.
template <typename T, int V>
__global__ void pool_bprop_tiled_kernel(PoolGeo g, const T* __restrict__ I, const T* __restrict__ E,
                                        T* __restrict__ dI, int mask_pos) {
  const int nvec = g.N / V;
  const long long total = 1ll * g.K * g.M * g.P * g.Q * nvec;
  for (long long i = blockIdx.x * 1ll * blockDim.x + threadIdx.x; i < total; i += 1ll * gridDim.x * blockDim.x) {
    long long r = i;
    const int nv = r % nvec; r /= nvec;
    const int q = r % g.Q; r /= g.Q;
    const int p = r % g.P; r /= g.P;
    const int m = r % g.M; r /= g.M;
    const int k = static_cast<int>(r);
    float best[V];
    int arg[V];
    window_max<T, V>(g, I, k, m, p, q, nv, best, arg);
    const Vec<T, V> e = *reinterpret_cast<const Vec<T, V>*>(E + i * V);
    for (int j = 0; j < g.J; ++j)
      for (int t = 0; t < g.T; ++t)
        for (int rr = 0; rr < g.R; ++rr)
          for (int s = 0; s < g.S; ++s) {
            const int flat = (((k * g.J + j) * g.D + m * g.T + t) * g.H + p * g.R + rr) * g.W + q * g.S + s;
            Vec<T, V> out;
#pragma unroll
            for (int l = 0; l < V; ++l)
              out.set(l, (arg[l] == flat && !(mask_pos && !(best[l] > 0.0f))) ? e.get(l) : 0.0f);
            *reinterpret_cast<Vec<T, V>*>(dI + (1ll * flat * g.N + nv * V)) = out;
          }
  }
}

// ------------------------------------------------------------------------------------------
// Average and L2 pooling. The reference declares both ops and defines them in numpy
// (benchmarks/pool_test.py:141-146: the mean, and the root of the sum of squares, over all
// J*T*R*S window positions, positions outside the tensor counting as zeros), but its device path
// runs the max kernel whatever the op (nervanagpu/nervanagpu.py:797). The backward passes are
// the derivatives of those definitions: dI += E / (J*T*R*S), and dI += E * I / O (0 where O is 0).
// ------------------------------------------------------------------------------------------
enum PoolOp : int { POOL_MAX = 0, POOL_AVG = 1, POOL_L2 = 2 };

// sum (avg) or sum of squares (l2) of window (k,m,p,q), per image lane
template <typename T, int V>
__device__ __forceinline__ void window_sum(const PoolGeo& g, const T* __restrict__ I, int k, int m, int p, int q,
                                           int nv, bool squares, float (&acc)[V]) {
#pragma unroll
  for (int i = 0; i < V; ++i) acc[i] = 0.0f;
  const int c0 = k * g.str_j - g.pad_j, z0 = m * g.str_d - g.pad_d, y0 = p * g.str_h - g.pad_h,
            x0 = q * g.str_w - g.pad_w;
  for (int j = 0; j < g.J; ++j) {
    const int c = c0 + j;
    if (c < 0 || c >= g.C) continue;
    for (int t = 0; t < g.T; ++t) {
      const int z = z0 + t;
      if (z < 0 || z >= g.D) continue;
      for (int r = 0; r < g.R; ++r) {
        const int y = y0 + r;
        if (y < 0 || y >= g.H) continue;
        for (int s = 0; s < g.S; ++s) {
          const int x = x0 + s;
          if (x < 0 || x >= g.W) continue;
          const long long flat = ((1ll * c * g.D + z) * g.H + y) * g.W + x;
          const Vec<T, V> v = *reinterpret_cast<const Vec<T, V>*>(I + (flat * g.N + nv * V));
#pragma unroll
          for (int i = 0; i < V; ++i) {
            const float f = v.get(i);
            acc[i] += squares ? f * f : f;
          }
        }
      }
    }
  }
}

template <typename T, int V>
__global__ void pool_fprop_op_kernel(PoolGeo g, int op, const T* __restrict__ I, T* __restrict__ O) {
  const int nvec = g.N / V;
  const long long total = 1ll * g.K * g.M * g.P * g.Q * nvec;
  const float inv = 1.0f / static_cast<float>(g.J * g.T * g.R * g.S);
  for (long long i = blockIdx.x * 1ll * blockDim.x + threadIdx.x; i < total; i += 1ll * gridDim.x * blockDim.x) {
    long long r = i;
    const int nv = r % nvec; r /= nvec;
    const int q = r % g.Q; r /= g.Q;
    const int p = r % g.P; r /= g.P;
    const int m = r % g.M; r /= g.M;
    const int k = static_cast<int>(r);
    float acc[V];
    window_sum<T, V>(g, I, k, m, p, q, nv, op == POOL_L2, acc);
    Vec<T, V> out;
#pragma unroll
    for (int j = 0; j < V; ++j) out.set(j, op == POOL_L2 ? sqrtf(acc[j]) : acc[j] * inv);
    *reinterpret_cast<Vec<T, V>*>(O + i * V) = out;
  }
}

// One thread per input element (and image lane group): sums over the windows that contain it, in
// increasing (k,m,p,q) order. The L2 pass recomputes each such window's norm.
template <typename T, int V>
__global__ void pool_bprop_op_kernel(PoolGeo g, int op, const T* __restrict__ I, const T* __restrict__ E,
                                     T* __restrict__ dI) {
  const int nvec = g.N / V;
  const long long total = 1ll * g.C * g.D * g.H * g.W * nvec;
  const float inv = 1.0f / static_cast<float>(g.J * g.T * g.R * g.S);
  for (long long i = blockIdx.x * 1ll * blockDim.x + threadIdx.x; i < total; i += 1ll * gridDim.x * blockDim.x) {
    long long r = i;
    const int nv = r % nvec; r /= nvec;
    const int x = r % g.W; r /= g.W;
    const int y = r % g.H; r /= g.H;
    const int z = r % g.D; r /= g.D;
    const int c = static_cast<int>(r);
    int k0, k1, m0, m1, p0, p1, q0, q1;
    window_range(c, g.pad_j, g.J, g.str_j, g.K, k0, k1);
    window_range(z, g.pad_d, g.T, g.str_d, g.M, m0, m1);
    window_range(y, g.pad_h, g.R, g.str_h, g.P, p0, p1);
    window_range(x, g.pad_w, g.S, g.str_w, g.Q, q0, q1);
    const Vec<T, V> own = *reinterpret_cast<const Vec<T, V>*>(I + i * V);
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.0f;
    for (int k = k0; k <= k1; ++k)
      for (int m = m0; m <= m1; ++m)
        for (int p = p0; p <= p1; ++p)
          for (int q = q0; q <= q1; ++q) {
            const long long o = ((((1ll * k * g.M + m) * g.P + p) * g.Q + q) * g.N) + nv * V;
            const Vec<T, V> e = *reinterpret_cast<const Vec<T, V>*>(E + o);
            if (op == POOL_AVG) {
#pragma unroll
              for (int j = 0; j < V; ++j) acc[j] += e.get(j) * inv;
            } else {
              float sq[V];
              window_sum<T, V>(g, I, k, m, p, q, nv, true, sq);
#pragma unroll
              for (int j = 0; j < V; ++j) {
                // the forward pass stored the norm rounded to T: divide by that value
                Vec<T, 1> o1;
                o1.set(0, sqrtf(sq[j]));
                const float norm = o1.get(0);
                if (norm > 0.0f) acc[j] += e.get(j) * own.get(j) / norm;
              }
            }
          }
    Vec<T, V> out;
#pragma unroll
    for (int j = 0; j < V; ++j) out.set(j, acc[j]);
    *reinterpret_cast<Vec<T, V>*>(dI + i * V) = out;
  }
}

template <typename T, int VW>
int run_pool_op(const PoolGeo& g, int op, const void* I, const void* E, void* out, bool backward, DeviceCtx* c,
                cudaStream_t stream) {
  const bool vec = g.N % VW == 0 && (reinterpret_cast<uintptr_t>(I) & 15u) == 0 &&
                   (reinterpret_cast<uintptr_t>(E) & 15u) == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
  const long long out_elems = 1ll * g.K * g.M * g.P * g.Q * g.N;
  const long long in_elems = 1ll * g.C * g.D * g.H * g.W * g.N;
  const T* in = static_cast<const T*>(I);
  if (!backward) {
    if (vec) pool_fprop_op_kernel<T, VW><<<grid_for(out_elems / VW, c), 256, 0, stream>>>(g, op, in, static_cast<T*>(out));
    else pool_fprop_op_kernel<T, 1><<<grid_for(out_elems, c), 256, 0, stream>>>(g, op, in, static_cast<T*>(out));
  } else {
    const T* err = static_cast<const T*>(E);
    if (vec) pool_bprop_op_kernel<T, VW><<<grid_for(in_elems / VW, c), 256, 0, stream>>>(g, op, in, err, static_cast<T*>(out));
    else pool_bprop_op_kernel<T, 1><<<grid_for(in_elems, c), 256, 0, stream>>>(g, op, in, err, static_cast<T*>(out));
  }
  NG_CHECK_LAUNCH();
  return NG_OK;
}

bool tiles_exactly(const PoolGeo& g) {
  return g.pad_j == 0 && g.pad_d == 0 && g.pad_h == 0 && g.pad_w == 0 && g.str_j == g.J && g.str_d == g.T &&
         g.str_h == g.R && g.str_w == g.S && g.C % g.J == 0 && g.D % g.T == 0 && g.H % g.R == 0 && g.W % g.S == 0;
}

template <typename T, int VW>
int run_pool(const PoolGeo& g, const void* I, const void* EO, void* out, int mode, DeviceCtx* c,
             cudaStream_t stream) {
  const bool vec = g.N % VW == 0 && (reinterpret_cast<uintptr_t>(I) & 15u) == 0 &&
                   (reinterpret_cast<uintptr_t>(EO) & 15u) == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
  const long long out_elems = 1ll * g.K * g.M * g.P * g.Q * g.N;
  const long long in_elems = 1ll * g.C * g.D * g.H * g.W * g.N;
  // backward = record each window's argmax (scratch: one int per output element, in the
  // library workspace), then gather
  int* arg_ws = nullptr;
  if (mode != 0) {
    int rc = ensure_workspace(c, stream, static_cast<size_t>(out_elems) * sizeof(int));
    if (rc != NG_OK) return rc;
    arg_ws = reinterpret_cast<int*>(c->ws);
  }
  if (sizeof(T) == 2) {
    const int rc = try_pool2d(g, I, EO, out, mode, arg_ws, stream);
    if (rc <= 0) return rc;
  }
  if (mode != 0 && tiles_exactly(g)) {
    if (vec)
      pool_bprop_tiled_kernel<T, VW><<<grid_for(out_elems / VW, c), 256, 0, stream>>>(
          g, static_cast<const T*>(I), static_cast<const T*>(EO), static_cast<T*>(out), mode == 2);
    else
      pool_bprop_tiled_kernel<T, 1><<<grid_for(out_elems, c), 256, 0, stream>>>(
          g, static_cast<const T*>(I), static_cast<const T*>(EO), static_cast<T*>(out), mode == 2);
    NG_CHECK_LAUNCH();
    return NG_OK;
  }
  if (mode == 0) {
    T* O = static_cast<T*>(const_cast<void*>(EO));
    if (vec)
      pool_fprop_kernel<T, VW><<<grid_for(out_elems / VW, c), 256, 0, stream>>>(g, static_cast<const T*>(I), O, nullptr, 0);
    else
      pool_fprop_kernel<T, 1><<<grid_for(out_elems, c), 256, 0, stream>>>(g, static_cast<const T*>(I), O, nullptr, 0);
    NG_CHECK_LAUNCH();
  } else {
    if (vec) {
      pool_fprop_kernel<T, VW><<<grid_for(out_elems / VW, c), 256, 0, stream>>>(g, static_cast<const T*>(I), nullptr,
                                                                               arg_ws, mode == 2);
      NG_CHECK_LAUNCH();
      pool_gather_kernel<T, VW><<<grid_for(in_elems / VW, c), 256, 0, stream>>>(g, arg_ws, static_cast<const T*>(EO),
                                                                                static_cast<T*>(out));
    } else {
      pool_fprop_kernel<T, 1><<<grid_for(out_elems, c), 256, 0, stream>>>(g, static_cast<const T*>(I), nullptr, arg_ws,
                                                                          mode == 2);
      NG_CHECK_LAUNCH();
      pool_gather_kernel<T, 1><<<grid_for(in_elems, c), 256, 0, stream>>>(g, arg_ws, static_cast<const T*>(EO),
                                                                          static_cast<T*>(out));
    }
    NG_CHECK_LAUNCH();
  }
  return NG_OK;
}

}  // namespace
}  // namespace ngb

using namespace ngb;

extern "C" {

int ng_pool_output_dims(const ng_pool_desc* d, int* K, int* M, int* P, int* Q) {
  PoolGeo g;
  int rc = make_pool_geo(d, g);
  if (rc != NG_OK) return rc;
  if (K) *K = g.K;
  if (M) *M = g.M;
  if (P) *P = g.P;
  if (Q) *Q = g.Q;
  return NG_OK;
}

int ng_pool_fprop(const ng_pool_desc* d, int dtype_bytes, const void* I, void* O, void* stream) {
  PoolGeo g;
  int rc = make_pool_geo(d, g);
  if (rc != NG_OK) return rc;
  if (!I || !O) return fail(NG_ERR_INVALID_ARG, "null tensor");
  if (1ll * g.C * g.D * g.H * g.W > 0x7fffffffll) return fail(NG_ERR_TOO_LARGE, "too many pixels");
  DeviceCtx* c = current_ctx();
  if (!c) return NG_ERR_CUDA;
  if (dtype_bytes == 2) return run_pool<__half, 8>(g, I, O, O, 0, c, static_cast<cudaStream_t>(stream));
  if (dtype_bytes == 4) return run_pool<float, 4>(g, I, O, O, 0, c, static_cast<cudaStream_t>(stream));
  return fail(NG_ERR_UNSUPPORTED, "pooling supports fp16 and fp32 tensors");
}

int ng_pool_bprop(const ng_pool_desc* d, int dtype_bytes, const void* I, const void* E, void* gradI, void* stream) {
  PoolGeo g;
  int rc = make_pool_geo(d, g);
  if (rc != NG_OK) return rc;
  if (!I || !E || !gradI) return fail(NG_ERR_INVALID_ARG, "null tensor");
  if (1ll * g.C * g.D * g.H * g.W > 0x7fffffffll) return fail(NG_ERR_TOO_LARGE, "too many pixels");
  DeviceCtx* c = current_ctx();
  if (!c) return NG_ERR_CUDA;
  if (dtype_bytes == 2) return run_pool<__half, 8>(g, I, E, gradI, 1, c, static_cast<cudaStream_t>(stream));
  if (dtype_bytes == 4) return run_pool<float, 4>(g, I, E, gradI, 1, c, static_cast<cudaStream_t>(stream));
  return fail(NG_ERR_UNSUPPORTED, "pooling supports fp16 and fp32 tensors");
}

int ng_pool_fprop_op(const ng_pool_desc* d, int op, int dtype_bytes, const void* I, void* O, void* stream) {
  if (op == POOL_MAX) return ng_pool_fprop(d, dtype_bytes, I, O, stream);
  if (op != POOL_AVG && op != POOL_L2) return fail(NG_ERR_INVALID_ARG, "pooling op must be 0 (max), 1 (avg) or 2 (l2)");
  PoolGeo g;
  int rc = make_pool_geo(d, g);
  if (rc != NG_OK) return rc;
  if (!I || !O) return fail(NG_ERR_INVALID_ARG, "null tensor");
  DeviceCtx* c = current_ctx();
  if (!c) return NG_ERR_CUDA;
  if (dtype_bytes == 2) return run_pool_op<__half, 8>(g, op, I, nullptr, O, false, c, static_cast<cudaStream_t>(stream));
  if (dtype_bytes == 4) return run_pool_op<float, 4>(g, op, I, nullptr, O, false, c, static_cast<cudaStream_t>(stream));
  return fail(NG_ERR_UNSUPPORTED, "pooling supports fp16 and fp32 tensors");
}

int ng_pool_bprop_op(const ng_pool_desc* d, int op, int dtype_bytes, const void* I, const void* E, void* gradI,
                     void* stream) {
  if (op == POOL_MAX) return ng_pool_bprop(d, dtype_bytes, I, E, gradI, stream);
  if (op != POOL_AVG && op != POOL_L2) return fail(NG_ERR_INVALID_ARG, "pooling op must be 0 (max), 1 (avg) or 2 (l2)");
  PoolGeo g;
  int rc = make_pool_geo(d, g);
  if (rc != NG_OK) return rc;
  if (!I || !E || !gradI) return fail(NG_ERR_INVALID_ARG, "null tensor");
  DeviceCtx* c = current_ctx();
  if (!c) return NG_ERR_CUDA;
  if (dtype_bytes == 2) return run_pool_op<__half, 8>(g, op, I, E, gradI, true, c, static_cast<cudaStream_t>(stream));
  if (dtype_bytes == 4) return run_pool_op<float, 4>(g, op, I, E, gradI, true, c, static_cast<cudaStream_t>(stream));
  return fail(NG_ERR_UNSUPPORTED, "pooling supports fp16 and fp32 tensors");
}

int ng_pool_argmax_bytes(const ng_pool_desc* d, int dtype_bytes, size_t* bytes) {
  PoolGeo g;
  int rc = make_pool_geo(d, g);
  if (rc != NG_OK) return rc;
  if (!bytes) return fail(NG_ERR_INVALID_ARG, "bytes is null");
  const bool plain = dtype_bytes == 2 && g.J == 1 && g.T == 1 && g.D == 1 && g.str_j == 1 && g.str_d == 1 &&
                     g.pad_j == 0 && g.pad_d == 0 && g.pad_h == 0 && g.pad_w == 0 && g.N % 8 == 0 && g.C <= 65535 &&
                     g.H <= 65535 && g.str_h == g.str_w && g.R == g.S &&
                     ((g.R == 3 && (g.str_h == 2 || g.str_h == 3)) || (g.R == 2 && g.str_h == 2));
  *bytes = plain ? static_cast<size_t>(g.K) * g.M * g.P * g.Q * g.N : 0;
  return NG_OK;
}

int ng_pool_fprop_argmax(const ng_pool_desc* d, int dtype_bytes, const void* I, void* O, void* argmax, void* stream) {
  PoolGeo g;
  int rc = make_pool_geo(d, g);
  if (rc != NG_OK) return rc;
  if (!I || !O || !argmax) return fail(NG_ERR_INVALID_ARG, "null tensor");
  if (dtype_bytes != 2 || (reinterpret_cast<uintptr_t>(argmax) & 7u))
    return fail(NG_ERR_UNSUPPORTED, "recorded argmax needs fp16 tensors and an 8-byte aligned buffer");
  if (!current_ctx()) return NG_ERR_CUDA;
  rc = try_pool2d(g, I, O, O, 3, static_cast<int*>(argmax), static_cast<cudaStream_t>(stream));
  if (rc > 0) return fail(NG_ERR_UNSUPPORTED, "this pooling shape has no recorded-argmax path (see ng_pool_argmax_bytes)");
  return rc;
}

int ng_pool_bprop_argmax(const ng_pool_desc* d, int dtype_bytes, const void* argmax, const void* E, void* gradI,
                         int relu_mask, void* stream) {
  PoolGeo g;
  int rc = make_pool_geo(d, g);
  if (rc != NG_OK) return rc;
  if (!argmax || !E || !gradI) return fail(NG_ERR_INVALID_ARG, "null tensor");
  if (dtype_bytes != 2 || (reinterpret_cast<uintptr_t>(argmax) & 7u))
    return fail(NG_ERR_UNSUPPORTED, "recorded argmax needs fp16 tensors and an 8-byte aligned buffer");
  if (!current_ctx()) return NG_ERR_CUDA;
  rc = try_pool2d(g, nullptr, E, gradI, relu_mask ? 5 : 4,
                  static_cast<int*>(const_cast<void*>(argmax)), static_cast<cudaStream_t>(stream));
  if (rc > 0) return fail(NG_ERR_UNSUPPORTED, "this pooling shape has no recorded-argmax path (see ng_pool_argmax_bytes)");
  return rc;
}

int ng_pool_bprop_relu(const ng_pool_desc* d, int dtype_bytes, const void* I, const void* E, void* gradI,
                       void* stream) {
  PoolGeo g;
  int rc = make_pool_geo(d, g);
  if (rc != NG_OK) return rc;
  if (!I || !E || !gradI) return fail(NG_ERR_INVALID_ARG, "null tensor");
  if (1ll * g.C * g.D * g.H * g.W > 0x7fffffffll) return fail(NG_ERR_TOO_LARGE, "too many pixels");
  DeviceCtx* c = current_ctx();
  if (!c) return NG_ERR_CUDA;
  if (dtype_bytes == 2) return run_pool<__half, 8>(g, I, E, gradI, 2, c, static_cast<cudaStream_t>(stream));
  if (dtype_bytes == 4) return run_pool<float, 4>(g, I, E, gradI, 2, c, static_cast<cudaStream_t>(stream));
  return fail(NG_ERR_UNSUPPORTED, "pooling supports fp16 and fp32 tensors");
}

}  // extern "C"
