// Output stage shared by the tensor-core kernel, the split-K reduction and the SIMT kernels.
// Order of operations follows the reference's GEMM epilogue
// (kernels/sass/hgemm_common_128x128.sass:183-272, documented at nervanagpu/nervanagpu.py:960-965):
//   c = acc * alpha;  c = relu ? max(c, 0) : c;  c += beta * C_old;  round.
#pragma once
#include "common.cuh"

namespace ngb {

struct EpiArgs {
  float alpha, beta;
  int relu;
  int sr_bits;
  uint32_t seed_lo, seed_hi, rng_offset;
};

// Random bits for the 8 consecutive outputs that start at linear element index e8*8.
// One Philox block serves 8 elements (16 bits each); formats that keep fewer than 7 mantissa
// bits need more than 16 random bits, so a second block is drawn for them.
__device__ __forceinline__ void sr_bits8(const EpiArgs& e, unsigned long long e8, uint32_t (&rnd)[8]) {
  const Philox4 a = philox4x32_10(static_cast<uint32_t>(e8), static_cast<uint32_t>(e8 >> 32), e.rng_offset, 0u,
                                  e.seed_lo, e.seed_hi);
  if (e.sr_bits >= 7) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      rnd[2 * i] = a.v[i] & 0xffffu;
      rnd[2 * i + 1] = a.v[i] >> 16;
    }
  } else {
    const Philox4 b = philox4x32_10(static_cast<uint32_t>(e8), static_cast<uint32_t>(e8 >> 32), e.rng_offset, 1u,
                                    e.seed_lo, e.seed_hi);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      rnd[i] = a.v[i];
      rnd[4 + i] = b.v[i];
    }
  }
}

// Stochastic rounding of 8 consecutive outputs to fp16, out of line: ten Philox rounds inlined at
// every use made the tensor-core kernel's code several times larger than the instruction cache
// (and the round-to-nearest path paid for it in instruction-cache misses). `lin` is the linear
// index of the first element; groups that do not start on a multiple of 8 (ragged rows) draw
// per element.
static __device__ __noinline__ uint4 sr_round8(EpiArgs e, unsigned long long lin, float v0, float v1, float v2, float v3,
                                        float v4, float v5, float v6, float v7) {
  const float v[8] = {v0, v1, v2, v3, v4, v5, v6, v7};
  __half h[8];
  if ((lin & 7ull) == 0ull) {
    uint32_t rnd[8];
    sr_bits8(e, lin >> 3, rnd);
#pragma unroll
    for (int i = 0; i < 8; ++i) h[i] = f2h_sr(v[i], rnd[i], e.sr_bits);
  } else {
#pragma unroll 1
    for (int i = 0; i < 8; ++i) {
      uint32_t r8[8];
      const unsigned long long li = lin + i;
      sr_bits8(e, li >> 3, r8);
      h[i] = f2h_sr(v[i], r8[li & 7ull], e.sr_bits);
    }
  }
  uint4 o;
  __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) oh[i] = __halves2half2(h[2 * i], h[2 * i + 1]);
  return o;
}

__device__ __forceinline__ float epi_scale(const EpiArgs& e, float acc) {
  float c = acc * e.alpha;
  if (e.relu) c = fmaxf(c, 0.0f);
  return c;
}

// Finish 8 consecutive outputs of one row. `v` holds raw accumulators. `lin` is the logical
// linear index of the first element (multiple of 8 when vec is true). `nvalid` <= 8.
template <bool F32OUT>
__device__ __forceinline__ void epi_store8(const EpiArgs& e, float (&v)[8], void* crow, const void* oldrow,
                                           int col, unsigned long long lin, int nvalid, bool vec) {
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = epi_scale(e, v[i]);

  if (F32OUT) {
    float* out = static_cast<float*>(crow) + col;
    if (e.beta != 0.0f) {
      const float* old = static_cast<const float*>(oldrow) + col;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (i < nvalid) v[i] = fmaf(e.beta, old[i], v[i]);
    }
    if (vec && nvalid == 8) {
      reinterpret_cast<float4*>(out)[0] = make_float4(v[0], v[1], v[2], v[3]);
      reinterpret_cast<float4*>(out)[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (i < nvalid) out[i] = v[i];
    }
    return;
  }

  __half* out = static_cast<__half*>(crow) + col;
  if (e.beta != 0.0f) {
    const __half* old = static_cast<const __half*>(oldrow) + col;
    if (vec && nvalid == 8) {
      const uint4 o = *reinterpret_cast<const uint4*>(old);
      const __half2* oh = reinterpret_cast<const __half2*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(oh[i]);
        v[2 * i] = fmaf(e.beta, f.x, v[2 * i]);
        v[2 * i + 1] = fmaf(e.beta, f.y, v[2 * i + 1]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (i < nvalid) v[i] = fmaf(e.beta, __half2float(old[i]), v[i]);
    }
  }
  __half h[8];
  if (e.sr_bits) {
    const uint4 packed = sr_round8(e, lin, v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7]);
    const __half* ph = reinterpret_cast<const __half*>(&packed);
#pragma unroll
    for (int i = 0; i < 8; ++i) h[i] = ph[i];
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) h[i] = f2h_rn(v[i]);
  }
  if (vec && nvalid == 8) {
    uint4 o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) oh[i] = __halves2half2(h[2 * i], h[2 * i + 1]);
    *reinterpret_cast<uint4*>(out) = o;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < nvalid) out[i] = h[i];
  }
}

// epi_store8 as a call, for the tensor-core kernel's register-store path (outputs that cannot be
// staged: ragged or unaligned rows). That path is rare and the kernel's hot loops must stay within
// the instruction cache, so its four uses share one copy of the code.
template <bool F32OUT>
__device__ __noinline__ void epi_store8_call(EpiArgs e, float v0, float v1, float v2, float v3, float v4, float v5,
                                             float v6, float v7, void* crow, const void* oldrow, int col,
                                             unsigned long long lin, int nvalid, bool vec) {
  float v[8] = {v0, v1, v2, v3, v4, v5, v6, v7};
  epi_store8<F32OUT>(e, v, crow, oldrow, col, lin, nvalid, vec);
}

// Same arithmetic as epi_store8 for 8 consecutive, fully valid, 16-byte aligned outputs, but the
// result is returned in registers (one 16-byte vector of fp16, or two of fp32) so the caller can
// stage it in shared memory for a bulk tensor store. `oldp` points at the 8 old values or is null.
template <bool F32OUT>
__device__ __forceinline__ void epi_pack8(const EpiArgs& e, float (&v)[8], const void* oldp, unsigned long long lin,
                                          uint4& lo, uint4& hi) {
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = epi_scale(e, v[i]);
  if (F32OUT) {
    if (e.beta != 0.0f && oldp) {
      const float4 a = reinterpret_cast<const float4*>(oldp)[0], b = reinterpret_cast<const float4*>(oldp)[1];
      v[0] = fmaf(e.beta, a.x, v[0]); v[1] = fmaf(e.beta, a.y, v[1]); v[2] = fmaf(e.beta, a.z, v[2]);
      v[3] = fmaf(e.beta, a.w, v[3]); v[4] = fmaf(e.beta, b.x, v[4]); v[5] = fmaf(e.beta, b.y, v[5]);
      v[6] = fmaf(e.beta, b.z, v[6]); v[7] = fmaf(e.beta, b.w, v[7]);
    }
    lo = make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
    hi = make_uint4(__float_as_uint(v[4]), __float_as_uint(v[5]), __float_as_uint(v[6]), __float_as_uint(v[7]));
    return;
  }
  if (e.beta != 0.0f && oldp) {
    const uint4 o = *reinterpret_cast<const uint4*>(oldp);
    const __half2* oh = reinterpret_cast<const __half2*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(oh[i]);
      v[2 * i] = fmaf(e.beta, f.x, v[2 * i]);
      v[2 * i + 1] = fmaf(e.beta, f.y, v[2 * i + 1]);
    }
  }
  __half2* oh = reinterpret_cast<__half2*>(&lo);
  if (e.sr_bits) {
    lo = sr_round8(e, lin, v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7]);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) oh[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
  }
  hi = lo;
}

}  // namespace ngb
