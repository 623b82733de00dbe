// Shared device-side helpers for the sm_100a kernels: mbarrier, TMA, tcgen05/TMEM
// wrappers (inline PTX), bounded waits, Philox, fp16 rounding modes.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "status.h"

namespace ngb {

// ----------------------------------------------------------------------------------------
// small utilities
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " elect.sync _|p, 0xffffffff;\n"
      " selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ----------------------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      " selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Every wait in these kernels is bounded: after `limit_ns` without progress (kWaitLimitNs unless
// the host set another limit) the waiter raises the CTA-wide abort flag, records `code` in the
// global status word (first error wins) and returns false; callers unwind to the common teardown.
constexpr uint64_t kWaitLimitNs = 2000000000ull;

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code, uint64_t limit_ns = kWaitLimitNs) {
  // The clock stays off the path of a wait that ends soon: it is first read after 1024 failed
  // polls (each of which already blocks for a while in hardware), and the limit counts from there.
  uint64_t t0 = 0;
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 0x3ff) == 0) {
      if (*abort_flag) return false;
      const uint64_t now = global_timer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > limit_ns) {
        *abort_flag = 1;
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}

// ----------------------------------------------------------------------------------------
// TMA (tiled mode, rank 5 everywhere; unused trailing dims have extent 1)
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0,
                                            int c1, int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
      "r"(c4)
      : "memory");
}

// Store of one box from shared memory (bulk async-group completion).
__device__ __forceinline__ void tma_store_5d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3,
                                             int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// wait until at most N of this thread's bulk groups still have to READ their shared-memory source
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// wait until all of this thread's bulk groups are complete (writes performed)
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// make generic-proxy writes to shared memory visible to the async proxy (TMA)
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// The same load issued by one CTA of a CTA pair (cta_group::2): the data lands in this CTA's
// shared memory, the bytes are counted on `bar`, a shared::cluster address that may name the
// barrier of the pair's other CTA. (No multicast: each CTA fetches what it holds.)
__device__ __forceinline__ void tma_load_5d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int c0,
                                                 int c1, int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
      "r"(c4)
      : "memory");
}

// ----------------------------------------------------------------------------------------
// thread-block clusters (CTA pairs)
// ----------------------------------------------------------------------------------------
// Programmatic dependent launch. A kernel launched with the programmatic-serialization attribute
// may start while the kernel before it in the stream still runs; grid_dependency_wait() returns
// once that kernel has finished and its writes are visible (at once when the launch carried no
// such attribute). grid_launch_dependents() lets the kernel after this one start being scheduled
// (it waits in turn, so nothing of it that matters runs early).
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the location `smem_addr` (a shared::cta address) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on a barrier given by its shared::cluster address (this CTA's or the peer's)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ----------------------------------------------------------------------------------------
// tcgen05 / TMEM
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
// CTA pairs: both CTAs allocate / free the same columns together (same warp index in each)
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], fp16 inputs, fp32 accumulate, issued by one thread.
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same with the descriptors given as (low, high) words, so that the issuing thread steps the
// start-address field with one 32-bit add per operand and K step. kPair: the two-SM form below.
template <bool kPair>
__device__ __forceinline__ void tc_mma_f16_words(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                                 uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  if (kPair) {
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " .reg .b64 da, db;\n"
        " setp.ne.b32 p, %6, 0;\n"
        " mov.b64 da, {%1, %2};\n"
        " mov.b64 db, {%3, %4};\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n"
        "}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " .reg .b64 da, db;\n"
        " setp.ne.b32 p, %6, 0;\n"
        " mov.b64 da, {%1, %2};\n"
        " mov.b64 db, {%3, %4};\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n"
        "}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// kCount (1..4) MMAs of one k-block into one accumulator as a single block of PTX: the first takes
// `accumulate`, the others add; the start-address fields step by a_kstep / b_kstep (16-byte units)
// from one to the next. One statement, so that no control flow of the surrounding loop ends up
// between the MMAs: the issuing thread has to get each of them out in well under the 128 cycles
// the tensor pipe spends on it.
template <bool kPair, int kCount>
__device__ __forceinline__ void tc_mma_f16_run(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                               uint32_t b_hi, uint32_t idesc, uint32_t accumulate, uint32_t a_kstep,
                                               uint32_t b_kstep) {
#define NG_MMA_OP(group) " tcgen05.mma.cta_group::" group ".kind::f16 [%0], da, db, %5, "
#define NG_MMA_STEP(group)                                       \
  " add.u32 al, al, %7;\n add.u32 bl, bl, %8;\n"                \
  " mov.b64 da, {al, %2};\n mov.b64 db, {bl, %4};\n" NG_MMA_OP(group) "q;\n"
#define NG_MMA_RUN(group, more)                                                                            \
  asm volatile(                                                                                            \
      "{\n .reg .pred p, q;\n .reg .b64 da, db;\n .reg .b32 al, bl;\n"                                    \
      " setp.ne.b32 p, %6, 0;\n setp.eq.b32 q, %6, %6;\n mov.b32 al, %1;\n mov.b32 bl, %3;\n"            \
      " mov.b64 da, {al, %2};\n mov.b64 db, {bl, %4};\n" NG_MMA_OP(group) "p;\n" more "}\n"               \
      ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(a_kstep), \
      "r"(b_kstep)                                                                                         \
      : "memory")
  if (kPair) {
    if (kCount == 1) NG_MMA_RUN("2", "");
    else if (kCount == 2) NG_MMA_RUN("2", NG_MMA_STEP("2"));
    else if (kCount == 3) NG_MMA_RUN("2", NG_MMA_STEP("2") NG_MMA_STEP("2"));
    else NG_MMA_RUN("2", NG_MMA_STEP("2") NG_MMA_STEP("2") NG_MMA_STEP("2"));
  } else {
    if (kCount == 1) NG_MMA_RUN("1", "");
    else if (kCount == 2) NG_MMA_RUN("1", NG_MMA_STEP("1"));
    else if (kCount == 3) NG_MMA_RUN("1", NG_MMA_STEP("1") NG_MMA_STEP("1"));
    else NG_MMA_RUN("1", NG_MMA_STEP("1") NG_MMA_STEP("1") NG_MMA_STEP("1"));
  }
#undef NG_MMA_RUN
#undef NG_MMA_STEP
#undef NG_MMA_OP
}
// The two-SM form: D is 256 rows (128 in the tensor memory of each CTA of the pair), A comes from
// both CTAs' shared memory (128 rows each), B likewise (half of the columns each), all at the
// same offsets; issued by one thread of the pair's first CTA.
__device__ __forceinline__ void tc_mma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on `bar_cluster` (shared::cluster address: either CTA's barrier) once all MMAs this
// thread issued for the pair have completed
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster)
               : "memory");
}
// mbarrier arrive once all previously issued MMAs of this thread have completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread t of the warp gets TMEM lane (base_lane + t).
__device__ __forceinline__ void tc_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// ----------------------------------------------------------------------------------------
// Philox4x32-10 (counter-based RNG): 128 random bits per (counter, key) pair.
// ----------------------------------------------------------------------------------------
struct Philox4 {
  uint32_t v[4];
};

__host__ __device__ __forceinline__ Philox4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                                          uint32_t k0, uint32_t k1) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = static_cast<uint64_t>(M0) * c0;
    const uint64_t p1 = static_cast<uint64_t>(M1) * c2;
    const uint32_t hi0 = static_cast<uint32_t>(p0 >> 32), lo0 = static_cast<uint32_t>(p0);
    const uint32_t hi1 = static_cast<uint32_t>(p1 >> 32), lo1 = static_cast<uint32_t>(p1);
    const uint32_t n0 = hi1 ^ c1 ^ k0;
    const uint32_t n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += W0; k1 += W1;
  }
  Philox4 out;
  out.v[0] = c0; out.v[1] = c1; out.v[2] = c2; out.v[3] = c3;
  return out;
}

// ----------------------------------------------------------------------------------------
// fp32 -> fp16 rounding
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ __half f2h_rn(float x) { return __float2half_rn(x); }

// Stochastic rounding to `mbits` (1..10) fp16 mantissa bits: add a uniform integer below one
// target ulp to the magnitude bits, then truncate toward zero. `rnd` supplies >= 23-mbits bits.
// The result is one of the two representable neighbours of x, upper one with probability equal
// to the fractional position of x between them. Below the fp16 normal range the target ulp is
// the fixed subnormal spacing 2^-24.
__device__ __forceinline__ __half f2h_sr(float x, uint32_t rnd, int mbits) {
  uint32_t b = __float_as_uint(x);
  const uint32_t expo = (b >> 23) & 0xffu;
  if (expo == 0xffu) return __float2half_rn(x);  // inf / nan pass through
  if (expo >= 113u) {                            // |x| >= 2^-14: fp16-normal range
    const int drop = 23 - mbits;
    const uint32_t mask = (1u << drop) - 1u;
    b += (rnd & mask);
    b &= ~mask;
    return __float2half_rz(__uint_as_float(b));
  }
  // subnormal fp16 range: spacing 2^-24 (scaled up by dropped mantissa bits if mbits < 10)
  const float ulp = __uint_as_float((103u + static_cast<uint32_t>(10 - mbits)) << 23);  // 2^(-24+10-mbits)
  const float u = static_cast<float>(rnd & 0xfffu) * (1.0f / 4096.0f);                  // [0,1)
  const float mag = fabsf(x) + u * ulp;
  const float q = floorf(mag / ulp) * ulp;
  return __float2half_rz(copysignf(q, x));
}

}  // namespace ngb
