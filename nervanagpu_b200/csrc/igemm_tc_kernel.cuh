// tcgen05 / TMEM / TMA implicit-GEMM engine for sm_100a.
//
// One persistent, warp-specialised kernel computes D[M x N] = A[M x Kred] * B[Kred x N] with fp16
// operands staged in 128-byte-swizzled shared memory by TMA, fp32 accumulation in tensor memory
// and a fused epilogue (alpha, ReLU, beta*C, round-to-nearest or stochastic rounding, fp16 or
// fp32 store, or raw fp32 split-K partials).
//
//   warp 0      TMA producer: one lane per box of a k-block issues the load
//   warp 1      allocates TMEM, one lane issues tcgen05.mma and the commits
//   warps 2..9  epilogue: two warps per group of 32 TMEM lanes, each takes half of the columns;
//               tcgen05.ld 32 lanes x 32 columns at a time, convert, then either a bulk tensor
//               store through swizzled shared memory or stores straight from registers
//
// TMEM holds 512 fp32 columns, used in one of three ways:
//   128-row tiles   two accumulators of block_n columns, double-buffered across tiles so that the
//                   epilogue of tile i overlaps the main loop of tile i+1
//   256-row tiles   two accumulators that share every B operand (half the B traffic per flop)
//   weight update   up to eight accumulators, one per group of filter taps, that share every
//                   chunk of the error tensor; taps with few rows are stacked inside one accumulator
// All waits are bounded (see mbar_wait).
//
// It replaces the reference's register-tiled FFMA kernels: hgemm_{nn,nt,tn}_* for ng.dot
// (nervanagpu/nervanagpu.py:959-1105), hconv_fprop_K64_N64, hconv_bprop_C64_N64/C32_N64 and
// hconv_updat_C128_K64/K128 for the convolution passes (nervanagpu/nervanagpu.py:642-734).
#pragma once
#include "igemm_tc.cuh"

#include "common.cuh"
#include "epilogue.cuh"

namespace ngb {

namespace {

__device__ __forceinline__ int fast_div(int n, const FastDiv& f) {
  return f.d == 1u ? n : static_cast<int>(__umulhi(static_cast<uint32_t>(n), f.mul) >> f.shr);
}

struct ChunkPos {
  int inner0, q, p, m;
  bool valid;
};

// Position of 64-element chunk `chunk` in a (m, p, q, n) pixel space. In flattened mode the
// (q, n) pair is one dimension of extent Q*N and dec_q == 1.
__device__ __forceinline__ ChunkPos decode_chunk(const TcParams& p, int chunk) {
  ChunkPos c;
  const int g = fast_div(chunk, p.fd_cpi);
  c.inner0 = (chunk - g * p.dec_cpi) * kChunk;
  const int g2 = fast_div(g, p.fd_q);
  c.q = g - g2 * p.dec_q;
  c.m = fast_div(g2, p.fd_p);
  c.p = g2 - c.m * p.dec_p;
  c.valid = c.m < p.dec_m;
  return c;
}

struct Tap {
  int t, r, s;
};
__device__ __forceinline__ Tap decode_tap(const TcParams& p, int trs) {
  Tap tp;
  tp.t = fast_div(trs, p.fd_RS);
  const int rs = trs - tp.t * p.RS;
  tp.r = fast_div(rs, p.fd_S);
  tp.s = rs - tp.r * p.S;
  return tp;
}

// Producer state that is stepped from one k-block to the next.
struct Walk {
  ChunkPos cp;
  Tap tap;
  int trs, rc, kb;
};

// Exact division for the strided gather of the backward pass: returns false when `num` is not
// a multiple of `den` (that tap does not touch this pixel).
__device__ __forceinline__ bool div_exact(int num, int den, int& out) {
  if (den == 1) {
    out = num;
    return true;
  }
  if (num < 0) {
    out = -1;  // out of range either way
    return true;
  }
  out = num / den;
  return out * den == num;
}

// Row coordinate of a box that must read zeros (a chunk past the end of the pixel space): this far
// beyond the last row, so that the per-tap steps added to it cannot bring it back inside.
constexpr int kFarRows = 1 << 16;

struct WorkItem {
  int tile_m, tile_n, z, split, kb0, kb1;
  int m0;     // first output row of the item
  int live;   // 256-row tiles: accumulators (row halves) the item computes, 0 = nothing to do; else 1
};
// Items [0, full_items) are whole tiles. With 256-row tiles the tiles of the last, partly filled
// wave are cut into their two 128-row halves, items full_items + 2 * t + h, so that this wave
// takes half a tile time on twice as many SMs.
__device__ __forceinline__ WorkItem decode_work(const TcParams& p, int w) {
  WorkItem it;
  int half = -1;
  if (w >= p.full_items) {
    const int hw = w - p.full_items;
    w = p.full_items + (hw >> 1);
    half = hw & 1;
  }
  int r = fast_div(w, p.fd_tiles_m);
  it.tile_m = w - r * p.tiles_m;
  const int r2 = fast_div(r, p.fd_tiles_n);
  it.tile_n = r - r2 * p.tiles_n;
  it.split = fast_div(r2, p.fd_nz);
  it.z = r2 - it.split * p.nz;
  it.kb0 = it.split * p.kb_per_split;
  it.kb1 = min(p.num_kb, it.kb0 + p.kb_per_split);
  it.m0 = it.tile_m * kTileM * p.m_halves + (half > 0 ? kTileM : 0);
  it.live = 1;
  if (p.m_halves == 2) {
    it.live = half >= 0 ? 1 : (it.m0 + kTileM < p.M ? 2 : 1);
    if (it.m0 >= p.M) it.live = 0;
  }
  return it;
}

}  // namespace

// One instance per mode (kMode = p.mode): the producer of each carries only its own coordinate
// code, which keeps the single-warp roles' loops short in the instruction cache.
// kLean instances serve the common output stage only (tiles staged through shared memory,
// alpha 1, no beta term, round to nearest, or raw split-K partials) and carry no other.
// kPair instances run as clusters of two CTAs on the two SMs of a pair (tcgen05 cta_group::2):
// a work item is a tile of 256 rows, 128 in the tensor memory of each CTA; each CTA loads its own
// 128 rows of A and its own half of the columns of B (plain TMA loads, no multicast) and the MMA,
// issued by one thread of the first CTA, reads both halves of B from the two shared memories. Per
// flop each SM takes in a third fewer operand bytes than with a 128-row tile of its own, and the
// accumulators stay double-buffered across tiles.
template <int kMode, bool kLean, bool kPair = false>
__global__ void __launch_bounds__(kTcThreads, 1)
igemm_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                const __grid_constant__ CUtensorMap mapBm, const __grid_constant__ TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  // ring buffer must be 1024-byte aligned for the 128-byte swizzle pattern
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t ring_bytes = static_cast<uint32_t>(p.stages) * p.stage_bytes;
  // output staging (staged epilogue only), then the control block
  const uint32_t epi_base = smem_base + ring_bytes;
  const bool staged = kLean || p.store_staged != 0;
  const uint32_t epi_bytes = staged ? kEpiStageBytes : 0u;

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + ring_bytes + epi_bytes);
  const uint32_t bar_base = smem_base + ring_bytes + epi_bytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
  auto accf_bar = [&](int a) { return bar_base + 8u * (2 * kMaxStages + a); };
  auto acce_bar = [&](int a) { return bar_base + 8u * (2 * kMaxStages + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_work = p.total_items;   // tiles_m * tiles_n * nz * splits, plus the halves of a cut last wave
  const uint32_t tmem_cols = 512;  // 2 accumulators of up to 256 columns
  // CTA pairs: rank of this CTA in its pair; both walk the pair's work items
  const uint32_t rank = kPair ? cluster_cta_rank() : 0u;
  const int w_first = kPair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int w_step = kPair ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  const int row_shift = kPair ? static_cast<int>(rank) * kTileM : 0;              // this CTA's rows of the tile
  const int col_shift = kPair ? static_cast<int>(rank) * (p.block_n >> 1) : 0;    // its columns of B

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(accf_bar(a), 1);
      mbar_init(acce_bar(a), kPair ? 2 * kEpiWarps : kEpiWarps);   // (pairs: both CTAs' epilogues report to the first)
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&mapA);
    tma_prefetch_desc(&mapB);
    if (p.b_merge == 1 || p.b_merge == 2) tma_prefetch_desc(&mapBm);
  }
  if (warp == 1) {
    if (kPair) {
      tmem_alloc_pair(smem_u32(tmem_slot), tmem_cols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_slot), tmem_cols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (kPair) cluster_sync_all();   // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above (barriers, tensor memory, descriptor prefetch) may run while the kernel
  // before this one in the stream drains; its results are needed from here on. (Letting the next
  // kernel in as soon as this one has started, griddepcontrol.launch_dependents here, made whole
  // training steps 4 % slower: its blocks wait on the SMs this kernel's tail still needs.)
  grid_dependency_wait();

  if (warp == 0) {
    // =========================== TMA producer ===========================
    const int nboxes = p.a_boxes + p.b_boxes;
    const bool active = lane < nboxes;
    const bool is_a = lane < p.a_boxes;
    const int bi = is_a ? lane : lane - p.a_boxes;
    const CUtensorMap* map = is_a ? &mapA : &mapB;
    bool merged = false;   // this item's B operand comes as one box (convolutions, see b_merge)
    const uint32_t box_off = is_a ? bi * p.a_box_bytes : p.a_bytes + bi * p.b_box_bytes;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    // steps of the box coordinates per tap (s, r, t) and per reduction chunk, see below
    const bool linear = (kMode == TC_FPROP || (kMode == TC_BPROP && p.str_w == 1 && p.str_h == 1 && p.str_d == 1));
    int ls[5] = {0, 0, 0, 0, 0}, lr[5] = {0, 0, 0, 0, 0}, lt[5] = {0, 0, 0, 0, 0}, lc[5] = {0, 0, 0, 0, 0};
    int steps_for = -1;   // form of the B box (0 per chunk, 1 merged) the steps were taken for; -1 = not yet
    for (int w = w_first; w < total_work && ok; w += w_step) {
      const WorkItem it = decode_work(p, w);
      if (it.live == 0) continue;
      const int m0 = it.m0 * (kPair ? 2 : 1) + row_shift;
      const int n0 = it.tile_n * p.block_n + col_shift;
      // an item that computes one half of a 256-row tile needs only that half's A boxes when they
      // are separate boxes (MN-major A); a K-major A box always carries all its rows
      const int a_live = (p.m_halves == 2 && it.live == 1 && p.a_mn_major) ? (p.a_boxes >> 1) : p.a_boxes;
      bool act = active && (!is_a || bi < a_live);
      const uint32_t tx_item = p.tx_bytes - static_cast<uint32_t>(p.a_boxes - a_live) * p.a_box_bytes;
      // Per-tile state of this lane's box. Everything that changes from one k-block to the next
      // is kept as counters that are stepped, not re-derived: integer division by run-time
      // values costs this single warp more than the MMAs of a k-block take.
      Walk wk;
      wk.cp = {0, 0, 0, 0, true};   // fprop/bprop: pixel chunk of this B box; update: walks
      wk.tap = {0, 0, 0};           // fprop/bprop: walks the filter taps; update: fixed (z)
      wk.trs = 0; wk.rc = 0;        // tap number and reduction-chunk number inside the tap
      wk.kb = it.kb0;
      bool tap_live = true;         // update: this A box's tap exists (last group may be short)
      if (kMode == TC_FPROP || kMode == TC_BPROP) {
        // (b_merge 4: a box carries the two chunks of one pixel)
        if (!is_a) wk.cp = decode_chunk(p, n0 / kChunk + (p.b_merge == 4 ? 2 * bi : bi));
        if (p.b_merge == 1 || p.b_merge == 2) {
          // A column tile that lies inside one image row arrives as one box (its chunks are
          // consecutive pixels / image groups of that row); other tiles chunk by chunk.
          const ChunkPos first = decode_chunk(p, n0 / kChunk);
          const int cpi0 = first.inner0 / kChunk;
          merged = first.valid && (p.dec_q - first.q) * p.dec_cpi - cpi0 >= p.b_boxes;
          if (merged && !is_a) {
            act = act && bi == 0;
            map = &mapBm;
          } else if (!is_a) {
            map = &mapB;
          }
        }
        wk.trs = fast_div(it.kb0, p.fd_red);
        wk.rc = it.kb0 - wk.trs * p.red_chunks;
        wk.tap = decode_tap(p, wk.trs);
      } else if (kMode == TC_UPDATE) {
        // item z owns taps [z * taps_per_z, (z + 1) * taps_per_z); A box `bi` carries the bi-th of them
        // (acc_taps consecutive boxes stack into one accumulator)
        // (swapped operands: column tile tile_n owns taps [tile_n * b_boxes, ...), one per B box)
        const int zt = p.swap_ab ? it.tile_n * p.b_boxes + (is_a ? 0 : bi) : it.z * p.taps_per_z + (is_a ? bi : 0);
        wk.tap = decode_tap(p, zt);
        tap_live = p.swap_ab ? zt < p.taps_per_z : (zt < p.nz_out && (!is_a || bi < p.taps_per_z));
        wk.cp = decode_chunk(p, it.kb0);
      }
      // box coordinates of this lane's box at walker position `s`
      auto coords = [&](const Walk& s, int& c0, int& c1, int& c2, int& c3, int& c4) {
        const ChunkPos& cp = s.cp;
        const Tap& tap = s.tap;
        const int trs = s.trs, rc = s.rc, kb = s.kb;
        c0 = c1 = c2 = c3 = c4 = 0;
        {
          if (kMode == TC_GEMM) {
            const int k0 = kb * kChunk;
            if (is_a) {
              if (p.a_merge) { c1 = k0; c2 = (m0 + kTileM * bi) / kChunk; c3 = it.z * p.a_zmul; }
              else if (p.a_mn_major) { c0 = m0 + kChunk * bi; c1 = k0; c2 = it.z * p.a_zmul; }
              else { c0 = k0; c1 = m0; c2 = it.z * p.a_zmul; }
            } else {
              if (p.b_merge == 3) { c1 = k0; c2 = n0 / kChunk; c3 = it.z * p.b_zmul; }
              else if (p.b_mn_major) { c0 = n0 + kChunk * bi; c1 = k0; c2 = it.z * p.b_zmul; }
              else { c0 = k0; c1 = n0; c2 = it.z * p.b_zmul; }
            }
          } else if (kMode == TC_FPROP) {
            if (is_a) {  // filter rows c of tap trs, 64 output channels wide
              if (p.a_merge) { c1 = rc * p.kb_rows; c2 = (m0 + kTileM * bi) / kChunk; c3 = trs; }
              else { c0 = m0 + kChunk * bi; c1 = trs; c2 = rc * p.kb_rows; }
            } else {     // input pixels of this chunk shifted by the tap
              c0 = cp.inner0 + (tap.s - p.pad_w) * p.inner_tap;
              c1 = (cp.q * p.str_w - p.pad_w + tap.s * p.tap_w) * p.x_tap;
              c2 = cp.valid ? cp.p * p.str_h - p.pad_h + tap.r * p.tap_h : p.oob_y + kFarRows;
              c3 = cp.m * p.str_d - p.pad_d + tap.t;
              c4 = rc * p.kb_rows;
            }
          } else if (kMode == TC_BPROP) {
            if (is_a) {  // filter rows c0.., 64 output channels k of tap trs
              c0 = rc * kChunk; c1 = trs; c2 = m0;
            } else {     // error pixels that reach this input pixel through tap trs
              bool v = cp.valid;
              int q = 0, pp = 0, mm = 0;
              if (p.x_tap) {
                v &= div_exact(cp.q + p.pad_w - tap.s, p.str_w, q);
                c0 = cp.inner0;
              } else {
                c0 = cp.inner0 + (p.pad_w - tap.s) * p.inner_tap;
              }
              v &= div_exact(cp.p + p.pad_h - tap.r, p.str_h, pp);
              v &= div_exact(cp.m + p.pad_d - tap.t, p.str_d, mm);
              c1 = q; c2 = v ? pp : p.oob_y + kFarRows; c3 = mm; c4 = rc * kChunk;
            }
          } else {  // TC_UPDATE: k-block = one 64-element chunk of the (m,p,q,n) space
            if (is_a != (p.swap_ab != 0)) {  // input pixels under tap z, 128 channels c
              c0 = cp.inner0 + (tap.s - p.pad_w) * p.inner_tap;
              c1 = (cp.q * p.str_w - p.pad_w + tap.s * p.tap_w) * p.x_tap;
              c2 = tap_live ? cp.p * p.str_h - p.pad_h + tap.r * p.tap_h : p.oob_y;
              c3 = cp.m * p.str_d - p.pad_d + tap.t;
              c4 = p.swap_ab ? 0 : m0;
            } else {     // error pixels, block_n output channels k
              c0 = cp.inner0; c1 = cp.q * p.x_tap; c2 = cp.p; c3 = cp.m; c4 = p.swap_ab ? m0 : n0;
            }
          }
        }
        if (merged && !is_a) {
          // the whole-tile box starts where the first chunk's box starts; its map orders the
          // dimensions (n, chan, x, y, z) or, with several chunks per pixel, (n_lo, chan, n_hi, x, y)
          const int n = c0, x = c1, y = c2, z = c3, ch = c4;
          if (p.b_merge == 1) { c0 = n; c1 = ch; c2 = x; c3 = y; c4 = z; }
          else { c0 = 0; c1 = ch; c2 = n / kChunk; c3 = x; c4 = y; }
        } else if (p.b_merge == 4 && !is_a) {
          // tap-block map with the image group last: (n_lo, x, y, chan, n_hi)
          c3 = c4; c4 = c0 / kChunk; c0 = 0;
        }
      };
      // step a walker to the next k-block
      auto advance = [&](Walk& s) {
        ++s.kb;
        if (kMode == TC_FPROP || kMode == TC_BPROP) {
          if (++s.rc == p.red_chunks) {
            s.rc = 0;
            ++s.trs;
            if (++s.tap.s == p.S) {
              s.tap.s = 0;
              if (++s.tap.r == p.R) { s.tap.r = 0; ++s.tap.t; }
            }
          }
        } else if (kMode == TC_UPDATE) {
          s.cp.inner0 += kChunk;
          if (s.cp.inner0 == p.dec_cpi * kChunk) {
            s.cp.inner0 = 0;
            if (++s.cp.q == p.dec_q) {
              s.cp.q = 0;
              if (++s.cp.p == p.dec_p) { s.cp.p = 0; ++s.cp.m; }
            }
          }
        }
      };
      // (Asking the L2 for the boxes of later k-blocks with prefetch copies was tried and was
      // slower everywhere: a prefetch costs the copy engine as much as the load it precedes.)
      // Forward pass, and backward pass with unit strides: inside one tile every coordinate of a
      // box is linear in the tap (t, r, s) and the reduction chunk. The offsets and the four
      // steps are taken once per tile, as differences of the general formula above, and a k-block
      // costs this warp five multiply-adds per coordinate instead of a walk through that formula
      // (which the A and the B lanes take one after the other): with it the producer took about
      // as long per k-block as the MMAs themselves and, being one serial warp, set the pace.
      // The steps depend on the tile only through the form of its B box (one merged box or one
      // per chunk), so they are kept from tile to tile; a tile costs one walk through the formula
      // for its offsets. (Tiles of a few k-blocks, e.g. a 3-channel first layer with one k-block
      // per tile, spent most of their time in this set-up when it took five walks.)
      int lb0 = 0, lb1 = 0, lb2 = 0, lb3 = 0, lb4 = 0;          // coordinates at tap (0, 0, 0), chunk 0
      if (linear && act) {
        Walk o = wk;
        o.tap = {0, 0, 0}; o.trs = 0; o.rc = 0;
        coords(o, lb0, lb1, lb2, lb3, lb4);
        if (steps_for != static_cast<int>(merged)) {
          steps_for = static_cast<int>(merged);
          // (taken on a chunk that exists: a chunk past the end has a constant, far row coordinate)
          o.cp.valid = true;
          int b0, b1, b2, b3, b4, d0, d1, d2, d3, d4;
          coords(o, b0, b1, b2, b3, b4);
          Walk q = o;
          q.tap.s = 1; q.trs = 1;
          coords(q, d0, d1, d2, d3, d4);
          ls[0] = d0 - b0; ls[1] = d1 - b1; ls[2] = d2 - b2; ls[3] = d3 - b3; ls[4] = d4 - b4;
          q = o; q.tap.r = 1; q.trs = p.S;
          coords(q, d0, d1, d2, d3, d4);
          lr[0] = d0 - b0; lr[1] = d1 - b1; lr[2] = d2 - b2; lr[3] = d3 - b3; lr[4] = d4 - b4;
          q = o; q.tap.t = 1; q.trs = p.RS;
          coords(q, d0, d1, d2, d3, d4);
          lt[0] = d0 - b0; lt[1] = d1 - b1; lt[2] = d2 - b2; lt[3] = d3 - b3; lt[4] = d4 - b4;
          q = o; q.rc = 1;
          coords(q, d0, d1, d2, d3, d4);
          lc[0] = d0 - b0; lc[1] = d1 - b1; lc[2] = d2 - b2; lc[3] = d3 - b3; lc[4] = d4 - b4;
        }
      }
      for (int kb = it.kb0; kb < it.kb1; ++kb) {
        // The coordinates are ready before the slot is, so the copy leaves as soon as it frees.
        // (All lanes poll: one polling lane plus a broadcast measured the same or slower.)
        int c0 = 0, c1 = 0, c2 = 0, c3 = 0, c4 = 0;
        if (linear) {
          const int ts = wk.tap.s, tr = wk.tap.r, tt = wk.tap.t, rc = wk.rc;
          c0 = lb0 + ts * ls[0] + tr * lr[0] + tt * lt[0] + rc * lc[0];
          c1 = lb1 + ts * ls[1] + tr * lr[1] + tt * lt[1] + rc * lc[1];
          c2 = lb2 + ts * ls[2] + tr * lr[2] + tt * lt[2] + rc * lc[2];
          c3 = lb3 + ts * ls[3] + tr * lr[3] + tt * lt[3] + rc * lc[3];
          c4 = lb4 + ts * ls[4] + tr * lr[4] + tt * lt[4] + rc * lc[4];
        } else if (act) {
          coords(wk, c0, c1, c2, c3, c4);
        }
        const int got = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, NG_DEV_TIMEOUT_PRODUCER, p.wait_limit_ns);
        // (pairs: the operands of both CTAs are counted on the first CTA's barrier)
        if (lane == 0 && got && rank == 0) mbar_expect_tx(full_bar(stage), kPair ? 2u * tx_item : tx_item);
        if (!__all_sync(0xffffffffu, got)) {
          ok = false;
          break;
        }
        if (act) {
          if (kPair)
            tma_load_5d_pair(smem_base + stage * p.stage_bytes + box_off, map, map_to_cta(full_bar(stage), 0u), c0, c1,
                             c2, c3, c4);
          else
            tma_load_5d(smem_base + stage * p.stage_bytes + box_off, map, full_bar(stage), c0, c1, c2, c3, c4);
        }
        advance(wk);
        if (++stage == p.stages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // =========================== MMA issuer ===========================
    // m_halves == 1: accumulator `local & 1` (double-buffered across tiles), barriers accf/acce[acc].
    // m_halves == 2: both accumulators belong to one 256-row tile; acce[h] says half h was drained,
    //                accf[0] says both halves are complete.
    // The whole warp walks the loop (every lane waits on the barriers) and lane 0 alone issues the
    // MMAs and commits: a warp that stays converged gets through an iteration in fewer cycles than
    // a single lane running inside a divergent branch does.
    if (rank == 0) {
      const bool issuer = lane == 0;
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      const bool wide = p.m_halves == 2;
      // acc_groups > 1 (weight update): one item accumulates several taps at once, accumulator g
      // for tap z*groups+g, all fed by the same B operand; TMEM is then one set, not two.
      const bool grouped = kMode == TC_UPDATE && (p.acc_groups > 1 || p.acc_taps > 1);
      // Everything the issue loop needs sits in registers, and the loop does as little as it can:
      // this one thread's instruction stream is serial, and every cycle it spends between two
      // MMAs beyond the 128 the tensor pipe needs for one is a cycle the pipe idles. Descriptors
      // are kept as (low, high) words whose start-address field is stepped by 32-bit adds (the
      // ring lies below 256 KB, so the 14-bit field never carries), barrier addresses and the
      // stage base are stepped, not recomputed, and a wait first tries the barrier once inline.
      const uint32_t a_lo0 = p.a_desc_lo, a_hi = p.a_desc_hi, b_lo0 = p.b_desc_lo, b_hi = p.b_desc_hi;
      const uint32_t a_kstep = p.a_kstep, b_kstep = p.b_kstep, a_half = p.a_half_step, idesc = p.idesc;
      const int mma_per_kb = p.mma_per_kb, stages = p.stages;
      const uint32_t ring0 = (smem_base >> 4) & 0x3fffu, stage_step = p.stage_bytes >> 4, b_off = p.a_bytes >> 4;
      const uint32_t block_n = static_cast<uint32_t>(p.block_n);
      const uint32_t full0 = full_bar(0);
      const uint32_t empty0 = kPair ? map_to_cta(empty_bar(0), 0u) : empty_bar(0);
      const uint32_t empty0_peer = kPair ? map_to_cta(empty_bar(0), 1u) : 0u;
      uint32_t sa = ring0, fbar = full0, ebar = empty0, ebar_peer = empty0_peer;
      for (int w = w_first; w < total_work && ok; w += w_step) {
        const WorkItem it = decode_work(p, w);
        if (it.live == 0) continue;     // `local` counts the items this CTA works on, in every role alike
        const int acc = (wide || grouped) ? 0 : (local & 1);
        const uint32_t acc_phase = (wide || grouped) ? (local & 1u) : ((local >> 1) & 1u);
        // rows of the second half that lie beyond M need no MMAs; taps beyond the last need none
        int halves = wide ? it.live : 1;
        if (grouped) {
          const int taps_here = min(p.taps_per_z, p.nz_out - it.z * p.taps_per_z);
          halves = min(p.acc_groups, (taps_here + p.acc_taps - 1) / p.acc_taps);
        }
        if (!wide) {
          if (!mbar_wait(acce_bar(acc), acc_phase ^ 1u, abort_flag, p.status, NG_DEV_TIMEOUT_ACC, p.wait_limit_ns)) break;
          tc_fence_after();
        }
        const uint32_t d_base = tmem_base + ((wide || grouped) ? 0u : static_cast<uint32_t>(acc) * block_n);
        // One k-block: wait for its operands, issue its MMAs accumulator by accumulator (measured
        // faster than interleaving them k-step by k-step), release the slot, step the ring.
        auto wait_operands = [&]() -> bool {
          if (!mbar_try_wait(fbar, phase) &&
              !mbar_wait(fbar, phase, abort_flag, p.status, NG_DEV_TIMEOUT_MMA, p.wait_limit_ns))
            return false;
          tc_fence_after();
          return true;
        };
        auto release_and_step = [&]() {
          // frees the smem slot (in both CTAs of a pair) once these MMAs have read it
          if (issuer) {
            if (kPair) {
              tc_commit_pair(ebar);
              tc_commit_pair(ebar_peer);
            } else {
              tc_commit(ebar);
            }
          }
          sa += stage_step; fbar += 8u; ebar += 8u; ebar_peer += 8u;
          if (++stage == stages) {
            stage = 0; phase ^= 1u;
            sa = ring0; fbar = full0; ebar = empty0; ebar_peer = empty0_peer;
          }
        };
        auto run_any = [&](uint32_t d_tmem, uint32_t alo, uint32_t blo, uint32_t accumulate) {
          switch (mma_per_kb) {   // (one block of PTX per accumulator and k-block: see tc_mma_f16_run)
            case 4: tc_mma_f16_run<kPair, 4>(d_tmem, alo, a_hi, blo, b_hi, idesc, accumulate, a_kstep, b_kstep); break;
            case 3: tc_mma_f16_run<kPair, 3>(d_tmem, alo, a_hi, blo, b_hi, idesc, accumulate, a_kstep, b_kstep); break;
            case 2: tc_mma_f16_run<kPair, 2>(d_tmem, alo, a_hi, blo, b_hi, idesc, accumulate, a_kstep, b_kstep); break;
            default: tc_mma_f16_run<kPair, 1>(d_tmem, alo, a_hi, blo, b_hi, idesc, accumulate, a_kstep, b_kstep); break;
          }
        };
        // general form: any number of accumulators, the first k-block of an item included (it
        // overwrites the accumulators, and with 256-row tiles waits for each half to be drained)
        auto general_kb = [&](uint32_t accumulate) -> bool {
          if (!wait_operands()) return false;
          const uint32_t blo0 = b_lo0 | (sa + b_off);
          uint32_t alo_h = a_lo0 | sa, d_tmem = d_base;
          for (int h = 0; h < halves; ++h, alo_h += a_half, d_tmem += block_n) {
            if (wide && accumulate == 0u) {   // half h of the previous tile must have been drained
              if (!mbar_wait(acce_bar(h), acc_phase ^ 1u, abort_flag, p.status, NG_DEV_TIMEOUT_ACC, p.wait_limit_ns))
                return false;
              tc_fence_after();
            }
            if (issuer) run_any(d_tmem, alo_h, blo0, accumulate);
          }
          release_and_step();
          return true;
        };
        int kb = it.kb0;
        ok = general_kb(0u);
        ++kb;
        // The steady state of the common tilings (one or two accumulators) runs in loops that hold
        // nothing but the wait, the MMAs of a fixed count and the commit: with the accumulator
        // loop, the count switch and the first-k-block test inside, the same work took the issuing
        // warp ~900 cycles per k-block of four MMAs instead of ~570 (the tensor pipe needs 512).
#define NG_STEADY_LOOP(count, two)                                                                                  \
  for (; ok && kb < it.kb1; ++kb) {                                                                                 \
    if (!wait_operands()) { ok = false; break; }                                                                    \
    if (issuer) {                                                                                                   \
      tc_mma_f16_run<kPair, count>(d_base, a_lo0 | sa, a_hi, b_lo0 | (sa + b_off), b_hi, idesc, 1u, a_kstep, b_kstep); \
      if (two)                                                                                                      \
        tc_mma_f16_run<kPair, count>(d_base + block_n, (a_lo0 | sa) + a_half, a_hi, b_lo0 | (sa + b_off), b_hi, idesc, \
                                     1u, a_kstep, b_kstep);                                                         \
    }                                                                                                               \
    release_and_step();                                                                                             \
  }
        if (halves == 1) {
          switch (mma_per_kb) {
            case 4: NG_STEADY_LOOP(4, false) break;
            case 3: NG_STEADY_LOOP(3, false) break;
            case 2: NG_STEADY_LOOP(2, false) break;
            default: NG_STEADY_LOOP(1, false) break;
          }
        } else if (halves == 2) {
          switch (mma_per_kb) {
            case 4: NG_STEADY_LOOP(4, true) break;
            case 3: NG_STEADY_LOOP(3, true) break;
            case 2: NG_STEADY_LOOP(2, true) break;
            default: NG_STEADY_LOOP(1, true) break;
          }
        } else {
          for (; ok && kb < it.kb1; ++kb) ok = general_kb(1u);
        }
#undef NG_STEADY_LOOP
        if (ok && issuer) {   // accumulator(s) complete
          if (kPair) {
            tc_commit_pair(map_to_cta(accf_bar(acc), 0u));
            tc_commit_pair(map_to_cta(accf_bar(acc), 1u));
          } else {
            tc_commit(accf_bar(acc));
          }
        }
        ++local;
      }
    }
    __syncwarp();
  } else {
    // =========================== epilogue ===========================
    const int lane_group = warp & 3;  // TMEM lanes [32*lane_group, +32) are visible to this warp
    // One set of output-stage scalars, held in registers: split-K partials leave as untouched
    // fp32 accumulators. (Choosing between two argument structs by reference put both in local
    // memory, and every use became a load.)
    // (The forward and backward passes always write rounded fp16 without a beta term, the weight
    // update never rounds stochastically: their instances leave those paths out.)
    constexpr bool kConvOut = kMode == TC_FPROP || kMode == TC_BPROP;
    constexpr bool kNoBetaSr = kMode != TC_GEMM;
    const bool partial = p.splits > 1;
    const bool f32 = partial || (!kConvOut && p.out_f32 != 0);
    EpiArgs ea;
    ea.alpha = partial ? 1.0f : p.alpha;
    ea.beta = (partial || kNoBetaSr) ? 0.0f : p.beta;
    ea.relu = (partial || kMode == TC_UPDATE) ? 0 : p.relu;
    ea.sr_bits = (partial || kNoBetaSr) ? 0 : p.sr_bits;
    ea.seed_lo = p.seed_lo; ea.seed_hi = p.seed_hi; ea.rng_offset = p.rng_offset;
    // the common case gets a short path of its own: the epilogue is bound by instruction latency
    // (two warps per scheduler), so every instruction fewer counts
    const bool plain = kLean || (ea.alpha == 1.0f && ea.beta == 0.0f && ea.sr_bits == 0);
    const bool wide = p.m_halves == 2;
    // two warps share each group of 32 TMEM lanes and split the columns between them
    const int col_group = (warp - 2) >> 2;
    const bool grouped = kMode == TC_UPDATE && (p.acc_groups > 1 || p.acc_taps > 1);
    const int n_acc = wide ? 2 : p.acc_groups;   // accumulators of one work item
    int local = 0;
    for (int w = w_first; w < total_work; w += w_step) {
      WorkItem it = decode_work(p, w);
      if (it.live == 0) continue;
      if (kPair) it.m0 = it.m0 * 2 + row_shift;
      const int acc = (wide || grouped) ? 0 : (local & 1);
      const uint32_t acc_phase = (wide || grouped) ? (local & 1u) : ((local >> 1) & 1u);
      if (!mbar_wait(accf_bar(acc), acc_phase, abort_flag, p.status, NG_DEV_TIMEOUT_EPILOGUE, p.wait_limit_ns)) break;
      tc_fence_after();
      const int n0 = it.tile_n * p.block_n;
      for (int h = 0; h < n_acc; ++h) {
        // accumulator h holds rows of row-tile `rt` of output slice `zt`; with stacked taps
        // (weight update, few rows per tap) every `pack_rows` lanes belong to the next slice
        const int rt = it.m0 / kTileM + (wide ? h : 0);
        int zt = it.z, row = rt * kTileM + lane_group * 32 + lane, row0 = rt * kTileM + lane_group * 32;
        int zt_warp = it.z;               // slice of this warp's first lane (bulk-store path)
        bool row_ok = row < p.M;
        int acc_first = zt;               // first slice of this accumulator
        int z_end = p.nz_out;             // one past the last slice this work item owns
        if (grouped) {
          acc_first = it.z * p.taps_per_z + h * p.acc_taps;
          z_end = min(p.nz_out, (it.z + 1) * p.taps_per_z);
          zt = acc_first;
          zt_warp = acc_first < z_end ? acc_first : p.nz_out;
          row_ok = row_ok && acc_first < z_end;
          if (p.acc_taps > 1) {
            const int r = lane_group * 32 + lane;
            const int sub = r / p.pack_rows;
            row = r - sub * p.pack_rows;
            zt = acc_first + sub;
            row_ok = sub < p.acc_taps && row < p.M && zt < z_end;
            const int sub_w = (lane_group * 32) / p.pack_rows;
            row0 = lane_group * 32 - sub_w * p.pack_rows;
            zt_warp = (sub_w < p.acc_taps && acc_first + sub_w < z_end) ? acc_first + sub_w : p.nz_out;
          }
        }
        // whole accumulator beyond M (or beyond the last tap): nothing accumulated, nothing to store
        const bool half_live = rt * kTileM < p.M && acc_first < z_end && (!wide || h < it.live);
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) +
                               static_cast<uint32_t>(((wide || grouped) ? h : acc) * p.block_n);
        // row base pointers
        uint8_t* crow = nullptr;
        const uint8_t* oldrow = nullptr;
        unsigned long long lin_row = 0;
        if (partial) {
          const long long off = ((static_cast<long long>(it.split) * p.nz_out + zt) * p.M + row) * p.N;
          crow = reinterpret_cast<uint8_t*>(p.ws + off);
        } else {
          const long long off = zt * p.c_zstride + static_cast<long long>(row) * p.ldc;
          const int esz = p.out_f32 ? 4 : 2;
          crow = static_cast<uint8_t*>(p.C) + off * esz;
          oldrow = p.Cold ? static_cast<const uint8_t*>(p.Cold) + off * esz : nullptr;
          lin_row = (static_cast<unsigned long long>(zt) * p.M + row) * static_cast<unsigned long long>(p.N);
        }
        if (staged) {
          // Staged path: 32 rows x 128 bytes per box, written to shared memory in the 128-byte
          // swizzle pattern (16-byte chunk j of row t lands at chunk j ^ (t & 7): conflict-free
          // for the per-row writes below), then written out by the warp in whole 128-byte rows.
          const int epi_warp = warp - 2;
          const int zc = partial ? it.split * p.nz_out + zt_warp : zt_warp;
          const int subs = p.c_box_cols / 32;            // tcgen05.ld groups per box: 2 (fp16) or 1 (fp32)
          const int n_boxes = p.block_n / p.c_box_cols;
          const int cb0 = col_group == 0 ? 0 : (n_boxes + 1) / 2;
          const int cb1 = col_group == 0 ? (n_boxes + 1) / 2 : n_boxes;
          const uint32_t buf = epi_base + static_cast<uint32_t>(epi_warp * 4096);
          for (int cb = cb0; half_live && cb < cb1; ++cb) {
            const int colb = n0 + cb * p.c_box_cols;
            for (int sub = 0; sub < subs; ++sub) {
              uint32_t r[32];
              tc_ld_32x32(taddr + static_cast<uint32_t>(cb * p.c_box_cols + sub * 32), r);
              tc_wait_ld();
              const uint32_t rowb = buf + static_cast<uint32_t>(lane) * 128u;
              const uint32_t swz = static_cast<uint32_t>(lane & 7);
              // (no "memory" clobber on the staging stores: they are ordered with the loads of the
              // write-out by being volatile and by the __syncwarp between them)
              if (plain && f32) {
                // raw fp32 (split-K partials; fp32 results with alpha 1, beta 0): registers to staging
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                  uint32_t a = r[g * 4], b = r[g * 4 + 1], c = r[g * 4 + 2], d = r[g * 4 + 3];
                  if (ea.relu) {
                    a = __float_as_uint(fmaxf(__uint_as_float(a), 0.0f));
                    b = __float_as_uint(fmaxf(__uint_as_float(b), 0.0f));
                    c = __float_as_uint(fmaxf(__uint_as_float(c), 0.0f));
                    d = __float_as_uint(fmaxf(__uint_as_float(d), 0.0f));
                  }
                  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowb + ((g ^ swz) << 4)), "r"(a),
                               "r"(b), "r"(c), "r"(d));
                }
                continue;
              }
              if (plain) {
                // fp16 with alpha 1, beta 0, round to nearest: convert pairs, ReLU on the packed halves
                // (rounding is monotonic, so max(round(x), 0) == round(max(x, 0)))
                const __half2 zero2 = __float2half2_rn(0.0f);
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                  uint32_t w[4];
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    __half2 h = __floats2half2_rn(__uint_as_float(r[g * 8 + 2 * i]), __uint_as_float(r[g * 8 + 2 * i + 1]));
                    if (ea.relu) h = __hmax2(h, zero2);
                    w[i] = *reinterpret_cast<uint32_t*>(&h);
                  }
                  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(
                                   rowb + ((static_cast<uint32_t>(sub * 4 + g) ^ swz) << 4)),
                               "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]));
                }
                continue;
              }
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                const int col = colb + sub * 32 + g * 8;
                float v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[g * 8 + i]);
                uint4 lo, hi;
                const bool live = row_ok && col < p.N;
                if (f32) {   // 8 fp32 = two chunks
                  epi_pack8<true>(ea, v, (live && oldrow) ? oldrow + static_cast<long long>(col) * 4 : nullptr,
                                  lin_row + col, lo, hi);
                  const int j = g * 2;
                  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowb + (((j) ^ (lane & 7)) << 4)),
                               "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w));
                  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowb + (((j + 1) ^ (lane & 7)) << 4)),
                               "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w));
                } else {                       // 8 fp16 = one chunk
                  epi_pack8<false>(ea, v, (live && oldrow) ? oldrow + static_cast<long long>(col) * 2 : nullptr,
                                   lin_row + col, lo, hi);
                  const int j = sub * 4 + g;
                  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowb + ((j ^ (lane & 7)) << 4)),
                               "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w));
                }
              }
            }
            {
              // Write-out by the warp itself: each instruction stores four whole 128-byte rows
              // (lane = row within the group of four, 16-byte chunk). (A bulk tensor store would
              // queue behind the operand loads of the copy engine; the wait for it to release the
              // staging buffer then cost ~2 us per box.)
              __syncwarp();
              const int esz = f32 ? 4 : 2;
              uint8_t* gbase;
              long long gstride;
              if (partial) {
                gbase = reinterpret_cast<uint8_t*>(p.ws + static_cast<long long>(zc) * p.M * p.N);
                gstride = static_cast<long long>(p.N) * 4;
              } else {
                gbase = static_cast<uint8_t*>(p.C) + static_cast<long long>(zt_warp) * p.c_zstride * esz;
                gstride = p.ldc * esz;
              }
              const int j = lane & 7;
              int gcol = colb + j * (16 / esz);
              bool col_live = gcol < p.N && zt_warp < p.nz_out;
              if (kConvOut && !partial && p.c_row_chunks) {
                // Flattened pixel space whose image rows are padded to whole 64-element chunks:
                // this box is chunk `ch` of the padded space; it holds elements [cq * 64, +64) of
                // image row r, of which only those below c_row_len exist in memory.
                const int ch = colb >> 6;
                const int r = fast_div(ch, p.fd_crow);
                const int cq = ch - r * p.c_row_chunks;
                gcol = r * p.c_row_len + cq * kChunk + j * 8;
                col_live = col_live && cq * kChunk + j * 8 < p.c_row_len;
              }
              uint8_t* gp = gbase + (row0 + (lane >> 3)) * gstride + static_cast<long long>(gcol) * esz;
              uint4 v[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int t = i * 4 + (lane >> 3);
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(v[i].x), "=r"(v[i].y), "=r"(v[i].z), "=r"(v[i].w)
                             : "r"(buf + static_cast<uint32_t>(t) * 128u + static_cast<uint32_t>((j ^ (t & 7)) << 4)));
              }
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                if (col_live && row0 + i * 4 + (lane >> 3) < p.M) *reinterpret_cast<uint4*>(gp) = v[i];
                gp += 4 * gstride;
              }
              __syncwarp();   // the buffer is free for the next box
            }
          }
        }
        const int n_chunks = p.block_n / 32;
        const int c_begin = col_group == 0 ? 0 : (n_chunks + 1) / 2;
        const int c_end = col_group == 0 ? (n_chunks + 1) / 2 : n_chunks;
        // (lean instances always stage: the loop bound is 0 for them)
        const int c_stop = (kLean || staged || !half_live) ? c_begin : c_end;
        for (int c = c_begin; c < c_stop; ++c) {
          uint32_t r[32];
          tc_ld_32x32(taddr + static_cast<uint32_t>(c * 32), r);
          tc_wait_ld();
          const int col0 = n0 + c * 32;
          if (row_ok && col0 < p.N) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int col = col0 + g * 8;
              const int nvalid = min(8, p.N - col);
              if (nvalid <= 0) break;
              float v[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[g * 8 + i]);
              const bool vec = partial ? (p.N & 3) == 0 : p.vec_ok != 0;
              if (f32) {
                epi_store8_call<true>(ea, v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7], crow, oldrow, col,
                                      lin_row + col, nvalid, vec);
              } else {
                epi_store8_call<false>(ea, v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7], crow, oldrow, col,
                                       lin_row + col, nvalid, vec);
              }
            }
          }
        }
        if (wide) {   // hand this half back as soon as it is drained
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(acce_bar(h));
        }
      }
      if (!wide) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (kPair) mbar_arrive_cluster(map_to_cta(acce_bar(acc), 0u));
          else mbar_arrive(acce_bar(acc));
        }
      }
      ++local;
    }
  }

  // =========================== teardown ===========================
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // a wait gave up: give copies that may still be in flight time to land before the
    // shared memory and TMEM are handed back
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (kPair) cluster_sync_all();   // neither CTA leaves while the other may still read its shared memory
  if (warp == 1) {
    tc_fence_after();
    if (kPair) tmem_dealloc_pair(tmem_base, tmem_cols);
    else tmem_dealloc(tmem_base, tmem_cols);
  }
}

// ------------------------------------------------------------------------------------------
// split-K second stage: sum the partials in a fixed order, then the fused epilogue.
// `lanes` (a power of two, at most 32) neighbouring threads share 8 consecutive columns of one
// row: thread j adds partitions j, j + lanes, ... in that order, then the lanes are combined by a
// butterfly. The order depends only on (splits, lanes), so results repeat bit for bit. Several
// lanes matter when there are many partitions of a small output: one thread walking 70 slices
// one after the other is a chain of 70 dependent memory latencies.
// ------------------------------------------------------------------------------------------
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, int splits, int lanes, int nz, int M, int N,
                                     void* C, const void* Cold, long long ldc, long long c_zstride, int out_f32,
                                     int vec_ok, EpiArgs ea, int c_row_chunks, int c_row_len) {
  grid_dependency_wait();     // (launched while the product that writes the partials drains)
  grid_launch_dependents();
  const int groups_per_row = (N + 7) / 8;
  const long long total = static_cast<long long>(nz) * M * groups_per_row;
  const long long slice = static_cast<long long>(nz) * M * N;
  const long long t = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const int sub = static_cast<int>(t % lanes);
  const long long i = t / lanes;
  const bool live = i < total;          // whole groups of `lanes` threads are live or not
  const long long ic = live ? i : 0;
  const int g = static_cast<int>(ic % groups_per_row);
  const long long zr = ic / groups_per_row;
  const int row = static_cast<int>(zr % M);
  const int z = static_cast<int>(zr / M);
  const int col = g * 8;
  const int nvalid = min(8, N - col);
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = 0.0f;
  const float* src = ws + zr * N + col + sub * slice;
  const long long step = slice * lanes;
  const bool v4 = (N & 3) == 0 && nvalid == 8;
  if (live) {
    if (v4) {
      int s = sub;
      // four partitions in flight per thread
      for (; s + 3 * lanes < splits; s += 4 * lanes, src += 4 * step) {
        float4 a[4], b[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          a[u] = reinterpret_cast<const float4*>(src + u * step)[0];
          b[u] = reinterpret_cast<const float4*>(src + u * step)[1];
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          v[0] += a[u].x; v[1] += a[u].y; v[2] += a[u].z; v[3] += a[u].w;
          v[4] += b[u].x; v[5] += b[u].y; v[6] += b[u].z; v[7] += b[u].w;
        }
      }
      for (; s < splits; s += lanes, src += step) {
        const float4 a = reinterpret_cast<const float4*>(src)[0];
        const float4 b = reinterpret_cast<const float4*>(src)[1];
        v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
        v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
      }
    } else {
      for (int s = sub; s < splits; s += lanes, src += step)
        for (int j = 0; j < nvalid; ++j) v[j] += src[j];
    }
  }
  for (int d = lanes >> 1; d > 0; d >>= 1) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] += __shfl_xor_sync(0xffffffffu, v[j], d);
  }
  if (!live || sub != 0) return;
  int gcol = col;
  if (c_row_chunks) {
    // padded image rows (see TcParams::c_row_chunks): the partials are laid out in the padded
    // column space, the output is not
    const int ch = col >> 6;
    const int r = ch / c_row_chunks;
    const int within = (ch - r * c_row_chunks) * kChunk + (col & 63);
    if (within >= c_row_len) return;
    gcol = r * c_row_len + within;
  }
  const long long off = z * c_zstride + static_cast<long long>(row) * ldc;
  const int esz = out_f32 ? 4 : 2;
  uint8_t* crow = static_cast<uint8_t*>(C) + off * esz;
  const uint8_t* oldrow = Cold ? static_cast<const uint8_t*>(Cold) + off * esz : nullptr;
  const unsigned long long lin = (static_cast<unsigned long long>(z) * M + row) * static_cast<unsigned long long>(N) + col;
  if (out_f32)
    epi_store8<true>(ea, v, crow, oldrow, gcol, lin, nvalid, vec_ok != 0);
  else
    epi_store8<false>(ea, v, crow, oldrow, gcol, lin, nvalid, vec_ok != 0);
}

}  // namespace ngb
