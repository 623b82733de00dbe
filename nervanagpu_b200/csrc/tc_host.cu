// Host side of the tensor-core engine: UMMA descriptor construction, ring sizing, split-K
// choice and the launch itself.
#include <algorithm>
#include <cstdio>
#include <mutex>
#include <vector>

#include "../../include/nervana_b200.h"
#include "epilogue.cuh"
#include "host.h"
#include "igemm_tc_kernel.cuh"

namespace ngb {

namespace {
constexpr uint32_t kSmemLimit = 232448;  // 227 KB opt-in dynamic shared memory per CTA
constexpr uint32_t kCtrlBytes = 512;     // barriers + TMEM slot + abort flag
constexpr uint32_t kLayoutSw128 = 2;     // UMMA shared-memory descriptor layout type

// Upper 32 bits of a shared-memory matrix descriptor: stride byte offset [32,46), descriptor
// version 1 in [46,48), base offset 0, layout type in [61,64).
uint32_t desc_hi(uint32_t sbo_bytes) {
  return ((sbo_bytes >> 4) & 0x3fffu) | (1u << 14) | (kLayoutSw128 << 29);
}
// Lower 32 bits without the start address: leading byte offset in [16,30).
uint32_t desc_lo(uint32_t lbo_bytes) { return ((lbo_bytes >> 4) & 0x3fffu) << 16; }
}  // namespace

static FastDiv make_fast_div(int d) {
  FastDiv f = {0u, 0u, 1u};
  if (d <= 1) return f;
  uint32_t lg = 0;
  while ((1u << lg) < static_cast<uint32_t>(d)) ++lg;        // ceil(log2 d), d >= 2 so lg >= 1
  const unsigned pw = 31u + lg;
  f.mul = static_cast<uint32_t>(((1ull << pw) + static_cast<uint32_t>(d) - 1u) / static_cast<uint32_t>(d));
  f.shr = pw - 32u;
  f.d = static_cast<uint32_t>(d);
  return f;
}

static void fill_fast_divs(TcParams& p) {
  p.fd_tiles_m = make_fast_div(p.tiles_m);
  p.fd_tiles_n = make_fast_div(p.tiles_n);
  p.fd_nz = make_fast_div(p.nz);
  p.fd_cpi = make_fast_div(p.dec_cpi);
  p.fd_q = make_fast_div(p.dec_q);
  p.fd_p = make_fast_div(p.dec_p);
  p.fd_RS = make_fast_div(p.RS);
  p.fd_S = make_fast_div(p.S);
  p.fd_red = make_fast_div(p.red_chunks);
  p.fd_crow = make_fast_div(p.c_row_chunks);
}

// Bytes a K-major A descriptor may read past its (short) slot; kept inside the allocation.
static uint32_t a_overread(const TcParams& p) {
  if (p.a_mn_major) return 0u;
  const uint32_t full = kTileM * p.m_halves * 128u;
  // the last accumulator's descriptor starts at its first box and spans a full tile
  const uint32_t acc_stride = static_cast<uint32_t>(std::max(1, p.acc_taps)) * p.a_box_bytes;
  const uint32_t last_end = (p.acc_groups > 1 ? (p.acc_groups - 1) * acc_stride : 0u) + full;
  return last_end > p.a_bytes ? last_end - p.a_bytes : 0u;
}

void tc_fill_mma(TcParams& p, const TcOperandLayout& lay) {
  p.a_mn_major = lay.a_mn_major;
  p.b_mn_major = lay.b_mn_major;
  p.kb_rows = lay.kb_rows;
  p.mma_per_kb = lay.kb_rows / 16;
  // Instruction descriptor (kind::f16): D fp32 [4,6)=1, A/B fp16 (format 0), major-ness bits
  // 15/16 (1 = MN-major), N>>3 in [17,23), M>>4 in [24,29).
  // (CTA pairs: M = 256, 128 rows in each CTA; N = block_n, half of the columns from each CTA)
  p.idesc = (1u << 4) | (static_cast<uint32_t>(lay.a_mn_major) << 15) |
            (static_cast<uint32_t>(lay.b_mn_major) << 16) | (static_cast<uint32_t>(p.block_n >> 3) << 17) |
            (static_cast<uint32_t>((p.pair ? 2 * kTileM : kTileM) >> 4) << 24);
  const int bn_cta = p.pair ? p.block_n / 2 : p.block_n;   // columns of B this CTA holds
  // K-major operand: one box of [rows][64 k] 128-byte rows; 8-row groups 1024 B apart; a K=16
  // step moves the start address 32 B inside the swizzled row.
  // MN-major operand: boxes of [kb_rows][64 mn]; 8 reduction rows = 1024 B (stride offset),
  // next 64-wide MN chunk = next box (leading offset); a K=16 step moves 16 rows = 2048 B.
  const uint32_t mn_box = static_cast<uint32_t>(lay.kb_rows) * 128u;
  if (p.m_halves != 2) p.m_halves = 1;
  const uint32_t tile_rows = kTileM * p.m_halves;
  if (lay.a_mn_major) {
    // one box per 64-row chunk, or (a_merge: the map has the chunk number as a dimension of its
    // own, behind the reduction rows) one box per 128-row half
    // (a_chunks: a 128-row tile over fewer than 128 real rows loads the real chunks only; the
    // MMA then reads stale shared memory for the others, rows that are never stored)
    int chunks = tile_rows / kChunk;
    if (!lay.a_merge && p.m_halves == 1 && lay.a_chunks > 0) chunks = std::min(chunks, lay.a_chunks);
    p.a_boxes = lay.a_merge ? p.m_halves : chunks;
    p.a_box_bytes = lay.a_merge ? 2u * mn_box : mn_box;
    p.a_merge = lay.a_merge;
    p.a_desc_lo = desc_lo(mn_box);
    p.a_kstep = 2048u >> 4;
    p.a_half_step = (2u * mn_box) >> 4;
  } else {
    if (p.acc_groups < 1) p.acc_groups = 1;
    if (p.acc_taps < 1) p.acc_taps = 1;
    p.a_boxes = p.acc_groups * p.acc_taps;   // grouped update: one A box per tap of every accumulator
    // a box may deliver fewer rows than the tile has (few-channel update): the rest of the
    // slot keeps stale data whose products land in rows that are never stored
    p.a_box_bytes = (lay.a_box_rows ? lay.a_box_rows : tile_rows) * 128u;
    p.a_desc_lo = desc_lo(16);
    p.a_kstep = 32u >> 4;
    p.a_half_step = ((p.acc_groups > 1 || p.acc_taps > 1) ? p.acc_taps * p.a_box_bytes : kTileM * 128u) >> 4;
  }
  if (p.acc_groups < 1) p.acc_groups = 1;
  if (p.acc_taps < 1) p.acc_taps = 1;
  p.a_desc_hi = desc_hi(1024);
  // A slot: the rows the box delivers. When that is fewer than the MMA's 128 rows the instruction
  // also reads what follows (the B slot, the next stage, the staging area: all inside this CTA's
  // allocation); those products fall in accumulator rows that are never stored.
  p.a_bytes = p.a_boxes * p.a_box_bytes;
  if (lay.b_mn_major) {
    // one box per 64-column chunk, or (b_merge_static) one box for the whole column tile
    // (b_pair: one box per pixel, its two image groups)
    const int per_box = lay.b_merge_static ? bn_cta / kChunk : (lay.b_pair ? 2 : 1);
    p.b_boxes = bn_cta / kChunk / per_box;
    p.b_box_bytes = per_box * mn_box;
    if (lay.b_merge_static) p.b_merge = 3;
    if (lay.b_pair) p.b_merge = 4;
    p.b_desc_lo = desc_lo(mn_box);
    p.b_kstep = 2048u >> 4;
  } else {
    // one box of block_n rows, or several shorter ones stacked (rows past the last box keep stale
    // data: their products are columns that the caller never reads)
    p.b_boxes = lay.b_box_count > 0 ? lay.b_box_count : 1;
    p.b_box_bytes = static_cast<uint32_t>(lay.b_box_count > 0 ? lay.b_box_rows : bn_cta) * 128u;
    p.b_desc_lo = desc_lo(16);
    p.b_kstep = 32u >> 4;
  }
  p.b_desc_hi = desc_hi(1024);
  // every box must start on a 1024-byte boundary for the 128-byte swizzle
  p.a_bytes = (p.a_bytes + 1023u) & ~1023u;
  uint32_t b_bytes = (p.b_boxes * p.b_box_bytes + 1023u) & ~1023u;
  if (!lay.b_mn_major) b_bytes = std::max(b_bytes, static_cast<uint32_t>(bn_cta) * 128u);
  p.stage_bytes = p.a_bytes + b_bytes;
  p.tx_bytes = p.a_boxes * p.a_box_bytes + p.b_boxes * p.b_box_bytes;
  p.stages = std::min<uint32_t>(kMaxStages, (kSmemLimit - 1024u - kCtrlBytes - kEpiStageBytes - a_overread(p)) /
                                               p.stage_bytes);
  if (tuning().max_stages > 0) p.stages = std::min<int>(p.stages, tuning().max_stages);
}

// How tiles leave the epilogue: 1 = staged through swizzled shared memory and written out by the
// warps in whole 128-byte rows, 0 = straight from registers (output not 16-byte addressable).
static int pick_store_mode(TcParams& p) {
  if ((p.N & 7) != 0) return 0;
  // stacked taps: a warp's 32 rows must belong to one tap
  if (p.acc_taps > 1 && (p.pack_rows & 31) != 0) return 0;
  const bool partial = p.splits > 1;
  const int esz = (partial || p.out_f32) ? 4 : 2;
  uint64_t row_bytes, z_bytes;
  const void* base;
  if (partial) {
    base = p.ws;
    row_bytes = static_cast<uint64_t>(p.N) * 4;
    z_bytes = row_bytes * p.M;
  } else {
    if (!p.vec_ok) return 0;
    base = p.C;
    row_bytes = static_cast<uint64_t>(p.ldc) * esz;
    z_bytes = p.nz_out > 1 ? static_cast<uint64_t>(p.c_zstride) * esz : row_bytes * p.M;
    if (z_bytes == 0) return 0;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15u) || (row_bytes & 15u) || (z_bytes & 15u)) return 0;
  p.c_box_cols = 128 / esz;
  return 1;
}

void tc_pick_tile_rows(const DeviceCtx* c, TcParams& p, long long col_tiles, int num_kb) {
  p.m_halves = 1;
  p.tiles_m = (p.M + kTileM - 1) / kTileM;
  if (p.M <= kTileM) return;
  const long long sm = c->sm_count;
  // cost model in "operand bytes per SM": waves x k-blocks x (rows + columns) of a k-block,
  // plus an un-overlapped epilogue worth about four k-blocks for the wide tile
  const long long t1 = p.tiles_m * col_tiles;
  const long long cost1 = ((t1 + sm - 1) / sm) * num_kb * (kTileM + p.block_n);
  const long long tm2 = (p.M + 2 * kTileM - 1) / (2 * kTileM);
  const long long t2 = tm2 * col_tiles;
  long long cost2 = ((t2 + sm - 1) / sm) * (num_kb + 4ll) * (2 * kTileM + p.block_n);
  if (t2 % sm > 0 && 2 * (t2 % sm) <= sm)   // the last wave runs as 128-row halves (see tc_launch)
    cost2 -= (num_kb + 4ll) * (2 * kTileM + p.block_n) - (num_kb + 2ll) * (kTileM + p.block_n);
  const int force = tuning().tile_rows;   // 128 | 256 overrides the choice
  const bool wide = force ? force == 256 : (cost2 < cost1);
  if (wide) {
    p.m_halves = 2;
    p.tiles_m = static_cast<int>(tm2);
  }
}

// Tile rows (128 / 256) and tile columns (256 / 192 / 128) of a convolution's forward or backward
// pass together, by modelled time: tiles run in waves of one per SM; a k-block costs the larger
// of its operand feed (copy engine: ~68 bytes/ns per SM) and its MMAs (~(rows + columns)/2 cycles
// per K=16 step); a 256-row tile pays for its epilogue (not overlapped), a 128-row tile does not.
// 85 tiles of 256 columns on 148 SMs (the 13x13 AlexNet layers) lose to 113 tiles of 192.
static double tuning_or(int value, double fallback) { return value > 0 ? static_cast<double>(value) : fallback; }

void tc_pick_tile(const DeviceCtx* c, TcParams& p, long long cols, int num_kb, int kb_rows) {
  const int force_rows = tuning().tile_rows, force_cols = tuning().tile_cols;
  double best = -1.0;
  int best_h = 1, best_bn = 256;
  for (int h = 1; h <= 2; ++h) {
    if (h == 2 && p.M <= kTileM) continue;
    if (force_rows && (force_rows == 256) != (h == 2) && p.M > kTileM) continue;
    for (int bn = 256; bn >= 128; bn -= 64) {
      if (force_cols && force_cols != bn) continue;
      const long long tm = (p.M + kTileM * h - 1) / (kTileM * h);
      const long long tn = (cols + bn - 1) / bn;
      const long long tiles = tm * tn;
      // (an MMA takes the tensor pipe ~128 cycles whatever its width up to 256 columns, so narrower
      // tiles only pay when they fill the last wave better; operands arrive at ~100 bytes/ns per SM)
      const double feed_ns = (kTileM * h + bn) * kb_rows * 2.0 / tuning_or(tuning().feed_bytes_per_ns, 100);
      const double mma_ns = h * (kb_rows / 16) * 66.0 + 30.0;
      const double epi_ns = h == 2 ? 5500.0 * bn / 256.0 : 600.0;
      const double tile_ns = num_kb * std::max(feed_ns, mma_ns) + epi_ns;
      double t = static_cast<double>((tiles + c->sm_count - 1) / c->sm_count) * tile_ns;
      const long long rem = tiles % c->sm_count;
      if (h == 2 && rem > 0 && 2 * rem <= c->sm_count) {
        // the last wave runs as 128-row halves (see tc_launch)
        const double half_feed = (kTileM + bn) * kb_rows * 2.0 / tuning_or(tuning().feed_bytes_per_ns, 100);
        t += num_kb * std::max(half_feed, mma_ns * 0.5) + epi_ns * 0.5 - tile_ns;
      }
      if (best < 0.0 || t < best) {
        best = t;
        best_h = h;
        best_bn = bn;
      }
    }
  }
  p.m_halves = best_h;
  p.block_n = best_bn;
  p.tiles_m = (p.M + kTileM * best_h - 1) / (kTileM * best_h);
  p.tiles_n = static_cast<int>((cols + best_bn - 1) / best_bn);
}

int choose_splits(const DeviceCtx* c, long long tiles, int num_kb, long long out_elems, bool charge_reduction) {
  if (charge_reduction && tuning().conv_splits > 0) return std::min(tuning().conv_splits, std::max(1, num_kb / 2));
  if (tiles >= c->sm_count || num_kb < 8) return 1;
  // Makespan model: items run in waves of one per SM; an item costs its k-blocks plus a fixed
  // start-up/drain charge. 17 splits of 9 tiles (153 items on 148 SMs) would take two waves;
  // 16 splits take one.
  const long long sm = c->sm_count;
  long long best = 1, best_cost = -1;
  for (long long s = 1; s <= kMaxSplits && s * 4 <= num_kb; ++s) {
    // partials cost 8 bytes of traffic per output element per split: keep them small next to
    // the operands (and bounded in absolute size)
    if (s > 1 && s * out_elems * 4 > (256ll << 20)) break;
    if (s > 32 && s * out_elems * 4 > (16ll << 20)) break;
    const long long items = tiles * s;
    const long long waves = (items + sm - 1) / sm;
    long long cost = waves * ((num_kb + s - 1) / s + 6);
    // (forward / backward passes: the output is large, so the second stage is not free: a launch
    // plus (s + 1) passes over the fp32 output at ~5 TB/s, in units of a k-block's ~0.5 us)
    if (charge_reduction && s > 1) cost += 8 + out_elems * 4 * (s + 1) / 2500000;
    if (best_cost < 0 || cost < best_cost) {
      best = s;
      best_cost = cost;
    }
  }
  return static_cast<int>(best);
}

// Threads that share one 8-column group of the split-K reduction: more when the output is small
// and the partitions many, so that the device is filled and no thread walks a long chain.
static int splitk_reduce_lanes(long long groups, int splits, int sm_count) {
  const int force = tuning().reduce_lanes;   // 1, 2, 4, ... 32
  if (force >= 1 && force <= 32 && (force & (force - 1)) == 0) return force;
  int lanes = 1;
  // only as many as it takes to occupy the SMs: with more, every thread holds fewer loads in flight
  // and the launch becomes several waves of short threads (AlexNet conv5: 49 -> 38 us for update + sum)
  while (lanes < 32 && lanes * 4 <= splits && groups * lanes < sm_count * 384ll) lanes *= 2;
  return lanes;
}

int tc_launch(DeviceCtx* c, const CUtensorMap& mapA, const CUtensorMap& mapB, TcParams& p, cudaStream_t stream,
              const CUtensorMap* mapBm) {
  if (p.num_kb < 1) return fail(NG_ERR_INVALID_ARG, "empty reduction");
  if (p.splits < 1) p.splits = 1;
  if (p.acc_groups < 1) p.acc_groups = 1;
  if (p.acc_taps < 1) p.acc_taps = 1;
  if (p.nz_out < 1) p.nz_out = p.nz;
  if (p.taps_per_z < 1) p.taps_per_z = p.acc_groups * p.acc_taps;
  if ((p.acc_groups > 1 || p.acc_taps > 1) &&
      (p.m_halves != 1 || p.tiles_m != 1 || p.acc_groups * p.block_n > 512 ||
       p.taps_per_z > p.acc_groups * p.acc_taps || static_cast<long long>(p.nz) * p.taps_per_z < p.nz_out ||
       (p.acc_taps > 1 && (p.pack_rows < 8 || p.acc_taps * p.pack_rows > kTileM)))) {
    return fail(NG_ERR_INVALID_ARG, "internal: grouped accumulators do not fit tensor memory");
  }
  p.kb_per_split = (p.num_kb + p.splits - 1) / p.splits;
  p.splits = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;  // no empty partitions
  p.status = c->status;
  // TMA counts the whole box (including zero-filled parts) against the barrier
  // stage_bytes was sized from padded regions; the bytes that actually land are:
  const uint32_t landed = p.a_boxes * p.a_box_bytes + p.b_boxes * p.b_box_bytes;
  if (p.splits > 1) {
    const size_t need = static_cast<size_t>(p.splits) * p.nz_out * p.M * p.N * sizeof(float);
    int rc = ensure_workspace(c, stream, need);
    if (rc != NG_OK) return rc;
    p.ws = c->ws;
  } else {
    p.ws = nullptr;
  }
  if (!c->smem_attr_set) {
#define NG_TC_SMEM_ATTR(mode)                                                                                        \
  NG_CUDA(cudaFuncSetAttribute(igemm_tc_kernel<mode, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit)); \
  NG_CUDA(cudaFuncSetAttribute(igemm_tc_kernel<mode, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit))
    NG_TC_SMEM_ATTR(TC_GEMM);
    NG_TC_SMEM_ATTR(TC_FPROP);
    NG_TC_SMEM_ATTR(TC_BPROP);
    NG_TC_SMEM_ATTR(TC_UPDATE);
#undef NG_TC_SMEM_ATTR
#define NG_TC_SMEM_ATTR_PAIR(mode)                                                                                 \
  NG_CUDA(cudaFuncSetAttribute(igemm_tc_kernel<mode, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                               kSmemLimit));                                                                       \
  NG_CUDA(cudaFuncSetAttribute(igemm_tc_kernel<mode, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit))
    NG_TC_SMEM_ATTR_PAIR(TC_GEMM);
    NG_TC_SMEM_ATTR_PAIR(TC_FPROP);
    NG_TC_SMEM_ATTR_PAIR(TC_BPROP);
#undef NG_TC_SMEM_ATTR_PAIR
    c->smem_attr_set = true;
  }
  long long total = static_cast<long long>(p.tiles_m) * p.tiles_n * p.nz * p.splits;
  if (total > 0x3fffffffll) return fail(NG_ERR_TOO_LARGE, "too many work items");
  p.full_items = static_cast<int>(total);
  // 256-row tiles: when the last wave fills at most half of the SMs, its tiles are handed out as
  // 128-row halves, so that the wave takes about half a tile time on twice as many SMs
  const bool split_tail = tuning().split_tail != 0;
  const long long rem = total % c->sm_count;
  if (split_tail && p.m_halves == 2 && rem > 0 && 2 * rem <= c->sm_count) {
    p.full_items = static_cast<int>(total - rem);
    total += rem;
  }
  p.total_items = static_cast<int>(total);
  int grid = static_cast<int>(std::min<long long>(total, c->sm_count));
  if (tuning().max_ctas > 0) grid = std::min(grid, tuning().max_ctas);
  if (p.pair) {
    if (p.m_halves != 1 || p.acc_groups > 1 || p.acc_taps > 1 || p.mode == TC_UPDATE || (p.block_n & 127))
      return fail(NG_ERR_INVALID_ARG, "internal: this tiling cannot run on CTA pairs");
    grid = 2 * static_cast<int>(std::min<long long>(total, c->sm_count / 2));   // one pair per work item in flight
  }
  p.store_staged = pick_store_mode(p);
  if (p.c_row_chunks && !p.store_staged)
    return fail(NG_ERR_UNSUPPORTED, "internal: padded image rows need the staged output stage");
  if (!p.wait_limit_ns) p.wait_limit_ns = c->wait_limit_ns;
  const uint32_t smem = p.stages * p.stage_bytes + 1024u + kCtrlBytes + (p.store_staged ? kEpiStageBytes : 0u) +
                        a_overread(p);
  fill_fast_divs(p);
  TcParams launch = p;
  launch.stage_bytes = p.stage_bytes;
  // expect_tx must equal the bytes the boxes deliver
  if (landed != p.tx_bytes || landed > p.stage_bytes) {
    return fail(NG_ERR_INVALID_ARG, "internal: stage layout and box sizes disagree");
  }
  if (!mapBm && (launch.b_merge == 1 || launch.b_merge == 2)) launch.b_merge = 0;
  const CUtensorMap& mapB2 = mapBm ? *mapBm : mapB;
  // the lean instances: staged tiles, and either raw split-K partials or alpha 1 / no beta / round to nearest
  const bool lean = tuning().lean_kernels != 0 && launch.store_staged &&
                    (launch.splits > 1 || (launch.alpha == 1.0f && launch.beta == 0.0f && launch.sr_bits == 0));
  if (launch.pair) {
    // clusters of two CTAs
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kTcThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
#define NG_TC_LAUNCH_PAIR(mode)                                                                              \
  if (lean) NG_CUDA(cudaLaunchKernelEx(&cfg, igemm_tc_kernel<mode, true, true>, mapA, mapB, mapB2, launch));  \
  else NG_CUDA(cudaLaunchKernelEx(&cfg, igemm_tc_kernel<mode, false, true>, mapA, mapB, mapB2, launch))
    switch (launch.mode) {
      case TC_GEMM: NG_TC_LAUNCH_PAIR(TC_GEMM); break;
      case TC_FPROP: NG_TC_LAUNCH_PAIR(TC_FPROP); break;
      case TC_BPROP: NG_TC_LAUNCH_PAIR(TC_BPROP); break;
      default: return fail(NG_ERR_INVALID_ARG, "internal: no CTA-pair instance of this mode");
    }
#undef NG_TC_LAUNCH_PAIR
  } else
  {
  // (may be set up while the kernel before it in the stream drains: see grid_dependency_wait)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kTcThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = tuning().dependent_launch != 0 ? 1 : 0;
#define NG_TC_LAUNCH(mode)                                                                                      \
  if (lean) NG_CUDA(cudaLaunchKernelEx(&cfg, igemm_tc_kernel<mode, true, false>, mapA, mapB, mapB2, launch));  \
  else NG_CUDA(cudaLaunchKernelEx(&cfg, igemm_tc_kernel<mode, false, false>, mapA, mapB, mapB2, launch))
  switch (launch.mode) {
    case TC_GEMM: NG_TC_LAUNCH(TC_GEMM); break;
    case TC_FPROP: NG_TC_LAUNCH(TC_FPROP); break;
    case TC_BPROP: NG_TC_LAUNCH(TC_BPROP); break;
    case TC_UPDATE: NG_TC_LAUNCH(TC_UPDATE); break;
    default: return fail(NG_ERR_INVALID_ARG, "internal: unknown tensor-core mode");
  }
#undef NG_TC_LAUNCH
  }
  NG_CHECK_LAUNCH();
  if (p.splits > 1) {
    EpiArgs ea;
    ea.alpha = p.alpha; ea.beta = p.beta; ea.relu = p.relu; ea.sr_bits = p.sr_bits;
    ea.seed_lo = p.seed_lo; ea.seed_hi = p.seed_hi; ea.rng_offset = p.rng_offset;
    const long long groups = static_cast<long long>(p.nz_out) * p.M * ((p.N + 7) / 8);
    const int lanes = splitk_reduce_lanes(groups, p.splits, c->sm_count);
    const long long blocks = (groups * lanes + 255) / 256;
    if (blocks > 0x7fffffffll) return fail(NG_ERR_TOO_LARGE, "output too large for the split-K reduction");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(blocks));
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tuning().dependent_launch != 0 ? 1 : 0;
    NG_CUDA(cudaLaunchKernelEx(&cfg, splitk_reduce_kernel, static_cast<const float*>(p.ws), p.splits, lanes, p.nz_out,
                               p.M, p.N, p.C, p.Cold, p.ldc, p.c_zstride, p.out_f32, p.vec_ok, ea, p.c_row_chunks,
                               p.c_row_len));
    NG_CHECK_LAUNCH();
  }
  return NG_OK;
}

}  // namespace ngb

// ------------------------------------------------------------------------------------------
// Split-K GEMM that allocates nothing.
//
// Some hosts of this library may not allocate device memory at the point where they call it: a
// process that has handed its whole memory budget to its own pool or arena, a real-time loop
// that must not take the allocator's lock or risk an implicit synchronisation, a plugin whose
// embedding application forbids cudaMalloc after start-up. ng_hgemm cannot serve them, because
// its split-K path keeps the fp32 partial tiles in a workspace that the library grows with
// cudaMalloc on demand (and its device status word is allocated on first use). This entry point
// keeps both in file-scope device arrays of fixed size, which every GPU that loads the library
// carries until the process exits.
// ------------------------------------------------------------------------------------------
namespace ngb {
namespace {

constexpr size_t kStaticScratchBytes = NG_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) float g_static_scratch[kStaticScratchBytes / sizeof(float)];
static __device__ __align__(256) int g_static_status[64];

// Device addresses of the two arrays, looked up once per device. In host code the array names
// are only handles for cudaGetSymbolAddress; a kernel must be given the looked-up pointers.
struct StaticSlots {
  float* scratch = nullptr;
  int* status = nullptr;
  int sm_count = 0;
  bool ready = false;
};
StaticSlots g_static_slots[64];
std::mutex g_static_mutex;

int static_setup(int dev, StaticSlots** out) {
  if (dev < 0 || dev >= 64) return fail(NG_ERR_INVALID_ARG, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  StaticSlots& s = g_static_slots[dev];
  if (!s.ready) {
    int major = 0;
    NG_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10) return fail(NG_ERR_UNSUPPORTED, "device %d is not sm_100", dev);
    NG_CUDA(cudaDeviceGetAttribute(&s.sm_count, cudaDevAttrMultiProcessorCount, dev));
    void* p = nullptr;
    NG_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    s.scratch = static_cast<float*>(p);
    NG_CUDA(cudaGetSymbolAddress(&p, g_static_status));
    s.status = static_cast<int*>(p);
    NG_CUDA(cudaFuncSetAttribute(igemm_tc_kernel<TC_GEMM, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    s.ready = true;
  }
  *out = &s;
  return NG_OK;
}

}  // namespace

// Status word of the static-scratch entry point on device `dev`: read and cleared. Nothing is
// allocated; returns NG_OK with *code = 0 when that entry point has never run on the device.
int static_scratch_status(int dev, int* code) {
  *code = 0;
  if (dev < 0 || dev >= 64) return NG_OK;
  int* status = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_slots[dev].ready) return NG_OK;
    status = g_static_slots[dev].status;
  }
  NG_CUDA(cudaMemcpy(code, status, sizeof(int), cudaMemcpyDeviceToHost));
  if (*code != 0) NG_CUDA(cudaMemset(status, 0, sizeof(int)));
  return NG_OK;
}

// One CTA, one thread: a bounded wait on an mbarrier that nothing ever arrives at. The wait runs
// out after `limit_ns`, records the site in the status word and the kernel returns normally.
__global__ void wait_expires_kernel(int* status, unsigned long long limit_ns, unsigned long long* waited_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  abort_flag = 0;
  mbar_init(smem_u32(&bar), 1);
  mbar_fence_init();
  const uint64_t t0 = global_timer_ns();
  const bool ok = mbar_wait(smem_u32(&bar), 0u, &abort_flag, status, NG_DEV_TIMEOUT_TEST, limit_ns);
  if (waited_ns) *waited_ns = ok ? 0ull : global_timer_ns() - t0;
}

}  // namespace ngb

using namespace ngb;

extern "C" int ng_static_scratch_status(int* code) {
  int dev = -1;
  NG_CUDA(cudaGetDevice(&dev));
  int v = 0;
  const int rc = static_scratch_status(dev, &v);
  if (rc != NG_OK) return rc;
  if (code) *code = v;
  if (v != 0) return fail(NG_ERR_TIMEOUT, "a static-scratch GEMM gave up a bounded wait (site %d)", v);
  return NG_OK;
}

extern "C" int ng_set_wait_limit_ns(unsigned long long limit_ns) {
  DeviceCtx* c = current_ctx();
  if (!c) return NG_ERR_CUDA;
  c->wait_limit_ns = limit_ns ? limit_ns : kWaitLimitNs;
  return NG_OK;
}

extern "C" int ng_test_wait_expires(unsigned long long limit_ns, unsigned long long* waited_ns_device, void* stream) {
  DeviceCtx* c = current_ctx();
  if (!c) return NG_ERR_CUDA;
  if (limit_ns == 0 || limit_ns > 100000000ull)
    return fail(NG_ERR_INVALID_ARG, "the test wait is limited to 100 ms");
  wait_expires_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(c->status, limit_ns, waited_ns_device);
  NG_CHECK_LAUNCH();
  return NG_OK;
}

extern "C" int ng_hgemm_static_scratch(const void* A, const void* B, void* C, int a_t, int b_t, int m, int n, int k,
                                       int lda, int ldb, int ldc, float alpha, float beta, int relu, int sr_bits,
                                       unsigned long long seed, unsigned int rng_offset, void* stream_) {
  if (!A || !B || !C) return fail(NG_ERR_INVALID_ARG, "null operand");
  if (m <= 0 || n <= 0 || k <= 0) return fail(NG_ERR_INVALID_ARG, "m, n, k must be positive");
  if (a_t && b_t) return fail(NG_ERR_UNSUPPORTED, "op 'tt' is not supported");
  if (sr_bits < 0 || sr_bits > 10) return fail(NG_ERR_INVALID_ARG, "stochastic rounding keeps 1..10 mantissa bits");
  if (lda < (a_t ? m : k) || ldb < (b_t ? k : n) || ldc < n) return fail(NG_ERR_INVALID_ARG, "leading dimension too small");
  auto tma_ok = [](const void* p, long long ld) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0 && (ld & 7) == 0; };
  if (!tma_ok(A, lda) || !tma_ok(B, ldb))
    return fail(NG_ERR_UNSUPPORTED, "operands must be 16-byte aligned with leading dimensions that are multiples of 8");
  // two partitions of fp32 partials is the least this variant uses
  const size_t tile_bytes = static_cast<size_t>(m) * n * sizeof(float);
  if (2 * tile_bytes > kStaticScratchBytes)
    return fail(NG_ERR_TOO_LARGE, "m*n = %lld exceeds the static scratch: 2 * m * n * 4 bytes must fit in %zu bytes",
                static_cast<long long>(m) * n, kStaticScratchBytes);
  int dev = -1;
  NG_CUDA(cudaGetDevice(&dev));
  StaticSlots* slots = nullptr;
  int rc = static_setup(dev, &slots);
  if (rc != NG_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);

  TcParams p = {};
  p.mode = TC_GEMM;
  p.block_n = n <= 64 ? 64 : (n <= 128 ? 128 : 256);
  p.M = m; p.N = n;
  p.tiles_m = (m + kTileM - 1) / kTileM;
  p.tiles_n = (n + p.block_n - 1) / p.block_n;
  p.nz = 1;
  p.nz_out = 1;
  p.acc_groups = 1;
  p.num_kb = (k + kChunk - 1) / kChunk;
  TcOperandLayout lay;
  lay.a_mn_major = a_t ? 1 : 0;
  lay.b_mn_major = b_t ? 0 : 1;
  lay.kb_rows = kChunk;
  tc_fill_mma(p, lay);
  p.C = C; p.Cold = beta != 0.0f ? C : nullptr;
  p.ldc = ldc; p.c_zstride = 0;
  p.alpha = alpha; p.beta = beta; p.relu = relu; p.sr_bits = sr_bits; p.out_f32 = 0;
  p.vec_ok = (reinterpret_cast<uintptr_t>(C) & 15u) == 0 && ldc % 8 == 0;
  p.seed_lo = static_cast<uint32_t>(seed); p.seed_hi = static_cast<uint32_t>(seed >> 32); p.rng_offset = rng_offset;

  // partitions: enough to occupy the SMs, never more than the scratch holds, at least two
  long long want = (slots->sm_count + static_cast<long long>(p.tiles_m) * p.tiles_n - 1) /
                   (static_cast<long long>(p.tiles_m) * p.tiles_n);
  want = std::min<long long>(want, static_cast<long long>(kStaticScratchBytes / tile_bytes));
  want = std::min<long long>(want, 32);
  want = std::max<long long>(want, 2);
  p.splits = static_cast<int>(std::min<long long>(want, p.num_kb));
  p.kb_per_split = (p.num_kb + p.splits - 1) / p.splits;
  p.splits = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;
  p.status = slots->status;
  p.ws = slots->scratch;     // device address from cudaGetSymbolAddress, never the symbol itself

  CUtensorMap mapA, mapB;
  {
    uint64_t dims[5] = {1, 1, 1, 1, 1};
    uint64_t str[4];
    uint32_t box[5] = {kChunk, 1, 1, 1, 1};
    if (a_t) { dims[0] = m; dims[1] = k; box[1] = kChunk; } else { dims[0] = k; dims[1] = m; box[1] = kTileM; }
    str[0] = static_cast<uint64_t>(lda) * 2; str[1] = str[0] * dims[1]; str[2] = str[1]; str[3] = str[1];
    rc = make_tensor_map(&mapA, A, dims, str, box);
    if (rc != NG_OK) return rc;
  }
  {
    uint64_t dims[5] = {1, 1, 1, 1, 1};
    uint64_t str[4];
    uint32_t box[5] = {kChunk, 1, 1, 1, 1};
    if (b_t) { dims[0] = k; dims[1] = n; box[1] = p.block_n; } else { dims[0] = n; dims[1] = k; box[1] = kChunk; }
    str[0] = static_cast<uint64_t>(ldb) * 2; str[1] = str[0] * dims[1]; str[2] = str[1]; str[3] = str[1];
    rc = make_tensor_map(&mapB, B, dims, str, box);
    if (rc != NG_OK) return rc;
  }

  const long long total = static_cast<long long>(p.tiles_m) * p.tiles_n * p.splits;
  const int grid = static_cast<int>(std::min<long long>(total, slots->sm_count));
  const uint32_t smem = p.stages * p.stage_bytes + 1024u + kCtrlBytes;
  p.store_staged = 0;   // this variant stores straight from registers
  p.wait_limit_ns = kWaitLimitNs;
  p.full_items = p.total_items = static_cast<int>(total);
  ngb::fill_fast_divs(p);
  igemm_tc_kernel<TC_GEMM, false><<<grid, kTcThreads, smem, stream>>>(mapA, mapB, mapB, p);
  NG_CHECK_LAUNCH();
  EpiArgs ea;
  ea.alpha = alpha; ea.beta = beta; ea.relu = relu; ea.sr_bits = sr_bits;
  ea.seed_lo = p.seed_lo; ea.seed_hi = p.seed_hi; ea.rng_offset = rng_offset;
  if (p.splits > 1) {
    const long long groups = static_cast<long long>(m) * ((n + 7) / 8);
    const int lanes = ngb::splitk_reduce_lanes(groups, p.splits, slots->sm_count);
    const int blocks = static_cast<int>((groups * lanes + 255) / 256);
    splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(p.ws, p.splits, lanes, 1, m, n, C, p.Cold, ldc, 0, 0, p.vec_ok,
                                                     ea, 0, 0);
    NG_CHECK_LAUNCH();
  }
  return NG_OK;
}
