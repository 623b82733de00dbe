// Host side of the tensor-core engine: UMMA descriptor construction, ring sizing, split-K
// choice and the launch itself.
#include <algorithm>

#include "epilogue.cuh"
#include "host.h"
#include "igemm_tc_kernel.cuh"

namespace ngb {

namespace {
constexpr uint32_t kSmemLimit = 232448;  // 227 KB opt-in dynamic shared memory per CTA
constexpr uint32_t kCtrlBytes = 256;     // barriers + TMEM slot + abort flag
constexpr uint32_t kLayoutSw128 = 2;     // UMMA shared-memory descriptor layout type

// Upper 32 bits of a shared-memory matrix descriptor: stride byte offset [32,46), descriptor
// version 1 in [46,48), base offset 0, layout type in [61,64).
uint32_t desc_hi(uint32_t sbo_bytes) {
  return ((sbo_bytes >> 4) & 0x3fffu) | (1u << 14) | (kLayoutSw128 << 29);
}
// Lower 32 bits without the start address: leading byte offset in [16,30).
uint32_t desc_lo(uint32_t lbo_bytes) { return ((lbo_bytes >> 4) & 0x3fffu) << 16; }
}  // namespace

void tc_fill_mma(TcParams& p, const TcOperandLayout& lay) {
  p.a_mn_major = lay.a_mn_major;
  p.b_mn_major = lay.b_mn_major;
  p.kb_rows = lay.kb_rows;
  p.mma_per_kb = lay.kb_rows / 16;
  // Instruction descriptor (kind::f16): D fp32 [4,6)=1, A/B fp16 (format 0), major-ness bits
  // 15/16 (1 = MN-major), N>>3 in [17,23), M>>4 in [24,29).
  p.idesc = (1u << 4) | (static_cast<uint32_t>(lay.a_mn_major) << 15) |
            (static_cast<uint32_t>(lay.b_mn_major) << 16) | (static_cast<uint32_t>(p.block_n >> 3) << 17) |
            (static_cast<uint32_t>(kTileM >> 4) << 24);
  // K-major operand: one box of [rows][64 k] 128-byte rows; 8-row groups 1024 B apart; a K=16
  // step moves the start address 32 B inside the swizzled row.
  // MN-major operand: boxes of [kb_rows][64 mn]; 8 reduction rows = 1024 B (stride offset),
  // next 64-wide MN chunk = next box (leading offset); a K=16 step moves 16 rows = 2048 B.
  const uint32_t mn_box = static_cast<uint32_t>(lay.kb_rows) * 128u;
  if (lay.a_mn_major) {
    p.a_boxes = kTileM / kChunk;
    p.a_box_bytes = mn_box;
    p.a_desc_lo = desc_lo(mn_box);
    p.a_kstep = 2048u >> 4;
  } else {
    p.a_boxes = 1;
    p.a_box_bytes = kTileM * 128u;
    p.a_desc_lo = desc_lo(16);
    p.a_kstep = 32u >> 4;
  }
  p.a_desc_hi = desc_hi(1024);
  p.a_bytes = p.a_boxes * p.a_box_bytes;
  if (lay.b_mn_major) {
    p.b_boxes = p.block_n / kChunk;
    p.b_box_bytes = mn_box;
    p.b_desc_lo = desc_lo(mn_box);
    p.b_kstep = 2048u >> 4;
  } else {
    p.b_boxes = 1;
    p.b_box_bytes = static_cast<uint32_t>(p.block_n) * 128u;
    p.b_desc_lo = desc_lo(16);
    p.b_kstep = 32u >> 4;
  }
  p.b_desc_hi = desc_hi(1024);
  // every box must start on a 1024-byte boundary for the 128-byte swizzle
  p.a_bytes = (p.a_bytes + 1023u) & ~1023u;
  const uint32_t b_bytes = (p.b_boxes * p.b_box_bytes + 1023u) & ~1023u;
  p.stage_bytes = p.a_bytes + b_bytes;
  p.stages = std::min<uint32_t>(kMaxStages, (kSmemLimit - 1024u - kCtrlBytes) / p.stage_bytes);
}

int choose_splits(const DeviceCtx* c, long long tiles, int num_kb, long long out_elems) {
  if (tiles * 2 > c->sm_count || num_kb < 8) return 1;
  long long s = (c->sm_count + tiles - 1) / tiles;
  s = std::min<long long>(s, num_kb / 4);
  s = std::min<long long>(s, 32);
  // partials cost 8 bytes of traffic per output element per split; keep them cheap relative
  // to the operand traffic
  while (s > 1 && s * out_elems * 4 > (512ll << 20)) --s;
  return static_cast<int>(std::max<long long>(s, 1));
}

int tc_launch(DeviceCtx* c, const CUtensorMap& mapA, const CUtensorMap& mapB, TcParams& p, cudaStream_t stream) {
  if (p.num_kb < 1) return fail(NG_ERR_INVALID_ARG, "empty reduction");
  if (p.splits < 1) p.splits = 1;
  p.kb_per_split = (p.num_kb + p.splits - 1) / p.splits;
  p.splits = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;  // no empty partitions
  p.status = c->status;
  // TMA counts the whole box (including zero-filled parts) against the barrier
  // stage_bytes was sized from padded regions; the bytes that actually land are:
  const uint32_t landed = p.a_boxes * p.a_box_bytes + p.b_boxes * p.b_box_bytes;
  if (p.splits > 1) {
    const size_t need = static_cast<size_t>(p.splits) * p.nz * p.M * p.N * sizeof(float);
    int rc = ensure_workspace(c, need);
    if (rc != NG_OK) return rc;
    p.ws = c->ws;
  } else {
    p.ws = nullptr;
  }
  if (!c->smem_attr_set) {
    NG_CUDA(cudaFuncSetAttribute(igemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    c->smem_attr_set = true;
  }
  const long long total = static_cast<long long>(p.tiles_m) * p.tiles_n * p.nz * p.splits;
  if (total > 0x7fffffffll) return fail(NG_ERR_TOO_LARGE, "too many work items");
  const int grid = static_cast<int>(std::min<long long>(total, c->sm_count));
  const uint32_t smem = p.stages * p.stage_bytes + 1024u + kCtrlBytes;
  TcParams launch = p;
  launch.stage_bytes = p.stage_bytes;
  // expect_tx must equal the bytes the boxes deliver; regions are box multiples already
  if (landed != p.stage_bytes) {
    // padded regions: the kernel's expect_tx uses stage_bytes, so keep them identical
    return fail(NG_ERR_INVALID_ARG, "internal: stage layout is not a whole number of boxes");
  }
  igemm_tc_kernel<<<grid, kTcThreads, smem, stream>>>(mapA, mapB, launch);
  NG_CHECK_LAUNCH();
  if (p.splits > 1) {
    EpiArgs ea;
    ea.alpha = p.alpha; ea.beta = p.beta; ea.relu = p.relu; ea.sr_bits = p.sr_bits;
    ea.seed_lo = p.seed_lo; ea.seed_hi = p.seed_hi; ea.rng_offset = p.rng_offset;
    const long long groups = static_cast<long long>(p.nz) * p.M * ((p.N + 7) / 8);
    const int threads = 256;
    const int blocks = static_cast<int>(std::min<long long>((groups + threads - 1) / threads, c->sm_count * 8ll));
    splitk_reduce_kernel<<<blocks, threads, 0, stream>>>(p.ws, p.splits, p.nz, p.M, p.N, p.C, p.Cold, p.ldc,
                                                         p.c_zstride, p.out_f32, p.vec_ok, ea);
    NG_CHECK_LAUNCH();
  }
  return NG_OK;
}

}  // namespace ngb
