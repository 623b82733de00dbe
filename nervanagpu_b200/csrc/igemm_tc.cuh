// Parameter block of the tcgen05 implicit-GEMM engine (one kernel serves ng.dot and the
// three convolution passes; they differ in how the TMA producer turns a k-block into box
// coordinates and in how work items map onto output tiles).
#pragma once
#include <stdint.h>

namespace ngb {

enum TcMode : int { TC_GEMM = 0, TC_FPROP = 1, TC_BPROP = 2, TC_UPDATE = 3 };

constexpr int kTileM = 128;        // UMMA M (TMEM lanes)
constexpr int kChunk = 64;         // fp16 elements per 128-byte swizzle row
constexpr int kMaxStages = 16;
constexpr int kEpiWarps = 8;       // two per group of 32 TMEM lanes, each takes half of the columns
constexpr int kTcThreads = 64 + 32 * kEpiWarps;    // warp 0 TMA, warp 1 MMA, then the epilogue warps
constexpr uint32_t kEpiStageBytes = kEpiWarps * 4096;  // one [32 rows][128 B] staging box per epilogue warp

// Division of a non-negative 31-bit number by a run-time constant as multiply-high and shift
// (round-up method: mul = ceil(2^(31+ceil(log2 d)) / d), quotient = umulhi(n, mul) >> shr). The
// single producer thread decodes a tile with a dozen divisions; as hardware-emulated divides they
// cost it about 0.8 us per tile.
struct FastDiv {
  uint32_t mul, shr, d;
};

struct TcParams {
  // ---- work decomposition: item = ((split * nz + z) * tiles_n + tile_n) * tiles_m + tile_m
  int tiles_m, tiles_n, nz, splits;
  int num_kb;          // k-blocks in the whole reduction
  int kb_per_split;    // ceil(num_kb / splits)
  int full_items;      // items [0, full_items) are whole tiles; from there on, item pairs are the two
  int total_items;     // 128-row halves of one 256-row tile (the cut last wave); all items
  int block_n;         // UMMA N: 64, 128 or 256
  int m_halves;        // 1: 128-row tiles, accumulator double-buffered across tiles
                       // 2: 256-row tiles, two accumulators that share every B operand
  int pair;            // 1: CTA pairs (cta_group::2): a work item is 256 rows x block_n columns, each CTA
                       // of the pair holds 128 rows of A and block_n / 2 columns of B; needs m_halves == 1
                       // and tiles_m counted in 256-row tiles
  int acc_groups;      // weight update only: accumulators per work item (taps z*g .. z*g+g-1 share
                       // every B operand); 1 otherwise. Needs m_halves == 1, g * block_n <= 512.
  int acc_taps;        // weight update only: taps stacked along the rows of one accumulator (each
                       // `pack_rows` rows: t * pack_rows <= 128), so that a tap with few rows does
                       // not cost a whole 128-row MMA; 1 otherwise
  int pack_rows;       // rows per stacked tap (= rows of one A box)
  int taps_per_z;      // weight update with groups / stacking: work item z owns output slices
                       // [z * taps_per_z, (z + 1) * taps_per_z), at most acc_groups * acc_taps of them
  int nz_out;          // number of output slices (= nz unless taps are grouped or stacked, then
                       // nz = ceil(nz_out / (acc_groups * acc_taps)))
  int M, N;            // logical output extent (rows, cols)

  // ---- MMA descriptors (host-built)
  uint32_t idesc;
  uint32_t a_desc_lo, a_desc_hi;   // lo: LBO field only; start address is or-ed in per stage
  uint32_t b_desc_lo, b_desc_hi;
  uint32_t a_kstep, b_kstep;       // start-address increment (16-byte units) per K=16 MMA
  uint32_t a_half_step;            // start-address increment (16-byte units) to the second 128 rows of A
  int mma_per_kb;                  // kb_rows / 16

  // ---- shared-memory ring
  int stages;
  uint32_t stage_bytes;            // distance between ring slots
  uint32_t tx_bytes;               // bytes the boxes of one k-block deliver (= expect_tx)
  uint32_t a_bytes;                // B region starts at this offset inside a stage
  int a_boxes, b_boxes;            // TMA boxes per stage per operand
  uint32_t a_box_bytes, b_box_bytes;

  // ---- producer
  int mode;
  int swap_ab;                     // weight update only: A = error pixels (rows k), B = the input boxes
                                   // of b_boxes taps per column tile (output transposed: few filters)
  int a_mn_major, b_mn_major;
  int a_merge;                     // MN-major A: one box per 128-row half, map (64, rows, chunk, ...)
  int b_merge;                     // MN-major B boxes that span the whole column tile:
                                   //   1 conv, map (n, chan, x, y, z)        } tiles inside one image row;
                                   //   2 conv, map (n_lo, chan, n_hi, x, y)  } per-chunk boxes otherwise
                                   //   3 GEMM, map (n_lo, k, n_hi, batch), every tile
                                   //   4 tap blocks, N = 128: a box per pixel, map (n_lo, x, y, chan, n_hi)
  int kb_rows;                     // reduction rows per k-block (64, or 16..64 for small C in fprop)
  int a_zmul, b_zmul;              // batched GEMM: coordinate in dim 2 = z * zmul
  // conv geometry (unused by TC_GEMM)
  int red_chunks;                  // fprop: ceil(C/kb_rows); bprop: ceil(K/64)
  int RS, S, R;                    // filter taps (tap blocks when tap_w/tap_h > 1)
  int tap_w, tap_h;                // input pixels per tap step: 1, or the tap-block size of the
                                   // few-channel modes where one box carries a block of taps
  int pad_d, pad_h, pad_w;
  int str_d, str_h, str_w;
  int inner_tap;                   // N in flattened-(W,N) mode else 0
  int x_tap;                       // 0 in flattened mode else 1
  int dec_cpi, dec_q, dec_p, dec_m;  // chunk decode of the pixel space the chunks walk
  int oob_y;                       // a y/p coordinate that is out of range (forces zero fill)

  // ---- epilogue
  void* C;                         // fp16 or fp32 output
  const void* Cold;                // source of the beta term (same type/shape as C) or null
  long long ldc;                   // elements
  long long c_zstride;             // elements, per z
  float alpha, beta;
  int relu;
  int sr_bits;                     // 0 = round to nearest even, else mantissa bits kept
  int out_f32;
  int vec_ok;                      // rows are 16-byte aligned for vector access
  int store_staged;                // 1: tiles leave through swizzled shared memory, written out in
                                   // whole 128-byte rows; 0: stored straight from registers
  int c_box_cols;                  // columns per staged box (128 bytes worth: 64 fp16 / 32 fp32)
  // Convolution outputs over a flattened (x, n) pixel space whose image rows are not a multiple
  // of 64 elements: the column space is padded to c_row_chunks chunks per image row, of which
  // the first c_row_len elements exist in memory (row r starts at column r * c_row_len of C).
  // 0 = columns are stored as they are numbered.
  int c_row_chunks, c_row_len;
  uint32_t seed_lo, seed_hi, rng_offset;
  float* ws;                       // split-K partials [split][z][M][N] when splits > 1
  int* status;                     // device status word
  // divisors of the tile / chunk / tap decodes, filled in by the launch code
  FastDiv fd_tiles_m, fd_tiles_n, fd_nz, fd_cpi, fd_q, fd_p, fd_RS, fd_S, fd_red, fd_crow;
  unsigned long long wait_limit_ns;   // bound of every wait inside the kernel
};

}  // namespace ngb
