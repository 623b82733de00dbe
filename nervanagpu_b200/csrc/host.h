// Host-side internals shared by the translation units of libnervana_b200.so.
#pragma once
#include <map>
#include <vector>
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "igemm_tc.cuh"
#include "status.h"

namespace ngb {

// Per-device state owned by the library: SM count, device status word, split-K workspace.
struct DeviceCtx {
  int device = -1;
  int sm_count = 0;
  int* status = nullptr;     // device int written by kernels whose bounded wait gave up
  // split-K / conv / pooling scratch, grown on demand, one buffer per stream; ws / ws_bytes name
  // the buffer of the stream the last ensure_workspace call was for
  struct Scratch {
    float* ptr = nullptr;
    size_t bytes = 0;
  };
  std::map<cudaStream_t, Scratch> scratch;
  // second buffer per stream, for operands that a call re-lays-out before it hands them to another
  // entry point of the library (which uses the first buffer as it likes)
  std::map<cudaStream_t, Scratch> aux;
  float* ws = nullptr;
  size_t ws_bytes = 0;
  // Recorded sequences (CUDA graphs) keep the scratch pointers of the calls they recorded: while
  // any is alive, a scratch buffer that has to grow is retired (kept allocated), not freed.
  int live_graphs = 0;
  std::vector<void*> retired;
  bool smem_attr_set = false;
  unsigned long long wait_limit_ns = 2000000000ull;   // bound of the kernels' waits (ng_set_wait_limit_ns)
  bool capturing = false;    // a stream capture is open: nothing may allocate or synchronise
  unsigned long long capture_launches0 = 0;
};

// Tuning aids, read from the environment once per process (none is needed in normal use):
// NG_TILE_ROWS=128|256, NG_TILE_COLS=128|192|256, NG_KB_ROWS=16|32|48|64, NG_MERGE_BOXES=0,
// NG_SPLIT_TAIL=0, NG_LEAN_KERNELS=0, NG_REDUCE_LANES=<power of two>, NG_UPDATE_GROUPS=<n>,
// NG_UPDATE_STACK=<n>, NG_UPDATE_MIN_STAGES=<n>, NG_UPDATE_SWAP=0, NG_PAIR_MMA=0|1, NG_CHAN_BLOCK=0|2 (never / always copy activations channel-blocked), NG_DEPENDENT_LAUNCH=0, NG_SPACE_TO_DEPTH=0, NG_MAX_CTAS=<n>,
// NG_CONV_SPLITS=<n> (partitions of the forward / backward reduction; 1 = never split). A field is 0
// (or -1 for the on/off switches) when its variable is not set.
struct Tuning {
  int tile_rows = 0, tile_cols = 0, kb_rows = 0, reduce_lanes = 0;
  int update_groups = 0, update_stack = 0, update_min_stages = 0, max_ctas = 0, conv_splits = -1, max_stages = 0, feed_bytes_per_ns = 0;
  int merge_boxes = -1, split_tail = -1, lean_kernels = -1, update_swap = -1, pair_mma = -1, chan_block = -1, dependent_launch = -1, space_to_depth = -1;
};
const Tuning& tuning();
Tuning& tuning_mutable();   // ng_tune

// Error reporting: returns `code` after storing a printf-style message for ng_last_error().
int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define NG_CUDA(expr)                                        \
  do {                                                       \
    cudaError_t _e = (expr);                                 \
    if (_e != cudaSuccess) return ::ngb::cuda_fail(_e, #expr); \
  } while (0)

// Count of kernels this library has launched (all devices, all streams); read by ng_launch_count.
void count_launch();
// Count of GEMM / convolution calls that ran on the plain CUDA-core fall-back kernels instead of
// the tensor-core engine; read by ng_fallback_launch_count.
void count_fallback_launch();
#define NG_CHECK_LAUNCH()            \
  do {                               \
    NG_CUDA(cudaGetLastError());     \
    ::ngb::count_launch();           \
  } while (0)

// Status word of ng_hgemm_static_scratch on device `dev`, read and cleared without allocating.
int static_scratch_status(int dev, int* code);

// Context of the current device (initialised on first use). Null + error set on failure.
DeviceCtx* current_ctx();
// Ensure the workspace of `stream` holds at least `bytes` and make c->ws point at it; may
// synchronise the device when it has to grow.
int ensure_workspace(DeviceCtx* c, cudaStream_t stream, size_t bytes);
int ensure_aux(DeviceCtx* c, cudaStream_t stream, size_t bytes, void** ptr);

// Rank-5 tiled tensor map over fp16 (elem_bytes 2) data. dims[0] is the contiguous dimension;
// strides_bytes[i] is the byte stride of dims[i+1]. Swizzle is chosen from the inner box width.
int make_tensor_map(CUtensorMap* out, const void* base, const uint64_t dims[5], const uint64_t strides_bytes[4],
                    const uint32_t box[5], int elem_bytes = 2);

// Fill the MMA/ring fields of a parameter block and launch the tensor-core kernel (+ split-K reduce).
struct TcOperandLayout {
  int a_mn_major, b_mn_major;
  int kb_rows;   // reduction rows per k-block
  int a_box_rows = 0;   // K-major A only: rows one box delivers (0 = the whole tile)
  int b_box_rows = 0;   // K-major B only: the column tile is made of b_box_count boxes of this many
  int b_box_count = 0;  // rows each (0 = one box of block_n rows)
  // MN-major operands whose tensor map carries the 64-wide chunk number as a dimension of its own
  // (behind the reduction rows), so that one box delivers several chunks in the order the MMA wants:
  int a_chunks = 0;        // MN-major A, 128-row tiles: 64-row chunks that hold real rows (0 = both)
  int a_merge = 0;         // A: one box per 128-row half
  int b_merge_static = 0;  // B: one box per column tile
  int b_pair = 0;          // B (tap-block map, N = 128): one box per pixel = its two chunks
};
void tc_fill_mma(TcParams& p, const TcOperandLayout& lay);
// mapBm (optional, convolutions): a second map over B whose box is the whole column tile; the
// kernel uses it for the tiles that lie inside one image row (p.b_merge says how its dimensions
// are ordered) and the per-chunk map for the others.
int tc_launch(DeviceCtx* c, const CUtensorMap& mapA, const CUtensorMap& mapB, TcParams& p, cudaStream_t stream,
              const CUtensorMap* mapBm = nullptr);

// 1 = 128-row tiles, 2 = 256-row tiles (two accumulators sharing each B operand: a third less
// L2 -> SM traffic per flop, but no overlap of the epilogue with the next tile and coarser waves).
// `col_tiles` = column tiles x z x splits. Sets p.m_halves and p.tiles_m.
void tc_pick_tile_rows(const DeviceCtx* c, TcParams& p, long long col_tiles, int num_kb);
// Chooses m_halves and block_n (256/192/128) together and sets tiles_m / tiles_n; p.M must be set.
void tc_pick_tile(const DeviceCtx* c, TcParams& p, long long cols, int num_kb, int kb_rows);

// Picks the number of split-K partitions for `tiles` output tiles and `num_kb` k-blocks.
constexpr int kMaxSplits = 160;
int choose_splits(const DeviceCtx* c, long long tiles, int num_kb, long long out_elems, bool charge_reduction = false);

// One GEMM request: C[m x n] = epilogue(op(A) * op(B)); see ng_hgemm for the conventions.
struct GemmCall {
  const void* A;
  const void* B;
  void* C;
  int a_t, b_t, m, n, k;
  long long lda, ldb, ldc;
  float alpha, beta;
  int relu, sr_bits;
  unsigned long long seed;
  unsigned rng_offset;
  int batch;                 // independent outputs (grid z)
  long long az, bz, cz;      // element strides between them (0 = shared operand)
  int loops;                 // batches accumulated into each output
  long long alz, blz;
  int out_f32;
  int force_simt;
};
int run_gemm(const GemmCall& g, cudaStream_t stream);

}  // namespace ngb
