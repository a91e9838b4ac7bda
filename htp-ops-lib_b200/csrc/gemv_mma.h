// Launch interface of the decode-side mat-vec kernel (gemv_mma.cu).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace htp {

constexpr int kGemvTileRows    = 32;  // output rows per tile (two 16-row MMA groups)
constexpr int kGemvMaxStages   = 8;
// Fixed part of the kernel's shared memory: barriers, per-token scales, the output staging tile and
// two copies (one on the wide path, token padding 8) of the 16 KB cross-warp reduction buffer.
constexpr int gemv_header_bytes(int mpad) {
  return mpad == 8 ? 17792 : 34176;
}
constexpr int kGemvSmemBudget  = 232448;  // 227 KiB opt-in dynamic shared memory per CTA on sm_100
constexpr int kGemvMaxGrid     = 1024;    // scratch is sized for this many CTAs

constexpr int kGemvErrProducerWait = 101;
constexpr int kGemvErrConsumerWait = 102;
constexpr int kGemvErrFlagWait     = 103;  // a peer's completion flag never arrived

// 32-weight blocks per pipeline stage and row: 64 for Q4_0 / IQ4_NL (1152 B), 32 for Q8_0 (1088 B), so a
// stage of 32 rows is ~36 KB in either format.
constexpr int gemv_stage_blocks(int wt) {
  return wt == 1 ? 32 : 64;
}

// Shared-memory pitch of one weight row inside a stage: the stage's bytes plus 16, an odd
// multiple of 16, so that eight consecutive rows start in eight different 16-byte bank groups.
constexpr int gemv_row_pitch(int wt) {
  return wt == 1 ? 1104 /* 32*34 = 1088 -> 69*16 */ : 1168 /* 64*18 = 1152 -> 73*16 */;
}

// Tokens per launch are padded to 1, 2 or 8 (8 = the wide integer path).
constexpr int gemv_mpad(int m) {
  return m <= 1 ? 1 : (m <= 2 ? 2 : 8);
}
// Pipeline stages a launch needs at least.  The wide path (8), whose activation fragments take 864
// bytes per block, runs K = 4096 on a two-stage ring: measured faster than more, smaller stages (the
// hand-over per stage is what costs) and than cutting K into launches that accumulate.
constexpr int gemv_min_stages(int mpad) {
  return mpad == 8 ? 2 : 3;
}

struct GemvArgs {
  float         *y;              // [M][N] fp32
  const void    *x;              // [M][x_stride] fp32 or fp16
  const uint8_t *w;              // N rows of blocks
  long long      w_row_bytes;    // bytes between weight rows
  long long      w_k_off_bytes;  // byte offset of this launch's K range inside a row
  int            x_k_off;        // element offset of this launch's K range inside an activation row
  int            x_stride;       // elements between activation rows
  int            M, N;
  int            kblocks;     // blocks in this launch's K range (multiple of 8)
  int            accumulate;  // add to y instead of overwriting it
  int            n_stages;    // ring depth
  int            stages_per_tile;
  long long      item_base;    // index of this operator's first item in the launch's item list (0 when alone)
  long long      total_items;  // items of the whole launch: (N / 32) * stages_per_tile when alone
  float         *partials;     // [grid][2][256] scratch for tiles cut by a CTA range boundary
  unsigned      *counters;     // [grid] arrival counters, zero between launches
  int           *err;          // first error code, 0 when none
  // Output placement (single-operator launches): the result is stored as the column band
  // [y_col0, y_col0 + N) of n_dst matrices of y_ld floats per token - y and y_more[0 .. n_dst - 2],
  // e.g. every rank's copy of a row-sharded output.  n_dst = 0 / y_ld = 0: plain y[M][N].
  int            n_dst;
  long long      y_ld, y_col0;
  float         *y_more[7];
  // Completion signal (optional, with several destinations): when the LAST CTA of the launch has
  // finished - every CTA's stores fenced at system scope - it writes `epoch` to sig_flags[d] for
  // every destination d (a word in that destination GPU's memory), so that a waiter there knows this
  // rank's band has landed.  done_counter: a zeroed word of this GPU, zero again afterwards.
  unsigned      *done_counter;
  unsigned      *sig_flags[8];
  unsigned       epoch;
  // Optional: after signalling, the last CTA waits (bounded) until wait_flags[r] has reached `epoch`
  // for r = 0 .. n_wait - 1 - this GPU's flag array, written by the peers' launches of the same step.
  const unsigned *wait_flags;
  int             n_wait;
};


// Waits (bounded) on `stream` until flags[r] has reached `epoch` for r = 0 .. n - 1; records
// kGemvErrFlagWait in *err when that does not happen.
cudaError_t flags_wait_launch(const unsigned *flags, int n, unsigned epoch, int *err, cudaStream_t stream);

// One operator of a batched launch: several independent mat-vecs of the same kind (weight format,
// activation type, token count) streamed by ONE persistent kernel as a single item list, so that
// small operators pay neither a launch nor a pipeline fill and drain each.
constexpr int kGemvBatchMaxOps = 128;

struct alignas(64) GemvBatchOp {
  unsigned char  wmap[128];   // CUtensorMap over the operator's weight bytes
  float         *y;
  const void    *x;
  long long      item_begin;  // first item of this operator in the launch's item list
  int            N, kblocks, x_stride, stages_per_tile;
  int            x_k_off;     // element offset of the operator's K range inside an activation row
  int            accumulate;  // add to y: a later K range of a matrix whose fragments do not fit one launch
};

struct GemvBatchArgs {
  GemvBatchOp ops[kGemvBatchMaxOps];
  long long   total_items;
  float      *partials;
  unsigned   *counters;
  int        *err;
  int         n_ops, M, n_stages, frag_bytes;  // frag_bytes: fragment region, sized for the largest K
};

// Fills op.wmap for a weight matrix of n rows and kblocks blocks per row (cached by geometry).
cudaError_t gemv_weight_map(void *wmap_out, const uint8_t *w, long long w_row_bytes, int kblocks, int n, int wt);

cudaError_t gemv_mma_batch_launch(const GemvBatchArgs &args, int wt, bool a16, int mpad, int grid, size_t smem,
                                  cudaStream_t stream, bool pdl);

// Bytes of shared memory the activation fragments of `kblocks` blocks occupy.
size_t gemv_frag_bytes(int wt, bool a16, int mpad, int kblocks);

// How a mat-vec of m (1..8) tokens over kblocks blocks (a multiple of 8) per row runs: token padding,
// stage geometry, and into how many equal K ranges it is cut so that the activation fragments of
// one range fit in shared memory beside enough pipeline stages (ranges after the first accumulate
// into the output, as launches of their own).  False when no split fits.
struct GemvPlan {
  int  mpad;
  int  stage_blocks, stage_bytes;
  int  nchunks, chunk_periods;  // K ranges; blocks of 256 weights per range (the last may be shorter)
  int  n_stages;                // ring depth the budget allows for one range
};
bool gemv_plan(int smem_budget, int wt, bool a16, int m, int kblocks, GemvPlan *out);

cudaError_t gemv_mma_launch(const GemvArgs &args, int wt, bool a16, int mpad, int grid, size_t smem,
                            cudaStream_t stream, bool pdl);

}  // namespace htp
