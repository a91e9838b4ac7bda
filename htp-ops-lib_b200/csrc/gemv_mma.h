// Launch interface of the decode-side mat-vec kernel (gemv_mma.cu).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace htp {

constexpr int kGemvTileRows    = 32;  // output rows per tile (two 16-row MMA groups)
constexpr int kGemvMaxStages   = 8;
constexpr int kGemvSmemHeader  = 33024;   // barriers, per-token scales, cross-warp reduction buffer
constexpr int kGemvSmemBudget  = 232448;  // 227 KiB opt-in dynamic shared memory per CTA on sm_100
constexpr int kGemvMaxGrid     = 1024;    // scratch is sized for this many CTAs

constexpr int kGemvErrProducerWait = 101;
constexpr int kGemvErrConsumerWait = 102;

// 32-weight blocks per pipeline stage and row: 64 for Q4_0 (1152 B), 32 for Q8_0 (1088 B), so a
// stage of 32 rows is ~36 KB in either format.
constexpr int gemv_stage_blocks(int wt) {
  return wt == 0 ? 64 : 32;
}

// Shared-memory pitch of one weight row inside a stage: the stage's bytes plus 16, an odd
// multiple of 16, so that eight consecutive rows start in eight different 16-byte bank groups.
constexpr int gemv_row_pitch(int wt) {
  return wt == 0 ? 1168 /* 64*18 = 1152 -> 73*16 */ : 1104 /* 32*34 = 1088 -> 69*16 */;
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
  long long      total_items;  // (N / 32) * stages_per_tile
  float         *partials;     // [grid][2][256] scratch for tiles cut by a CTA range boundary
  unsigned      *counters;     // [grid] arrival counters, zero between launches
  int           *err;          // first error code, 0 when none
};

// Bytes of shared memory the activation fragments of `kblocks` blocks occupy.
size_t gemv_frag_bytes(int wt, bool a16, int mpad, int kblocks);

cudaError_t gemv_mma_launch(const GemvArgs &args, int wt, bool a16, int mpad, int grid, size_t smem,
                            cudaStream_t stream, bool pdl);

}  // namespace htp
