// Launch interface of the prefill-side GEMM (gemm_tcgen05.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace htp {

constexpr int kGemmErrProducer = 201;
constexpr int kGemmErrMma      = 202;
constexpr int kGemmErrEpilogue = 203;
constexpr int kGemmErrDequant  = 204;
constexpr int kGemmErrFixup    = 205;  // the other contributor of a split tile never raised its flag

constexpr int kGemmMaxDst = 8;

// `wt` of gemm_tcgen05_launch beyond the block formats (0 Q4_0, 1 Q8_0, 2 IQ4_NL): fp16 weights in the
// reference's 32 x 32 tile order (tile (n/32, k/32) at tile number (n/32) * (K/32) + k/32, element
// (k, n) of a tile at halfword (k & ~1) * 32 + 2 n + (k & 1)); K a multiple of 128.
constexpr int kGemmWtF16Tiled = 3;
// The reference's permuted super-blocks (my_block_q4_0 144 bytes / my_block_q8_0 272 bytes, four per
// tile of the same tile order; include/dsp/quants.h:16-31, expanded slot by slot at
// src/dsp/ops/mat_mul.c:308-510): Q4_0, Q8_0, IQ4_NL values.  K a multiple of 128.
constexpr int kGemmWtPermQ4  = 4;
constexpr int kGemmWtPermQ8  = 5;
constexpr int kGemmWtPermIQ4 = 6;

struct GemmArgs {
  float         *y;  // [M][N] fp32 (destination 0)
  const void    *x;  // [M][K] fp16
  const uint8_t *w;  // N rows of K/32 blocks, or fp16 tiles
  int            M, N, K;  // K a multiple of 256 (tile-order formats: 128), N a multiple of 32
  int           *err;      // first error code, 0 when none
  // Scratch for tiles whose K range is split between two workers (gemm_scratch_bytes() bytes at
  // `part`, 256-byte aligned, zero before the first launch; the flags are zero again after every
  // launch).  nullptr: tiles are never split.
  float         *part;
  int           *flags;  // set by the launcher
  int            split;  // set by the launcher
  // Output placement.  The result is stored into n_dst destination matrices (destination 0 = y,
  // the others = y_more[0 .. n_dst - 2]; 0 means 1), each row-major with y_ld elements per token
  // (0 means N), at column y_col0: this is how a rank of a row-sharded matmul writes its column
  // band straight into every rank's full output (peer pointers), instead of a gather afterwards.
  int            n_dst;
  float         *y_more[kGemmMaxDst - 1];
  long long      y_ld, y_col0;
  // Optional per-token output scale (fp32 activations arrive as scaled fp16 copies): output row m is
  // multiplied by tok_scale[m].  Readable up to the next multiple of 256 tokens.  nullptr: none.
  const float   *tok_scale;
};

// Bytes of split-tile scratch a device with `sm_count` SMs needs (partial tiles, then flags).
size_t gemm_scratch_bytes(int sm_count);

cudaError_t gemm_tcgen05_launch(const GemmArgs &args, int wt, int sm_count, cudaStream_t stream);

}  // namespace htp
