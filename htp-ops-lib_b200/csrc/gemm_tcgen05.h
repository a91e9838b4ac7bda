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

struct GemmArgs {
  float         *y;  // [M][N] fp32
  const void    *x;  // [M][K] fp16
  const uint8_t *w;  // N rows of K/32 blocks
  int            M, N, K;  // K a multiple of 256, N a multiple of 32
  int           *err;      // first error code, 0 when none
  // Scratch for tiles whose K range is split between two workers (gemm_scratch_bytes() bytes at
  // `part`, 256-byte aligned, zero before the first launch; the flags are zero again after every
  // launch).  nullptr: tiles are never split.
  float         *part;
  int           *flags;  // set by the launcher
  int            split;  // set by the launcher
#ifdef HTP_GEMM_PROF
  int            dbg;      // instrumented builds only: bit mask of waits to skip (timing experiments)
#endif
};

// Bytes of split-tile scratch a device with `sm_count` SMs needs (partial tiles, then flags).
size_t gemm_scratch_bytes(int sm_count);

cudaError_t gemm_tcgen05_launch(const GemmArgs &args, int wt, int sm_count, cudaStream_t stream);

}  // namespace htp
