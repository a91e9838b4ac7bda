// Per-device state shared by the compute entry points: SM count and, per stream, the small
// scratch area the mat-vec kernel finishes boundary tiles through.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace htp {

struct StreamScratch {
  float    *partials = nullptr;  // [kGemvMaxGrid][2][256]
  unsigned *counters = nullptr;  // [kGemvMaxGrid], zero between launches
  int      *err      = nullptr;  // first kernel error code
  int      *err_host = nullptr;  // pinned host word the error code is copied to when the stream is waited for
  float    *gemm_part = nullptr;  // split-tile scratch of the prefill GEMM, allocated on its first use
  uint8_t  *act16     = nullptr;  // fp16 copies of fp32 activations for the GEMM + their per-token scales
  size_t    act16_bytes = 0;
  uint8_t  *kslab      = nullptr;  // partial outputs of the K ranges of batched mat-vecs, summed afterwards
  size_t    kslab_bytes = 0;
};

struct DeviceCtx {
  int device   = -1;
  int sm_count = 0;
  int max_smem = 0;
};

// Context of the current device (created on first use).  nullptr when no device is usable.
DeviceCtx *current_device_ctx();

// Scratch bound to (current device, stream); allocated on first use.  nullptr on failure.
StreamScratch *stream_scratch(DeviceCtx *ctx, cudaStream_t stream);

// Frees every scratch area (used at session close).
void release_all_scratch();

// The checked matmul behind htp_b200_mul_mat.  allow_pdl = false forces plain stream ordering for
// this launch (needed when the weight buffer may still be written by earlier work on the stream).
int mul_mat_checked(void *dst, const void *activation, const void *weight, int m, int k, int n, int weight_type,
                    int act_type, cudaStream_t stream, bool allow_pdl);

// Several independent mat-vecs of one kind (same weight format, activation type and token count
// m <= 8) in one persistent launch.  The caller guarantees that no operator reads what another one
// of the batch writes.
struct MatMulDesc {
  float         *y;
  const void    *x;
  const uint8_t *w;
  int            k, n;
};
bool mul_mat_batchable(int m, int k, int n, int weight_type, int act_type);
int  mul_mat_batch_checked(const MatMulDesc *d, int n_ops, int m, int weight_type, int act_type, cudaStream_t stream,
                           bool allow_pdl);

extern int      g_opt_pdl;
extern int      g_opt_force_generic;
extern int      g_opt_gemm_min_m;
extern int      g_opt_gemm_tile_n;
extern int      g_opt_gemm_split;
extern int      g_opt_gemv_whole_tiles;
extern int      g_opt_permuted_weights;
extern int      g_opt_a32_exact;
void            count_launch(int n = 1);

}  // namespace htp
