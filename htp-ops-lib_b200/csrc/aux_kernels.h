// Launchers of the shape-agnostic fallback matmul, the integer block-sum probe and RMSNorm
// (aux_kernels.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace htp {

cudaError_t mul_mat_generic_launch(float *y, const void *x, const uint8_t *w, int M, int K, int N, int wt, bool a16,
                                   cudaStream_t stream);

cudaError_t block_sums_launch(const uint8_t *w, int32_t *s, int32_t *t, long long n_blocks, int wt,
                              cudaStream_t stream);

// y[j][i] = x[j][i] / sqrt(mean_i(x[j][i]^2) + 1e-5) for ne1 rows of ne0 floats (rows 16-byte aligned
// when ne0 % 4 == 0, which selects the vector path).
// src[m][k] fp32 -> dst[m][k] fp16, every token scaled by its own power of two (largest magnitude into
// [2^14, 2^15)); inv_scale[token] undoes the scale on the outputs.  k % 4 == 0, rows 16-byte aligned.
cudaError_t act_f32_to_f16_launch(void *dst_f16, float *inv_scale, const float *src, int m, int k, cudaStream_t stream);

// Sums of K-range slabs: y[i] = sum over c < n_parts of part[c * count + i], i < count, in that order.
constexpr int kKSumMaxOps = 64;
struct KSumOp {
  float       *y;
  const float *part;
  long long    count;
  int          n_parts;
};
struct KSumArgs {
  KSumOp ops[kKSumMaxOps];
  int    n_ops;
};
cudaError_t k_range_sum_launch(const KSumArgs &args, cudaStream_t stream);

cudaError_t rms_norm_f32_launch(float *dst, const float *src, int ne0, int ne1, cudaStream_t stream);

}  // namespace htp
