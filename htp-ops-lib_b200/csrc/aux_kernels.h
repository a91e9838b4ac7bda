// Launchers of the shape-agnostic fallback matmul and the integer block-sum probe (aux_kernels.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace htp {

cudaError_t mul_mat_generic_launch(float *y, const void *x, const uint8_t *w, int M, int K, int N, int wt, bool a16,
                                   cudaStream_t stream);

cudaError_t block_sums_launch(const uint8_t *w, int32_t *s, int32_t *t, long long n_blocks, int wt,
                              cudaStream_t stream);

}  // namespace htp
