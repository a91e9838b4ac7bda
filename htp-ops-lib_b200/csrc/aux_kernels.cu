// Two small kernels beside the main ones:
//   * mul_mat_generic - shape-agnostic quantised matmul for the shapes the streaming kernels do
//     not take (K not a multiple of 256, i.e. weight rows that are not 16-byte aligned).  One warp
//     per output row, 2-byte loads, fp32 arithmetic in dequantise-then-dot order
//     (reference semantics: src/dsp/ops/mat_mul.c:260-306).
//   * block_sums - integer probe of the unpack: S_b = sum_i v_i and T_b = sum_i (i+1) v_i for every
//     block, computed through the same unpack routines and element-order functions (unpack.cuh)
//     the matmul kernels use, so a wrong nibble order or sign shows up as an integer mismatch.
#include "aux_kernels.h"

#include <cuda_fp16.h>

#include "unpack.cuh"

namespace htp {

namespace {

__device__ __forceinline__ uint32_t ld_word_2b(const uint8_t *p) {  // p is 2-byte aligned
  const uint16_t *h = reinterpret_cast<const uint16_t *>(p);
  return (uint32_t) h[0] | ((uint32_t) h[1] << 16);
}

template <int WT>
__device__ __forceinline__ void unpack_block_values(const uint8_t *blk, float (&v)[32]) {
  if constexpr (WT == kQ4) {
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      uint32_t h[4];
      q4_0_unpack_word(ld_word_2b(blk + 2 + 4 * t), h);
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const __half2 p            = u32_as_h2(h[r]);
        v[q4_0_word_elem(t, r, 0)] = __low2float(p);
        v[q4_0_word_elem(t, r, 1)] = __high2float(p);
      }
    }
  } else {
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      uint32_t h[2];
      q8_0_unpack_word(ld_word_2b(blk + 2 + 4 * u), h);
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const __half2 p            = u32_as_h2(h[r]);
        v[q8_0_word_elem(u, r, 0)] = __low2float(p);
        v[q8_0_word_elem(u, r, 1)] = __high2float(p);
      }
    }
  }
}

template <int WT, bool A16>
__global__ void __launch_bounds__(256) mul_mat_generic_kernel(float *__restrict__ y, const void *__restrict__ x,
                                                              const uint8_t *__restrict__ w, int M, int K, int N) {
  constexpr int BB   = BlockTraits<WT>::kBytes;
  const int     lane = threadIdx.x & 31;
  const int     nb   = K / 32;
  const long long row = (long long) blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= N) {
    return;
  }
  const uint8_t *wrow = w + row * nb * BB;
  for (int m0 = 0; m0 < M; m0 += 8) {
    float acc[8] = { 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f };
    for (int b = lane; b < nb; b += 32) {
      const uint8_t *blk = wrow + (long long) b * BB;
      const float    d   = __half2float(*reinterpret_cast<const __half *>(blk));
      float          v[32];
      unpack_block_values<WT>(blk, v);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        v[i] *= d;  // dequantise ...
      }
      for (int mm = 0; mm < 8 && m0 + mm < M; ++mm) {
        float s = 0.f;
        if constexpr (A16) {
          const __half *xr = static_cast<const __half *>(x) + (long long) (m0 + mm) * K + b * 32;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            s = fmaf(__half2float(xr[i]), v[i], s);  // ... then dot
          }
        } else {
          const float *xr = static_cast<const float *>(x) + (long long) (m0 + mm) * K + b * 32;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            s = fmaf(xr[i], v[i], s);
          }
        }
        acc[mm] += s;
      }
    }
    for (int mm = 0; mm < 8 && m0 + mm < M; ++mm) {
      float s = acc[mm];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        s += __shfl_xor_sync(0xffffffffu, s, o);
      }
      if (lane == 0) {
        y[(long long) (m0 + mm) * N + row] = s;
      }
    }
  }
}

template <int WT>
__global__ void block_sums_kernel(const uint8_t *__restrict__ w, int32_t *__restrict__ s_out,
                                  int32_t *__restrict__ t_out, long long n_blocks) {
  constexpr int   BB = BlockTraits<WT>::kBytes;
  const long long b  = (long long) blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n_blocks) {
    return;
  }
  float v[32];
  unpack_block_values<WT>(w + b * BB, v);
  int s = 0, t = 0;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int q = __float2int_rn(v[i]);
    s += q;
    t += (i + 1) * q;
  }
  s_out[b] = s;
  t_out[b] = t;
}

}  // namespace

cudaError_t mul_mat_generic_launch(float *y, const void *x, const uint8_t *w, int M, int K, int N, int wt, bool a16,
                                   cudaStream_t stream) {
  const dim3 grid((N + 7) / 8), block(256);
  if (wt == kQ4) {
    if (a16) {
      mul_mat_generic_kernel<kQ4, true><<<grid, block, 0, stream>>>(y, x, w, M, K, N);
    } else {
      mul_mat_generic_kernel<kQ4, false><<<grid, block, 0, stream>>>(y, x, w, M, K, N);
    }
  } else {
    if (a16) {
      mul_mat_generic_kernel<kQ8, true><<<grid, block, 0, stream>>>(y, x, w, M, K, N);
    } else {
      mul_mat_generic_kernel<kQ8, false><<<grid, block, 0, stream>>>(y, x, w, M, K, N);
    }
  }
  return cudaGetLastError();
}

cudaError_t block_sums_launch(const uint8_t *w, int32_t *s, int32_t *t, long long n_blocks, int wt,
                              cudaStream_t stream) {
  if (n_blocks <= 0) {
    return cudaSuccess;
  }
  const int       threads = 256;
  const long long grid    = (n_blocks + threads - 1) / threads;
  if (wt == kQ4) {
    block_sums_kernel<kQ4><<<(unsigned) grid, threads, 0, stream>>>(w, s, t, n_blocks);
  } else {
    block_sums_kernel<kQ8><<<(unsigned) grid, threads, 0, stream>>>(w, s, t, n_blocks);
  }
  return cudaGetLastError();
}

}  // namespace htp
