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
  } else if constexpr (WT == kIQ4) {
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      uint32_t r[2];
      iq4nl_unpack_word(ld_word_2b(blk + 2 + 4 * t), r[0], r[1]);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          v[iq4nl_word_elem(t, h, i)] = (float) (int8_t) (r[h] >> (8 * i));
        }
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
  } else if (wt == kIQ4) {
    if (a16) {
      mul_mat_generic_kernel<kIQ4, true><<<grid, block, 0, stream>>>(y, x, w, M, K, N);
    } else {
      mul_mat_generic_kernel<kIQ4, false><<<grid, block, 0, stream>>>(y, x, w, M, K, N);
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
  } else if (wt == kIQ4) {
    block_sums_kernel<kIQ4><<<(unsigned) grid, threads, 0, stream>>>(w, s, t, n_blocks);
  } else {
    block_sums_kernel<kQ8><<<(unsigned) grid, threads, 0, stream>>>(w, s, t, n_blocks);
  }
  return cudaGetLastError();
}

// ---------------------------------------------------------------- RMSNorm (fp32)
//
// Replaces the reference's hvx_rms_norm_f32 (src/dsp/ops/rms_norm.c:8-84; scalar statement
// src/host/test.c:60-80): per row, scale = 1 / sqrt(sum(x^2) / ne0 + 1e-5), y = x * scale.  HBM-bound:
// one CTA per row (grid-stride over rows), the row is read once into registers when it has at most
// kRmsRegElems elements (16-byte loads), otherwise read twice.  The sum of squares is added in a
// fixed order (per-thread strided partial sums, warp tree, then the warps in order), so results
// do not depend on the launch.
namespace {

constexpr int kRmsThreads  = 256;
constexpr int kRmsVecs     = 8;                               // float4 per thread kept in registers
constexpr int kRmsRegElems = kRmsThreads * kRmsVecs * 4;      // 8192
constexpr float kRmsEps    = 1e-5f;

__device__ __forceinline__ float rms_block_sum(float v, float *warp_sums) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    v += __shfl_xor_sync(0xffffffffu, v, o);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // warp_sums may still be read by the previous row
  if (lane == 0) {
    warp_sums[warp] = v;
  }
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int w = 0; w < kRmsThreads / 32; ++w) {
    s += warp_sums[w];
  }
  return s;
}

template <bool VEC>
__global__ void __launch_bounds__(kRmsThreads) rms_norm_f32_kernel(float *__restrict__ dst, const float *__restrict__ src,
                                                                  int ne0, int ne1) {
  __shared__ float warp_sums[kRmsThreads / 32];
  for (int row = blockIdx.x; row < ne1; row += gridDim.x) {
    const float *x = src + (long long) row * ne0;
    float       *y = dst + (long long) row * ne0;
    if constexpr (VEC) {
      // ne0 % 4 == 0 and ne0 <= kRmsRegElems: the row lives in registers between the two passes
      const int    nv = ne0 >> 2;
      const float4 *xv = reinterpret_cast<const float4 *>(x);
      float4       r[kRmsVecs];
      float        ss = 0.f;
#pragma unroll
      for (int j = 0; j < kRmsVecs; ++j) {
        const int i = threadIdx.x + j * kRmsThreads;
        r[j]        = i < nv ? __ldcs(xv + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        ss += r[j].x * r[j].x + r[j].y * r[j].y + r[j].z * r[j].z + r[j].w * r[j].w;
      }
      const float sum   = rms_block_sum(ss, warp_sums);
      const float scale = 1.0f / sqrtf(sum / (float) ne0 + kRmsEps);
      float4     *yv    = reinterpret_cast<float4 *>(y);
#pragma unroll
      for (int j = 0; j < kRmsVecs; ++j) {
        const int i = threadIdx.x + j * kRmsThreads;
        if (i < nv) {
          __stcs(yv + i, make_float4(r[j].x * scale, r[j].y * scale, r[j].z * scale, r[j].w * scale));
        }
      }
    } else {
      float ss = 0.f;
      for (int i = threadIdx.x; i < ne0; i += kRmsThreads) {
        const float v = x[i];
        ss += v * v;
      }
      const float sum   = rms_block_sum(ss, warp_sums);
      const float scale = 1.0f / sqrtf(sum / (float) ne0 + kRmsEps);
      for (int i = threadIdx.x; i < ne0; i += kRmsThreads) {
        y[i] = x[i] * scale;
      }
    }
  }
}

// fp32 activations -> fp16 for the tensor-core GEMM, one CTA per token.  The token is scaled by a
// power of two that puts its largest magnitude into [2^14, 2^15) - no overflow for large inputs, no
// loss to subnormals for small ones - and the inverse of that scale is kept per token for the
// GEMM's epilogue.  (The reference converts its fp32 activations to fp16 as they are,
// src/dsp/ops/mat_mul.c:89-128.)
__global__ void __launch_bounds__(256) act_f32_to_f16_kernel(__half *dst, float *inv_scale, const float *src, int k) {
  __shared__ float red[8];
  const int        m   = blockIdx.x;
  const float     *x   = src + (size_t) m * k;
  __half          *y   = dst + (size_t) m * k;
  float            a   = 0.f;
  for (int i = threadIdx.x; i < k / 4; i += 256) {
    const float4 v = reinterpret_cast<const float4 *>(x)[i];
    a              = fmaxf(a, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
  }
  if ((threadIdx.x & 31) == 0) {
    red[threadIdx.x >> 5] = a;
  }
  __syncthreads();
  a = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) {
    a = fmaxf(a, red[i]);
  }
  int sh = ((__float_as_int(a) >> 23) & 0xff) - 127 - 14;  // floor(log2(amax)) - 14
  sh     = a == 0.f ? 0 : (sh < -100 ? -100 : (sh > 100 ? 100 : sh));
  const float s = __int_as_float((127 - sh) << 23);
  if (threadIdx.x == 0) {
    inv_scale[m] = __int_as_float((127 + sh) << 23);
  }
  for (int i = threadIdx.x; i < k / 4; i += 256) {
    const float4 v = reinterpret_cast<const float4 *>(x)[i];
    const __half2 lo = __floats2half2_rn(v.x * s, v.y * s), hi = __floats2half2_rn(v.z * s, v.w * s);
    uint2         o;
    o.x = *reinterpret_cast<const uint32_t *>(&lo);
    o.y = *reinterpret_cast<const uint32_t *>(&hi);
    reinterpret_cast<uint2 *>(y)[i] = o;
  }
}

// y[i] = part[0][i] + part[1][i] + ... (fixed order) for up to kKSumMaxOps outputs at once: the K
// ranges of a batched mat-vec whose activation fragments do not fit one launch each write their own
// slab, this adds them.  blockIdx.y = output, blockIdx.x strides over its elements.
__global__ void __launch_bounds__(256) k_range_sum_kernel(const __grid_constant__ KSumArgs a) {
  const KSumOp &op = a.ops[blockIdx.y];
  for (long long i = (long long) blockIdx.x * 256 + threadIdx.x; i < op.count; i += (long long) gridDim.x * 256) {
    float v = op.part[i];
    for (int c = 1; c < op.n_parts; ++c) {
      v += op.part[(long long) c * op.count + i];
    }
    op.y[i] = v;
  }
}

}  // namespace

cudaError_t k_range_sum_launch(const KSumArgs &args, cudaStream_t stream) {
  long long most = 0;
  for (int i = 0; i < args.n_ops; ++i) {
    most = args.ops[i].count > most ? args.ops[i].count : most;
  }
  const int bx = (int) ((most + 2047) / 2048 < 1 ? 1 : ((most + 2047) / 2048 > 64 ? 64 : (most + 2047) / 2048));
  k_range_sum_kernel<<<dim3(bx, args.n_ops), 256, 0, stream>>>(args);
  return cudaGetLastError();
}

cudaError_t act_f32_to_f16_launch(void *dst_f16, float *inv_scale, const float *src, int m, int k,
                                  cudaStream_t stream) {
  act_f32_to_f16_kernel<<<m, 256, 0, stream>>>(static_cast<__half *>(dst_f16), inv_scale, src, k);
  return cudaGetLastError();
}

cudaError_t rms_norm_f32_launch(float *dst, const float *src, int ne0, int ne1, cudaStream_t stream) {
  const bool vec  = (ne0 % 4 == 0) && ne0 <= kRmsRegElems;
  const int  grid = ne1 < 148 * 8 ? ne1 : 148 * 8;  // up to eight resident CTAs per SM, rows strided over them
  if (vec) {
    rms_norm_f32_kernel<true><<<grid, kRmsThreads, 0, stream>>>(dst, src, ne0, ne1);
  } else {
    rms_norm_f32_kernel<false><<<grid, kRmsThreads, 0, stream>>>(dst, src, ne0, ne1);
  }
  return cudaGetLastError();
}

}  // namespace htp
