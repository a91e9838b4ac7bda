// Matmul over weights kept in the reference's 32 x 32 TILE ORDER, read in place (no repack):
//
//   * fp16 tiles - the weight format of hmx_mat_mul_permuted_w16a32 (reference
//     src/dsp/ops/mat_mul.c:758-855; the layout is written out by its host test,
//     src/host/test.c:303-313): tile (n/32, k/32) is tile number (n/32) * (K/32) + k/32, 1024
//     halfwords each; element (k, n) of the tile sits at halfword (k & ~1) * 32 + n * 2 + (k & 1),
//     i.e. 16 row-pairs of 128 bytes, each a run of 32 {k even, k odd} pairs, one per column.
//   * permuted super-blocks my_block_q4_0 (144 B) / my_block_q8_0 (272 B) (reference
//     include/dsp/quants.h:16-19, 28-31): 8 fp16 scales, then the quants of 256 consecutive
//     halfword SLOTS of the same tile order, four super-blocks per tile
//     (mat_mul.c:308-405 and :407-510 expand them slot by slot).  Slot t of a super-block is
//     k-row 2 * (t / 64) + (t & 1) of its eight k-rows and column (t % 64) / 2; its scale is
//     scales[t / 32] (the index tables at mat_mul.c:318-325), so one scale covers 2 k-rows x 16
//     columns.  Q8_0: slot t = (int8) quants[t].  Q4_0 / IQ4_NL: with s = t % 64, the slots of
//     k-row pairs 0..3 come from quants[2s] & 15, quants[2s+1] & 15, quants[2s] >> 4,
//     quants[2s+1] >> 4 (the 16-entry lookup sends even bytes to the first and odd bytes to the
//     second result vector, mat_mul.c:386-387, 402-405).
//
// The kernel is a streaming mat-vec: HBM-bound for a few tokens, which is the case the reference
// exercises (m = 1, test.c:281).  One CTA per 32 output columns (a cluster of up to 8 CTAs that
// split K when the matrix has few column tiles); its 16 warps walk the k-tiles of that column
// tile (contiguous bytes), every lane owning 4 columns and a share of the k-rows, so
// a warp-wide load instruction covers a contiguous 256..512-byte run.  Products and sums are
// fp32; nothing is rounded to fp16 (the reference rounds activations and outputs, the contract
// here is the exact dequantise-then-dot).  Partial sums meet in a fixed order (lane shuffles,
// warps in index order, then the cluster's CTAs in rank order through distributed shared
// memory): results do not depend on scheduling, and the kernel needs no scratch memory.
#include "tiled_weights.h"

#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include "unpack.cuh"

namespace cg = cooperative_groups;

namespace htp {

namespace {

constexpr int kWarps   = 16;
constexpr int kThreads = kWarps * 32;

// Two consecutive activations (idx even) as fp32.
template <bool A16>
__device__ __forceinline__ float2 ld_act2(const void *x, size_t idx) {
  if constexpr (A16) {
    return __half22float2(__ldg(reinterpret_cast<const __half2 *>(static_cast<const __half *>(x) + idx)));
  } else {
    return __ldg(reinterpret_cast<const float2 *>(static_cast<const float *>(x) + idx));
  }
}

// Eight consecutive activations (idx a multiple of 8) as fp32.
template <bool A16>
__device__ __forceinline__ void ld_act8(const void *x, size_t idx, float (&a)[8]) {
  if constexpr (A16) {
    const uint4 v = __ldg(reinterpret_cast<const uint4 *>(static_cast<const __half *>(x) + idx));
    const float2 p0 = __half22float2(u32_as_h2(v.x)), p1 = __half22float2(u32_as_h2(v.y));
    const float2 p2 = __half22float2(u32_as_h2(v.z)), p3 = __half22float2(u32_as_h2(v.w));
    a[0] = p0.x, a[1] = p0.y, a[2] = p1.x, a[3] = p1.y, a[4] = p2.x, a[5] = p2.y, a[6] = p3.x, a[7] = p3.y;
  } else {
    const float4 *p = reinterpret_cast<const float4 *>(static_cast<const float *>(x) + idx);
    const float4  u = __ldg(p), v = __ldg(p + 1);
    a[0] = u.x, a[1] = u.y, a[2] = u.z, a[3] = u.w, a[4] = v.x, a[5] = v.y, a[6] = v.z, a[7] = v.w;
  }
}

__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i) {
  return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}

// Four 4-bit table indices, one in the low nibble of each byte of `x`, gathered into the low 16
// bits (index of byte j in bits 4j .. 4j+3), the form iq4nl_lookup4 takes.
__device__ __forceinline__ uint32_t gather_nibbles(uint32_t x) {
  const uint32_t y = (x | (x >> 4)) & 0x00FF00FFu;
  return (y | (y >> 8)) & 0xFFFFu;
}

// 2^23 + byte j of x as an fp32 number: the byte lands in the low mantissa bits of 0x4B000000
// (2^23, whose unit in the last place is 1).  Subtracting 2^23 (+ the offset of the encoding) is
// exact.  One byte permute and one fp32 add on the full-rate pipes; an integer-to-float or
// half-to-float conversion instruction runs at a quarter of that rate, and with one conversion per
// weight that pipe, not HBM, set the pace of the 4- and 8-bit formats (ncu: 0.40 / 0.72 of the
// copy bandwidth).
__device__ __forceinline__ float biased_byte(uint32_t x, int j) {
  return __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7540u | (uint32_t) j));
}

// Eight consecutive slots of a Q8_0 super-block (one row pair, four columns) -> out[i] =
// {k even, k odd} of column i as exact fp32 integers.  Shared by the matmul and the integer probe.
__device__ __forceinline__ void decode_byte_pairs(uint2 q, float2 (&out)[4]) {
  const float2   nbias = make_float2(-(8388608.f + 128.f), -(8388608.f + 128.f));
  const uint32_t ux = q.x ^ 0x80808080u, uy = q.y ^ 0x80808080u;  // byte + 128 is unsigned
  out[0] = __fadd2_rn(make_float2(biased_byte(ux, 0), biased_byte(ux, 1)), nbias);
  out[1] = __fadd2_rn(make_float2(biased_byte(ux, 2), biased_byte(ux, 3)), nbias);
  out[2] = __fadd2_rn(make_float2(biased_byte(uy, 0), biased_byte(uy, 1)), nbias);
  out[3] = __fadd2_rn(make_float2(biased_byte(uy, 2), biased_byte(uy, 3)), nbias);
}

// One quant word of a 4-bit super-block (quants[4c .. 4c+3]: column c, all eight k-rows) -> out[v] =
// {k-row 2v, k-row 2v + 1} as exact fp32 integers.  Bytes B0..B3 of the word hold k-rows (0, 4)
// (2, 6) (1, 5) (3, 7) as (low, high) nibbles.  Shared by the matmul and the integer probe.
template <int FMT>
__device__ __forceinline__ void decode_nibble_word(uint32_t w, float2 (&out)[4]) {
  uint32_t lo = w & 0x0F0F0F0Fu, up = (w >> 4) & 0x0F0F0F0Fu;  // k-rows 0 2 1 3 / 4 6 5 7
  if constexpr (FMT == kTileIQ4) {
    lo = iq4nl_lookup4(gather_nibbles(lo)) ^ 0x80808080u;  // table bytes + 128
    up = iq4nl_lookup4(gather_nibbles(up)) ^ 0x80808080u;
  }
  const float  bias  = FMT == kTileIQ4 ? 8388608.f + 128.f : 8388608.f + 8.f;  // value = table byte / nibble - 8
  const float2 nbias = make_float2(-bias, -bias);
  out[0] = __fadd2_rn(make_float2(biased_byte(lo, 0), biased_byte(lo, 2)), nbias);
  out[1] = __fadd2_rn(make_float2(biased_byte(lo, 1), biased_byte(lo, 3)), nbias);
  out[2] = __fadd2_rn(make_float2(biased_byte(up, 0), biased_byte(up, 2)), nbias);
  out[3] = __fadd2_rn(make_float2(biased_byte(up, 1), biased_byte(up, 3)), nbias);
}

// Raw bytes one lane holds of one tile, per format.
template <int FMT>
struct LaneTile;
template <>
struct LaneTile<kTileF16> {
  uint4 q[4];  // load j: row-pair 4j + lane/8, columns 4 * (lane % 8) .. +3 as {k even, k odd} pairs
};
template <>
struct LaneTile<kTileQ8> {
  uint2  q[4];  // super-block sb: slots 8 * lane .. +7 = row-pair lane/8, columns 4 * (lane % 8) .. +3
  __half d[4];  // scales[lane / 4] of super-block sb
};
template <>
struct LaneTile<kTileQ4> {
  uint4 q;  // super-block lane/8, quants 16 * (lane % 8) .. +15: all 8 k-rows of columns 4 * (lane % 8) .. +3
  uint4 d;  // that super-block's eight scales
};
template <>
struct LaneTile<kTileIQ4> : LaneTile<kTileQ4> {};

template <int FMT>
__device__ __forceinline__ void load_tile(const uint8_t *tile, int lane, LaneTile<FMT> &t) {
  if constexpr (FMT == kTileF16) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      t.q[j] = __ldcs(reinterpret_cast<const uint4 *>(tile + j * 512 + lane * 16));
    }
  } else if constexpr (FMT == kTileQ8) {
#pragma unroll
    for (int sb = 0; sb < 4; ++sb) {
      t.q[sb] = __ldcs(reinterpret_cast<const uint2 *>(tile + sb * 272 + 16 + lane * 8));
      t.d[sb] = __ldg(reinterpret_cast<const __half *>(tile + sb * 272) + (lane >> 2));
    }
  } else {
    const uint8_t *sb = tile + (lane >> 3) * 144;
    t.q               = __ldcs(reinterpret_cast<const uint4 *>(sb + 16 + (lane & 7) * 16));
    t.d               = __ldg(reinterpret_cast<const uint4 *>(sb));
  }
}

// acc[mm][i] += { even k-rows, odd k-rows } of this lane's share of tile `kt`:
// x[token mm][k] * W[k][4 * (lane % 8) + i].  Weights and activations sit in registers as
// {k even, k odd} pairs, so every multiply-add is the packed two-lane fp32 instruction of sm_100
// (fma.rn.f32x2): half the instructions of scalar FMAs; the two halves are added once at the end.
template <int FMT, bool A16, int MT>
__device__ __forceinline__ void fma_tile(const LaneTile<FMT> &t, int kt, int lane, const void *x,
                                         const size_t (&xrow)[MT], float2 (&acc)[MT][4]) {
  if constexpr (FMT == kTileF16) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k0 = kt * 32 + 2 * (4 * j + (lane >> 3));
      float2    wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        wv[i] = __half22float2(u32_as_h2(word_of(t.q[j], i)));
      }
#pragma unroll
      for (int mm = 0; mm < MT; ++mm) {
        const float2 a = ld_act2<A16>(x, xrow[mm] + k0);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[mm][i] = __ffma2_rn(wv[i], a, acc[mm][i]);
        }
      }
    }
  } else if constexpr (FMT == kTileQ8) {
#pragma unroll
    for (int sb = 0; sb < 4; ++sb) {
      const int    k0 = kt * 32 + sb * 8 + 2 * (lane >> 3);
      const float  d  = __half2float(t.d[sb]);
      const float2 d2 = make_float2(d, d);
      float2       wv[4];  // {k even, k odd} of columns 0..3
      decode_byte_pairs(t.q[sb], wv);
#pragma unroll
      for (int mm = 0; mm < MT; ++mm) {
        // the scale goes onto the two activations, not onto the eight weights
        const float2 a = __fmul2_rn(ld_act2<A16>(x, xrow[mm] + k0), d2);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[mm][i] = __ffma2_rn(wv[i], a, acc[mm][i]);
        }
      }
    }
  } else {
    const int  k0 = kt * 32 + (lane >> 3) * 8;
    const bool hi = (lane & 7) >= 4;  // columns 16..31 use the odd scales
    float2     d2[4];                 // scale of k-rows 2v, 2v+1, twice
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const __half2 p = u32_as_h2(word_of(t.d, v));
      const float   d = hi ? __high2float(p) : __low2float(p);
      d2[v]           = make_float2(d, d);
    }
    float2 wv[4][4];  // [column][k-row pair] = {row 2v, row 2v + 1}, integer values
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      decode_nibble_word<FMT>(word_of(t.q, i), wv[i]);
    }
#pragma unroll
    for (int mm = 0; mm < MT; ++mm) {
      float a[8];
      ld_act8<A16>(x, xrow[mm] + k0, a);
      float2 a2[4];
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        a2[v] = __fmul2_rn(make_float2(a[2 * v], a[2 * v + 1]), d2[v]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          acc[mm][i] = __ffma2_rn(wv[i][v], a2[v], acc[mm][i]);
        }
      }
    }
  }
}

// Tiles a warp fetches before it starts on their arithmetic: enough bytes in flight per warp
// (2 to 4 KB) whatever the tile size.  Build-time knobs; measured on 32768 x 4096 fp16 tiles: 1 tile
// in flight 5.30 TB/s, 2 tiles 5.91 TB/s, 3 tiles 5.18 TB/s (each tile costs 16 registers per
// thread, and three push the kernel to two CTAs per SM); permuted Q4_0 65536 x 4096: 2 tiles 2.89,
// 3 tiles 2.83, 4 tiles 2.84 TB/s; permuted IQ4_NL: 2 tiles 1.63, 4 tiles 1.38 TB/s.
#ifndef HTP_TILE_F16_INFLIGHT
#define HTP_TILE_F16_INFLIGHT 2
#endif
#ifndef HTP_TILE_Q8_INFLIGHT
#define HTP_TILE_Q8_INFLIGHT 2
#endif
#ifndef HTP_TILE_Q4_INFLIGHT
#define HTP_TILE_Q4_INFLIGHT 2
#endif
#ifndef HTP_TILE_IQ4_INFLIGHT
#define HTP_TILE_IQ4_INFLIGHT 2
#endif
template <int FMT>
__host__ __device__ constexpr int tiles_in_flight() {
  return FMT == kTileF16 ? HTP_TILE_F16_INFLIGHT
                         : (FMT == kTileQ8 ? HTP_TILE_Q8_INFLIGHT
                                           : (FMT == kTileQ4 ? HTP_TILE_Q4_INFLIGHT : HTP_TILE_IQ4_INFLIGHT));
}

// grid = (N / 32, token groups, S).  S > 1: the launch is made of clusters of S CTAs along z that
// share one column tile and token group and split its k-tiles into S contiguous ranges; their
// partial sums meet in the first CTA through distributed shared memory, in rank order.
template <int FMT, bool A16, int MT>
__global__ void __launch_bounds__(kThreads)
    tiled_mul_mat_kernel(float *__restrict__ y, const void *__restrict__ x, const uint8_t *__restrict__ w, int M, int K,
                         int N) {
  __shared__ float red[kWarps][MT][32];
  __shared__ float part[MT][32];
  constexpr int    U    = tiles_in_flight<FMT>();
  const int        lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int        KT   = K >> 5;
  const int        nt   = blockIdx.x;
  const int        m0   = blockIdx.y * MT;
  const int        S    = gridDim.z, rank = blockIdx.z;
  const int        kt_begin = (int) ((long long) KT * rank / S), kt_end = (int) ((long long) KT * (rank + 1) / S);
  const uint8_t   *wt   = w + (size_t) nt * (size_t) KT * tile_bytes(FMT);

  size_t xrow[MT];  // first element of each token's activation row; tokens past M repeat the last
#pragma unroll
  for (int mm = 0; mm < MT; ++mm) {
    const int tok = m0 + mm < M ? m0 + mm : M - 1;
    xrow[mm]      = (size_t) tok * (size_t) K;
  }
  float2 acc[MT][4];  // {sum over even k-rows, sum over odd k-rows}
#pragma unroll
  for (int mm = 0; mm < MT; ++mm) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[mm][i] = make_float2(0.f, 0.f);
    }
  }

  for (int kt0 = kt_begin + warp * U; kt0 < kt_end; kt0 += kWarps * U) {
    LaneTile<FMT> t[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (kt0 + u < kt_end) {  // warp-uniform
        load_tile<FMT>(wt + (size_t) (kt0 + u) * tile_bytes(FMT), lane, t[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (kt0 + u < kt_end) {
        fma_tile<FMT, A16, MT>(t[u], kt0 + u, lane, x, xrow, acc);
      }
    }
  }

  // lanes l, l ^ 8, l ^ 16, l ^ 24 hold the same four columns over different k-rows
#pragma unroll
  for (int mm = 0; mm < MT; ++mm) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float v = acc[mm][i].x + acc[mm][i].y;
      v += __shfl_xor_sync(0xFFFFFFFFu, v, 8);
      v += __shfl_xor_sync(0xFFFFFFFFu, v, 16);
      if (lane < 8) {
        red[warp][mm][lane * 4 + i] = v;
      }
    }
  }
  __syncthreads();
  float s = 0.f;
  if (threadIdx.x < MT * 32) {  // MT * 32 <= 128 < kThreads: one output per thread
    const int mm = threadIdx.x >> 5, c = threadIdx.x & 31;
#pragma unroll
    for (int wi = 0; wi < kWarps; ++wi) {
      s += red[wi][mm][c];
    }
    part[mm][c] = s;
  }
  if (S > 1) {
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();  // every CTA's part[][] is written
    if (rank == 0 && threadIdx.x < MT * 32) {
      for (int r = 1; r < S; ++r) {
        const float *peer = cluster.map_shared_rank(&part[0][0], r);
        s += peer[threadIdx.x];
      }
    }
    cluster.sync();  // peers keep their shared memory until it has been read
    if (rank != 0) {
      return;
    }
  }
  if (threadIdx.x < MT * 32) {
    const int mm = threadIdx.x >> 5, c = threadIdx.x & 31;
    if (m0 + mm < M) {
      y[(size_t) (m0 + mm) * (size_t) N + (size_t) nt * 32 + c] = s;
    }
  }
}

// CTAs per cluster along K: enough CTAs to fill the GPU about three times over when the matrix has
// few column tiles, while every CTA keeps at least one round of tiles for each of its warps.
template <int FMT>
int k_split(int ctas, int KT, int sm_count) {
  int s = 1;
  while (s < 8 && ctas * s * 2 <= 3 * sm_count && KT / (s * 2) >= kWarps * tiles_in_flight<FMT>()) {
    s *= 2;
  }
  return s;
}

template <int FMT, bool A16, int MT>
cudaError_t launch_mt(float *y, const void *x, const uint8_t *w, int M, int K, int N, int sm_count,
                      cudaStream_t stream) {
  const int groups = (M + MT - 1) / MT;
  const int split  = k_split<FMT>((N / 32) * groups, K / 32, sm_count);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim          = dim3((unsigned) (N / 32), (unsigned) groups, (unsigned) split);
  cfg.blockDim         = dim3(kThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream           = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id               = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = (unsigned) split;
  cfg.attrs    = attr;
  cfg.numAttrs = split > 1 ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, tiled_mul_mat_kernel<FMT, A16, MT>, y, x, w, M, K, N);
}

template <int FMT, bool A16>
cudaError_t launch_fmt(float *y, const void *x, const uint8_t *w, int M, int K, int N, cudaStream_t stream) {
  int dev = 0, sm_count = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) {
    e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  if (e != cudaSuccess) {
    return e;
  }
  if (M == 1) {
    return launch_mt<FMT, A16, 1>(y, x, w, M, K, N, sm_count, stream);
  }
  if (M == 2) {
    return launch_mt<FMT, A16, 2>(y, x, w, M, K, N, sm_count, stream);
  }
  return launch_mt<FMT, A16, 4>(y, x, w, M, K, N, sm_count, stream);
}

// Integer probe of the super-block decode: for every scale group (32 consecutive slots of a
// super-block: 2 k-rows x 16 columns) S = sum_j q_j and T = sum_j (j + 1) q_j over its slots j in
// slot order, through the decode routines the matmul uses.  One warp per super-block.
template <int FMT>
__global__ void __launch_bounds__(256)
    tiled_group_sums_kernel(const uint8_t *__restrict__ w, int32_t *__restrict__ s, int32_t *__restrict__ t,
                            long long n_sb) {
  const long long sb   = (long long) blockIdx.x * 8 + (threadIdx.x >> 5);
  const int       lane = threadIdx.x & 31;
  if (sb >= n_sb) {  // warp-uniform
    return;
  }
  const uint8_t *blk = w + sb * (tile_bytes(FMT) / 4);
  float2         v[4];
  if constexpr (FMT == kTileQ8) {
    // slots 8 * lane .. +7: group lane / 4, first index in the group (8 * lane) % 32
    decode_byte_pairs(*reinterpret_cast<const uint2 *>(blk + 16 + lane * 8), v);
    int S = 0, T = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int a = __float2int_rn(v[i].x), b = __float2int_rn(v[i].y), j = ((8 * lane) & 31) + 2 * i;
      S += a + b;
      T += (j + 1) * a + (j + 2) * b;
    }
#pragma unroll
    for (int m = 1; m <= 2; m <<= 1) {
      S += __shfl_xor_sync(0xFFFFFFFFu, S, m);
      T += __shfl_xor_sync(0xFFFFFFFFu, T, m);
    }
    if ((lane & 3) == 0) {
      s[sb * 8 + (lane >> 2)] = S;
      t[sb * 8 + (lane >> 2)] = T;
    }
  } else {
    // word `lane` = column `lane`, k-row pairs 0..3: slot 64 * pair + 2 * lane + parity,
    // group 2 * pair + lane / 16, index in the group (2 * lane) % 32 + parity
    decode_nibble_word<FMT>(*reinterpret_cast<const uint32_t *>(blk + 16 + lane * 4), v);
    const int j = (2 * lane) & 31;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const int a = __float2int_rn(v[p].x), b = __float2int_rn(v[p].y);
      int       S = a + b, T = (j + 1) * a + (j + 2) * b;
#pragma unroll
      for (int m = 1; m <= 8; m <<= 1) {
        S += __shfl_xor_sync(0xFFFFFFFFu, S, m);
        T += __shfl_xor_sync(0xFFFFFFFFu, T, m);
      }
      if ((lane & 15) == 0) {
        s[sb * 8 + 2 * p + (lane >> 4)] = S;
        t[sb * 8 + 2 * p + (lane >> 4)] = T;
      }
    }
  }
}

template <int FMT>
cudaError_t launch_act(float *y, const void *x, const uint8_t *w, int M, int K, int N, bool a16, cudaStream_t stream) {
  return a16 ? launch_fmt<FMT, true>(y, x, w, M, K, N, stream) : launch_fmt<FMT, false>(y, x, w, M, K, N, stream);
}

}  // namespace

cudaError_t tiled_mul_mat_launch(float *y, const void *x, const uint8_t *w, int M, int K, int N, int fmt, bool a16,
                                 cudaStream_t stream) {
  if (M <= 0 || K <= 0 || N <= 0 || K % 32 != 0 || N % 32 != 0 || (M + 3) / 4 > 65535) {
    return cudaErrorInvalidValue;
  }
  switch (fmt) {
    case kTileF16: return launch_act<kTileF16>(y, x, w, M, K, N, a16, stream);
    case kTileQ4: return launch_act<kTileQ4>(y, x, w, M, K, N, a16, stream);
    case kTileQ8: return launch_act<kTileQ8>(y, x, w, M, K, N, a16, stream);
    case kTileIQ4: return launch_act<kTileIQ4>(y, x, w, M, K, N, a16, stream);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t tiled_group_sums_launch(const uint8_t *w, int32_t *s, int32_t *t, long long n_super_blocks, int fmt,
                                    cudaStream_t stream) {
  if (n_super_blocks <= 0) {
    return n_super_blocks == 0 ? cudaSuccess : cudaErrorInvalidValue;
  }
  const unsigned grid = (unsigned) ((n_super_blocks + 7) / 8);
  switch (fmt) {
    case kTileQ4: tiled_group_sums_kernel<kTileQ4><<<grid, 256, 0, stream>>>(w, s, t, n_super_blocks); break;
    case kTileQ8: tiled_group_sums_kernel<kTileQ8><<<grid, 256, 0, stream>>>(w, s, t, n_super_blocks); break;
    case kTileIQ4: tiled_group_sums_kernel<kTileIQ4><<<grid, 256, 0, stream>>>(w, s, t, n_super_blocks); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace htp
