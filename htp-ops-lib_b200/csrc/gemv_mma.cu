// K1 - decode-side quantised mat-vec (M <= 8 tokens): y[M][N] = x[M][K] . W[N][K]^T.
//
// Replaces the reference's DMA -> HVX dequantise -> HMX tile -> store schedule
// (src/dsp/ops/mat_mul.c:928-1005) for small M.  The kernel is HBM-bound by design:
//
//   * One persistent CTA per SM.  The work is the list of (32-row tile, 1024-weight K stage)
//     items in tile-major order; CTA c owns the contiguous item range [T c / G, T (c+1) / G), so
//     every SM streams the same number of bytes whatever N is.  A tile cut by a range boundary is
//     finished through a small scratch area: each part is written in a fixed slot, the last CTA to
//     arrive adds the parts in ascending order (bit-reproducible, no floating-point atomics).
//   * A producer thread streams the raw 18-/34-byte blocks with ONE tiled TMA copy per stage
//     (32 rows x one stage of blocks, through a tensor map over the weight bytes) into a
//     shared-memory ring (mbarrier full/empty pairs, L2 evict-first).  The box is 16 bytes wider
//     than a stage, which makes the shared-memory row pitch an odd multiple of 16 bytes: the
//     fragment reads below are bank-conflict-free, and the 16 extra bytes are simply the start of
//     the next stage (zero fill past the end of the row).
//   * Sixteen consumer warps split a stage along K.  Quants stay INTEGERS: a lane turns one 32-bit
//     word of nibbles/bytes into fp16 pairs (unpack.cuh) that are the A fragment of a warp MMA
//     (m16n8k16, fp32 accumulate) whose B fragment holds the activations.  The block scale is
//     applied to the 32-weight partial sum in fp32, i.e. sum_k (q_k x_k) * d - the same value as
//     dequantise-then-dot, without rounding q*d to fp16.
//   * fp32 activations are split as x = hi + lo with hi = fp16(x), lo = fp16(x - hi), so the
//     product is exact to ~2^-22; hi and lo occupy separate MMA columns (M <= 4) or two chained
//     MMAs (M <= 8).  Each token is normalised by a power of two first (undone on output).
//   * The activation fragments for the whole K range live in shared memory, built once per CTA.
//   * Programmatic dependent launch: the weight prefetch starts before the previous kernel in
//     the stream has finished; activations are read, and outputs written, only after it has.
//
// Every mbarrier wait is bounded; a wait that runs out stores an error code and the CTA leaves.
#include "gemv_mma.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstring>
#include <functional>
#include <mutex>
#include <unordered_map>

#include "ptx.cuh"
#include "unpack.cuh"

namespace htp {

namespace {

constexpr int kConsumerWarps   = 16;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kReduceWarp0     = kConsumerWarps + 1;  // two warps finish the tiles, one per 16-row group
constexpr int kReduceThreads   = 64;
constexpr int kThreads         = kConsumerThreads + 32 + kReduceThreads;

template <int WT, bool A16, int MPAD>
struct Cfg {
  static constexpr int  BB       = BlockTraits<WT>::kBytes;
  // Three to eight tokens (MPAD = 8), every weight format: the WIDE integer path.  A token, scaled by
  // a power of two, is the 23-bit fixed-point integer D2 * 2^16 + D1 * 2^8 + D0 with signed
  // base-256 digits; MMA number d of a block multiplies the weights by digit d of all eight tokens
  // (MMA column = token), so the three results of one (row, token) pair sit in the same lane.
  static constexpr bool WIDE     = MPAD == 8;
  // Q4_0 / IQ4_NL with one or two tokens run on the INTEGER tensor-core path too: nibbles are
  // masked into unsigned bytes (3 instructions per 8 weights instead of 9 for exact fp16), the
  // activations are four signed base-256 digits of a 31-bit fixed-point value (column = 4 m +
  // digit), one m16n8k32 MMA covers a whole block, and the -8 offset of the format comes out with
  // the float bias of the integer result.
  static constexpr bool I8       = WIDE || ((WT == kQ4 || WT == kIQ4) && MPAD <= 2);
  static constexpr bool DIGCOL   = I8 && !WIDE;  // MMA column = 4 m + digit
  static_assert(MPAD == 1 || MPAD == 2 || MPAD == 8, "token paddings built: 1, 2, 8");
  static constexpr int  NC       = WIDE ? 8 : (I8 ? 4 * MPAD : (A16 ? MPAD : 2 * MPAD));  // MMA columns in use
  static constexpr bool SPLITCOL = !I8 && !A16;                                         // column = 2 m + piece
  static constexpr int  SB       = gemv_stage_blocks(WT);  // blocks per stage and row
  static constexpr int  BPW      = SB / kConsumerWarps;          // blocks per consumer warp and stage
  static_assert(BPW >= 1 && BPW * kConsumerWarps == SB, "a stage splits evenly over the consumer warps");
  static constexpr int  PSTRIDE  = gemv_row_pitch(WT);
  static constexpr int  STAGE    = kGemvTileRows * PSTRIDE;
  // uint2 entries per block: two k-steps of fp16 fragments, or one int8 fragment per column and lane
  // position (per MMA) followed by the columns' accumulator inputs (one int each)
  // (the wide path needs no offsets: its Q4_0 nibbles go in as signed bytes 16 (q - 8))
  static constexpr int  FRAG_U2  = WIDE ? 3 * 32 : (I8 ? NC * 4 + NC / 2 : 2 * NC * 4);
  static constexpr int  CIN_OFF  = NC * 4;  // where a block's offsets start (one or two tokens)
  // Copies of the cross-warp reduction buffer: two, so that a tile is handed over while the one before
  // is still being added up; the wide path gives the second copy's 16 KB to the pipeline (a third
  // stage at K = 4096) - its tiles are far enough apart.
  static constexpr int  RED_BUFS = WIDE ? 1 : 2;
  static constexpr int  HEADER   = gemv_header_bytes(MPAD);
};

struct Smem {
  uint64_t full[kGemvMaxStages];
  uint64_t empty[kGemvMaxStages];
  float    tok_scale[8];
  float    tok_inv[8];
  int      tok_amax_bits[8];
  int      last_flag;
  int      abort_flag;
  int      pad[6];
  // Tile completion runs on two warps of its own: the consumer warps drop their partial sums of a
  // tile into red[n & 1] and carry on; red_full counts the 16 warps in, red_empty tells them the
  // copy has been read.
  uint64_t red_full[2];
  uint64_t red_empty[2];
  uint64_t op_bar;  // batched launch: the consumer warps meet here before an operator's activations replace the last one's
  uint8_t  pad2[88];
  // finished tile [token][row] of a launch with several destinations: staged here so that the copies
  // leave as 16-byte stores, 128 contiguous bytes per token and destination
  float    out_tile[8][kGemvTileRows];
  // (last: a path that uses one copy only starts its fragments where the second copy would be)
  float    red[2][kConsumerWarps][256];
};
static_assert(sizeof(Smem) % 128 == 0, "keep the regions after the header 128-byte aligned");
static_assert(sizeof(Smem) == gemv_header_bytes(1) && sizeof(Smem) - sizeof(float) * kConsumerWarps * 256 == gemv_header_bytes(8),
              "host-side size computation must match");

__device__ __forceinline__ void record_error(const GemvArgs &p, int code) {
  atomicCAS(p.err, 0, code);
}

__device__ __forceinline__ uint32_t lds32(const uint8_t *p) {
  return *reinterpret_cast<const uint32_t *>(p);
}
__device__ __forceinline__ float lds_scale(const uint8_t *p) {
  return __half2float(*reinterpret_cast<const __half *>(p));
}

// owner CTA of item i when T items are dealt to G CTAs as [T c / G, T (c+1) / G)
__device__ __forceinline__ long long item_owner(long long i, long long T, long long G) {
  return ((i + 1) * G - 1) / T;
}

// ------------------------------------------------------------------ activation fragments

// float 12582912 = 2^23 + 2^22: added to an integer |v| < 2^22 in the integer domain, the bit
// pattern is the float 12582912 + v exactly
constexpr int   kMagicBits = 0x4B400000;
constexpr float kMagic     = 12582912.0f;

// Integer paths.  Token m, scaled by a power of two so that |x| < 1, becomes a fixed-point integer
// that is split into signed base-256 digits, one MMA column each:
//   one or two tokens (Q4_0, IQ4_NL):  X = round(x * 2^30) = D3 * 2^24 + D2 * 2^16 + D1 * 2^8 + D0,
//     column = 4 m + digit;
//   wide path (three to eight tokens, every format):  X = round(x * 2^22) = D2 * 2^16 + D1 * 2^8 + D0,
//     MMA number d of a block = digit d of the eight tokens (column = token), so the three results
//     of one (row, token) pair sit in the same lane.
// D0 .. are in [-128, 127], the top digit within [-65, 65].  The digits are simply the bytes of
// (X + 0x8080..) ^ 0x8080..: adding 128 per lower digit makes the lower bytes unsigned digits + 128
// with the carries where they belong, the xor takes the 128 off again as a signed byte.
// The MMA starts from the integer kMagicBits in every accumulator, so its int32 result is the bit
// pattern of the float 12582912 + sum_k q_k D_k exactly; per block and column the fragments carry
// the float offset -12582912 - 8 * sum_k D (Q4_0: value = nibble - 8) that one packed add removes.
// The rounding of x - at most 2^-31 (2^-23 on the wide path) of the power of two above the token's
// largest magnitude per element - is the only inexact step.
constexpr int kWideShift   = 22;
constexpr int kNarrowShift = 30;

// Elements k0 .. k0 + 3 and k0 + 16 .. k0 + 19 of token m as floats (two 16- or 8-byte loads).
template <bool A16>
__device__ __forceinline__ void load_x8(const GemvArgs &p, int m, int k0, float (&v)[8]) {
  const long long i = (long long) m * p.x_stride + p.x_k_off + k0;
  if constexpr (A16) {
    const __half *x = static_cast<const __half *>(p.x) + i;
    const uint2   a = *reinterpret_cast<const uint2 *>(x), b = *reinterpret_cast<const uint2 *>(x + 16);
    const float2  a0 = __half22float2(u32_as_h2(a.x)), a1 = __half22float2(u32_as_h2(a.y));
    const float2  b0 = __half22float2(u32_as_h2(b.x)), b1 = __half22float2(u32_as_h2(b.y));
    v[0] = a0.x, v[1] = a0.y, v[2] = a1.x, v[3] = a1.y, v[4] = b0.x, v[5] = b0.y, v[6] = b1.x, v[7] = b1.y;
  } else {
    const float *x = static_cast<const float *>(p.x) + i;
    const float4 a = *reinterpret_cast<const float4 *>(x), b = *reinterpret_cast<const float4 *>(x + 16);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
  }
}

// Per-token largest magnitude over the launch's K range -> tok_amax_bits (16-byte loads, every
// token's loads independent of the others').
template <bool A16>
__device__ __forceinline__ void token_amax(const GemvArgs &p, Smem *sm, int tid) {
  if (tid < 8) {
    sm->tok_amax_bits[tid] = 0;
  }
  named_bar_sync(1, kConsumerThreads);
  const int nvec = p.kblocks * 32 / (A16 ? 8 : 4);  // 16-byte pieces per token
  float     amax[8];
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    amax[m] = 0.f;
    if (m < p.M) {
      for (int c = tid; c < nvec; c += kConsumerThreads) {
        const long long i = (long long) m * p.x_stride + p.x_k_off;
        if constexpr (A16) {
          const uint4 q = *reinterpret_cast<const uint4 *>(static_cast<const __half *>(p.x) + i + 8 * c);
          __half2     h = __hmax2(__habs2(u32_as_h2(q.x)), __habs2(u32_as_h2(q.y)));
          h             = __hmax2(h, __hmax2(__habs2(u32_as_h2(q.z)), __habs2(u32_as_h2(q.w))));
          amax[m]       = fmaxf(amax[m], fmaxf(__low2float(h), __high2float(h)));
        } else {
          const float4 q = *reinterpret_cast<const float4 *>(static_cast<const float *>(p.x) + i + 4 * c);
          amax[m] = fmaxf(amax[m], fmaxf(fmaxf(fabsf(q.x), fabsf(q.y)), fmaxf(fabsf(q.z), fabsf(q.w))));
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    if (m < p.M) {  // (uniform over the block)
      float a = amax[m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
      }
      if ((tid & 31) == 0) {
        atomicMax(&sm->tok_amax_bits[m], __float_as_int(a));
      }
    }
  }
  named_bar_sync(1, kConsumerThreads);
}

template <int WT, bool A16, int MPAD>
__device__ void build_x_frags_int(const GemvArgs &p, Smem *sm, uint2 *frags, int tid) {
  using C = Cfg<WT, A16, MPAD>;
  constexpr int      ND    = C::WIDE ? 3 : 4;                       // digits per token
  constexpr int      SHIFT = C::WIDE ? kWideShift : kNarrowShift;  // fixed-point position
  constexpr int      NTOK  = C::WIDE ? 8 : MPAD;
  constexpr uint32_t BIAS  = C::WIDE ? 0x00008080u : 0x00808080u;  // 128 per digit below the top one
  token_amax<A16>(p, sm, tid);
  if (tid < 8) {
    const int bits = sm->tok_amax_bits[tid];
    int       sh   = ((bits >> 23) & 0xff) - 127 + 1;  // amax < 2^sh
    sh             = sh < -90 ? -90 : (sh > 90 ? 90 : sh);
    sm->tok_scale[tid] = __int_as_float((127 + SHIFT - sh) << 23);  // x -> fixed point
    // wide path: the digit weights 256^d are applied as they are, the common 2^-22 here - and 2^-4
    // for Q4_0, whose nibbles go into the MMA as 16 (q - 8)
    sm->tok_inv[tid]   = __int_as_float((127 + sh - (C::WIDE ? SHIFT + (WT == kQ4 ? 4 : 0) : 0)) << 23);
  }
  named_bar_sync(1, kConsumerThreads);

  const int n_units = p.kblocks * 4;  // (block, t): a multiple of 32, so warps stay whole
  for (int u = tid; u < n_units; u += kConsumerThreads) {
    const int b = u >> 2, t = u & 3;
    uint2    *dst = frags + (size_t) b * C::FRAG_U2;
    // this lane position multiplies block elements 4t .. 4t+3 and 16+4t .. 19+4t of every token;
    // the loads of (up to) four tokens are in flight together
    constexpr int TG = NTOK < 4 ? NTOK : 4;
#pragma unroll 1
    for (int m0 = 0; m0 < NTOK; m0 += TG) {
      float xv[TG][8];
#pragma unroll
      for (int j = 0; j < TG; ++j) {
        if (m0 + j < p.M) {
          load_x8<A16>(p, m0 + j, b * 32 + 4 * t, xv[j]);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            xv[j][i] = 0.f;
          }
        }
      }
#pragma unroll
      for (int j = 0; j < TG; ++j) {
        const int   m  = m0 + j;
        const float sc = sm->tok_scale[m];
        // y[h][i]: the digits of the element that byte i of A register h (rows g / g + 8) of this
        // lane position multiplies - block element 16 h + 4 t + i (Q4_0, Q8_0) or
        // iq4nl_word_elem(t, h, i) = 4 t + 2 h + (i >> 1) + 16 (i & 1) - one digit per byte
        uint32_t y[2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int src = WT == kIQ4 ? 4 * (i & 1) + 2 * h + (i >> 1) : 4 * h + i;
            y[h][i]       = ((uint32_t) __float2int_rn(xv[j][src] * sc) + BIAS) ^ BIAS;
          }
        }
#pragma unroll
        for (int d = 0; d < ND; ++d) {
          // byte d of the four elements of each register, in element order
          uint32_t w[2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t lo = __byte_perm(y[h][0], y[h][1], 0x0040 + 0x0011 * d);  // bytes d of elements 0, 1
            const uint32_t hi = __byte_perm(y[h][2], y[h][3], 0x0040 + 0x0011 * d);  // bytes d of elements 2, 3
            w[h]              = __byte_perm(lo, hi, 0x5410);
          }
          const int col    = C::WIDE ? 8 * d + m : 4 * m + d;
          dst[col * 4 + t] = make_uint2(w[0], w[1]);
          if constexpr (!C::WIDE) {
            int sd = __dp4a((int) w[0], 0x01010101, __dp4a((int) w[1], 0x01010101, 0));  // sum of the 8 digits
            sd += __shfl_xor_sync(0xffffffffu, sd, 1);
            sd += __shfl_xor_sync(0xffffffffu, sd, 2);
            if (t == 0) {
              // (Q4_0: value = nibble - 8; IQ4_NL bytes are the values themselves)
              reinterpret_cast<float *>(dst + C::CIN_OFF)[col] = -kMagic - (WT == kQ4 ? 8.f * (float) sd : 0.f);
            }
          }
        }
      }
    }
  }
}

template <int WT, bool A16, int MPAD>
__device__ void build_x_frags(const GemvArgs &p, Smem *sm, uint2 *frags, int tid) {
  using C = Cfg<WT, A16, MPAD>;
  if constexpr (C::I8) {
    build_x_frags_int<WT, A16, MPAD>(p, sm, frags, tid);
    return;
  }
  if constexpr (!A16) {
    // per-token power-of-two normalisation: the largest |x| of a token lands in [2^14, 2^15), so
    // fp16(x) neither overflows nor drops into the subnormal range for small-magnitude tokens
    token_amax<false>(p, sm, tid);
    if (tid < 8) {
      const int bits = sm->tok_amax_bits[tid];
      const int e    = ((bits >> 23) & 0xff) - 127;  // floor(log2(amax))
      int       sh   = e - 14;
      sh             = sh < -100 ? -100 : (sh > 100 ? 100 : sh);
      sm->tok_scale[tid] = __int_as_float((127 - sh) << 23);
      sm->tok_inv[tid]   = __int_as_float((127 + sh) << 23);
    }
    named_bar_sync(1, kConsumerThreads);
  }

  const int n_units = p.kblocks * 8;  // (block, mma j, t)
  for (int u = tid; u < n_units; u += kConsumerThreads) {
    const int b = u >> 3, j = (u >> 2) & 1, t = u & 3;
    // the four activations this lane position multiplies: block elements
    // mma_frag_elem(j, t, hi, s) for (hi, s) in {0,1}^2; they always lie in one aligned group of 4
    const int e00 = mma_frag_elem<WT>(j, t, 0, 0);
    const int k0  = b * 32 + (e00 & ~3);
    const int i00 = e00 & 3;
    const int i01 = mma_frag_elem<WT>(j, t, 0, 1) & 3;
    const int i10 = mma_frag_elem<WT>(j, t, 1, 0) & 3;
    const int i11 = mma_frag_elem<WT>(j, t, 1, 1) & 3;
    uint2    *dst = frags + (size_t) (b * 2 + j) * C::NC * 4;
    for (int m = 0; m < MPAD; ++m) {
      if constexpr (A16) {
        __half v[4] = { __half(0.f), __half(0.f), __half(0.f), __half(0.f) };
        if (m < p.M) {
          const __half *x = static_cast<const __half *>(p.x) + (long long) m * p.x_stride + p.x_k_off + k0;
          const uint2   r = *reinterpret_cast<const uint2 *>(x);
          *reinterpret_cast<uint2 *>(v) = r;
        }
        uint2 f;
        f.x = h2_as_u32(__halves2half2(v[i00], v[i01]));
        f.y = h2_as_u32(__halves2half2(v[i10], v[i11]));
        dst[m * 4 + t] = f;
      } else {
        float v[4] = { 0.f, 0.f, 0.f, 0.f };
        if (m < p.M) {
          const float *x = static_cast<const float *>(p.x) + (long long) m * p.x_stride + p.x_k_off + k0;
          const float4 r = *reinterpret_cast<const float4 *>(x);
          const float  s = sm->tok_scale[m];
          v[0] = r.x * s, v[1] = r.y * s, v[2] = r.z * s, v[3] = r.w * s;
        }
        __half hi[4], lo[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          hi[i] = __float2half_rn(v[i]);
          lo[i] = __float2half_rn(v[i] - __half2float(hi[i]));
        }
        uint2 fh, fl;
        fh.x = h2_as_u32(__halves2half2(hi[i00], hi[i01]));
        fh.y = h2_as_u32(__halves2half2(hi[i10], hi[i11]));
        fl.x = h2_as_u32(__halves2half2(lo[i00], lo[i01]));
        fl.y = h2_as_u32(__halves2half2(lo[i10], lo[i11]));
        dst[(2 * m) * 4 + t]     = fh;
        dst[(2 * m + 1) * 4 + t] = fl;
      }
    }
  }
}

// ------------------------------------------------------------------ one block x 16 rows

template <int WT, bool A16, int MPAD, bool EVEN>
__device__ __forceinline__ void block_rows16(const uint8_t *ra, const uint2 (&bf)[2], int t, float (&acc)[4]) {
  using C = Cfg<WT, A16, MPAD>;
  // ra: this lane's row g of the 16-row group, at the block's first byte; row g+8 is 8 pitches on
  const uint8_t *rb = ra + 8 * C::PSTRIDE;
  uint32_t       a0[4], a1[4];  // A fragments of MMA 0 and 1: {row g lo, row g+8 lo, row g hi, row g+8 hi}
  if constexpr (WT == kQ4) {
    uint32_t qa, qb;
    if constexpr (EVEN) {  // quants start 2 bytes past a word boundary
      qa = __byte_perm(lds32(ra + 4 * t), lds32(ra + 4 * t + 4), 0x5432);
      qb = __byte_perm(lds32(rb + 4 * t), lds32(rb + 4 * t + 4), 0x5432);
    } else {  // block starts 2 bytes past a word boundary, quants are word aligned
      qa = lds32(ra + 2 + 4 * t);
      qb = lds32(rb + 2 + 4 * t);
    }
    uint32_t ha[4], hb[4];
    q4_0_unpack_word(qa, ha);
    q4_0_unpack_word(qb, hb);
    a0[0] = ha[0], a0[1] = hb[0], a0[2] = ha[1], a0[3] = hb[1];
    a1[0] = ha[2], a1[1] = hb[2], a1[2] = ha[3], a1[3] = hb[3];
  } else {
    uint32_t qa0, qa1, qb0, qb1;
    if constexpr (EVEN) {
      qa0 = __byte_perm(lds32(ra + 4 * t), lds32(ra + 4 * t + 4), 0x5432);
      qa1 = __byte_perm(lds32(ra + 4 * t + 16), lds32(ra + 4 * t + 20), 0x5432);
      qb0 = __byte_perm(lds32(rb + 4 * t), lds32(rb + 4 * t + 4), 0x5432);
      qb1 = __byte_perm(lds32(rb + 4 * t + 16), lds32(rb + 4 * t + 20), 0x5432);
    } else {
      qa0 = lds32(ra + 2 + 4 * t);
      qa1 = lds32(ra + 2 + 4 * t + 16);
      qb0 = lds32(rb + 2 + 4 * t);
      qb1 = lds32(rb + 2 + 4 * t + 16);
    }
    uint32_t ha0[2], ha1[2], hb0[2], hb1[2];
    q8_0_unpack_word(qa0, ha0);
    q8_0_unpack_word(qa1, ha1);
    q8_0_unpack_word(qb0, hb0);
    q8_0_unpack_word(qb1, hb1);
    a0[0] = ha0[0], a0[1] = hb0[0], a0[2] = ha0[1], a0[3] = hb0[1];
    a1[0] = ha1[0], a1[1] = hb1[0], a1[2] = ha1[1], a1[3] = hb1[1];
  }
  const float da = lds_scale(ra);
  const float db = lds_scale(rb);

  float c[4];
  mma_16816_zero(c, a0, bf[0].x, bf[0].y);
  mma_16816(c, a1, bf[1].x, bf[1].y);
  acc[0] = fmaf(da, c[0], acc[0]);
  acc[1] = fmaf(da, c[1], acc[1]);
  acc[2] = fmaf(db, c[2], acc[2]);
  acc[3] = fmaf(db, c[3], acc[3]);
}

// Integer path: one Q4_0 block x 16 rows = ONE m16n8k32 MMA (unsigned nibbles x signed digits,
// int32 accumulate starting from kMagicBits).  off2: the float offsets of columns 2t, 2t + 1.
template <int WT, bool A16, int MPAD, bool EVEN>
__device__ __forceinline__ void block_rows16_i8(const uint8_t *ra, uint2 bf, uint64_t off2, const int (&mg)[4], int t,
                                                float (&acc)[4]) {
  using C = Cfg<WT, A16, MPAD>;
  const uint8_t *rb = ra + 8 * C::PSTRIDE;
  uint32_t       qa, qb;
  if constexpr (EVEN) {  // quants start 2 bytes past a word boundary
    qa = __byte_perm(lds32(ra + 4 * t), lds32(ra + 4 * t + 4), 0x5432);
    qb = __byte_perm(lds32(rb + 4 * t), lds32(rb + 4 * t + 4), 0x5432);
  } else {
    qa = lds32(ra + 2 + 4 * t);
    qb = lds32(rb + 2 + 4 * t);
  }
  uint32_t a0, a1, a2, a3;
  int      d0, d1, d2, d3;
  if constexpr (WT == kIQ4) {
    // table values as signed bytes, in the element order of iq4nl_word_elem
    iq4nl_unpack_word(qa, a0, a2);
    iq4nl_unpack_word(qb, a1, a3);
    asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=r"(d0), "=r"(d1), "=r"(d2), "=r"(d3)
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(bf.x), "r"(bf.y), "r"(mg[0]), "r"(mg[1]), "r"(mg[2]), "r"(mg[3]));
  } else {
    // byte i of the word: low nibble = element 4t + i, high nibble = element 16 + 4t + i
    a0 = qa & 0x0F0F0F0Fu, a2 = (qa >> 4) & 0x0F0F0F0Fu;
    a1 = qb & 0x0F0F0F0Fu, a3 = (qb >> 4) & 0x0F0F0F0Fu;
    asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=r"(d0), "=r"(d1), "=r"(d2), "=r"(d3)
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(bf.x), "r"(bf.y), "r"(mg[0]), "r"(mg[1]), "r"(mg[2]), "r"(mg[3]));
  }
  const float da = lds_scale(ra);
  const float db = lds_scale(rb);
  // int bits -> float: add the offset, two results per instruction (packed fp32 add)
  float f0, f1, f2, f3;
  asm("{\n\t.reg .b64 p, q;\n\t"
      "mov.b64 p, {%4, %5};\n\t"
      "mov.b64 q, {%6, %7};\n\t"
      "add.rn.f32x2 p, p, %8;\n\t"
      "add.rn.f32x2 q, q, %8;\n\t"
      "mov.b64 {%0, %1}, p;\n\t"
      "mov.b64 {%2, %3}, q;\n\t}"
      : "=f"(f0), "=f"(f1), "=f"(f2), "=f"(f3)
      : "r"(d0), "r"(d1), "r"(d2), "r"(d3), "l"(off2));
  acc[0] = fmaf(da, f0, acc[0]);
  acc[1] = fmaf(da, f1, acc[1]);
  acc[2] = fmaf(db, f2, acc[2]);
  acc[3] = fmaf(db, f3, acc[3]);
}

// Packed pairs of floats (sm_100 has two-lane fp32 add and fma on 64-bit registers).
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
// acc += d2 * (bits as floats + off2), both lanes: the integer MMA results of one row leave their
// float bias (and Q4_0's -8 offset) behind and are scaled by the row's block scale
__device__ __forceinline__ void scale_add2(uint64_t &acc, int b0, int b1, uint64_t d2, uint64_t off2) {
  asm("{\n\t.reg .b64 p;\n\t"
      "mov.b64 p, {%1, %2};\n\t"
      "add.rn.f32x2 p, p, %4;\n\t"
      "fma.rn.f32x2 %0, %3, p, %0;\n\t}"
      : "+l"(acc)
      : "r"(b0), "r"(b1), "l"(d2), "l"(off2));
}

// Wide integer path: one block x 16 rows x eight tokens = THREE m16n8k32 MMAs on the same weight
// registers, one per activation digit.  acc[d][0]: row g, tokens 2t and 2t + 1 of digit d; acc[d][1]: row g + 8.
template <int WT, bool A16, bool EVEN>
__device__ __forceinline__ void block_rows16_wide(const uint8_t *ra, const uint2 (&bf)[3], uint64_t neg_magic2,
                                                  const int (&mg)[4], int t, uint64_t (&acc)[3][2]) {
  using C = Cfg<WT, A16, 8>;
  const uint8_t *rb = ra + 8 * C::PSTRIDE;
  uint32_t       a0, a1, a2, a3;
  if constexpr (WT == kQ8) {
    // lane position t owns quant words t and t + 4 of the block: bytes are the values (signed)
    if constexpr (EVEN) {  // quants start 2 bytes past a word boundary
      a0 = __byte_perm(lds32(ra + 4 * t), lds32(ra + 4 * t + 4), 0x5432);
      a2 = __byte_perm(lds32(ra + 4 * t + 16), lds32(ra + 4 * t + 20), 0x5432);
      a1 = __byte_perm(lds32(rb + 4 * t), lds32(rb + 4 * t + 4), 0x5432);
      a3 = __byte_perm(lds32(rb + 4 * t + 16), lds32(rb + 4 * t + 20), 0x5432);
    } else {
      a0 = lds32(ra + 2 + 4 * t);
      a2 = lds32(ra + 2 + 4 * t + 16);
      a1 = lds32(rb + 2 + 4 * t);
      a3 = lds32(rb + 2 + 4 * t + 16);
    }
  } else {
    uint32_t qa, qb;
    if constexpr (EVEN) {
      qa = __byte_perm(lds32(ra + 4 * t), lds32(ra + 4 * t + 4), 0x5432);
      qb = __byte_perm(lds32(rb + 4 * t), lds32(rb + 4 * t + 4), 0x5432);
    } else {
      qa = lds32(ra + 2 + 4 * t);
      qb = lds32(rb + 2 + 4 * t);
    }
    if constexpr (WT == kIQ4) {
      iq4nl_unpack_word(qa, a0, a2);
      iq4nl_unpack_word(qb, a1, a3);
    } else {
      // q - 8 is the nibble q ^ 8 read as a signed 4-bit number: in the high half of a byte that is the
      // signed byte 16 (q - 8) - no offset to take out afterwards (the 16 leaves with the output scale)
      const uint32_t ta = qa ^ 0x88888888u, tb = qb ^ 0x88888888u;
      a0 = (ta << 4) & 0xF0F0F0F0u, a2 = ta & 0xF0F0F0F0u;
      a1 = (tb << 4) & 0xF0F0F0F0u, a3 = tb & 0xF0F0F0F0u;
    }
  }
  const float    da  = lds_scale(ra);
  const float    db  = lds_scale(rb);
  const uint64_t da2 = pack2(da, da), db2 = pack2(db, db);
  // the three MMAs first, then their results: nothing waits on an MMA that was only just issued
  int r[3][4];
#pragma unroll
  for (int d = 0; d < 3; ++d) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(r[d][0]), "=r"(r[d][1]), "=r"(r[d][2]), "=r"(r[d][3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(bf[d].x), "r"(bf[d].y), "r"(mg[0]), "r"(mg[1]), "r"(mg[2]), "r"(mg[3]));
  }
#pragma unroll
  for (int d = 0; d < 3; ++d) {
    scale_add2(acc[d][0], r[d][0], r[d][1], da2, neg_magic2);
    scale_add2(acc[d][1], r[d][2], r[d][3], db2, neg_magic2);
  }
}

// Per-lane partial sums of the tile in progress: rows g, g + 8 of both 16-row groups x MMA columns
// 2t, 2t + 1.  The wide path keeps one packed pair per digit, row and group and weighs the digits
// when the tile is handed over.
template <class C, bool WIDE = C::WIDE>
struct TileAcc {
  float v[2][4];
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int rg = 0; rg < 2; ++rg) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[rg][i] = 0.f;
      }
    }
  }
  __device__ __forceinline__ void sums(float (&o)[2][4]) const {
#pragma unroll
    for (int rg = 0; rg < 2; ++rg) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        o[rg][i] = v[rg][i];
      }
    }
  }
};
template <class C>
struct TileAcc<C, true> {
  uint64_t v[2][3][2];
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int rg = 0; rg < 2; ++rg) {
#pragma unroll
      for (int d = 0; d < 3; ++d) {
        v[rg][d][0] = v[rg][d][1] = 0ull;  // the bit pattern of (0.f, 0.f)
      }
    }
  }
  // digit d weighs 256^d (the common factor 2^-22 is part of the token's output scale)
  __device__ __forceinline__ void sums(float (&o)[2][4]) const {
#pragma unroll
    for (int rg = 0; rg < 2; ++rg) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        float a0, a1, b0, b1, c0, c1;
        unpack2(v[rg][0][r], a0, a1);
        unpack2(v[rg][1][r], b0, b1);
        unpack2(v[rg][2][r], c0, c1);
        o[rg][2 * r]     = fmaf(c0, 65536.f, fmaf(b0, 256.f, a0));
        o[rg][2 * r + 1] = fmaf(c1, 65536.f, fmaf(b1, 256.f, a1));
      }
    }
  }
};

// This warp's blocks of one stage, both 16-row groups.  sb: the lane's row g at the warp's first
// block of the stage; fp: the lane's fragment entry (column g, lane position t) of that block;
// cp (integer paths): the lane's pair of accumulator inputs (columns 2t, 2t + 1) of that block;
// par: parity of the warp's first block inside the stage (it decides which blocks start on a word
// boundary; always 0 when a warp owns an even number of blocks).
template <int WT, bool A16, int MPAD>
__device__ __forceinline__ void stage_blocks(const uint8_t *sb, const uint2 *fp, const uint2 *cp, int t, int par,
                                             TileAcc<Cfg<WT, A16, MPAD>> &acc) {
  using C = Cfg<WT, A16, MPAD>;
  uint64_t neg_magic2;  // the pair (-kMagic, -kMagic)
  asm("mov.b64 %0, {%1, %1};" : "=l"(neg_magic2) : "f"(-kMagic));
  // the accumulator input of every integer MMA: four registers of their own, so that the compiler
  // keeps ONE register quad for all of them instead of assembling it before each MMA
  int mg[4];
  asm volatile("mov.b32 %0, %4;\n\tmov.b32 %1, %4;\n\tmov.b32 %2, %4;\n\tmov.b32 %3, %4;"
               : "=r"(mg[0]), "=r"(mg[1]), "=r"(mg[2]), "=r"(mg[3])
               : "r"(kMagicBits));
#pragma unroll
  for (int i = 0; i < C::BPW; ++i) {
    const bool even = (((C::BPW % 2 == 0) ? 0 : par) + i) % 2 == 0;
    if constexpr (C::WIDE) {
      uint2 bf[3];
#pragma unroll
      for (int d = 0; d < 3; ++d) {
        bf[d] = fp[i * C::FRAG_U2 + d * 32];
      }
#pragma unroll
      for (int rg = 0; rg < 2; ++rg) {
        const uint8_t *ra = sb + rg * 16 * C::PSTRIDE + i * C::BB;
        if (even) {
          block_rows16_wide<WT, A16, true>(ra, bf, neg_magic2, mg, t, acc.v[rg]);
        } else {
          block_rows16_wide<WT, A16, false>(ra, bf, neg_magic2, mg, t, acc.v[rg]);
        }
      }
    } else if constexpr (C::I8) {
      const uint2    bf   = fp[i * C::FRAG_U2];
      const uint64_t off2 = WT == kQ4 ? *reinterpret_cast<const uint64_t *>(cp + i * C::FRAG_U2) : neg_magic2;
#pragma unroll
      for (int rg = 0; rg < 2; ++rg) {
        const uint8_t *ra = sb + rg * 16 * C::PSTRIDE + i * C::BB;
        if (even) {
          block_rows16_i8<WT, A16, MPAD, true>(ra, bf, off2, mg, t, acc.v[rg]);
        } else {
          block_rows16_i8<WT, A16, MPAD, false>(ra, bf, off2, mg, t, acc.v[rg]);
        }
      }
    } else if constexpr (WT != kIQ4) {
      uint2 bf[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        bf[j] = fp[(i * 2 + j) * C::NC * 4];
      }
#pragma unroll
      for (int rg = 0; rg < 2; ++rg) {
        const uint8_t *ra = sb + rg * 16 * C::PSTRIDE + i * C::BB;
        if (even) {
          block_rows16<WT, A16, MPAD, true>(ra, bf, t, acc.v[rg]);
        } else {
          block_rows16<WT, A16, MPAD, false>(ra, bf, t, acc.v[rg]);
        }
      }
    }
  }
}

// ------------------------------------------------------------------ tile completion

// Bounded wait that also gives up when another role of the CTA has raised the abort flag.
// A failed try_wait comes back within tens of cycles, so a waiting warp would otherwise spin at full
// speed and take issue slots from the warps that have work: after a few polls it sleeps between them
// (NS nanoseconds: short for the consumers, whose data is usually a moment away, longer for the tile
// completion warps, which have a tile every few microseconds).
template <int NS = 32>
__device__ __forceinline__ bool mbar_wait_abort(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
  for (uint32_t i = 0; i < kWaitCap; ++i) {
    if (mbar_try_wait(bar, parity)) {
      return true;
    }
    if (i >= 4) {
      if (i > 64 && *abort_flag) {
        return false;
      }
      __nanosleep(NS);
    }
  }
  return false;
}

// Consumer side of a tile completion, n = how many tiles this CTA has completed before: the warp
// drops its partial sums into copy n & 1 of the reduction buffer and carries on.  Copy n & 1 was
// last used by completion n - 2, which the completion warps have read once red_empty says so.
template <class C>
__device__ __forceinline__ bool publish_tile(Smem *sm, const TileAcc<C> &tile_acc, int warp, int lane, unsigned n) {
  constexpr unsigned NB  = C::RED_BUFS;
  const int          buf = (int) (n % NB);
  if (n >= NB && !mbar_wait_abort(&sm->red_empty[buf], ((n / NB) - 1) & 1, &sm->abort_flag)) {
    return false;
  }
  float acc[2][4];
  tile_acc.sums(acc);
#pragma unroll
  for (int rg = 0; rg < 2; ++rg) {
    *reinterpret_cast<float4 *>(&sm->red[buf][warp][rg * 128 + lane * 4]) =
      make_float4(acc[rg][0], acc[rg][1], acc[rg][2], acc[rg][3]);
  }
  __syncwarp();
  if (lane == 0) {
    mbar_arrive(&sm->red_full[buf]);  // release: the warp's stores above are visible to the waiter
  }
  return true;
}

// Completion-warp side: warp rg (0, 1) finishes the 16-row group rg of the tile, lane (g, t) the
// four sums the consumer lanes (g, t) hold: rows g and g + 8, MMA columns 2t and 2t + 1.
// Returns false when a wait ran out (error recorded, abort flag raised).
template <int WT, bool A16, int MPAD>
__device__ bool complete_tile(const GemvArgs &p, Smem *sm, long long tile, long long it0, long long it1, int S, int rg,
                              int lane, unsigned n) {
  using C = Cfg<WT, A16, MPAD>;
  constexpr unsigned NB  = C::RED_BUFS;
  const int          buf = (int) (n % NB);
  const int g = lane >> 2, t = lane & 3;
  // which token the lane's results belong to, and whether this lane writes them out
  int  m0, m1;  // tokens of (column 2t, column 2t + 1); equal when the columns are pieces of one token
  bool writer = true;
  if constexpr (C::DIGCOL) {
    m0 = m1 = t >> 1;
    writer  = (t & 1) == 0;
  } else if constexpr (C::SPLITCOL) {
    m0 = m1 = t;
  } else {
    m0 = 2 * t, m1 = 2 * t + 1;
  }
  const bool arrived = mbar_wait_abort<256>(&sm->red_full[buf], (n / NB) & 1, &sm->abort_flag);
  // (both completion warps leave together: the barriers further down need all 64 threads)
  if (!named_bar_and(2, kReduceThreads, arrived)) {
    record_error(p, kGemvErrConsumerWait);
    sm->abort_flag = 1;
    return false;
  }
  // per-token output scale of this operator (read before the buffer is handed back: a batched
  // launch rebuilds the scales for its next operator only after that)
  float inv0 = 1.f, inv1 = 1.f;
  if constexpr (!A16 || C::I8) {
    inv0 = sm->tok_inv[m0 & 7], inv1 = sm->tok_inv[m1 & 7];
  }
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int w = 0; w < kConsumerWarps; ++w) {
    const float4 r = *reinterpret_cast<const float4 *>(&sm->red[buf][w][rg * 128 + lane * 4]);
    v.x += r.x, v.y += r.y, v.z += r.z, v.w += r.w;
  }
  __syncwarp();
  if (lane == 0) {
    mbar_arrive(&sm->red_empty[buf]);
  }

  const long long first = p.item_base + tile * S, last = first + S - 1;
  bool            write_out = true;
  if (first < it0 || last >= it1) {
    // this CTA holds only part of the tile
    const long long T = p.total_items, G = gridDim.x;
    const int       c_first = (int) item_owner(first, T, G);
    const int       c_last  = (int) item_owner(last, T, G);
    const int       slot    = (first < it0) ? 0 : 1;
    const int       off     = rg * 128 + lane * 4;
    float          *mine    = p.partials + ((size_t) blockIdx.x * 2 + slot) * 256;
    __stcg(reinterpret_cast<float4 *>(mine + off), v);
    __threadfence();
    named_bar_sync(2, kReduceThreads);
    if (rg == 0 && lane == 0) {
      const unsigned old  = atomicAdd(p.counters + c_first, 1u);
      const int      done = (old == (unsigned) (c_last - c_first));
      if (done) {
        p.counters[c_first] = 0;  // ready for the next launch
      }
      sm->last_flag = done;
    }
    named_bar_sync(2, kReduceThreads);
    write_out = sm->last_flag != 0;
    if (write_out) {
      __threadfence();
      v = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int c = c_first; c <= c_last; ++c) {
        const int    s = (c == c_first) ? 1 : 0;
        const float4 r = __ldcg(reinterpret_cast<const float4 *>(p.partials + ((size_t) c * 2 + s) * 256 + off));
        v.x += r.x, v.y += r.y, v.z += r.z, v.w += r.w;
      }
    }
    named_bar_sync(2, kReduceThreads);  // last_flag may be rewritten by the next completion
  }
  // v.x, v.y: row g, columns 2t, 2t + 1;  v.z, v.w: row g + 8, same columns
  float lo0 = v.x, lo1 = v.y, hi0 = v.z, hi1 = v.w;
  if constexpr (C::DIGCOL) {
    // column 2t + c = 4 m + digit: weigh the digits (2^(8 digit - 30)) and add the four columns
    const float w0 = __int_as_float((127 + 8 * ((t & 1) << 1) - kNarrowShift) << 23);
    const float w1 = __int_as_float((127 + 8 * (((t & 1) << 1) | 1) - kNarrowShift) << 23);
    lo0 = lo0 * w0 + lo1 * w1;
    hi0 = hi0 * w0 + hi1 * w1;
    lo0 += __shfl_xor_sync(0xffffffffu, lo0, 1);
    hi0 += __shfl_xor_sync(0xffffffffu, hi0, 1);
  } else if constexpr (C::SPLITCOL) {
    lo0 += lo1;  // hi-piece column + lo-piece column
    hi0 += hi1;
  }
  const long long ld = p.y_ld > 0 ? p.y_ld : p.N;
  if (p.n_dst > 1) {
    // Several destinations (every rank's copy of a row-sharded output): the two completion warps put
    // the tile together in shared memory, then all 64 threads send it out as 16-byte stores - eight
    // consecutive lanes cover the 128 bytes one token has in one destination.  (write_out is the same
    // for all 64 threads.)
    if (write_out && writer) {
      auto stage = [&](int m, int r, float val, float inv) {
        if (m < p.M) {
          sm->out_tile[m][r] = val * inv;
        }
      };
      stage(m0, rg * 16 + g, lo0, inv0);
      stage(m0, rg * 16 + g + 8, hi0, inv0);
      if constexpr (!C::DIGCOL && !C::SPLITCOL) {
        stage(m1, rg * 16 + g, lo1, inv1);
        stage(m1, rg * 16 + g + 8, hi1, inv1);
      }
    }
    named_bar_sync(2, kReduceThreads);
    if (write_out) {
      const int       per_dst = p.M * (kGemvTileRows / 4);
      const long long col     = p.y_col0 + tile * kGemvTileRows;
      for (int i = rg * 32 + lane; i < p.n_dst * per_dst; i += kReduceThreads) {
        const int    d = i / per_dst, r = i - d * per_dst;
        const int    m = r >> 3, c = r & 7;
        const float4 val  = *reinterpret_cast<const float4 *>(&sm->out_tile[m][4 * c]);
        float       *base = d == 0 ? p.y : p.y_more[d - 1];
        *reinterpret_cast<float4 *>(base + (long long) m * ld + col + 4 * c) = val;
      }
    }
    named_bar_sync(2, kReduceThreads);  // the next tile may overwrite the staging area
    return true;
  }
  if (!write_out || !writer) {
    return true;
  }
  const long long row = tile * kGemvTileRows + rg * 16 + g;
  auto            put = [&](int m, long long r, float val, float inv) {
    if (m < p.M) {
      const long long at = (long long) m * ld + p.y_col0 + r;
      val *= inv;
      p.y[at] = p.accumulate ? (p.y[at] + val) : val;
    }
  };
  put(m0, row, lo0, inv0);
  put(m0, row + 8, hi0, inv0);
  if constexpr (!C::DIGCOL && !C::SPLITCOL) {
    put(m1, row, lo1, inv1);
    put(m1, row + 8, hi1, inv1);
  }
  return true;
}

// ------------------------------------------------------------------ the kernel

template <int WT, bool A16, int MPAD>
__global__ void __launch_bounds__(kThreads, 1)
  gemv_mma_kernel(const GemvArgs p, const __grid_constant__ CUtensorMap wmap) {
  using C = Cfg<WT, A16, MPAD>;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  Smem    *sm     = reinterpret_cast<Smem *>(smem_raw);
  uint2   *frags  = reinterpret_cast<uint2 *>(smem_raw + C::HEADER);
  uint8_t *stages = smem_raw + C::HEADER + (((size_t) p.kblocks * C::FRAG_U2 * 8 + 127) & ~(size_t) 127);

  const int       warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int       S   = p.stages_per_tile;
  const int       NST = p.n_stages;
  const long long T = p.total_items, G = gridDim.x;
  const long long it0 = T * blockIdx.x / G, it1 = T * (blockIdx.x + 1) / G;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) {
      mbar_init(&sm->full[s], 1);
      mbar_init(&sm->empty[s], kConsumerWarps);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm->red_full[i], kConsumerWarps);
      mbar_init(&sm->red_empty[i], kReduceThreads / 32);
    }
    mbar_init(&sm->op_bar, kConsumerWarps);
    sm->abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == kConsumerWarps) {
    // ---------------- producer: weights only, may run ahead of the previous kernel's completion
    if (lane == 0) {
      tma_prefetch_descriptor(&wmap);
      const uint64_t pol = l2_policy_evict_first();
      long long      tile = it0 / S;
      int            st   = (int) (it0 - tile * S);
      int            slot = 0, ph = 0;
      for (long long it = it0; it < it1; ++it) {
        if (!mbar_wait(&sm->empty[slot], ph ^ 1)) {
          record_error(p, kGemvErrProducerWait);
          break;
        }
        mbar_arrive_expect_tx(&sm->full[slot], (uint32_t) C::STAGE);
        // box = 32 rows x PSTRIDE bytes, in 8-byte elements
        tma_load_2d(stages + (size_t) slot * C::STAGE, &wmap, st * (C::SB * C::BB / 8),
                    (int) (tile * kGemvTileRows), &sm->full[slot], pol);
        if (++slot == NST) {
          slot = 0;
          ph ^= 1;
        }
        if (++st == S) {
          st = 0;
          ++tile;
        }
      }
    }
  } else if (warp >= kReduceWarp0) {
    // ---------------- tile completion: the tiles this CTA touches, in order
    pdl_wait_prior_grids();  // outputs and scratch belong to the stream order
    if (it1 > it0) {
      const long long last_tile = (it1 - 1) / S;
      unsigned        n         = 0;
      for (long long tile = it0 / S; tile <= last_tile; ++tile, ++n) {
        if (!complete_tile<WT, A16, MPAD>(p, sm, tile, it0, it1, S, warp - kReduceWarp0, lane, n)) {
          break;
        }
      }
      if (p.n_dst > 1) {
        __threadfence_system();  // stores into other GPUs' memory are ordered before this kernel's end
      }
    }
    if (p.done_counter) {
      // this CTA's bands are out (both completion warps, each thread's stores fenced at system scope
      // above): count the CTA in; the last CTA of the launch tells every destination that this rank is
      // done.  The counter's acquire-release, the warp shuffle and the fence before each flag store
      // carry the ordering.
      named_bar_sync(2, kReduceThreads);
      if (warp == kReduceWarp0) {
        unsigned last = 0;
        if (lane == 0) {
          unsigned old;
          asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(p.done_counter) : "memory");
          if (old == gridDim.x - 1) {
            *p.done_counter = 0;  // ready for the next launch
            last = 1;
          }
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        // Lane d tells destination d: ONE system-scope fence per lane, all lanes at once, then a relaxed
        // store.  (A release store per destination from one thread is a system-scope fence per
        // destination, one after the other: about two microseconds each across NVLink.)
        if (last && lane < p.n_dst) {
          asm volatile("fence.acq_rel.sys;\n\tst.relaxed.sys.global.u32 [%0], %1;" ::"l"(p.sig_flags[lane]), "r"(p.epoch)
                       : "memory");
        }
        // Optionally the launch also WAITS (bounded, about a second) until every rank's flag of this epoch
        // is in this GPU's flag array: the kernel's end is then the end of the step on this GPU - every
        // rank's band has landed here - without a separate wait kernel and its kernel boundary.  The
        // last CTA waits; lane r watches rank r.  (Kernels of DIFFERENT GPUs wait for each other here;
        // each rank's launch depends only on its own earlier steps, so no cycle can form.)
        if (last && p.wait_flags && lane < p.n_wait) {
          bool seen = false;
          for (uint32_t i = 0; i < (1u << 23) && !seen; ++i) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.wait_flags + lane) : "memory");
            seen = (int) (v - p.epoch) >= 0;
            if (!seen) {
              __nanosleep(100);
            }
          }
          if (!seen) {
            atomicCAS(p.err, 0, kGemvErrFlagWait);
          }
        }
      }
    }
  } else {
    // ---------------- consumers
    const int tid = threadIdx.x;
    const int g = lane >> 2, t = lane & 3;
    pdl_wait_prior_grids();  // activations and outputs belong to the stream order
    build_x_frags<WT, A16, MPAD>(p, sm, frags, tid);
    named_bar_sync(1, kConsumerThreads);

    TileAcc<C> acc;
    acc.zero();
    // item -> (tile, stage) and ring position are tracked incrementally: no divisions in the loop
    long long tile = it0 / S;
    int       st   = (int) (it0 - tile * S);
    int       slot = 0, ph = 0;
    bool      ok   = true;
    unsigned  n_done = 0;  // tiles completed so far
    // lanes whose MMA column is beyond the columns in use read a valid fragment of another column:
    // their output columns are never stored, so what they multiply is irrelevant
    const uint2   *frag_lane = frags + (g & (C::NC - 1)) * 4 + t;
    const uint8_t *warp_base = stages + g * C::PSTRIDE + warp * C::BPW * C::BB;
    const uint2   *warp_frag = frag_lane + (size_t) (warp * C::BPW) * C::FRAG_U2;
    // (integer path) accumulator inputs of columns 2t, 2t + 1; positions past the columns in use
    // read another pair, their outputs are never stored
    const uint2   *warp_cin  = frags + C::CIN_OFF + (t & (C::NC / 2 - 1)) + (size_t) (warp * C::BPW) * C::FRAG_U2;
    for (long long it = it0; it < it1; ++it) {
      if (!mbar_wait_abort(&sm->full[slot], ph, &sm->abort_flag)) {
        record_error(p, kGemvErrConsumerWait);
        sm->abort_flag = 1;
        ok             = false;
        break;
      }
      const int nblk = min(C::SB, p.kblocks - st * C::SB);
      if (warp * C::BPW < nblk) {
        const uint8_t *sb = warp_base + (size_t) slot * C::STAGE;
        const uint2   *fp = warp_frag + (size_t) (st * C::SB) * C::FRAG_U2;
        const uint2   *cp = warp_cin + (size_t) (st * C::SB) * C::FRAG_U2;
        stage_blocks<WT, A16, MPAD>(sb, fp, cp, t, warp & 1, acc);
      }
      // The stage goes back to the TMA producer here.  An mbarrier arrive does not wait for this
      // thread's outstanding shared-memory loads, and the arithmetic that consumes the last loads
      // (the block scales) may be scheduled after it, so a fence makes sure every load of the
      // stage has been performed before the slot can be overwritten.
      asm volatile("fence.acq_rel.cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&sm->empty[slot]);
      }
      if (++slot == NST) {
        slot = 0;
        ph ^= 1;
      }
      if (++st == S) {
        st = 0;
        if (it + 1 < it1) {
          if (!publish_tile(sm, acc, warp, lane, n_done++)) {
            ok = false;
            break;
          }
          acc.zero();
          ++tile;
        }
      }
    }
    if (ok && it1 > it0) {
      publish_tile(sm, acc, warp, lane, n_done++);
    }
  }
}

template <int WT, bool A16, int MPAD>
cudaError_t launch_one(const GemvArgs &args, const CUtensorMap &wmap, int grid, size_t smem, cudaStream_t stream,
                       bool pdl) {
  auto kern = gemv_mma_kernel<WT, A16, MPAD>;
  // the opt-in shared-memory size is set once per device and instantiation, not per launch
  static bool attr_set[64] = {};
  int         dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvSmemBudget);
    if (e != cudaSuccess) {
      return e;
    }
    if (dev >= 0 && dev < 64) {
      attr_set[dev] = true;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim            = dim3(grid);
  cfg.blockDim           = dim3(kThreads);
  cfg.dynamicSmemBytes   = smem;
  cfg.stream             = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs                                          = attr;
  cfg.numAttrs                                       = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, args, wmap);
}

template <int WT, bool A16>
cudaError_t launch_mpad(const GemvArgs &a, const CUtensorMap &wm, int mpad, int grid, size_t smem, cudaStream_t s,
                        bool pdl) {
  switch (mpad) {
    case 1: return launch_one<WT, A16, 1>(a, wm, grid, smem, s, pdl);
    case 2: return launch_one<WT, A16, 2>(a, wm, grid, smem, s, pdl);
    case 8: return launch_one<WT, A16, 8>(a, wm, grid, smem, s, pdl);
    default: return cudaErrorInvalidValue;
  }
}

// ------------------------------------------------------------------ completion flags

// One warp; lane r watches flag r.  Launched with programmatic stream serialisation so that it is
// already resident and polling while the mat-vec before it in the stream is still running (it depends
// on that kernel only through the flags, this GPU's own included): no launch gap after the mat-vec.
__global__ void flags_wait_kernel(const unsigned *flags, int n, unsigned epoch, int *err) {
  // the next kernel in the stream may start its own prologue (a mat-vec prefetches weights) while this
  // one waits; whatever it does behind its own griddepcontrol.wait still comes after this kernel
  pdl_launch_dependents();
  const int r = threadIdx.x;
  if (r >= n) {
    return;
  }
  for (uint32_t i = 0; i < (1u << 23); ++i) {  // about a second
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + r) : "memory");
    if ((int) (v - epoch) >= 0) {
      return;
    }
    __nanosleep(100);
  }
  atomicCAS(err, 0, kGemvErrFlagWait);
}

// ------------------------------------------------------------------ the batched kernel
//
// Same pipeline, but the item list is the concatenation of the items of up to 128 independent
// operators of one kind.  CTA c still owns the contiguous range [T c / G, T (c+1) / G) of the WHOLE
// list, so it touches only one or two operators; the activation fragments are rebuilt when its
// range crosses into the next operator (all consumer warps have passed the tile-completion barrier
// by then, i.e. nobody reads the old fragments any more).  Tiles cut by a range boundary are
// finished exactly as in the single-operator kernel, with list-wide item indices.

template <int WT, bool A16, int MPAD>
__global__ void __launch_bounds__(kThreads, 1) gemv_mma_batch_kernel(const __grid_constant__ GemvBatchArgs b) {
  using C = Cfg<WT, A16, MPAD>;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  Smem    *sm     = reinterpret_cast<Smem *>(smem_raw);
  uint2   *frags  = reinterpret_cast<uint2 *>(smem_raw + C::HEADER);
  uint8_t *stages = smem_raw + C::HEADER + b.frag_bytes;

  const int       warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int       NST = b.n_stages;
  const long long T = b.total_items, G = gridDim.x;
  const long long it0 = T * blockIdx.x / G, it1 = T * (blockIdx.x + 1) / G;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) {
      mbar_init(&sm->full[s], 1);
      mbar_init(&sm->empty[s], kConsumerWarps);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm->red_full[i], kConsumerWarps);
      mbar_init(&sm->red_empty[i], kReduceThreads / 32);
    }
    mbar_init(&sm->op_bar, kConsumerWarps);
    sm->abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  // operator that holds item it0
  int oi = 0;
  while (oi + 1 < b.n_ops && b.ops[oi + 1].item_begin <= it0) {
    ++oi;
  }

  auto op_args = [&](int i) {
    GemvArgs p        = {};
    p.y               = b.ops[i].y;
    p.x               = b.ops[i].x;
    p.x_k_off         = b.ops[i].x_k_off;
    p.x_stride        = b.ops[i].x_stride;
    p.M               = b.M;
    p.N               = b.ops[i].N;
    p.kblocks         = b.ops[i].kblocks;
    p.accumulate      = b.ops[i].accumulate;
    p.stages_per_tile = b.ops[i].stages_per_tile;
    p.item_base       = b.ops[i].item_begin;
    p.total_items     = b.total_items;
    p.partials        = b.partials;
    p.counters        = b.counters;
    p.err             = b.err;
    return p;
  };

  if (warp == kConsumerWarps) {
    // ---------------- producer
    if (lane == 0) {
      const uint64_t pol  = l2_policy_evict_first();
      int            S    = b.ops[oi].stages_per_tile;
      long long      li   = it0 - b.ops[oi].item_begin;
      long long      tile = li / S;
      int            st   = (int) (li - tile * S);
      long long      tiles_in_op = b.ops[oi].N / kGemvTileRows;
      int            slot = 0, ph = 0;
      tma_prefetch_descriptor(b.ops[oi].wmap);
      for (long long it = it0; it < it1; ++it) {
        if (!mbar_wait(&sm->empty[slot], ph ^ 1)) {
          atomicCAS(b.err, 0, kGemvErrProducerWait);
          break;
        }
        mbar_arrive_expect_tx(&sm->full[slot], (uint32_t) C::STAGE);
        tma_load_2d(stages + (size_t) slot * C::STAGE, b.ops[oi].wmap, st * (C::SB * C::BB / 8),
                    (int) (tile * kGemvTileRows), &sm->full[slot], pol);
        if (++slot == NST) {
          slot = 0;
          ph ^= 1;
        }
        if (++st == S) {
          st = 0;
          if (++tile == tiles_in_op && oi + 1 < b.n_ops) {
            ++oi;
            tile        = 0;
            S           = b.ops[oi].stages_per_tile;
            tiles_in_op = b.ops[oi].N / kGemvTileRows;
            tma_prefetch_descriptor(b.ops[oi].wmap);
          }
        }
      }
    }
  } else if (warp >= kReduceWarp0) {
    // ---------------- tile completion: the (operator, tile) sequence of this CTA's item range
    pdl_wait_prior_grids();
    GemvArgs  p    = op_args(oi);
    int       S    = p.stages_per_tile;
    long long tile = (it0 - p.item_base) / S;
    long long tiles_in_op = p.N / kGemvTileRows;
    unsigned  n    = 0;
    for (long long it = it0; it < it1; ++n) {
      if (!complete_tile<WT, A16, MPAD>(p, sm, tile, it0, it1, S, warp - kReduceWarp0, lane, n)) {
        break;
      }
      it = p.item_base + (tile + 1) * S;  // first item after this tile
      if (++tile == tiles_in_op && oi + 1 < b.n_ops) {
        ++oi;
        p           = op_args(oi);
        tile        = 0;
        S           = p.stages_per_tile;
        tiles_in_op = p.N / kGemvTileRows;
      }
    }
  } else {
    // ---------------- consumers
    const int tid = threadIdx.x;
    const int g = lane >> 2, t = lane & 3;
    pdl_wait_prior_grids();

    GemvArgs p = op_args(oi);
    build_x_frags<WT, A16, MPAD>(p, sm, frags, tid);
    named_bar_sync(1, kConsumerThreads);

    TileAcc<C> acc;
    acc.zero();
    int       S    = p.stages_per_tile;
    long long li   = it0 - p.item_base;
    long long tile = li / S;
    int       st   = (int) (li - tile * S);
    long long tiles_in_op = p.N / kGemvTileRows;
    int       slot = 0, ph = 0;
    bool      ok   = true;
    unsigned  n_done = 0;  // tiles completed so far
    unsigned  n_ops_done = 0;  // operator changes so far
    const uint2   *frag_lane = frags + (g & (C::NC - 1)) * 4 + t;
    const uint8_t *warp_base = stages + g * C::PSTRIDE + warp * C::BPW * C::BB;
    const uint2   *warp_frag = frag_lane + (size_t) (warp * C::BPW) * C::FRAG_U2;
    // (integer path) accumulator inputs of columns 2t, 2t + 1; positions past the columns in use
    // read another pair, their outputs are never stored
    const uint2   *warp_cin  = frags + C::CIN_OFF + (t & (C::NC / 2 - 1)) + (size_t) (warp * C::BPW) * C::FRAG_U2;
    for (long long it = it0; it < it1; ++it) {
      if (!mbar_wait_abort(&sm->full[slot], ph, &sm->abort_flag)) {
        atomicCAS(b.err, 0, kGemvErrConsumerWait);
        sm->abort_flag = 1;
        ok             = false;
        break;
      }
      const int nblk = min(C::SB, p.kblocks - st * C::SB);
      if (warp * C::BPW < nblk) {
        const uint8_t *sb = warp_base + (size_t) slot * C::STAGE;
        const uint2   *fp = warp_frag + (size_t) (st * C::SB) * C::FRAG_U2;
        const uint2   *cp = warp_cin + (size_t) (st * C::SB) * C::FRAG_U2;
        stage_blocks<WT, A16, MPAD>(sb, fp, cp, t, warp & 1, acc);
      }
      // The stage goes back to the TMA producer here.  An mbarrier arrive does not wait for this
      // thread's outstanding shared-memory loads, and the arithmetic that consumes the last loads
      // (the block scales) may be scheduled after it, so a fence makes sure every load of the
      // stage has been performed before the slot can be overwritten.
      asm volatile("fence.acq_rel.cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&sm->empty[slot]);
      }
      if (++slot == NST) {
        slot = 0;
        ph ^= 1;
      }
      if (++st == S) {
        st = 0;
        if (it + 1 < it1) {
          if (!publish_tile(sm, acc, warp, lane, n_done++)) {
            ok = false;
            break;
          }
          acc.zero();
          if (++tile == tiles_in_op && oi + 1 < b.n_ops) {
            // next operator: its activations and token scales replace the old ones - once the
            // completion warps have taken the last tile of this one (its token scales with it) and
            // every consumer warp has stopped reading the fragments (the barriers below)
            // (an mbarrier, not bar.sync: a warp that has given up a wait never gets here, and the
            // others must not wait for it for ever)
            bool go = mbar_wait_abort(&sm->red_empty[(n_done - 1) % C::RED_BUFS], ((n_done - 1) / C::RED_BUFS) & 1,
                                      &sm->abort_flag);
            if (go) {
              __syncwarp();
              if (lane == 0) {
                mbar_arrive(&sm->op_bar);
              }
              go = mbar_wait_abort(&sm->op_bar, n_ops_done & 1, &sm->abort_flag);
              ++n_ops_done;
            }
            if (!go) {
              sm->abort_flag = 1;
              ok             = false;
              break;
            }
            ++oi;
            p           = op_args(oi);
            tile        = 0;
            S           = p.stages_per_tile;
            tiles_in_op = p.N / kGemvTileRows;
            build_x_frags<WT, A16, MPAD>(p, sm, frags, tid);
            named_bar_sync(1, kConsumerThreads);
          }
        }
      }
    }
    if (ok && it1 > it0) {
      publish_tile(sm, acc, warp, lane, n_done++);
    }
  }
}

template <int WT, bool A16, int MPAD>
cudaError_t batch_one(const GemvBatchArgs &args, int grid, size_t smem, cudaStream_t stream, bool pdl) {
  auto kern = gemv_mma_batch_kernel<WT, A16, MPAD>;
  static bool attr_set[64] = {};
  int         dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvSmemBudget);
    if (e != cudaSuccess) {
      return e;
    }
    if (dev >= 0 && dev < 64) {
      attr_set[dev] = true;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim            = dim3(grid);
  cfg.blockDim           = dim3(kThreads);
  cfg.dynamicSmemBytes   = smem;
  cfg.stream             = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs                                          = attr;
  cfg.numAttrs                                       = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, args);
}

template <int WT, bool A16>
cudaError_t batch_mpad(const GemvBatchArgs &a, int mpad, int grid, size_t smem, cudaStream_t s, bool pdl) {
  switch (mpad) {
    case 1: return batch_one<WT, A16, 1>(a, grid, smem, s, pdl);
    case 2: return batch_one<WT, A16, 2>(a, grid, smem, s, pdl);
    case 8: return batch_one<WT, A16, 8>(a, grid, smem, s, pdl);
    default: return cudaErrorInvalidValue;
  }
}

// cuTensorMapEncodeTiled through the runtime's driver-entry-point lookup (no link against libcuda)
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void                           *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      p = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

}  // namespace

cudaError_t flags_wait_launch(const unsigned *flags, int n, unsigned epoch, int *err, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim            = dim3(1);
  cfg.blockDim           = dim3(32);
  cfg.stream             = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs                                          = attr;
  cfg.numAttrs                                       = 1;
  return cudaLaunchKernelEx(&cfg, flags_wait_kernel, flags, n, epoch, err);
}

size_t gemv_frag_bytes(int wt, bool a16, int mpad, int kblocks) {
  size_t b;
  if (mpad == 8) {  // wide integer path: three digit sets of 8 columns
    b = (size_t) kblocks * (3 * 32) * 8;
  } else if (wt == kQ4 || wt == kIQ4) {  // integer path: 4 digit columns per token + their accumulator inputs
    const int nc = 4 * mpad;
    b            = (size_t) kblocks * (nc * 4 + nc / 2) * 8;
  } else {
    const int nc = a16 ? mpad : 2 * mpad;
    b            = (size_t) kblocks * 2 * nc * 4 * 8;
  }
  return (b + 127) & ~(size_t) 127;
}

bool gemv_plan(int smem_budget, int wt, bool a16, int m, int kblocks, GemvPlan *out) {
  GemvPlan pl;
  pl.mpad          = gemv_mpad(m);
  pl.stage_blocks  = gemv_stage_blocks(wt);
  pl.stage_bytes   = kGemvTileRows * gemv_row_pitch(wt);
  const int periods = kblocks / 8;
  const int budget  = smem_budget < kGemvSmemBudget ? smem_budget : kGemvSmemBudget;
  if (m < 1 || m > 8 || kblocks <= 0 || kblocks % 8 != 0) {
    return false;
  }
  auto stages_for = [&](int chunk_periods) {
    const size_t frag = gemv_frag_bytes(wt, a16, pl.mpad, chunk_periods * 8);
    const long   room = (long) budget - gemv_header_bytes(pl.mpad) - (long) frag;
    const int    nst  = room > 0 ? (int) (room / pl.stage_bytes) : 0;
    return nst > kGemvMaxStages ? kGemvMaxStages : nst;
  };
  const int need = gemv_min_stages(pl.mpad);
  pl.chunk_periods = periods;
  pl.n_stages      = stages_for(periods);
  if (pl.n_stages < need) {
    // K does not fit one launch: ranges of whole pipeline stages (a partly filled stage costs the
    // consumers as much as a full one), the longest that leave room for the ring
    const int spb = pl.stage_blocks / 8;  // blocks of 256 weights per stage
    int       cp  = (periods - 1) / spb * spb;
    for (; cp >= spb; cp -= spb) {
      if (stages_for(cp) >= need) {
        break;
      }
    }
    if (cp < spb) {
      cp = 1;  // (not reached with 227 KB of shared memory: one stage of K always fits)
      if (stages_for(cp) < 2) {
        return false;
      }
    }
    pl.chunk_periods = cp;
    pl.n_stages      = stages_for(cp);
  }
  pl.nchunks = (periods + pl.chunk_periods - 1) / pl.chunk_periods;
  *out       = pl;
  return true;
}

cudaError_t gemv_weight_map(void *wmap_out, const uint8_t *w, long long w_row_bytes, int kblocks, int n, int wt) {
  // Tensor map over a K range of the weight bytes, as 8-byte elements: inner dimension = bytes of
  // the K range per row / 8, outer = n rows, row pitch = w_row_bytes.  Encoding costs about a
  // microsecond of host time, comparable to a small launch, and a decoder re-issues the same few
  // hundred weight matrices every token: the maps are cached by what they describe.
  struct Key {
    const void *base;
    long long   row_bytes;
    int         kblocks, n, wt, dev;
    bool operator==(const Key &o) const {
      return base == o.base && row_bytes == o.row_bytes && kblocks == o.kblocks && n == o.n && wt == o.wt &&
             dev == o.dev;
    }
  };
  struct KeyHash {
    size_t operator()(const Key &k) const {
      size_t h = std::hash<const void *>()(k.base);
      h ^= std::hash<long long>()(k.row_bytes * 131 + k.kblocks) + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
      h ^= std::hash<long long>()(((long long) k.n << 8) ^ (k.wt << 4) ^ k.dev) + (h << 6) + (h >> 2);
      return h;
    }
  };
  static std::mutex                                    cache_mu;
  static std::unordered_map<Key, CUtensorMap, KeyHash> cache;
  int                                                  dev = 0;
  cudaGetDevice(&dev);
  const Key key{ w, w_row_bytes, kblocks, n, wt, dev };
  {
    std::lock_guard<std::mutex> lk(cache_mu);
    auto                        it = cache.find(key);
    if (it != cache.end()) {
      memcpy(wmap_out, &it->second, sizeof(CUtensorMap));
      return cudaSuccess;
    }
  }
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) {
    return cudaErrorNotSupported;
  }
  CUtensorMap      wmap;
  const int        bb         = wt == kQ8 ? 34 : 18;
  const cuuint64_t gdim[2]    = { (cuuint64_t) kblocks * bb / 8, (cuuint64_t) n };
  const cuuint64_t gstride[1] = { (cuuint64_t) w_row_bytes };
  const cuuint32_t box[2]     = { (cuuint32_t) gemv_row_pitch(wt) / 8, (cuuint32_t) kGemvTileRows };
  const cuuint32_t estr[2]    = { 1, 1 };
  if (enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint8_t *>(w), gdim, gstride, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
    return cudaErrorInvalidValue;
  }
  {
    std::lock_guard<std::mutex> lk(cache_mu);
    if (cache.size() >= 8192) {
      cache.clear();
    }
    cache.emplace(key, wmap);
  }
  memcpy(wmap_out, &wmap, sizeof(CUtensorMap));
  return cudaSuccess;
}

cudaError_t gemv_mma_launch(const GemvArgs &args, int wt, bool a16, int mpad, int grid, size_t smem,
                            cudaStream_t stream, bool pdl) {
  CUtensorMap wmap;
  cudaError_t e = gemv_weight_map(&wmap, args.w + args.w_k_off_bytes, args.w_row_bytes, args.kblocks, args.N, wt);
  if (e != cudaSuccess) {
    return e;
  }
  if (wt == kQ4) {
    return a16 ? launch_mpad<kQ4, true>(args, wmap, mpad, grid, smem, stream, pdl)
               : launch_mpad<kQ4, false>(args, wmap, mpad, grid, smem, stream, pdl);
  }
  if (wt == kIQ4) {
    return a16 ? launch_mpad<kIQ4, true>(args, wmap, mpad, grid, smem, stream, pdl)
               : launch_mpad<kIQ4, false>(args, wmap, mpad, grid, smem, stream, pdl);
  }
  return a16 ? launch_mpad<kQ8, true>(args, wmap, mpad, grid, smem, stream, pdl)
             : launch_mpad<kQ8, false>(args, wmap, mpad, grid, smem, stream, pdl);
}

cudaError_t gemv_mma_batch_launch(const GemvBatchArgs &args, int wt, bool a16, int mpad, int grid, size_t smem,
                                  cudaStream_t stream, bool pdl) {
  if (wt == kQ4) {
    return a16 ? batch_mpad<kQ4, true>(args, mpad, grid, smem, stream, pdl)
               : batch_mpad<kQ4, false>(args, mpad, grid, smem, stream, pdl);
  }
  if (wt == kIQ4) {
    return a16 ? batch_mpad<kIQ4, true>(args, mpad, grid, smem, stream, pdl)
               : batch_mpad<kIQ4, false>(args, mpad, grid, smem, stream, pdl);
  }
  return a16 ? batch_mpad<kQ8, true>(args, mpad, grid, smem, stream, pdl)
             : batch_mpad<kQ8, false>(args, mpad, grid, smem, stream, pdl);
}

}  // namespace htp
