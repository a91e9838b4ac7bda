// Device-side unpack of the standard 32-weight blocks, shared by every kernel on the path
// (GEMV fragments, GEMM tile dequantisation, integer block-sum probe).
//
// Block semantics follow the reference (src/dsp/ops/mat_mul.c:25-27, 266-271, 300-301):
//   Q4_0: element i (0..15) = (qs[i] & 0xF) - 8, element i+16 = (qs[i] >> 4) - 8
//   Q8_0: element i (0..31) = (int8) qs[i]
// The routines below turn one 32-bit word of quants into fp16 pairs holding those integer
// values exactly (no scale applied), using the 0x6400 exponent-bias trick: the bit pattern
// 0x6400 | v is the fp16 number 1024 + v for 0 <= v < 1024.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace htp {

constexpr int kQ4  = 0;
constexpr int kQ8  = 1;
constexpr int kIQ4 = 2;  // IQ4_NL: the Q4_0 block with a 16-entry value table instead of q - 8

template <int WT>
struct BlockTraits;
template <>
struct BlockTraits<kQ4> {
  static constexpr int kBytes = 18;
};
template <>
struct BlockTraits<kQ8> {
  static constexpr int kBytes = 34;
};
template <>
struct BlockTraits<kIQ4> {
  static constexpr int kBytes = 18;
};

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) {
  return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) {
  return *reinterpret_cast<__half2 *>(&u);
}

// Word `w` holds quant bytes B0..B3 (B0 in the low byte).  Output pairs {low half, high half}:
//   h[0] = {lo(B0), lo(B2)}   h[1] = {lo(B1), lo(B3)}   h[2] = {hi(B0), hi(B2)}   h[3] = {hi(B1), hi(B3)}
// with lo(B) = (B & 15) - 8 and hi(B) = (B >> 4) - 8, exact in fp16.
__device__ __forceinline__ void q4_0_unpack_word(uint32_t w, uint32_t (&h)[4]) {
  const __half2 k1032 = u32_as_h2(0x64086408u);  // 1024 + 8
  const __half2 k16th = u32_as_h2(0x2C002C00u);  // 1/16
  const __half2 km72  = u32_as_h2(0xD480D480u);  // -(64 + 8)
  const uint32_t w8   = w >> 8;
  h[0] = h2_as_u32(__hsub2(u32_as_h2((w & 0x000F000Fu) | 0x64006400u), k1032));
  h[1] = h2_as_u32(__hsub2(u32_as_h2((w8 & 0x000F000Fu) | 0x64006400u), k1032));
  // the high nibble sits 4 bits up: 0x6400 | (q << 4) = 1024 + 16 q; (1024 + 16 q) / 16 - 72 = q - 8
  h[2] = h2_as_u32(__hfma2(u32_as_h2((w & 0x00F000F0u) | 0x64006400u), k16th, km72));
  h[3] = h2_as_u32(__hfma2(u32_as_h2((w8 & 0x00F000F0u) | 0x64006400u), k16th, km72));
}

// Element index (0..31, within the block) of half `s` (0 = low 16 bits) of output pair `r`
// when the word is the block's quant word `t` (0..3).
__device__ __host__ __forceinline__ constexpr int q4_0_word_elem(int t, int r, int s) {
  return 4 * t + (r & 1) + 2 * s + ((r >> 1) << 4);
}

// Word `w` holds signed bytes B0..B3.  h[0] = {B0, B1}, h[1] = {B2, B3}, exact in fp16.
__device__ __forceinline__ void q8_0_unpack_word(uint32_t w, uint32_t (&h)[2]) {
  const __half2  k1152 = u32_as_h2(0x64806480u);  // 1024 + 128
  const uint32_t x     = w ^ 0x80808080u;         // byte + 128 in 0..255
  h[0] = h2_as_u32(__hsub2(u32_as_h2(__byte_perm(x, 0x64646464u, 0x4140)), k1152));
  h[1] = h2_as_u32(__hsub2(u32_as_h2(__byte_perm(x, 0x64646464u, 0x4342)), k1152));
}

// Element index of half `s` of output pair `r` when the word is quant word `u` (0..7).
__device__ __host__ __forceinline__ constexpr int q8_0_word_elem(int u, int r, int s) {
  return 4 * u + 2 * r + s;
}

// IQ4_NL (reference table: src/dsp/ops/mat_mul.c:29-32): four 4-bit indices in the low 16 bits of
// `idx16` (index j in bits 4j .. 4j+3) -> byte j of the result = table[index j] as a signed byte.
// The table does not fit one byte permute (8 entries): the two halves are looked up with the low
// three index bits and a third permute picks per byte by the fourth bit.
__device__ __forceinline__ uint32_t iq4nl_lookup4(uint32_t idx16) {
  constexpr uint32_t T0 = 0xBFAD9881u;  // -127 -104  -83  -65
  constexpr uint32_t T1 = 0xF6EADDCFu;  //  -49  -35  -22  -10
  constexpr uint32_t T2 = 0x26190D01u;  //    1   13   25   38
  constexpr uint32_t T3 = 0x71594535u;  //   53   69   89  113
  const uint32_t     s  = idx16 & 0x7777u;
  const uint32_t     lo = __byte_perm(T0, T1, s);
  const uint32_t     hi = __byte_perm(T2, T3, s);
  return __byte_perm(lo, hi, 0x3210u + ((idx16 >> 1) & 0x4444u));  // byte j of lo, or byte j of hi (4 + j)
}
// Quant word `w` of a block (bytes 4t .. 4t+3; low nibble of byte j = element j, high nibble =
// element j + 16) -> r0 = values of elements (4t, 16+4t, 4t+1, 17+4t), r1 = (4t+2, 18+4t, 4t+3, 19+4t).
__device__ __forceinline__ void iq4nl_unpack_word(uint32_t w, uint32_t &r0, uint32_t &r1) {
  r0 = iq4nl_lookup4(w);
  r1 = iq4nl_lookup4(w >> 16);
}
// Element (0..31) of byte `i` of register `h` (0 = r0, 1 = r1) above, for quant word `t`.
__device__ __host__ __forceinline__ constexpr int iq4nl_word_elem(int t, int h, int i) {
  return 4 * t + 2 * h + (i >> 1) + ((i & 1) << 4);
}

// Which block element feeds the warp-MMA (m16n8k16) A fragment of the lane with thread-in-group
// `t`, for MMA number `j` (0, 1) of the block: `hi` selects the k-columns 2t+8.. (registers a2, a3)
// instead of 2t.. (a0, a1); `s` the half within the register.  The activation (B) fragments are
// permuted with the same function, which is what makes the per-lane unpack order irrelevant.
template <int WT>
__device__ __host__ __forceinline__ constexpr int mma_frag_elem(int j, int t, int hi, int s) {
  if (WT == kQ4) {
    return q4_0_word_elem(t, 2 * j + hi, s);  // lane t owns quant word t
  }
  return q8_0_word_elem(t + 4 * j, hi, s);  // lane t owns quant words t and t + 4
}

}  // namespace htp
