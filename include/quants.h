/*
 * Quantised weight block formats on the MUL_MAT path.
 *
 * Layout-compatible with the reference's include/dsp/quants.h: block_q4_0 (:11-14, 18 B),
 * block_q8_0 (:23-26, 34 B) are the standard ggml blocks; my_block_q4_0 (:16-19, 144 B) and
 * my_block_q8_0 (:28-31, 272 B) are the reference-private 256-weight super-blocks. The fp16
 * scale is carried as raw bits (uint16_t) so the header compiles with any host compiler.
 *
 * Semantics (reference src/dsp/ops/mat_mul.c:25-27, 266-271, 290, 300-304):
 *   Q4_0: element i (0..15) = (quants[i] & 0x0F) - 8, element i+16 = (quants[i] >> 4) - 8
 *   Q8_0: element i (0..31) = (int8_t) quants[i]
 *   weight = element * scale
 * A weight matrix W[N][K] is N rows of K/32 consecutive blocks.
 */
#ifndef HTP_OPS_QUANTS_H
#define HTP_OPS_QUANTS_H

#include <stdint.h>

#define QK_K  256 /* weights per super-block */
#define QK_0  32  /* weights per block       */
#define QK4_0 32
#define QK8_0 32

typedef uint16_t htp_fp16_bits;

typedef struct {
  htp_fp16_bits scale;
  uint8_t       quants[QK4_0 / 2];
} __attribute__((packed)) block_q4_0;

typedef struct {
  htp_fp16_bits scales[8];
  uint8_t       quants[8 * QK4_0 / 2];
} __attribute__((packed)) my_block_q4_0;

typedef struct {
  htp_fp16_bits scale;
  uint8_t       quants[QK8_0]; /* consumed as signed bytes */
} __attribute__((packed)) block_q8_0;

typedef struct {
  htp_fp16_bits scales[8];
  int8_t        quants[8 * QK8_0];
} __attribute__((packed)) my_block_q8_0;

/* Subset of the ggml type numbering the reference re-declares (quants.h:33-74); only the
 * values this path dispatches on are named. */
enum htp_weight_type {
  HTP_TYPE_F32    = 0,
  HTP_TYPE_F16    = 1,
  HTP_TYPE_Q4_0   = 2,
  HTP_TYPE_Q8_0   = 8,
  HTP_TYPE_IQ4_NL = 20,
};

#if defined(__cplusplus)
static_assert(sizeof(block_q4_0) == 18 && sizeof(block_q8_0) == 34, "ggml block size");
static_assert(sizeof(my_block_q4_0) == 144 && sizeof(my_block_q8_0) == 272, "super-block size");
#else
_Static_assert(sizeof(block_q4_0) == 18 && sizeof(block_q8_0) == 34, "ggml block size");
_Static_assert(sizeof(my_block_q4_0) == 144 && sizeof(my_block_q8_0) == 272, "super-block size");
#endif

#endif /* HTP_OPS_QUANTS_H */
