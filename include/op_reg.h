/*
 * Operator registry and parameter descriptors of the htp-ops dispatch surface.
 *
 * Wire-compatible restatement of the reference's include/op_reg.h (enum at :5-13,
 * RpcmemBufAddr :15-18, RmsNormF32Params :20-25, MatMulParams :27-34, FlashAttnParams
 * :36-47): same names, same enumerator values 0..5, same packed sizes (8/24/36/60 B).
 *
 * Additions, all AFTER the reference's six indices so their values never move:
 *   - fp16-activation quantised matmuls (the reference registry only has fp32-activation
 *     "A32" ops, but the lm_head / prefill workloads feed fp16 activations);
 *   - HTP_OPS_COUNT therefore grows from 6 to 8; HTP_OPS_REFERENCE_COUNT keeps the old value.
 *
 * Weight layout consumed by indices 2, 3, 4, 6, 7 in this library: standard ggml block_q4_0 /
 * block_q8_0 (quants.h; index 4 = the Q4_0 block with the IQ4_NL value table), N rows of K/32
 * consecutive blocks, the layout walked by the reference's dequantize_common_weight_* routines
 * (src/dsp/ops/mat_mul.c:572-640); with the library option "permuted_weights" indices 2, 3, 4 read the
 * reference-private permuted super-blocks instead.  Index 1 reads fp16 weights in the reference's
 * 32 x 32 tile order (src/host/test.c:303-313).  Index 0 is RMSNorm.  Index 5 (FlashAttention) is
 * not built: the dispatcher answers -1.
 */
#ifndef HTP_OPS_OP_REG_H
#define HTP_OPS_OP_REG_H

#include <stdint.h>

enum HtpOpsIndex {
  HTP_OPS_RMS_NORM_F32                     = 0,
  HTP_OPS_MAT_MUL_PERMUTED_W16A32          = 1,
  HTP_OPS_MAT_MUL_PERMUTED_W4D16A32        = 2, /* Q4_0 weights, fp16 scale, fp32 activations */
  HTP_OPS_MAT_MUL_PERMUTED_W8D16A32        = 3, /* Q8_0 weights, fp16 scale, fp32 activations */
  HTP_OPS_MAT_MUL_PERMUTED_W4D16A32_IQ4_NL = 4,
  HTP_OPS_FLASH_ATTN_QO_F32_KV_F16         = 5,
  /* ---- appended by the B200 library ---- */
  HTP_OPS_MAT_MUL_W4D16A16                 = 6, /* Q4_0 weights, fp16 activations, fp32 output */
  HTP_OPS_MAT_MUL_W8D16A16                 = 7, /* Q8_0 weights, fp16 activations, fp32 output */
  HTP_OPS_COUNT,
};

#define HTP_OPS_REFERENCE_COUNT 6

#define HTP_OPS_PACKED __attribute__((packed))

/* A buffer is named by the handle the buffer table gave out (the reference's rpcmem fd)
 * plus a byte offset into it. */
struct RpcmemBufAddr {
  int32_t fd;
  int32_t offset;
} HTP_OPS_PACKED;

struct RmsNormF32Params {
  struct RpcmemBufAddr dst;
  struct RpcmemBufAddr src;
  int32_t ne0; /* row length  */
  int32_t ne1; /* row count   */
} HTP_OPS_PACKED;

/* output[m][n] (fp32) = activation[m][k] * weight[n][k]^T */
struct MatMulParams {
  struct RpcmemBufAddr output;
  struct RpcmemBufAddr activation;
  struct RpcmemBufAddr weight;
  int32_t m;
  int32_t k;
  int32_t n;
} HTP_OPS_PACKED;

struct FlashAttnParams {
  struct RpcmemBufAddr o;
  struct RpcmemBufAddr q;
  struct RpcmemBufAddr k;
  struct RpcmemBufAddr v;
  struct RpcmemBufAddr mask;
  int32_t qo_len;
  int32_t kv_len;
  int32_t n_heads;
  int32_t n_kv_heads;
  int32_t head_dim;
} HTP_OPS_PACKED;

#if defined(__cplusplus)
static_assert(sizeof(struct RpcmemBufAddr) == 8, "wire size");
static_assert(sizeof(struct RmsNormF32Params) == 24, "wire size");
static_assert(sizeof(struct MatMulParams) == 36, "wire size");
static_assert(sizeof(struct FlashAttnParams) == 60, "wire size");
#else
_Static_assert(sizeof(struct RpcmemBufAddr) == 8, "wire size");
_Static_assert(sizeof(struct RmsNormF32Params) == 24, "wire size");
_Static_assert(sizeof(struct MatMulParams) == 36, "wire size");
_Static_assert(sizeof(struct FlashAttnParams) == 60, "wire size");
#endif

#endif /* HTP_OPS_OP_REG_H */
