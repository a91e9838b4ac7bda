/*
 * Compute entry points of the B200 library: raw device pointers, plain sizes, one CUDA stream.
 * This is the C-ABI the host layer (session / message channel / execute_op_simple) is built on
 * and the one a foreign-language binding would target for zero-copy use.
 *
 * All functions act on the CUDA device that is current on the calling thread and return
 *   0   success (work is enqueued on `stream`, not necessarily finished),
 *  -1   invalid arguments (the reference's only failure code, src/dsp/ops/mat_mul.c:878-892),
 *  -2   a CUDA runtime call failed,
 *  -3   (htp_b200_mul_mat_static_scratch only) valid arguments outside that entry point's range,
 *  >0   (htp_b200_stream_status only) a kernel reported a bounded wait that ran out.
 * There is no CPU fallback: without a usable CUDA device every call fails.
 */
#ifndef HTP_OPS_B200_H
#define HTP_OPS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* activation element types */
#define HTP_B200_ACT_F32 0
#define HTP_B200_ACT_F16 1

/*
 * weight_type codes.  2, 8 and 20 are ggml's type numbers (Q4_0, Q8_0, IQ4_NL) and mean standard
 * ggml blocks, n rows of k/32 blocks.  The codes below mean weights in the reference's own 32 x 32
 * TILE ORDER, tile (n/32, k/32) at tile number (n/32) * (k_total/32) + k/32, read in place:
 *   HTP_B200_WT_F16_TILED        fp16 tiles of 2048 B, element (k, n) of a tile at halfword
 *                                (k & ~1) * 32 + n * 2 + (k & 1) - the weight buffer of
 *                                hmx_mat_mul_permuted_w16a32 (reference src/dsp/ops/mat_mul.c:758-855,
 *                                layout written by src/host/test.c:303-313);
 *   HTP_B200_WT_PERMUTED | type  the reference-private super-blocks my_block_q4_0 (144 B) /
 *                                my_block_q8_0 (272 B), four per tile (reference
 *                                include/dsp/quants.h:16-31, expanded at mat_mul.c:308-510) - the
 *                                buffers the reference's own ops 2, 3 and 4 consume; type = 2, 8 or 20.
 * These go through htp_b200_mul_mat only (any m, either activation type: a streaming kernel for a few
 * tokens; with k a multiple of 128, the tensor-core GEMM from 9 fp16 / 17 fp32 tokens up, which unpacks
 * tiles and super-blocks in place, weights rounded to fp16 once as the reference does); the batch,
 * multi-destination and static-scratch calls reject them.
 */
#define HTP_B200_WT_F16_TILED 1
#define HTP_B200_WT_PERMUTED 0x100

/*
 * dst[m][n] (fp32) = activation[m][k] . weight[n][k]^T, weight in standard ggml Q4_0
 * (weight_type 2) or Q8_0 (weight_type 8) blocks, n rows of k/32 blocks.
 * Replaces hmx_mat_mul_permuted_qk_0_d16a32 (reference include/dsp/ops.h:19-20,
 * src/dsp/ops/mat_mul.c:875-1153) and keeps its argument checks: non-null pointers, non-zero
 * sizes, k % 32 == 0, n % 32 == 0, all three pointers 128-byte aligned; anything else -> -1.
 * Kernel by token count: m <= 8 one launch of the decode kernel (fp32 activations, m = 9 .. 16: two),
 * which keeps the weights exact and meets 1e-5 against an fp64 dequantise-then-dot for fp32
 * activations; from m = 9 (fp16 activations) or m = 17 (fp32 activations) the tensor-core GEMM, whose weights are rounded to fp16 once (value * scale, as the reference's
 * dequantisation does, mat_mul.c:290, 304) and which takes fp32 activations as fp16 copies, each token
 * scaled by its own power of two (the reference converts them to fp16 as they are, mat_mul.c:89-128):
 * 1e-3.  Outputs are never rounded to fp16.  Option "a32_exact" keeps fp32-activation matmuls of any
 * m on the decode kernel.  `stream` is a cudaStream_t (NULL = the default stream).
 */
int htp_b200_mul_mat(void *dst, const void *activation, const void *weight, int m, int k, int n, int weight_type,
                     int act_type, void *stream);

/*
 * n_ops INDEPENDENT decode mat-vecs of one kind (same weight_type, act_type and token count
 * m <= 8; k[i] % 256 == 0) as one persistent launch: dst[i][m][n[i]] = activation[i][m][k[i]] .
 * weight[i][n[i]][k[i]]^T.  The operators are streamed as a single work list, so small matrices pay
 * neither a launch nor a pipeline fill and drain each (a decoder layer's q/k/v or gate/up
 * projections).  The caller guarantees that no operator reads a buffer another one of the batch
 * writes.  Closest reference behaviour: a message carrying several requests, executed in order
 * (src/dsp/commu.c:91-126); the message channel of this library forms such batches itself.
 * Returns -1 when an operator cannot be batched (m > 8, k % 256, a fragment set that does not fit
 * one launch, misaligned pointers): issue it with htp_b200_mul_mat instead.
 */
int htp_b200_mul_mat_batch(int n_ops, void *const *dst, const void *const *activation, const void *const *weight,
                           const int *k, const int *n, int m, int weight_type, int act_type, void *stream);

/*
 * The decode mat-vec (m <= 8) for callers that must not allocate device memory once they are
 * running - a server that has handed all of device memory to its own pools, or a decode loop that
 * cannot take the device-wide synchronisation an allocation implies.  Same arguments and checks as
 * htp_b200_mul_mat for the row-major block formats (weight_type 2, 8, 20), the same kernel, launch
 * plan and results, but the kernel's scratch is a static device array inside the library (about
 * 0.4 MB per GPU, held until the process exits) and the call makes no cudaMalloc, cudaFree or other
 * allocating call.  No counterpart in the reference.
 *   - Range: m <= 8, k % 256 == 0, and the activation fragments of the whole k must fit in one
 *     launch's shared memory (htp_b200_mul_mat cuts a longer k into launches that accumulate; this
 *     call does not).  That holds for every k <= 4096, and beyond it up to:
 *       m = 1:      k <= 18944 (Q4_0, IQ4_NL), 23040 (Q8_0, fp32 act.), 46080 (Q8_0, fp16 act.)
 *       m = 2:      k <=  9472 (Q4_0, IQ4_NL), 11520 (Q8_0, fp32 act.), 23040 (Q8_0, fp16 act.)
 *       m = 3 .. 8: k <=  5632 (Q4_0, IQ4_NL),  5888 (Q8_0)
 *     Outside the range the call prints the reason to stderr and returns -3.
 *   - All calls on a device share the one array, which keeps the previous call's contents; what
 *     must start at zero is cleared on `stream` at the start of each call.  Calls that overlap on
 *     the GPU (two streams, two threads) race on it: keep them ordered, e.g. on one stream.
 *   - The first call on each device resolves the array's device address; make that call during
 *     set-up, before any stream capture.
 *   - A bounded wait that runs out inside the kernel is not reported by this entry point.
 */
int htp_b200_mul_mat_static_scratch(void *dst, const void *activation, const void *weight, int m, int k, int n,
                                    int weight_type, int act_type, void *stream);

/*
 * How the decode kernel would run m (1..8) tokens over k (a multiple of 256) weights per row of a block
 * format on a device with 227 KB of shared memory per CTA: into how many K ranges the row is cut
 * (*k_ranges; 1 = the activation fragments of the whole k fit one launch, which is what
 * htp_b200_mul_mat_static_scratch requires), the weights per range (*range_k, whole pipeline stages; the
 * last range may be shorter) and the depth of the shared-memory ring (*stages).  Pure host arithmetic:
 * needs no GPU, launches nothing.  Any of the three pointers may be NULL.  -1 for arguments the decode
 * kernel does not take.  No counterpart in the reference (its chunk sizes are found by find_chunk_size,
 * src/dsp/ops/mat_mul.c:72-86, for a scratchpad of a different shape).
 */
int htp_b200_decode_plan(int m, int k, int weight_type, int act_type, int *k_ranges, int *range_k, int *stages);

/*
 * Integer probe of the block unpack: for each of n_blocks consecutive blocks writes
 * s[b] = sum_i v_i and t[b] = sum_i (i + 1) * v_i (int32), v_i the block's 32 integer values in
 * element order.  No counterpart in the reference (it has no integer path); exists so the
 * unpack the matmul kernels use can be checked bit-exactly.  For the permuted super-blocks
 * (weight_type HTP_B200_WT_PERMUTED | type) a "block" is a scale group - 32 consecutive slots of a
 * super-block, eight per super-block, element order = slot order; n_blocks must be a multiple of 8
 * and `weight` 16-byte aligned.
 */
int htp_b200_block_sums(const void *weight, int32_t *s, int32_t *t, int64_t n_blocks, int weight_type, void *stream);

/* Bytes of an n x k weight matrix; the size rule of the dispatcher (reference
 * src/dsp/op_executor.cc:124-126) evaluated in 64 bits.  0 for an unknown type or k % 32 != 0. */
size_t htp_b200_weight_bytes(int weight_type, int64_t k, int64_t n);

/* Matmul for m <= 8 (decode kernel, either activation type) or for fp16 activations with m >= 9
 * (tensor-core kernel), k % 256 == 0, whose result y[m][n] is stored as the column band [dst_col0, dst_col0 + n) of n_dst (1..8) destination matrices
 * of dst_ld floats per token: the fused form of "matmul on my row shard, then all-gather".  A rank of
 * a row-sharded lm_head passes every rank's full logits buffer (its own and the peers' mapped
 * pointers, e.g. from CUDA IPC or symmetric memory) with dst_col0 = its first row: the epilogue's
 * tiled stores go to all of them while the next tile is being computed, and no gather kernel or copy
 * follows - only a cross-rank barrier before the logits are read.  No counterpart in the reference
 * (single DSP).  -1 for arguments outside this range; dst_ld, dst_col0 multiples of 32; every
 * destination 128-byte aligned. */
int htp_b200_mul_mat_multi_dst(void *const *dsts, int n_dst, int64_t dst_ld, int64_t dst_col0, const void *activation,
                               const void *weight, int m, int k, int n, int weight_type, int act_type, void *stream);

/* Decode form (m <= 8, one launch) of the call above that also SIGNALS: when the whole launch has
 * finished and its stores are visible system-wide, the kernel writes `epoch` to flags[d] for every
 * destination d - a 4-byte word in that destination GPU's memory reserved for THIS rank.  Together
 * with htp_b200_wait_flags on each GPU this replaces the all-gather AND the barrier of a row-sharded
 * decode step: rank r passes flags[d] = &(flag array of the GPU that owns dsts[d])[r].  Epochs must
 * increase from call to call (wrap-around safe).  The kernel stores each finished 32-row tile to every
 * destination as 16-byte stores (128 contiguous bytes per token and destination).  The flag says that
 * THIS rank's band has landed; it does not hold back the next step - see the caller's obligation at
 * htp_b200_mul_mat_gather_step.  No counterpart in the reference. */
int htp_b200_mul_mat_multi_dst_signal(void *const *dsts, int n_dst, int64_t dst_ld, int64_t dst_col0,
                                      const void *activation, const void *weight, int m, int k, int n, int weight_type,
                                      int act_type, uint32_t *const *flags, uint32_t epoch, void *stream);

/* One decode step of a row-sharded matrix in ONE call and ONE launch: htp_b200_mul_mat_multi_dst_signal
 * whose last CTA, after raising this rank's flags, waits (bounded to about a second, then error 103)
 * until local_flags[r] has reached `epoch` for r = 0 .. n_dst - 1.  local_flags is THIS GPU's flag
 * array (word r = rank r's flag), i.e. the array the peers' flags[] entries point into.  When the
 * stream reaches the end of the launch, every rank's band of this epoch is in this GPU's copy of the
 * output.  Every rank must issue the same sequence of steps (a rank's launch depends only on its own
 * earlier steps, so the ranks cannot wait for each other in a circle).  The caller's obligation: a rank may start step e + 1 - and overwrite its band in the
 * PEERS' copies - as soon as its own wait of step e has passed, so a consumer that still reads the
 * output of step e when the next step is issued needs two output buffers used in turn (or its own
 * cross-rank barrier).  No counterpart in the reference. */
int htp_b200_mul_mat_gather_step(void *const *dsts, int n_dst, int64_t dst_ld, int64_t dst_col0, const void *activation,
                                 const void *weight, int m, int k, int n, int weight_type, int act_type,
                                 uint32_t *const *flags, const uint32_t *local_flags, uint32_t epoch, void *stream);

/* Enqueues on `stream` a bounded wait until flags[r] has reached `epoch` for r = 0 .. n-1 (n <= 32):
 * every rank's band of this step has landed in this GPU's copy.  If a flag does not arrive within
 * about a second the stream's error word gets 103 (see htp_b200_stream_status); nothing hangs. */
int htp_b200_wait_flags(const uint32_t *flags, int n, uint32_t epoch, void *stream);

/* RMSNorm over ne1 rows of ne0 floats: y = x / sqrt(mean(x^2) + 1e-5) (eps fixed as in the reference).
 * Replaces hvx_rms_norm_f32 (reference include/dsp/ops.h:15, src/dsp/ops/rms_norm.c:68-84): same argument
 * rules (non-null, non-zero sizes, 128-byte aligned pointers -> else -1), device pointers + stream. */
int htp_b200_rms_norm_f32(float *dst, const float *src, int ne0, int ne1, void *stream);

/* Waits for `stream`, then returns and clears the first error code a kernel recorded on it
 * (0 = none), or -2 when the stream itself is in error. */
int htp_b200_stream_status(void *stream);

/* Tuning / debugging switches: "pdl" (programmatic dependent launch, default 1),
 * "force_generic" (route every matmul to the shape-agnostic kernel, default 0), "gemm_min_m"
 * (matmuls with at least this many tokens use the tensor-core GEMM - fp32 activations from 17 on at
 * the earliest -, default 9), "a32_exact" (1 = fp32
 * activations never go through the GEMM's fp16 conversion, default 0),
 * "gemm_tile_n" (tokens per GEMM tile: 0 = automatic, 128 or 256), "gemm_split" (when the GEMM's
 * tiles do not divide evenly among the SMs, cut the work into equal K ranges and finish the split
 * tiles through a scratch area, default 0), "permuted_weights" (op indices 2, 3 and 4 of
 * execute_op_simple / the message channel read HTP_B200_WT_PERMUTED buffers, as the reference's
 * ops of those numbers do, instead of standard ggml blocks; default 0).  Returns the previous value, or -1 for an unknown name. */
int htp_b200_set_option(const char *name, int value);

/* Number of kernel launches this process has issued through the library (all devices). */
uint64_t htp_b200_launch_count(void);

const char *htp_b200_version(void);

#ifdef __cplusplus
}
#endif

#endif /* HTP_OPS_B200_H */
