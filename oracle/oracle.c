/*
 * CPU oracle for the quantised MUL_MAT path.  TEST INFRASTRUCTURE ONLY: nothing in the
 * shipped library links or calls this file; only the test-suite, the smoke check and the
 * CPU-baseline leg of the benchmark may load it.
 *
 * PARITY UNPINNED: the reference's own tests never issue a Q4_0/Q8_0 matmul and hold no
 * golden vectors for it, and its implementation (HVX intrinsics + HMX inline asm) cannot be
 * compiled on a host compiler, so this restatement is anchored on the reference SOURCE
 * semantics cited below, not on reference outputs.
 *
 * What is restated, and from where (paths inside the reference project):
 *   - block layouts: include/dsp/quants.h:11-14 (block_q4_0, 18 B), :23-26 (block_q8_0, 34 B);
 *   - Q4_0 element order and value: element j<16 is the low nibble of byte j, element j+16 the
 *     high nibble of byte j (src/dsp/ops/mat_mul.c:266-271), value = nibble - 8 (LUT at :25-27);
 *   - Q8_0 element = signed byte (mat_mul.c:300-301);
 *   - dequantised weight = value * fp16 scale (mat_mul.c:290, 304);
 *   - W is N rows of K/32 consecutive blocks (mat_mul.c:580-581, 594-600);
 *   - activation [M][K] and output [M][N] row-major, output fp32 (include/op_reg.h:27-34,
 *     src/dsp/op_executor.cc:124-125, mat_mul.c:747-748);
 *   - loop shape out[i][j] += a[i][l] * w[l][j] of the in-tree scalar check (src/host/test.c:319-327).
 * The reference additionally rounds dequantised weights, activations and outputs to fp16 on its
 * matrix unit; the oracle does NOT: it is the exact fp64 dequantise-then-dot the tolerances are
 * stated against.
 *
 * The quantiser (fp32 -> blocks) exists nowhere in the reference; it follows the workload
 * description only:  Q4_0: d = (signed value of max |w|) / -8 stored as fp16,
 * q = clamp(round(w/d) + 8, 0, 15);  Q8_0: d = max|w| / 127 stored as fp16, q = round(w/d).
 * Free choices pinned here: the division uses the fp16-ROUNDED d (what the block stores),
 * round() is round-half-away-from-zero (roundf), a zero d gives q = 8 (Q4_0) / 0 (Q8_0),
 * Q8_0 q is clamped to [-128, 127].
 */
#define _GNU_SOURCE
#include <math.h>
#include <pthread.h>
#include <sched.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef _Float16 f16;

static inline float f16_bits_to_f32(uint16_t b) {
  f16 h;
  memcpy(&h, &b, 2);
  return (float) h;
}

static inline uint16_t f32_to_f16_bits(float f) {
  f16      h = (f16) f; /* round to nearest even */
  uint16_t b;
  memcpy(&b, &h, 2);
  return b;
}

/* ---------------------------------------------------------------- thread fan-out helper */

typedef void (*range_fn)(void *ctx, int64_t begin, int64_t end);

struct range_job {
  range_fn fn;
  void    *ctx;
  int64_t  begin, end;
};

static void *range_thread(void *p) {
  struct range_job *j = (struct range_job *) p;
  j->fn(j->ctx, j->begin, j->end);
  return NULL;
}

int htp_oracle_usable_cores(void) {
  cpu_set_t set;
  CPU_ZERO(&set);
  if (sched_getaffinity(0, sizeof(set), &set) != 0) {
    return 1;
  }
  int c = CPU_COUNT(&set);
  return c > 0 ? c : 1;
}

static void parallel_ranges(range_fn fn, void *ctx, int64_t total, int n_threads) {
  if (n_threads <= 0) {
    n_threads = htp_oracle_usable_cores();
  }
  if (n_threads > 256) {
    n_threads = 256;
  }
  if (n_threads > total) {
    n_threads = total > 0 ? (int) total : 1;
  }
  if (n_threads == 1) {
    fn(ctx, 0, total);
    return;
  }
  pthread_t        tids[256];
  struct range_job jobs[256];
  int64_t          chunk = (total + n_threads - 1) / n_threads;
  int              started = 0;
  for (int t = 0; t < n_threads; ++t) {
    int64_t b = t * chunk, e = b + chunk;
    if (b >= total) {
      break;
    }
    if (e > total) {
      e = total;
    }
    jobs[t] = (struct range_job){ fn, ctx, b, e };
    if (pthread_create(&tids[t], NULL, range_thread, &jobs[t]) != 0) {
      fn(ctx, b, e);
      tids[t] = 0;
      jobs[t].fn = NULL;
    }
    started = t + 1;
  }
  for (int t = 0; t < started; ++t) {
    if (jobs[t].fn) {
      pthread_join(tids[t], NULL);
    }
  }
}

/* ---------------------------------------------------------------- fp16 helpers (exported) */

void htp_oracle_f32_to_f16(const float *src, uint16_t *dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    dst[i] = f32_to_f16_bits(src[i]);
  }
}

void htp_oracle_f16_to_f32(const uint16_t *src, float *dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    dst[i] = f16_bits_to_f32(src[i]);
  }
}

/* ---------------------------------------------------------------- quantiser */

struct quant_ctx {
  const float *w;
  uint8_t     *out;
  int64_t      k;
};

static void quantize_rows_q4_0(void *p, int64_t r0, int64_t r1) {
  struct quant_ctx *c  = (struct quant_ctx *) p;
  const int64_t     nb = c->k / 32;
  for (int64_t r = r0; r < r1; ++r) {
    for (int64_t b = 0; b < nb; ++b) {
      const float *x   = c->w + r * c->k + b * 32;
      uint8_t     *blk = c->out + (r * nb + b) * 18;
      float        amax = 0.0f, vmax = 0.0f;
      for (int i = 0; i < 32; ++i) {
        float a = fabsf(x[i]);
        if (a > amax) {
          amax = a;
          vmax = x[i];
        }
      }
      uint16_t dbits = f32_to_f16_bits(vmax / -8.0f);
      float    d     = f16_bits_to_f32(dbits);
      memcpy(blk, &dbits, 2);
      for (int i = 0; i < 16; ++i) {
        int q0 = 8, q1 = 8;
        if (d != 0.0f) {
          q0 = (int) roundf(x[i] / d) + 8;
          q1 = (int) roundf(x[i + 16] / d) + 8;
        }
        q0 = q0 < 0 ? 0 : (q0 > 15 ? 15 : q0);
        q1 = q1 < 0 ? 0 : (q1 > 15 ? 15 : q1);
        blk[2 + i] = (uint8_t) (q0 | (q1 << 4));
      }
    }
  }
}

static void quantize_rows_q8_0(void *p, int64_t r0, int64_t r1) {
  struct quant_ctx *c  = (struct quant_ctx *) p;
  const int64_t     nb = c->k / 32;
  for (int64_t r = r0; r < r1; ++r) {
    for (int64_t b = 0; b < nb; ++b) {
      const float *x    = c->w + r * c->k + b * 32;
      uint8_t     *blk  = c->out + (r * nb + b) * 34;
      float        amax = 0.0f;
      for (int i = 0; i < 32; ++i) {
        float a = fabsf(x[i]);
        if (a > amax) {
          amax = a;
        }
      }
      uint16_t dbits = f32_to_f16_bits(amax / 127.0f);
      float    d     = f16_bits_to_f32(dbits);
      memcpy(blk, &dbits, 2);
      for (int i = 0; i < 32; ++i) {
        int q = 0;
        if (d != 0.0f) {
          q = (int) roundf(x[i] / d);
        }
        q = q < -128 ? -128 : (q > 127 ? 127 : q);
        blk[2 + i] = (uint8_t) (int8_t) q;
      }
    }
  }
}

/* IQ4_NL: the 18-byte block of Q4_0 with a non-linear value table instead of q - 8
 * (reference table: src/dsp/ops/mat_mul.c:29-32; it is ggml's kvalues_iq4nl). */
static const int8_t kIq4nlValues[16] = { -127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113 };

/* Packer for synthetic IQ4_NL weights: d = (signed value of max |w|) / -127 rounded to fp16, each
 * element takes the table entry nearest to w / d (ggml's quantiser without its scale search). */
static void quantize_rows_iq4_nl(void *p, int64_t r0, int64_t r1) {
  struct quant_ctx *c  = (struct quant_ctx *) p;
  const int64_t     nb = c->k / 32;
  for (int64_t r = r0; r < r1; ++r) {
    for (int64_t b = 0; b < nb; ++b) {
      const float *x   = c->w + r * c->k + b * 32;
      uint8_t     *blk = c->out + (r * nb + b) * 18;
      float        amax = 0.0f, vmax = 0.0f;
      for (int i = 0; i < 32; ++i) {
        float a = fabsf(x[i]);
        if (a > amax) {
          amax = a;
          vmax = x[i];
        }
      }
      uint16_t dbits = f32_to_f16_bits(vmax / -127.0f);
      float    d     = f16_bits_to_f32(dbits);
      memcpy(blk, &dbits, 2);
      uint8_t q[32];
      for (int i = 0; i < 32; ++i) {
        int best = 8;  /* value 1, the entry nearest to 0 */
        if (d != 0.0f) {
          const float t    = x[i] / d;
          float       berr = fabsf(t - (float) kIq4nlValues[0]);
          best             = 0;
          for (int j = 1; j < 16; ++j) {
            const float e = fabsf(t - (float) kIq4nlValues[j]);
            if (e < berr) {
              berr = e;
              best = j;
            }
          }
        }
        q[i] = (uint8_t) best;
      }
      for (int i = 0; i < 16; ++i) {
        blk[2 + i] = (uint8_t) (q[i] | (q[i + 16] << 4));
      }
    }
  }
}

/* type: 2 = Q4_0, 8 = Q8_0, 20 = IQ4_NL (ggml numbering).  Returns bytes written, or -1. */
int64_t htp_oracle_quantize(const float *w, uint8_t *out, int64_t n_rows, int64_t k, int type, int n_threads) {
  if (k % 32 != 0 || (type != 2 && type != 8 && type != 20)) {
    return -1;
  }
  struct quant_ctx c = { w, out, k };
  parallel_ranges(type == 2 ? quantize_rows_q4_0 : (type == 8 ? quantize_rows_q8_0 : quantize_rows_iq4_nl), &c, n_rows,
                  n_threads);
  return n_rows * (k / 32) * (type == 8 ? 34 : 18);
}

/* ---------------------------------------------------------------- unpack (the contract) */

static inline void unpack_block(const uint8_t *blk, int type, int8_t v[32], float *d) {
  uint16_t dbits;
  memcpy(&dbits, blk, 2);
  *d = f16_bits_to_f32(dbits);
  if (type == 2) {
    for (int i = 0; i < 16; ++i) {
      v[i]      = (int8_t) ((blk[2 + i] & 0x0F) - 8);
      v[i + 16] = (int8_t) ((blk[2 + i] >> 4) - 8);
    }
  } else if (type == 20) {  /* same nibble order, table values (mat_mul.c:316, 583) */
    for (int i = 0; i < 16; ++i) {
      v[i]      = kIq4nlValues[blk[2 + i] & 0x0F];
      v[i + 16] = kIq4nlValues[blk[2 + i] >> 4];
    }
  } else {
    for (int i = 0; i < 32; ++i) {
      v[i] = (int8_t) blk[2 + i];
    }
  }
}

static inline int block_bytes(int type) {
  return (type == 2 || type == 20) ? 18 : (type == 8 ? 34 : 0);
}

/* dequantise rows [0, n_rows) to fp32 (exact: |value| <= 128 times an fp16 fits fp32). */
int htp_oracle_dequantize(const uint8_t *wq, float *out, int64_t n_rows, int64_t k, int type) {
  const int bb = block_bytes(type);
  if (!bb || k % 32) {
    return -1;
  }
  const int64_t nb = k / 32;
  for (int64_t r = 0; r < n_rows; ++r) {
    for (int64_t b = 0; b < nb; ++b) {
      int8_t v[32];
      float  d;
      unpack_block(wq + (r * nb + b) * bb, type, v, &d);
      for (int i = 0; i < 32; ++i) {
        out[r * k + b * 32 + i] = (float) v[i] * d;
      }
    }
  }
  return 0;
}

/* Per-block integer sums: S_b = sum_i value_i, T_b = sum_i (i+1) * value_i, int32.
 * The plain sum is blind to element order, the weighted one is not. */
int htp_oracle_block_sums(const uint8_t *wq, int32_t *s_out, int32_t *t_out, int64_t n_blocks, int type) {
  const int bb = block_bytes(type);
  if (!bb) {
    return -1;
  }
  for (int64_t b = 0; b < n_blocks; ++b) {
    int8_t v[32];
    float  d;
    unpack_block(wq + b * bb, type, v, &d);
    int32_t s = 0, t = 0;
    for (int i = 0; i < 32; ++i) {
      s += v[i];
      t += (i + 1) * v[i];
    }
    s_out[b] = s;
    t_out[b] = t;
  }
  return 0;
}

/* ---------------------------------------------------------------- matmul */

struct mm_ctx {
  const uint8_t *wq;
  const void    *act;
  int            act_is_f16;
  void          *out; /* double* (oracle) or float* (baseline) */
  double        *absdot; /* optional: sum_l |x_l * w_l| per output, for condition-normalised error */
  int64_t        m, k, n;
  int            type;
  int64_t        row_begin; /* first output row (column of y) this call covers */
};

static inline double act_at(const struct mm_ctx *c, int64_t i, int64_t l) {
  if (c->act_is_f16) {
    return (double) f16_bits_to_f32(((const uint16_t *) c->act)[i * c->k + l]);
  }
  return (double) ((const float *) c->act)[i * c->k + l];
}

/* fp64 oracle: exact dequantised weight (value * d, in double), fp64 accumulate. */
static void mm_rows_f64(void *p, int64_t j0, int64_t j1) {
  struct mm_ctx *c  = (struct mm_ctx *) p;
  const int      bb = block_bytes(c->type);
  const int64_t  nb = c->k / 32;
  double        *y  = (double *) c->out;
  double        *wrow = (double *) malloc(sizeof(double) * c->k);
  for (int64_t j = j0; j < j1; ++j) {
    for (int64_t b = 0; b < nb; ++b) {
      int8_t v[32];
      float  d;
      unpack_block(c->wq + (j * nb + b) * bb, c->type, v, &d);
      for (int i = 0; i < 32; ++i) {
        wrow[b * 32 + i] = (double) v[i] * (double) d;
      }
    }
    for (int64_t i = 0; i < c->m; ++i) {
      double acc = 0.0, aabs = 0.0;
      for (int64_t l = 0; l < c->k; ++l) {
        double t = act_at(c, i, l) * wrow[l];
        acc += t;
        aabs += fabs(t);
      }
      y[i * c->n + j] = acc;
      if (c->absdot) {
        c->absdot[i * c->n + j] = aabs;
      }
    }
  }
  free(wrow);
}

/* y[m][n] (double) = act[m][k] . W[n][k]^T.  act_is_f16: activations are fp16 bit patterns.
 * absdot may be NULL. */
int htp_oracle_mul_mat_f64(double *y, double *absdot, const void *act, int act_is_f16, const uint8_t *wq, int64_t m,
                           int64_t k, int64_t n, int type, int n_threads) {
  if (!block_bytes(type) || k % 32 || m <= 0 || n <= 0 || k <= 0) {
    return -1;
  }
  struct mm_ctx c = { wq, act, act_is_f16, y, absdot, m, k, n, type, 0 };
  parallel_ranges(mm_rows_f64, &c, n, n_threads);
  return 0;
}

/* ---------------------------------------------------------------- weights in tile order
 *
 * The reference's own weight buffers are stored in 32 x 32 tile order: tile (n/32, k/32) is tile
 * number (n/32) * (K/32) + k/32, and inside a tile element (k, n) is halfword slot
 * T = (k & ~1) * 32 + n * 2 + (k & 1) (src/host/test.c:303-313 writes fp16 weights that way for
 * hmx_mat_mul_permuted_w16a32; src/dsp/ops/mat_mul.c:594-605 scatters dequantised groups the same
 * way).  Formats, by the library's weight_type code:
 *   1      fp16 tiles, 2048 B each: the slot holds the weight.
 *   0x102  my_block_q4_0 (include/dsp/quants.h:16-19): 144-byte super-blocks, four per tile, each
 *          8 fp16 scales then quants[128] covering slots T = 256 * sb + t.  With v = t / 64 and
 *          s = t % 64 the nibble of slot t is quants[2s] & 15 (v = 0), quants[2s + 1] & 15 (v = 1),
 *          quants[2s] >> 4 (v = 2), quants[2s + 1] >> 4 (v = 3): mat_mul.c:373-376 looks up the low
 *          and the high nibbles of all 128 bytes, the lookup returns even bytes in its first and odd
 *          bytes in its second vector, and :402-405 stores the four vectors in that order.  value =
 *          nibble - 8 (table at :25-27), scale = scales[t / 32] (index tables :318-325, :396-400).
 *   0x114  the same block with the IQ4_NL table (:29-32, selected at :316).
 *   0x108  my_block_q8_0 (quants.h:28-31): 272-byte super-blocks, 8 fp16 scales then quants[256];
 *          slot t = (int8) quants[t] in order (:472-489), scale = scales[t / 32].
 * PARITY UNPINNED for the three permuted formats: no producer, test or fixture of them exists in
 * the reference; the slot order above is read off the vector code and rests on the lookup
 * instruction's even/odd split, which the un-coalesced branch of the same function (:345-372,
 * eight standard groups -> four vectors) agrees with.  The fp16 format is pinned by test.c's
 * index formula.
 */
static int tiled_tile_bytes(int fmt) {
  return fmt == 1 ? 2048 : (fmt == 0x108 ? 1088 : ((fmt == 0x102 || fmt == 0x114) ? 576 : 0));
}

/* out[j * k + l] (fp32, exact) = weight of input l for output j, for all n outputs. */
int htp_oracle_tiled_dequantize(const uint8_t *w, float *out, int64_t k, int64_t n, int fmt) {
  const int tb = tiled_tile_bytes(fmt);
  if (!tb || k <= 0 || n <= 0 || k % 32 || n % 32) {
    return -1;
  }
  const int64_t kt_n = k / 32;
  for (int64_t nt = 0; nt < n / 32; ++nt) {
    for (int64_t kt = 0; kt < kt_n; ++kt) {
      const uint8_t *tile = w + (nt * kt_n + kt) * tb;
      for (int T = 0; T < 1024; ++T) {
        const int r = (T / 64) * 2 + (T & 1); /* k within the tile */
        const int c = (T % 64) / 2;           /* n within the tile */
        float     val;
        if (fmt == 1) {
          uint16_t h;
          memcpy(&h, tile + 2 * T, 2);
          val = f16_bits_to_f32(h);
        } else {
          const int      sb   = T / 256, t = T % 256;
          const int      sbb  = tb / 4;
          const uint8_t *blk  = tile + sb * sbb;
          uint16_t       dbits;
          memcpy(&dbits, blk + 2 * (t / 32), 2);
          const float d = f16_bits_to_f32(dbits);
          int         q;
          if (fmt == 0x108) {
            q = (int8_t) blk[16 + t];
          } else {
            const int     v = t / 64, s = t % 64;
            const uint8_t b   = blk[16 + 2 * s + (v & 1)];
            const int     nib = v < 2 ? (b & 0x0F) : (b >> 4);
            q = fmt == 0x102 ? nib - 8 : kIq4nlValues[nib];
          }
          val = (float) q * d;
        }
        out[(nt * 32 + c) * k + kt * 32 + r] = val;
      }
    }
  }
  return 0;
}

/* Integer sums per scale group of the permuted super-blocks (fmt 0x102, 0x108, 0x114): group g of
 * super-block sb covers its slots t = 32 g .. 32 g + 31; S = sum_j q_j, T = sum_j (j + 1) q_j with
 * j = t % 32 and q the slot's integer value read exactly as in htp_oracle_tiled_dequantize. */
int htp_oracle_tiled_group_sums(const uint8_t *w, int32_t *s_out, int32_t *t_out, int64_t n_super_blocks, int fmt) {
  if (fmt != 0x102 && fmt != 0x108 && fmt != 0x114) {
    return -1;
  }
  const int sbb = tiled_tile_bytes(fmt) / 4;
  for (int64_t sb = 0; sb < n_super_blocks; ++sb) {
    const uint8_t *blk = w + sb * sbb;
    for (int g = 0; g < 8; ++g) {
      int32_t S = 0, T = 0;
      for (int j = 0; j < 32; ++j) {
        const int t = 32 * g + j;
        int       q;
        if (fmt == 0x108) {
          q = (int8_t) blk[16 + t];
        } else {
          const int     v = t / 64, sl = t % 64;
          const uint8_t b   = blk[16 + 2 * sl + (v & 1)];
          const int     nib = v < 2 ? (b & 0x0F) : (b >> 4);
          q = fmt == 0x102 ? nib - 8 : kIq4nlValues[nib];
        }
        S += q;
        T += (j + 1) * q;
      }
      s_out[sb * 8 + g] = S;
      t_out[sb * 8 + g] = T;
    }
  }
  return 0;
}

struct mmd_ctx {
  const float *wd;
  const void  *act;
  int          act_is_f16;
  double      *y, *absdot;
  int64_t      m, k, n;
};

static void mmd_rows_f64(void *p, int64_t j0, int64_t j1) {
  struct mmd_ctx *c = (struct mmd_ctx *) p;
  for (int64_t j = j0; j < j1; ++j) {
    for (int64_t i = 0; i < c->m; ++i) {
      double acc = 0.0, aabs = 0.0;
      for (int64_t l = 0; l < c->k; ++l) {
        const double a = c->act_is_f16 ? (double) f16_bits_to_f32(((const uint16_t *) c->act)[i * c->k + l])
                                       : (double) ((const float *) c->act)[i * c->k + l];
        const double t = a * (double) c->wd[j * c->k + l];
        acc += t;
        aabs += fabs(t);
      }
      c->y[i * c->n + j] = acc;
      if (c->absdot) {
        c->absdot[i * c->n + j] = aabs;
      }
    }
  }
}

/* fp64 oracle over a dense fp32 weight matrix wd[n][k] (as htp_oracle_tiled_dequantize returns):
 * y[m][n] = act[m][k] . wd^T in the loop shape of src/host/test.c:319-327, double accumulate. */
int htp_oracle_mul_mat_dense_f64(double *y, double *absdot, const void *act, int act_is_f16, const float *wd,
                                 int64_t m, int64_t k, int64_t n, int n_threads) {
  if (m <= 0 || n <= 0 || k <= 0) {
    return -1;
  }
  struct mmd_ctx c = { wd, act, act_is_f16, y, absdot, m, k, n };
  parallel_ranges(mmd_rows_f64, &c, n, n_threads);
  return 0;
}

/* Timed CPU baseline: same dequantise-then-dot, fp32 weights and fp32 accumulation, threads
 * over output rows.  The activation rows are converted to fp32 once up front. */
struct mm32_ctx {
  const uint8_t *wq;
  const float   *act32;
  float         *y;
  int64_t        m, k, n;
  int            type;
};

static void mm_rows_f32(void *p, int64_t j0, int64_t j1) {
  struct mm32_ctx *c  = (struct mm32_ctx *) p;
  const int        bb = block_bytes(c->type);
  const int64_t    nb = c->k / 32;
  float           *wrow = (float *) malloc(sizeof(float) * c->k);
  for (int64_t j = j0; j < j1; ++j) {
    const uint8_t *row = c->wq + j * nb * bb;
    if (c->type == 2) {
      for (int64_t b = 0; b < nb; ++b) {
        const uint8_t *blk = row + b * 18;
        uint16_t       dbits;
        memcpy(&dbits, blk, 2);
        const float d  = f16_bits_to_f32(dbits);
        float      *wo = wrow + b * 32;
        for (int i = 0; i < 16; ++i) {
          wo[i]      = (float) ((int) (blk[2 + i] & 0x0F) - 8) * d;
          wo[i + 16] = (float) ((int) (blk[2 + i] >> 4) - 8) * d;
        }
      }
    } else if (c->type == 8) {
      for (int64_t b = 0; b < nb; ++b) {
        const uint8_t *blk = row + b * 34;
        uint16_t       dbits;
        memcpy(&dbits, blk, 2);
        const float d  = f16_bits_to_f32(dbits);
        float      *wo = wrow + b * 32;
        for (int i = 0; i < 32; ++i) {
          wo[i] = (float) (int8_t) blk[2 + i] * d;
        }
      }
    } else {
      for (int64_t b = 0; b < nb; ++b) {
        int8_t v[32];
        float  d;
        unpack_block(row + b * bb, c->type, v, &d);
        for (int i = 0; i < 32; ++i) {
          wrow[b * 32 + i] = (float) v[i] * d;
        }
      }
    }
    for (int64_t i = 0; i < c->m; ++i) {
      const float *a = c->act32 + i * c->k;
      float        acc[8] = { 0 };
      for (int64_t l = 0; l < c->k; l += 8) {
        for (int u = 0; u < 8; ++u) {
          acc[u] += a[l + u] * wrow[l + u];
        }
      }
      c->y[i * c->n + j] = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
    }
  }
  free(wrow);
}

int htp_oracle_mul_mat_f32(float *y, const void *act, int act_is_f16, const uint8_t *wq, int64_t m, int64_t k,
                           int64_t n, int type, int n_threads) {
  if (!block_bytes(type) || k % 32 || m <= 0 || n <= 0 || k <= 0) {
    return -1;
  }
  float *act32 = NULL;
  if (act_is_f16) {
    act32 = (float *) malloc(sizeof(float) * m * k);
    htp_oracle_f16_to_f32((const uint16_t *) act, act32, m * k);
  }
  struct mm32_ctx c = { wq, act_is_f16 ? act32 : (const float *) act, y, m, k, n, type };
  parallel_ranges(mm_rows_f32, &c, n, n_threads);
  free(act32);
  return 0;
}

/* ---------------------------------------------------------------- RMSNorm (next-row f1)
 *
 * Restates the reference's scalar statement rms_norm_f32_ref (src/host/test.c:60-80): per row
 * sum of squares, mean = sum / ne0, scale = 1 / sqrt(mean + 1e-5), y = x * scale.  wide != 0
 * accumulates the sum in double (the gate the GPU kernel is held to); wide == 0 is the reference's
 * own float loop, term by term.  Argument rules as hvx_rms_norm_f32 (src/dsp/ops/rms_norm.c:69-71). */
int htp_oracle_rms_norm_f32(float *dst, const float *src, int64_t ne0, int64_t ne1, int wide) {
  if (!dst || !src || ne0 <= 0 || ne1 <= 0) {
    return -1;
  }
  const float eps = 1e-5f;
  for (int64_t j = 0; j < ne1; ++j) {
    const float *x = src + j * ne0;
    float       *y = dst + j * ne0;
    float        scale;
    if (wide) {
      double sum = 0.0;
      for (int64_t i = 0; i < ne0; ++i) {
        sum += (double) x[i] * (double) x[i];
      }
      scale = (float) (1.0 / sqrt(sum / (double) ne0 + (double) eps));
    } else {
      float sum = 0;
      for (int64_t i = 0; i < ne0; ++i) {
        sum += x[i] * x[i];
      }
      const float mean = sum / ne0;
      scale            = 1.0f / sqrtf(mean + eps);
    }
    for (int64_t i = 0; i < ne0; ++i) {
      y[i] = x[i] * scale;
    }
  }
  return 0;
}
