// K2 - prefill-side quantised GEMM (M >= 64, fp16 activations): y[M][N] = x[M][K] . W[N][K]^T with
// fp32 accumulation on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM).
//
// Replaces the reference's HVX dequantise -> HMX 32x32 tile loop (src/dsp/ops/mat_mul.c:702-726,
// 928-1005).  Like the reference the weights are dequantised to fp16, value * scale rounded once
// (mat_mul.c:290, 304); unlike it the accumulator and the output stay fp32.
//
// The product is computed transposed, D[weight row][token] = W . x^T, so that the dequantised
// weights are the MMA's A operand and can live in TENSOR MEMORY: the dequantisation warps write
// their fp16 values straight into TMEM with tcgen05.st and the MMA reads them from there
// (tcgen05.mma with A in TMEM, B = the activation tile in shared memory).  Compared with putting
// the dequantised tile in shared memory this removes the 128-byte-swizzled stores, the proxy
// fences and two thirds of the shared-memory traffic per K step, which is what bounds a
// one-CTA UMMA pipeline.
//
// Two flavours.  M <= 128: one persistent CTA per SM, tile = 128 weight rows x 128 tokens,
// tcgen05.mma.cta_group::1.  M > 128: persistent CTA PAIRS (a cluster of two SMs), pair tile = 256
// weight rows x 256 tokens, tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 16): each CTA dequantises
// its own 128 weight rows into its own tensor memory and loads only ITS half (128 tokens) of the
// activation tile - the tensor cores of both SMs read both halves.  No multicast loads: every CTA
// fetches its own operands; the other CTA's copy engine and dequantisation warps signal the
// leader's barriers directly, and tcgen05.commit multicasts its arrival to the pair.
//
// K advances in steps of 64 through ONE ring of 8 slots; slot i holds the activation tile
// (shared memory) and the dequantised weight tile (32 TMEM columns) of one K step.  A group of
// consecutive slots (two for CTA pairs, a raw stage for single-CTA tiles) is filled behind one `full`
// barrier and released by one tcgen05.commit on one `empty` barrier: the issuing thread's waits and
// commits cost it hundreds of clocks each.
//
// Roles per CTA:
//   warp 0      TMA producer of the activation tile (128 tokens x 64 fp16, 128-byte swizzle)
//   warp 1      MMA issuer (leader CTA of a pair only): the whole warp runs the loop, one elected
//               lane issues; one wait and one commit per group of K steps, four MMAs per step
//   warp 2      TMEM allocation: columns 0..255 accumulator, 256..511 the ring of A tiles
//   warps 4-7   epilogue: tcgen05.ld of the accumulator 16 tokens at a time -> shared-memory
//               staging -> TMA store to y[token][weight row]; the accumulator is released after
//               the last load, the stores drain under the next tile
//   warps 8-15  dequantisation, two groups of four warps; group g takes the raw stages (256 weights
//               per row) whose running index is g (mod 2).  A warp fetches the 144 / 272 raw bytes
//               of its 32 rows itself (coalesced cp.async, one stage ahead); thread = one weight
//               row: 9 / 17 conflict-free 16-byte loads to registers, then per K step 64 weights to
//               fp16 (value * scale, rounded once) stored as 32 TMEM columns of its lane
// Weight formats: the row-major 32-weight blocks (Q4_0, Q8_0, IQ4_NL) and, read in place, the
// reference's 32 x 32 tile order - fp16 tiles (its W16A32 op) and the permuted super-blocks its
// quantised ops consume (include/dsp/quants.h:16-31, src/dsp/ops/mat_mul.c:308-510): there a warp's
// 32 rows are one column tile, a raw stage is 128 of K = four contiguous tiles, and the unpack is a
// copy (fp16) or one 16-byte chunk per super-block (eight k-rows of the thread's column).
// Optionally (off by default) tiles that do not divide among the SMs are cut into equal K ranges
// and finished through a global scratch tile.
// All waits are bounded; a wait that runs out records an error code, raises the CTA's abort flag
// and every role leaves its loop; TMEM is freed before the CTA exits.
#include "gemm_tcgen05.h"

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdlib.h>

#include "device_ctx.h"
#include "ptx.cuh"
#include "unpack.cuh"

namespace htp {

namespace {

constexpr int kBW        = 128;  // weight rows per tile (UMMA M, the TMEM lanes)
constexpr int kBK        = 64;   // K per pipeline step: one 128-byte swizzled row of fp16
constexpr int kF16T      = 3;    // weight "format" of this file only: fp16 values in the reference's 32 x 32 tile order
constexpr int kPQ4       = 4;    // the reference's permuted super-blocks in the same tile order: Q4_0 (144 bytes),
constexpr int kPQ8       = 5;    // Q8_0 (272 bytes),
constexpr int kPIQ4      = 6;    // IQ4_NL values in Q4_0's layout
constexpr int kNAT       = 8;    // A tiles (32 TMEM columns each) in the tensor-memory ring
constexpr int kThreads   = 512;
constexpr int kEpiWarp0  = 4;
constexpr int kDeqWarp0  = 8;    // warps 8-11: group 0, warps 12-15: group 1
constexpr int kTmemCols  = 512;
constexpr int kTmemA     = 256;  // first column of the A ring
constexpr int kOutTok    = 16;      // tokens per output store (one TMA box of 32 weight rows x 16 tokens)
constexpr int kSmemLimit = 232448;  // opt-in dynamic shared memory per CTA
constexpr uint32_t kFlagWaitCap = 1u << 22;  // polls of the other contributor's flag (about a second)

}  // namespace
template <>
struct BlockTraits<3> {  // kF16T: 32 fp16 weights of a row
  static constexpr int kBytes = 64;
};
// permuted super-blocks: the bytes per row and 32 of K come to the same 18 / 34 as the row-major blocks
template <>
struct BlockTraits<4> {
  static constexpr int kBytes = 18;
};
template <>
struct BlockTraits<5> {
  static constexpr int kBytes = 34;
};
template <>
struct BlockTraits<6> {
  static constexpr int kBytes = 18;
};
namespace {

template <int WT, int BT, bool TWO>
struct GCfg {
  static constexpr bool TILED    = WT == kF16T;
  static constexpr bool PERM     = WT >= kPQ4;  // permuted super-blocks, four per 32 x 32 tile
  // A raw stage = the bytes of RAWK weights per row, fetched and unpacked as one unit: 256 weights of
  // the block formats (a 16-byte aligned period of 8 blocks), 128 of the tile-order formats (four
  // tiles of 2048 / 576 / 1088 bytes per 32 rows).
  static constexpr int RAWK      = (TILED || PERM) ? 128 : 256;
  static constexpr int TILE_B    = TILED ? 2048 : (WT == kPQ8 ? 1088 : 576);  // bytes of a tile (tile-order formats)
  static constexpr int PIECES    = (RAWK / 32) * TILE_B / 16;  // 16-byte pieces of a warp's raw stage (tile-order formats)
  static_assert(TILE_B % 16 == 0 && PIECES > 0, "tiles are copied in 16-byte pieces");
  static constexpr int Q         = RAWK / kBK;  // K steps per raw stage
  static constexpr int NG        = kNAT / Q;    // raw stages the ring of K steps holds
  static constexpr int BB        = BlockTraits<WT>::kBytes;
  static constexpr int RB        = (RAWK / 32) * BB;  // raw bytes per row and raw stage: 144 / 272 / 256
  static constexpr int RW        = RB / 16;           // 16-byte words per row: 9 / 17 / 16 (row-major blocks, fp16 tiles)
  static constexpr int XROWS     = TWO ? BT / 2 : BT;  // activation rows this CTA loads per K step
  static constexpr int X_BYTES   = XROWS * 128;
  static constexpr int RAW_BYTES = kBW * RB;
  static constexpr int STAGE_OUT = 4 * 2 * kOutTok * 32 * 4;  // 4 epilogue warps x 2 buffers x 16 tokens x 32 rows
  static constexpr int FIXED     = 2 * ((RAW_BYTES + 127) & ~127) + 1024 + 512 + STAGE_OUT;  // raw ring, slack, barriers, output staging
  static constexpr int NX        = kNAT;  // activation stages: the same ring as the A tiles
  // K steps that share one full / empty barrier pair: two for CTA pairs (their MMAs take longer than the
  // issuing thread's wait and commit), a whole raw stage for single-CTA tiles, whose small MMAs leave the
  // issuing thread as the limit
  static constexpr int BSTEPS    = TWO ? 2 : Q;
  static_assert(Q % BSTEPS == 0 && kNAT % BSTEPS == 0, "barrier groups do not straddle raw stages");
  static_assert(NX * X_BYTES + FIXED <= kSmemLimit, "shared memory");
};

// One ring of kNAT K steps.  Slot i holds the activation tile (shared memory) and the dequantised
// weight tile (tensor memory) of one K step; both are filled behind ONE barrier and released by
// ONE tcgen05.commit, so the MMA issuer waits once and commits once per K step.
// tensor maps of the output destinations (one per destination matrix, all of the same shape)
struct GemmDstMaps {
  CUtensorMap m[kGemmMaxDst];
};

struct GSmemBar {
  uint64_t full[kNAT], empty[kNAT];
  uint64_t acc_full, acc_empty;
  uint32_t tmem_base;
  int      abort_flag;
};
static_assert(sizeof(GSmemBar) <= 512, "barrier block");

// ---------------------------------------------------------------- tcgen05 wrappers

template <bool TWO>
__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t ncols) {
  if constexpr (TWO) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
                 "r"(ncols)
                 : "memory");
  } else {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
                 "r"(ncols)
                 : "memory");
  }
}
template <bool TWO>
__device__ __forceinline__ void tmem_relinquish() {
  if constexpr (TWO) {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  } else {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
}
template <bool TWO>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (TWO) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
  } else {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
  }
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// all threads of both CTAs of the pair
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// one arrival on the mbarrier at the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ void mbar_arrive_remote(uint64_t *bar, uint32_t rank) {
  asm volatile(
    "{\n\t.reg .b32 ra;\n\t"
    "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
    "mbarrier.arrive.shared::cluster.b64 _, [ra];\n\t}" ::"r"(smem_u32(bar)),
    "r"(rank)
    : "memory");
}
// true in exactly one lane of the (converged) warp
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
    "{\n\t.reg .pred p;\n\t"
    "elect.sync _|p, 0xffffffff;\n\t"
    "selp.u32 %0, 1, 0, p;\n\t}"
    : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Tiled TMA load whose completion is signalled on the LEADER CTA's mbarrier (the barrier at this
// shared-memory offset in the even CTA of the pair); the data goes to this CTA's shared memory.
// No multicast: each CTA fetches its own box.
__device__ __forceinline__ void tma_load_2d_pair(void *dst_smem, const void *tmap, int x, int y, uint64_t *bar,
                                                 uint64_t policy) {
  const uint32_t leader_bar = smem_u32(bar) & 0xFEFFFFFFu;  // bit 24 of a shared::cluster address: CTA rank
  asm volatile(
    "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
    "[%0], [%1, {%2, %3}], [%4], %5;" ::"r"(smem_u32(dst_smem)),
    "l"(tmap), "r"(x), "r"(y), "r"(leader_bar), "l"(policy)
    : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem desc]; issued by ONE thread (of the leader CTA for a pair)
template <bool TWO>
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  if constexpr (TWO) {
    asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
  } else {
    asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
  }
}
// The mbarrier gets one arrival when every MMA issued so far by this thread has completed; for a
// pair the arrival is delivered to the barrier at this offset in BOTH CTAs.
template <bool TWO>
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
  if constexpr (TWO) {
    asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
        smem_u32(bar)),
      "h"((uint16_t) 3)
      : "memory");
  } else {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
  }
}
// 16 columns of this thread's TMEM lane -> 16 registers, asynchronously: the registers hold the
// values only after tmem_ld_wait on the same array
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr)
               : "memory");
}
// Waits for every tcgen05.ld of this thread.  The registers pass through the statement so that
// the compiler cannot read or move them before the wait.
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
}
// 2-D tiled tensor store shared memory -> global through a tensor map (elements outside the
// tensor are not written); completion is tracked by the issuing thread's bulk groups (bulk_commit).
__device__ __forceinline__ void tma_store_2d(const void *tmap, int x, int y, uint32_t src_smem) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(tmap), "r"(x), "r"(y),
               "r"(src_smem)
               : "memory");
}
// closes the bulk group of the stores issued since the last commit
__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// at most N of this thread's bulk groups still have to READ their shared-memory source
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
// generic-proxy writes to shared memory before this fence are visible to the copy engine after it
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// 32 columns of this thread's TMEM lane <- 32 registers, asynchronously: complete after tmem_st_wait
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint4 (&o)[8]) {
  asm volatile(
    "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
    "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
    "%30,%31,%32};" ::"r"(taddr),
    "r"(o[0].x), "r"(o[0].y), "r"(o[0].z), "r"(o[0].w), "r"(o[1].x), "r"(o[1].y), "r"(o[1].z), "r"(o[1].w),
    "r"(o[2].x), "r"(o[2].y), "r"(o[2].z), "r"(o[2].w), "r"(o[3].x), "r"(o[3].y), "r"(o[3].z), "r"(o[3].w),
    "r"(o[4].x), "r"(o[4].y), "r"(o[4].z), "r"(o[4].w), "r"(o[5].x), "r"(o[5].y), "r"(o[5].z), "r"(o[5].w),
    "r"(o[6].x), "r"(o[6].y), "r"(o[6].z), "r"(o[6].w), "r"(o[7].x), "r"(o[7].y), "r"(o[7].z), "r"(o[7].w)
    : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// K-major, 128-byte swizzled operand tile: rows of 128 bytes, 8-row atoms of 1024 bytes.
__device__ __forceinline__ uint64_t smem_desc_sw128(const void *tile) {
  const uint64_t addr = smem_u32(tile);
  return ((addr & 0x3FFFFull) >> 4) | (1ull << 16) /* leading byte offset: unused in this mode */ |
         ((1024ull >> 4) << 32) /* stride between 8-row atoms */ | (1ull << 46) /* descriptor version */ |
         (2ull << 61) /* SWIZZLE_128B */;
}

// c = fp32, a = b = fp16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
__host__ __device__ constexpr uint32_t instr_desc_f16(int m, int n) {
  return (1u << 4) | ((uint32_t) (n >> 3) << 17) | ((uint32_t) (m >> 4) << 24);
}

// Bounded wait that also gives up when another role has raised the abort flag.  The hand-offs
// between the roles are on the critical path of every K step, so the wait spins on try_wait (which
// itself suspends the thread for a short hardware-defined time) and only backs off, and looks at
// the abort flag, once the wait has become long.
__device__ __forceinline__ bool wait_or_abort(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *err,
                                              int code) {
  for (uint32_t i = 0; i < kWaitCap; ++i) {
    if (mbar_try_wait(bar, parity)) {
      return true;
    }
    if (i >= 4096) {
      if (*abort_flag) {
        return false;
      }
      __nanosleep(128);
    }
  }
  atomicCAS(err, 0, code);
  *abort_flag = 1;
  return false;
}


struct Ring {
  int slot = 0, phase = 0, n;
  __device__ explicit Ring(int n_) : n(n_) {}
  __device__ void next() {
    if (++slot == n) {
      slot = 0;
      phase ^= 1;
    }
  }
};

// ---------------------------------------------------------------- dequantisation of one K step

// 64 weights (two blocks) of one row -> eight 16-byte chunks of fp16 (value * scale, rounded once).
// `raw` holds the words of the row's raw stage; for Q8_0 every word has been XORed with 0x80808080
// (quant bytes biased to 0..255; the scale halfwords are un-biased again where they are used).
template <int WT>
__device__ __forceinline__ void dequant_two_blocks(const uint32_t *raw, int q, uint4 (&out)[8]) {
  static_assert(WT == kQ4 || WT == kQ8 || WT == kIQ4, "block formats only");
  // block b of the raw stage starts at byte b * BB; its scale is the first halfword
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int      b    = 2 * q + h;
    const int      off  = b * BlockTraits<WT>::kBytes;  // even; a multiple of 4 when b is even
    const uint32_t sw   = raw[off >> 2] ^ (WT == kQ8 ? 0x80808080u : 0u);
    const uint16_t sbit = (off & 2) ? (uint16_t) (sw >> 16) : (uint16_t) (sw & 0xffff);
    const __half2  d2   = __half2half2(__ushort_as_half(sbit));
    if constexpr (WT == kIQ4) {
      // table values as signed bytes (unpack.cuh), biased to 0..255, then the 0x6400 trick as for Q8_0
      const __half2 k1152 = u32_as_h2(0x64806480u);
      uint32_t      lo[8], hi[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int      o = off + 2 + 4 * i;
        const uint32_t w = (o & 2) ? __byte_perm(raw[o >> 2], raw[(o >> 2) + 1], 0x5432) : raw[o >> 2];
        uint32_t       r0, r1;  // r0 = elements (4i, 16+4i, 4i+1, 17+4i), r1 = (4i+2, 18+4i, 4i+3, 19+4i)
        iq4nl_unpack_word(w, r0, r1);
        r0 ^= 0x80808080u, r1 ^= 0x80808080u;
        auto pair = [&](uint32_t r, uint32_t sel) {
          return h2_as_u32(__hmul2(__hsub2(u32_as_h2(__byte_perm(r, 0x64646464u, sel)), k1152), d2));
        };
        lo[2 * i]     = pair(r0, 0x4240);  // bytes 0, 2
        hi[2 * i]     = pair(r0, 0x4341);  // bytes 1, 3
        lo[2 * i + 1] = pair(r1, 0x4240);
        hi[2 * i + 1] = pair(r1, 0x4341);
      }
      out[4 * h + 0] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      out[4 * h + 1] = make_uint4(lo[4], lo[5], lo[6], lo[7]);
      out[4 * h + 2] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      out[4 * h + 3] = make_uint4(hi[4], hi[5], hi[6], hi[7]);
    } else if constexpr (WT == kQ4) {
      uint32_t lo[8], hi[8];  // fp16 pairs in element order: lo = elements 0..15, hi = 16..31
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        // quant bytes (B0, B1, B2, B3) of word i -> (B0, B2, B1, B3), taken straight from the one or
        // two raw words that hold them; the unpack then yields {B0,B1} and {B2,B3}
        const int      o = off + 2 + 4 * i;
        const uint32_t w = (o & 2) ? __byte_perm(raw[o >> 2], raw[(o >> 2) + 1], 0x5342)
                                   : __byte_perm(raw[o >> 2], 0u, 0x3120);
        uint32_t       u[4];
        q4_0_unpack_word(w, u);
        lo[2 * i]     = h2_as_u32(__hmul2(u32_as_h2(u[0]), d2));
        lo[2 * i + 1] = h2_as_u32(__hmul2(u32_as_h2(u[1]), d2));
        hi[2 * i]     = h2_as_u32(__hmul2(u32_as_h2(u[2]), d2));
        hi[2 * i + 1] = h2_as_u32(__hmul2(u32_as_h2(u[3]), d2));
      }
      out[4 * h + 0] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      out[4 * h + 1] = make_uint4(lo[4], lo[5], lo[6], lo[7]);
      out[4 * h + 2] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      out[4 * h + 3] = make_uint4(hi[4], hi[5], hi[6], hi[7]);
    } else {
      // elements 2p, 2p + 1 are two adjacent bytes of ONE raw word (the quants start on an even
      // byte): 0x6400 | (byte + 128) = 1024 + 128 + value, exact in fp16
      const __half2 k1152 = u32_as_h2(0x64806480u);
      uint32_t      v[16];
#pragma unroll
      for (int pr = 0; pr < 16; ++pr) {
        const int      o  = off + 2 + 2 * pr;
        const uint32_t hh = __byte_perm(raw[o >> 2], 0x64646464u, (o & 2) ? 0x4342 : 0x4140);
        v[pr]             = h2_as_u32(__hmul2(__hsub2(u32_as_h2(hh), k1152), d2));
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        out[4 * h + c] = make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
      }
    }
  }
}

// ---------------------------------------------------------------- the kernel

template <int WT, int BT, bool TWO>
__global__ void __launch_bounds__(kThreads, 1)
  gemm_tcgen05_kernel(const GemmArgs p, const __grid_constant__ CUtensorMap xmap,
                      const __grid_constant__ GemmDstMaps ymaps, const __grid_constant__ CUtensorMap pmap) {
  using C = GCfg<WT, BT, TWO>;
  static_assert((!TWO && BT == 128) || (TWO && BT == 256), "token tile");
  constexpr int      NX        = C::NX;
  constexpr int      X_BYTES   = C::X_BYTES;
  constexpr int      RAW_BYTES = C::RAW_BYTES;
  constexpr int      RAW_PITCH = (RAW_BYTES + 127) & ~127;
  constexpr int      ROWS_TILE = TWO ? 2 * kBW : kBW;  // weight rows per (pair) tile
  constexpr uint32_t IDESC     = instr_desc_f16(ROWS_TILE, BT);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // swizzled operand tiles need 1024-byte alignment in the shared address space
  uint8_t  *sX   = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t  *sRaw = sX + NX * X_BYTES;
  GSmemBar *bar  = reinterpret_cast<GSmemBar *>(sRaw + 2 * RAW_PITCH);
  uint8_t  *sOut = sRaw + 2 * RAW_PITCH + 512;  // output staging, 128-byte aligned

  const int      warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = TWO ? cluster_ctarank() : 0u;  // 0 = leader of the pair
  volatile int  *abort_flag = &bar->abort_flag;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kNAT / C::BSTEPS; ++i) {  // one barrier pair per group of K steps
      // the TMA producer's expect_tx arrival and the four warps of the writing group, of both CTAs
      // for a pair
      mbar_init(&bar->full[i], TWO ? 1 + 4 + 4 : 1 + 4);
      mbar_init(&bar->empty[i], 1);  // one tcgen05.commit
    }
    mbar_init(&bar->acc_full, 1);
    mbar_init(&bar->acc_empty, TWO ? 8 : 4);  // the epilogue warps of every CTA of the tile
    bar->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc<TWO>(&bar->tmem_base, kTmemCols);
    tmem_relinquish<TWO>();
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (TWO) {
    cluster_sync_all();  // both CTAs' barriers and tensor memory exist before anyone signals across
  }
  tc_fence_after();
  const uint32_t tmem_base = bar->tmem_base;

  const int t_tiles = (p.M + BT - 1) / BT;                // token tiles
  const int w_tiles = (p.N + ROWS_TILE - 1) / ROWS_TILE;  // weight-row tiles
  const int tiles   = t_tiles * w_tiles;
  const int k_raws  = p.K / C::RAWK;
  const int worker  = TWO ? (int) (blockIdx.x >> 1) : (int) blockIdx.x;  // CTA, or CTA pair
  const int workers = TWO ? (int) (gridDim.x >> 1) : (int) gridDim.x;
  const int row_off = (int) rank * kBW;        // this CTA's weight rows inside the tile
  const int tok_off = (int) rank * C::XROWS;   // this CTA's tokens inside the activation tile
  // Work is counted in STAGES of one raw stage (256 of K) of one tile.  A worker first takes whole
  // tiles, interleaved with the other workers' (tile = i * workers + worker: neighbours work on
  // neighbouring tiles at the same time, which share weight rows or activations in L2).  When
  // the tiles do not divide evenly among the workers (p.split) only all but the last FULL wave is
  // handed out that way; the remaining tiles (between one and two per worker) are laid end to end
  // and cut into `workers` contiguous ranges of equal length, anywhere inside a tile.  A tile cut
  // in two has two contributors - the worker whose range ENDS in it (it has the head of the tile's
  // K range and reaches it last) and the next worker, whose range STARTS in it (the tail of K,
  // done first) - and the second hands its partial sums to the first through global scratch.  A
  // range is at least one tile long, so no tile has more than two contributors.
  const int dp_tiles  = p.split ? tiles / workers - 1 : (tiles - worker + workers - 1) / workers;  // whole tiles first
  const int dp_stages = dp_tiles * k_raws;
  const int sk_tile0  = dp_tiles * workers;  // first tile of the part that is cut into ranges
  int       sk_begin = 0, sk_end = 0;        // this worker's range of that part, in stages
  if (p.split) {
    const long long sk_stages = (long long) (tiles - sk_tile0) * k_raws;
    sk_begin = (int) (sk_stages * worker / workers);
    sk_end   = (int) (sk_stages * (worker + 1) / workers);
  }
  const int n_stages = dp_stages + (sk_end - sk_begin);  // stages this worker goes through, in order
  // stage li of this worker -> (tile, raw stage of the tile)
  auto stage_at = [&](int li, int &t, int &rs) {
    if (li < dp_stages) {
      const int i = li / k_raws;
      rs = li - i * k_raws;
      t  = i * workers + worker;
    } else {
      const int u = sk_begin + (li - dp_stages), tt = u / k_raws;
      rs = u - tt * k_raws;
      t  = sk_tile0 + tt;
    }
  };
  // segment = the stages of ONE tile that follow each other in this worker's order: stages
  // rs0 .. rs1 - 1 of tile t, starting at the worker's stage li
  auto segment = [&](int li, int &t, int &rs0, int &rs1) {
    stage_at(li, t, rs0);
    rs1 = rs0 + (n_stages - li) < k_raws ? rs0 + (n_stages - li) : k_raws;
  };

  if (warp == 0) {
    // ---------------- TMA producer of the activation tiles (this CTA's share of the tokens)
    if (lane == 0) {
      tma_prefetch_descriptor(&xmap);
      const uint64_t pol = l2_policy_evict_last();  // re-read by the other weight-row tiles
      Ring           rx(NX);
      bool           ok = true;
      for (int li = 0; li < n_stages && ok;) {
        int t, rs0, rs1;
        segment(li, t, rs0, rs1);
        li += rs1 - rs0;
        const int m0 = (t % t_tiles) * BT + tok_off;
        for (int kb = rs0 * C::Q; kb < rs1 * C::Q; ++kb) {
          // BSTEPS K steps share one full / empty barrier pair (a segment holds whole raw stages): the MMA
          // issuer's waits and commits, which cost it hundreds of clocks each, come once per group
          const int hb = rx.slot / C::BSTEPS;
          if (rx.slot % C::BSTEPS == 0) {
            ok = wait_or_abort(&bar->empty[hb], rx.phase ^ 1, abort_flag, p.err, kGemmErrProducer);
            if (!ok) {
              break;
            }
            if constexpr (TWO) {
              // both halves of both activation tiles complete on the leader's barrier
              if (rank == 0) {
                mbar_arrive_expect_tx(&bar->full[hb], 2 * C::BSTEPS * X_BYTES);
              }
            } else {
              mbar_arrive_expect_tx(&bar->full[hb], C::BSTEPS * X_BYTES);
            }
          }
          if constexpr (TWO) {
            tma_load_2d_pair(sX + rx.slot * X_BYTES, &xmap, kb * kBK, m0, &bar->full[hb], pol);
          } else {
            tma_load_2d(sX + rx.slot * X_BYTES, &xmap, kb * kBK, m0, &bar->full[hb], pol);
          }
          rx.next();
        }
      }
    }
  } else if (warp == 1) {
    if (rank == 0) {
      // ---------------- MMA issuer (leader CTA).  The whole warp runs the loop so that control
      // flow and operands stay warp-uniform; one elected lane issues the tensor-core instructions.
      unsigned gs = 0;
      int      it = 0;
      bool     ok = true;
      for (int li = 0; li < n_stages && ok; ++it) {
        int t, rs0, rs1;
        segment(li, t, rs0, rs1);
        li += rs1 - rs0;
        // the accumulator must have been read out by the epilogue(s) of the previous segment
        ok = wait_or_abort(&bar->acc_empty, (it & 1) ^ 1, abort_flag, p.err, kGemmErrMma);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          break;
        }
        tc_fence_after();
        for (int rs = rs0; rs < rs1 && ok; ++rs, ++gs) {
          const int sg = (int) (gs % C::NG), gph = (int) (gs / C::NG) & 1;  // ring position of the raw stage
#pragma unroll
          for (int q = 0; q < C::Q; ++q) {
            const int slot = sg * C::Q + q;  // (slot % BSTEPS == q % BSTEPS)
            if (q % C::BSTEPS == 0) {
              ok = wait_or_abort(&bar->full[slot / C::BSTEPS], gph, abort_flag, p.err, kGemmErrMma);
              ok = __all_sync(0xffffffffu, ok);
              if (!ok) {
                break;
              }
              tc_fence_after();
            }
            if (elect_one()) {
              const uint64_t bdesc  = smem_desc_sw128(sX + slot * X_BYTES);
              const uint32_t a_tmem = tmem_base + kTmemA + slot * 32;
#pragma unroll
              for (int s = 0; s < kBK / 16; ++s) {
                // A: 16 fp16 per lane = 8 TMEM columns per step; B: +32 bytes inside the swizzled row
                umma_f16_ts<TWO>(tmem_base, a_tmem + 8 * s, bdesc + 2 * s, IDESC, ((rs - rs0) | q | s) ? 1u : 0u);
              }
              if (q % C::BSTEPS == C::BSTEPS - 1) {
                umma_commit<TWO>(&bar->empty[slot / C::BSTEPS]);
              }
            }
            __syncwarp();
          }
        }
        if (ok && elect_one()) {
          umma_commit<TWO>(&bar->acc_full);
        }
        __syncwarp();
      }
    }
  } else if (warp >= kEpiWarp0 && warp < kEpiWarp0 + 4) {
    // ---------------- epilogue: TMEM -> registers -> shared memory -> y[token][weight row].
    // Each warp drains its 32 TMEM lanes (weight rows) 16 tokens at a time into a private
    // [16 tokens][32 rows] staging buffer (two of them, alternating) and hands the buffer to the
    // copy engine as one tiled store; the accumulator is released as soon as the last load has
    // completed, the stores drain while the next tile is being computed.
    const int q4 = warp & 3;  // a warp may only touch TMEM lanes 32 * (warp % 4) .. + 31
    int       it = 0;
    bool      ok = true;
    unsigned  nbuf = 0;  // running count of staged chunks: buffer = nbuf & 1
    const uint32_t stage0 = smem_u32(sOut + q4 * (2 * kOutTok * 128));
    if (lane == 0) {
      tma_prefetch_descriptor(&ymaps.m[0]);
    }
    for (int li = 0; li < n_stages && ok; ++it) {
      int t, rs0, rs1;
      segment(li, t, rs0, rs1);
      li += rs1 - rs0;
      // whole tile: store y.  Tail of the K range (the other contributor finishes the tile): store
      // the partial sums to this worker's scratch tile and raise this warp's flag.  Head of the K
      // range: wait for the flag of the next worker's same warp, add its partial sums, store y.
      const bool is_tail = rs0 > 0, is_head = rs0 == 0 && rs1 < k_raws;
      const int n0 = (t / t_tiles) * ROWS_TILE + row_off, m0 = (t % t_tiles) * BT;
      ok = wait_or_abort(&bar->acc_full, it & 1, abort_flag, p.err, kGemmErrEpilogue);
      ok = __all_sync(0xffffffffu, ok);  // tensor-memory loads are warp-wide
      if (!ok) {
        break;
      }
      tc_fence_after();
      const int      col0   = n0 + q4 * 32;  // first output column (weight row) of this warp
      const uint32_t taddr  = tmem_base + ((uint32_t) (q4 * 32) << 16);
      const bool     col_ok = col0 < p.N;  // N is a multiple of 32: a warp is in or out
      const int      m_end  = p.M - m0 < BT ? p.M - m0 : BT;  // tokens of this tile inside the matrix
      const float   *other  = nullptr;  // the other contributor's partial sums of this thread's row
      int           *flag   = nullptr;
      if (is_head) {
        flag  = p.flags + ((worker + 1) * 2 + (int) rank) * 4 + q4;
        other = p.part + (size_t) (worker + 1) * BT * ROWS_TILE + row_off + q4 * 32 + lane;
        bool seen = false;
        for (uint32_t i = 0; i < kFlagWaitCap && !seen; ++i) {
          int f;
          asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(f) : "l"(flag) : "memory");
          seen = f != 0;
          if (!seen) {
            if (*abort_flag) {
              break;
            }
            __nanosleep(256);
          }
        }
        if (!seen) {
          atomicCAS(p.err, 0, kGemmErrFixup);
          *abort_flag = 1;
        }
        ok = __all_sync(0xffffffffu, seen);
        if (!ok) {
          break;  // (the accumulator is not released: every other role runs into the abort flag)
        }
      }
      uint32_t va[16], vb[16];
      // v = tokens c0 .. c0 + 15 of this thread's row; tokens past M are cut off by the tensor map
      // (the other contributor's sums of a chunk are requested one chunk ahead, with the chunk's
      // tensor-memory load)
      float adda[16], addb[16];
      auto  load_other = [&](int c0, float (&add)[16]) {
        if (is_head) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            add[i] = __ldcg(other + (size_t) (c0 + i) * ROWS_TILE);
          }
        }
      };
      auto store16 = [&](int c0, uint32_t (&v)[16], const float (&add)[16]) {
        if (is_head) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            v[i] = __float_as_uint(__uint_as_float(v[i]) + add[i]);
          }
        }
        if (p.tok_scale && !is_tail) {  // (partial sums travel unscaled)
          const float4 *ts = reinterpret_cast<const float4 *>(p.tok_scale + m0 + c0);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 sc = __ldg(ts + i);
            v[4 * i]     = __float_as_uint(__uint_as_float(v[4 * i]) * sc.x);
            v[4 * i + 1] = __float_as_uint(__uint_as_float(v[4 * i + 1]) * sc.y);
            v[4 * i + 2] = __float_as_uint(__uint_as_float(v[4 * i + 2]) * sc.z);
            v[4 * i + 3] = __float_as_uint(__uint_as_float(v[4 * i + 3]) * sc.w);
          }
        }
        const uint32_t buf = stage0 + (nbuf & 1) * (kOutTok * 128);
        ++nbuf;
        if (lane == 0) {
          bulk_wait_read<1>();  // the store that last used this buffer has read it
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          asm volatile("st.shared.b32 [%0], %1;" ::"r"(buf + i * 128 + lane * 4), "r"(v[i]) : "memory");
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (is_tail) {
            tma_store_2d(&pmap, row_off + q4 * 32, worker * BT + c0, buf);
          } else if (col_ok) {
            // every destination gets the same box (the others are other GPUs' copies of the output)
            for (int d = 0; d < p.n_dst; ++d) {
              tma_store_2d(&ymaps.m[d], (int) p.y_col0 + col0, m0 + c0, buf);
            }
          }
          bulk_commit();
        }
      };
      auto release_acc = [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (TWO && rank != 0) {
            mbar_arrive_remote(&bar->acc_empty, 0);  // the leader issues the next segment's first MMA
          } else {
            mbar_arrive(&bar->acc_empty);
          }
        }
      };
      tmem_ld16_issue(taddr, va);
      load_other(0, adda);
#pragma unroll 1
      for (int c0 = 0; c0 < m_end; c0 += 32) {
        tmem_ld_wait(va);
        if (c0 + 16 < m_end) {
          tmem_ld16_issue(taddr + c0 + 16, vb);
          load_other(c0 + 16, addb);
        } else {
          release_acc();
        }
        store16(c0, va, adda);
        if (c0 + 16 < m_end) {
          tmem_ld_wait(vb);
          if (c0 + 32 < m_end) {
            tmem_ld16_issue(taddr + c0 + 32, va);
            load_other(c0 + 32, adda);
          } else {
            release_acc();
          }
          store16(c0 + 16, vb, addb);
        }
      }
      if (is_tail) {
        // the partial sums are in global memory before the flag is: the stores have completed
        // (wait_group), the copy engine's writes are ordered before this thread's release
        if (lane == 0) {
          bulk_wait_all();
          asm volatile("fence.proxy.async;" ::: "memory");
          __threadfence();
          asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p.flags + (worker * 2 + (int) rank) * 4 + q4), "r"(1)
                       : "memory");
        }
      } else if (is_head) {
        __syncwarp();
        if (lane == 0) {
          *flag = 0;  // ready for the next launch on this stream
        }
      }
    }
    if (lane == 0) {
      bulk_wait_all();  // the staging buffers stay valid until the copy engine is done with them
      if (p.n_dst > 1) {
        __threadfence_system();  // stores into other GPUs' memory are ordered before this kernel's end
      }
    }
  } else if (warp >= kDeqWarp0) {
    // ---------------- dequantisation: group g, thread = weight row r of this CTA's 128 rows.
    // Each WARP also fetches the raw stages of its own 32 rows (32 x 144 / 272 bytes) with 16-byte
    // asynchronous copies (cp.async), one stage of the group ahead, into its slice of the group's
    // buffer; the pieces are taken in linear order (lane after lane along a row, 2-4 rows per warp
    // instruction) so that one instruction touches a handful of cache lines rather than 32.  Only
    // the warp itself reads or writes the slice: __syncwarp is all the ordering the stage needs.
    // (A tiled TMA copy of 128 such short rows was the bottleneck of an earlier version: the copy
    // engine's cost is per row, about the same for 144 bytes as for a kilobyte.)
    const int      g     = (warp - kDeqWarp0) >> 2;
    const uint32_t tlane = tmem_base + kTmemA + ((uint32_t) ((warp & 3) * 32) << 16);
    const uint32_t warp_smem = smem_u32(sRaw + g * RAW_PITCH + (warp & 3) * 32 * C::RB);
    const uint32_t slot_smem = warp_smem + lane * C::RB;  // this thread's row
    const long long row_bytes = (long long) (p.K / 32) * C::BB;

    // this group's stages: g, g + 2, ... of the worker's order
    // piece j = 32 i + lane of the warp's stage (i = 0 .. RW - 1) is piece j % RW of row j / RW and
    // lands at byte 16 j of the slice; row and piece advance incrementally (32 = kA * RW + kB)
    constexpr int kA = 32 / C::RW, kB = 32 % C::RW;
    const int     row_first = lane / C::RW, pc_first = lane % C::RW;
    auto fetch = [&](int li) {
      int t, rs;
      stage_at(li, t, rs);
      const long long row0 = (long long) (t / t_tiles) * ROWS_TILE + row_off + (warp & 3) * 32;
      if (row0 >= p.N) {
        return;  // N is a multiple of 32: the warp's rows are all inside or all outside the matrix;
                 // rows outside are computed on whatever the slice holds and never stored
      }
      if constexpr (C::TILED || C::PERM) {
        // the warp's 32 rows are ONE column tile of the reference's tile order, and the RAWK / 32
        // k-tiles of a raw stage are consecutive tiles: one contiguous run, copied as it lies
        const uint8_t *src = p.w + ((row0 >> 5) * (long long) (p.K / 32) + (long long) rs * (C::RAWK / 32)) * C::TILE_B + 16 * lane;
        uint32_t       dst = warp_smem + 16 * lane;
#pragma unroll
        for (int i = 0; i < (C::PIECES + 31) / 32; ++i) {
          if (C::PIECES % 32 == 0 || i * 32 + lane < C::PIECES) {
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
          }
          src += 512, dst += 512;
        }
      } else {
        const uint8_t *src = p.w + (row0 + row_first) * row_bytes + (long long) rs * C::RB + 16 * pc_first;
        int            pc  = pc_first;
        uint32_t       dst = warp_smem + 16 * lane;
#pragma unroll
        for (int i = 0; i < C::RW; ++i) {
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
          const bool wrap = pc + kB >= C::RW;
          pc += wrap ? kB - C::RW : kB;
          src += wrap ? (kA + 1) * row_bytes + 16 * (kB - C::RW) : kA * row_bytes + 16 * kB;
          dst += 512;
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (g < n_stages) {
      fetch(g);
    }
    bool ok = true;
    for (int li = g; li < n_stages; li += 2) {
      const unsigned gs  = (unsigned) li;  // running stage index
      const int      sg = (int) (gs % C::NG), gph = (int) (gs / C::NG) & 1;  // ring position of the raw stage
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      // every lane's pieces of the stage have landed; the warp also leaves TOGETHER here once a
      // lane has given up a wait
      if (!__all_sync(0xffffffffu, ok)) {
        break;
      }
      // the thread's row of the raw stage, out of the slice into registers
      constexpr int RAW_WORDS = C::PERM ? 64 : (C::TILED ? C::RAWK / 2 : C::RW * 4);
      uint32_t      raw[RAW_WORDS + 1];
      if constexpr (C::PERM) {
        // Super-block sb (0..15: four per tile, four tiles) holds k-rows 8 (sb % 4) .. + 7 of its tile
        // for all 32 columns.  Its scale for column n and k-row pair v is halfword 2 v + n / 16 of the
        // 16-byte header: kept as raw[4 sb + 2] = pairs 0, 1 and raw[4 sb + 3] = pairs 2, 3.  Quants:
        //   Q4_0 / IQ4_NL: ONE word per column, nibbles (low to high) = k-rows 0, 4, 2, 6, 1, 5, 3, 7
        //                  (raw[4 sb]);
        //   Q8_0: k-row pair v = bytes 64 v + 2 n, + 1; raw[4 sb] = pairs 0, 1, raw[4 sb + 1] = pairs 2, 3,
        //         biased to 0..255.
        constexpr int  SBB  = C::TILE_B / 4;
        const uint32_t hsel = (lane & 16) ? 0x7632u : 0x5410u;  // the column's half of two scale words
        const uint32_t qsel = (lane & 1) ? 0x7632u : 0x5410u;   // the column's halfword of two quant words
#pragma unroll
        for (int sb = 0; sb < 16; ++sb) {
          const uint32_t at = warp_smem + sb * SBB;
          uint32_t       s0, s1, s2, s3;
          asm volatile("ld.volatile.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(s0), "=r"(s1), "=r"(s2), "=r"(s3)
                       : "r"(at)
                       : "memory");
          raw[4 * sb + 2] = __byte_perm(s0, s1, hsel);
          raw[4 * sb + 3] = __byte_perm(s2, s3, hsel);
          if constexpr (WT == kPQ8) {
            uint32_t w[4];
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              asm volatile("ld.volatile.shared.u32 %0, [%1];"
                           : "=r"(w[v])
                           : "r"(at + 16 + 64 * v + (lane >> 1) * 4)
                           : "memory");
            }
            raw[4 * sb]     = __byte_perm(w[0], w[1], qsel) ^ 0x80808080u;
            raw[4 * sb + 1] = __byte_perm(w[2], w[3], qsel) ^ 0x80808080u;
          } else {
            asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(raw[4 * sb]) : "r"(at + 16 + lane * 4) : "memory");
            raw[4 * sb + 1] = 0;
          }
        }
      } else if constexpr (C::TILED) {
        // tile order: the k-pair (2 kp, 2 kp + 1) of column n of a tile is the 32-bit word kp * 32 + n;
        // a lane's words are the fp16 pairs of its row in K order - what the tensor memory wants
#pragma unroll
        for (int i = 0; i < RAW_WORDS; ++i) {
          asm volatile("ld.volatile.shared.u32 %0, [%1];"
                       : "=r"(raw[i])
                       : "r"(warp_smem + (i >> 4) * 2048 + (i & 15) * 128 + lane * 4)
                       : "memory");
        }
      } else {
#pragma unroll
        for (int i = 0; i < C::RW; ++i) {
          asm volatile("ld.volatile.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(raw[4 * i]), "=r"(raw[4 * i + 1]), "=r"(raw[4 * i + 2]), "=r"(raw[4 * i + 3])
                       : "r"(slot_smem + 16 * i)
                       : "memory");
        }
        if constexpr (WT == kQ8) {
#pragma unroll
          for (int i = 0; i < C::RW * 4; ++i) {
            raw[i] ^= 0x80808080u;  // quant bytes biased to 0..255, once per word
          }
        }
      }
      raw[RAW_WORDS] = 0;  // the word past the end is only ever the unused half of a byte_perm
      // the fp16 values of a K step are computed before waiting for their TMEM slot
      uint4 out[8];
      auto  k_step = [&](int q) {
        if constexpr (C::PERM) {
          // K step q = tiles 2 q, 2 q + 1 = super-blocks 8 q .. 8 q + 7; a super-block's eight k-rows are
          // one 16-byte chunk: pairs (0,1), (2,3), (4,5), (6,7), value * scale rounded once
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const int      sb = 8 * q + c;
            const uint32_t pa = raw[4 * sb + 2], pb = raw[4 * sb + 3];
            const __half2  d0 = u32_as_h2(__byte_perm(pa, pa, 0x1010)), d1 = u32_as_h2(__byte_perm(pa, pa, 0x3232));
            const __half2  d2 = u32_as_h2(__byte_perm(pb, pb, 0x1010)), d3 = u32_as_h2(__byte_perm(pb, pb, 0x3232));
            uint32_t       v0, v1, v2, v3;
            if constexpr (WT == kPQ8) {
              const __half2  k1152 = u32_as_h2(0x64806480u);
              const uint32_t qa = raw[4 * sb], qb = raw[4 * sb + 1];
              v0 = h2_as_u32(__hmul2(__hsub2(u32_as_h2(__byte_perm(qa, 0x64646464u, 0x4140)), k1152), d0));
              v1 = h2_as_u32(__hmul2(__hsub2(u32_as_h2(__byte_perm(qa, 0x64646464u, 0x4342)), k1152), d1));
              v2 = h2_as_u32(__hmul2(__hsub2(u32_as_h2(__byte_perm(qb, 0x64646464u, 0x4140)), k1152), d2));
              v3 = h2_as_u32(__hmul2(__hsub2(u32_as_h2(__byte_perm(qb, 0x64646464u, 0x4342)), k1152), d3));
            } else if constexpr (WT == kPIQ4) {
              // table values of nibbles 0..3 (k-rows 0, 4, 2, 6) and 4..7 (k-rows 1, 5, 3, 7), biased
              const __half2  k1152 = u32_as_h2(0x64806480u);
              const uint32_t w  = raw[4 * sb];
              const uint32_t e  = iq4nl_lookup4(w) ^ 0x80808080u, o = iq4nl_lookup4(w >> 16) ^ 0x80808080u;
              const uint32_t t0 = __byte_perm(e, o, 0x5140);  // k-rows 0, 1, 4, 5
              const uint32_t t1 = __byte_perm(e, o, 0x7362);  // k-rows 2, 3, 6, 7
              v0 = h2_as_u32(__hmul2(__hsub2(u32_as_h2(__byte_perm(t0, 0x64646464u, 0x4140)), k1152), d0));
              v1 = h2_as_u32(__hmul2(__hsub2(u32_as_h2(__byte_perm(t1, 0x64646464u, 0x4140)), k1152), d1));
              v2 = h2_as_u32(__hmul2(__hsub2(u32_as_h2(__byte_perm(t0, 0x64646464u, 0x4342)), k1152), d2));
              v3 = h2_as_u32(__hmul2(__hsub2(u32_as_h2(__byte_perm(t1, 0x64646464u, 0x4342)), k1152), d3));
            } else {
              const __half2  k1032 = u32_as_h2(0x64086408u);  // 1024 + 8
              const uint32_t w = raw[4 * sb];
              v0 = h2_as_u32(__hmul2(__hsub2(u32_as_h2((w & 0x000F000Fu) | 0x64006400u), k1032), d0));
              v1 = h2_as_u32(__hmul2(__hsub2(u32_as_h2(((w >> 8) & 0x000F000Fu) | 0x64006400u), k1032), d1));
              v2 = h2_as_u32(__hmul2(__hsub2(u32_as_h2(((w >> 4) & 0x000F000Fu) | 0x64006400u), k1032), d2));
              v3 = h2_as_u32(__hmul2(__hsub2(u32_as_h2(((w >> 12) & 0x000F000Fu) | 0x64006400u), k1032), d3));
            }
            out[c] = make_uint4(v0, v1, v2, v3);
          }
        } else if constexpr (C::TILED) {
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            out[c] = make_uint4(raw[32 * q + 4 * c], raw[32 * q + 4 * c + 1], raw[32 * q + 4 * c + 2],
                                raw[32 * q + 4 * c + 3]);
          }
        } else {
          dequant_two_blocks<WT>(raw, q, out);
        }
      };
      k_step(0);
      // Next stage of this group into the same slice.
      // The loads above are volatile (they stay where they are written) and the copies below go
      // down the same in-order load/store pipe behind them, writing shared memory only after a
      // global-memory round trip.
      __syncwarp();  // every lane has taken its row out of the slice
      if (li + 2 < n_stages) {
        fetch(li + 2);
      }
#pragma unroll
      for (int q = 0; q < C::Q; ++q) {
        const int slot = sg * C::Q + q;
        if (q % C::BSTEPS == 0) {
          ok = ok && wait_or_abort(&bar->empty[slot / C::BSTEPS], gph ^ 1, abort_flag, p.err, kGemmErrDequant);
        }
        ok = __all_sync(0xffffffffu, ok);  // a warp stores to tensor memory as a whole or not at all
        if (ok) {
          tc_fence_after();
          tmem_st32(tlane + slot * 32, out);  // 64 fp16 = 32 columns of this thread's lane
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();  // every lane's store has completed (wait::st above)
          if (lane == 0 && q % C::BSTEPS == C::BSTEPS - 1) {  // the group's K steps are all in tensor memory
            if (TWO && rank != 0) {
              mbar_arrive_remote(&bar->full[slot / C::BSTEPS], 0);  // the MMA is issued by the leader CTA
            } else {
              mbar_arrive(&bar->full[slot / C::BSTEPS]);
            }
          }
        }
        if (q + 1 < C::Q) {
          k_step(q + 1);
        }
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  }

  // ---------------- teardown
  tc_fence_before();
  __syncthreads();
  if constexpr (TWO) {
    cluster_sync_all();  // nobody leaves while the other CTA may still signal or read this one
  }
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc<TWO>(tmem_base, kTmemCols);
  }
}

// one partial tile per worker: 74 pairs x 256 x 256 or 148 CTAs x 128 x 128 floats
size_t gemm_part_bytes(int sm_count) {
  const size_t pair = (size_t) (sm_count / 2) * 256 * 256 * 4, one = (size_t) sm_count * 128 * 128 * 4;
  return pair > one ? pair : one;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
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

template <int WT, int BT, bool TWO>
cudaError_t launch(const GemmArgs &a, int sm_count, cudaStream_t stream) {
  using C = GCfg<WT, BT, TWO>;
  EncodeTiledFn enc = encode_fn();
  if (!enc) {
    return cudaErrorNotSupported;
  }
  CUtensorMap xmap;
  {
    const cuuint64_t gdim[2] = { (cuuint64_t) a.K, (cuuint64_t) a.M };
    const cuuint64_t gstr[1] = { (cuuint64_t) a.K * 2 };
    const cuuint32_t box[2]  = { kBK, (cuuint32_t) C::XROWS };
    const cuuint32_t es[2]   = { 1, 1 };
    if (enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(a.x), gdim, gstr, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      return cudaErrorInvalidValue;
    }
  }
  GemmArgs args = a;
  if (args.n_dst <= 0) {
    args.n_dst = 1;
  }
  if (args.y_ld <= 0) {
    args.y_ld = a.N, args.y_col0 = 0;
  }
  if (args.n_dst > kGemmMaxDst || args.y_col0 < 0 || args.y_col0 % 32 != 0 || args.y_col0 + a.N > args.y_ld ||
      args.y_ld % 4 != 0) {
    return cudaErrorInvalidValue;
  }
  GemmDstMaps ymaps;
  for (int d = 0; d < kGemmMaxDst; ++d) {
    if (d >= args.n_dst) {
      ymaps.m[d] = ymaps.m[0];  // unused slots
      continue;
    }
    // output [M][y_ld] fp32, stored in boxes of 32 weight rows (128 bytes) x 16 tokens
    float *base = d == 0 ? a.y : a.y_more[d - 1];
    const cuuint64_t gdim[2] = { (cuuint64_t) args.y_ld, (cuuint64_t) a.M };
    const cuuint64_t gstr[1] = { (cuuint64_t) args.y_ld * 4 };
    const cuuint32_t box[2]  = { 32, kOutTok };
    const cuuint32_t es[2]   = { 1, 1 };
    if (!base || enc(&ymaps.m[d], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, gdim, gstr, box, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      return cudaErrorInvalidValue;
    }
  }
  const int rows_tile = TWO ? 2 * kBW : kBW;
  const int tiles     = ((a.M + BT - 1) / BT) * ((a.N + rows_tile - 1) / rows_tile);
  const int max_w     = TWO ? sm_count / 2 : sm_count;
  const int workers   = tiles < max_w ? tiles : max_w;
  // uneven tile counts: cut the work into equal ranges (needs the scratch)
  args.split = (a.part != nullptr && tiles > workers && tiles % workers != 0) ? 1 : 0;
  args.flags = a.part ? reinterpret_cast<int *>(reinterpret_cast<uint8_t *>(a.part) + gemm_part_bytes(sm_count)) : nullptr;
  CUtensorMap pmap = ymaps.m[0];
  if (args.split) {
    // partial tiles: [worker][token][weight row of the tile] fp32, stored in the same boxes as y
    const cuuint64_t gdim[2] = { (cuuint64_t) rows_tile, (cuuint64_t) BT * workers };
    const cuuint64_t gstr[1] = { (cuuint64_t) rows_tile * 4 };
    const cuuint32_t box[2]  = { 32, kOutTok };
    const cuuint32_t es[2]   = { 1, 1 };
    if (enc(&pmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, a.part, gdim, gstr, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      return cudaErrorInvalidValue;
    }
  }
  const size_t smem = (size_t) C::NX * C::X_BYTES + C::FIXED;
  auto         kern = gemm_tcgen05_kernel<WT, BT, TWO>;
  cudaError_t  e    = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
  if (e != cudaSuccess) {
    return e;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim            = dim3(TWO ? 2 * workers : workers);
  cfg.blockDim           = dim3(kThreads);
  cfg.dynamicSmemBytes   = smem;
  cfg.stream             = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id               = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs                = attr;
  cfg.numAttrs             = TWO ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, args, xmap, ymaps, pmap);
}

}  // namespace


size_t gemm_scratch_bytes(int sm_count) {
  return gemm_part_bytes(sm_count) + (size_t) sm_count * 8 * sizeof(int);
}

cudaError_t gemm_tcgen05_launch(const GemmArgs &args_in, int wt, int sm_count, cudaStream_t stream) {
  GemmArgs args = args_in;
  // up to 128 tokens: single-CTA tiles of 128 tokens; more: CTA pairs on 256 x 256 tiles
  const bool one = g_opt_gemm_tile_n ? g_opt_gemm_tile_n == 128 : args.M <= 128;
  if (wt == kQ4) {
    return one ? launch<kQ4, 128, false>(args, sm_count, stream) : launch<kQ4, 256, true>(args, sm_count, stream);
  }
  if (wt == kIQ4) {
    return one ? launch<kIQ4, 128, false>(args, sm_count, stream) : launch<kIQ4, 256, true>(args, sm_count, stream);
  }
  if (wt == kGemmWtF16Tiled) {
    return one ? launch<kF16T, 128, false>(args, sm_count, stream) : launch<kF16T, 256, true>(args, sm_count, stream);
  }
  if (wt == kGemmWtPermQ4) {
    return one ? launch<kPQ4, 128, false>(args, sm_count, stream) : launch<kPQ4, 256, true>(args, sm_count, stream);
  }
  if (wt == kGemmWtPermQ8) {
    return one ? launch<kPQ8, 128, false>(args, sm_count, stream) : launch<kPQ8, 256, true>(args, sm_count, stream);
  }
  if (wt == kGemmWtPermIQ4) {
    return one ? launch<kPIQ4, 128, false>(args, sm_count, stream) : launch<kPIQ4, 256, true>(args, sm_count, stream);
  }
  return one ? launch<kQ8, 128, false>(args, sm_count, stream) : launch<kQ8, 256, true>(args, sm_count, stream);
}

}  // namespace htp
