// K2 - prefill-side quantised GEMM (M >= 64, fp16 activations): y[M][N] = x[M][K] . W[N][K]^T with
// fp32 accumulation on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM).
//
// Replaces the reference's HVX dequantise -> HMX 32x32 tile loop (src/dsp/ops/mat_mul.c:702-726,
// 928-1005).  Like the reference the weights are dequantised to fp16, value * scale rounded once
// (mat_mul.c:290, 304); unlike it the accumulator and the output stay fp32.
//
// One persistent CTA per SM, tile = 128 tokens x BN weight rows, K in steps of 64:
//   warp 0      TMA producer: the activation tile (128 x 64 fp16, 128-byte swizzle) per K step and
//               the RAW weight bytes (BN rows x 256 weights = 144 / 272 bytes per row) per 4 K steps
//   warp 1      MMA issuer: one thread issues tcgen05.mma.cta_group::1.kind::f16 (M = 128, N = BN,
//               K = 16) four times per K step, operands through shared-memory descriptors
//   warp 2      TMEM allocation (512 columns = two BN-column accumulators)
//   warps 4-7   epilogue: tcgen05.ld of an accumulator, fp32 stores to y (row-major)
//   warps 8-15  dequantisation: thread r owns weight row r of the tile; 9 / 17 conflict-free 16-byte
//               loads bring its 256 raw weights into registers, then per K step it writes 64 fp16
//               values as eight 16-byte chunks into the K-major SWIZZLE_128B operand tile
// Two accumulators let the epilogue of one tile overlap the main loop of the next.  All waits are
// bounded; a wait that runs out records an error code, raises the CTA's abort flag and every role
// leaves its loop; TMEM is freed before the CTA exits.  No cluster launch, no multicast.
#include "gemm_tcgen05.h"

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "device_ctx.h"
#include "ptx.cuh"
#include "unpack.cuh"

namespace htp {

namespace {

constexpr int kBM          = 128;  // tokens per tile (UMMA M)
constexpr int kBK          = 64;   // K per pipeline step: one 128-byte swizzled row of fp16
constexpr int kKPerRaw     = 256;  // weights per row in one raw stage (a 16-byte aligned period)
constexpr int kNB          = 3;    // dequantised-weight stages
constexpr int kMaxNA       = 8;    // activation stages: as many as fit (see GCfg)
constexpr int kSmemLimit   = 232448;  // opt-in dynamic shared memory per CTA
constexpr int kThreads     = 512;
constexpr int kDeqWarp0    = 8;    // first dequantisation warp
constexpr int kDeqWarps    = 8;
constexpr int kEpiWarp0    = 4;
constexpr int kTmemCols    = 512;

struct GSmemBar;

template <int WT, int BN>
struct GCfg {
  static constexpr int BB  = BlockTraits<WT>::kBytes;
  static constexpr int RB  = 8 * BB;  // raw bytes per row and raw stage: 144 / 272
  static constexpr int NR  = 1;       // raw stages: the bytes move to registers at once, one is enough
  static constexpr int RW  = RB / 16;  // 16-byte words per row: 9 / 17
  static constexpr int A_BYTES   = 128 * 128;
  static constexpr int B_BYTES   = BN * 128;
  static constexpr int RAW_BYTES = BN * RB;
  // everything but the activation ring, plus alignment slack and the barrier block
  static constexpr int FIXED = kNB * B_BYTES + ((NR * RAW_BYTES + 127) & ~127) + 1024 + 512;
  static constexpr int NA_FIT = (kSmemLimit - FIXED) / A_BYTES;
  static constexpr int NA     = NA_FIT > kMaxNA ? kMaxNA : NA_FIT;  // 5 / 6 (Q4_0), 3 / 5 (Q8_0) for BN 256 / 224
  static_assert(NA >= 3, "activation ring too shallow");
};

struct GSmemBar {
  uint64_t a_full[kMaxNA], a_empty[kMaxNA];
  uint64_t b_full[kNB], b_empty[kNB];
  uint64_t raw_full[2], raw_empty[2];
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int      abort_flag;
};

// ---------------------------------------------------------------- tcgen05 wrappers

__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; issued by ONE thread
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
    "{\n\t.reg .pred p;\n\t"
    "setp.ne.b32 p, %4, 0;\n\t"
    "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
    "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
    : "memory");
}
// the mbarrier gets one arrival when every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
    "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
    "%29,%30,%31}, [%32];"
    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
      "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
      "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
      "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
    : "r"(taddr)
    : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    v[i] = __uint_as_float(r[i]);
  }
}

// K-major, 128-byte swizzled operand tile: rows of 128 bytes, 8-row atoms of 1024 bytes.
__device__ __forceinline__ uint64_t smem_desc_sw128(const void *tile) {
  const uint64_t addr = smem_u32(tile);
  return ((addr & 0x3FFFFull) >> 4) | (1ull << 16) /* leading byte offset: unused in this mode */ |
         ((1024ull >> 4) << 32) /* stride between 8-row atoms */ | (1ull << 46) /* descriptor version */ |
         (2ull << 61) /* SWIZZLE_128B */;
}

// c = fp32, a = b = fp16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
__host__ __device__ constexpr uint32_t instr_desc_f16(int n) {
  return (1u << 4) | ((uint32_t) (n >> 3) << 17) | ((uint32_t) (kBM >> 4) << 24);
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

// 64 weights (two blocks) of one row -> eight 16-byte chunks of fp16 (value * scale, rounded once)
template <int WT>
__device__ __forceinline__ void dequant_two_blocks(const uint32_t *raw /* words of the row's raw stage */, int q,
                                                   uint4 (&out)[8]) {
  // block b of the raw stage starts at byte b * BB; its scale is the first halfword
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int      b    = 2 * q + h;
    const int      off  = b * BlockTraits<WT>::kBytes;  // even, multiple of 4 when b is even
    const uint32_t sw   = raw[off >> 2];
    const uint16_t sbit = (off & 2) ? (uint16_t) (sw >> 16) : (uint16_t) (sw & 0xffff);
    const __half2  d2   = __half2half2(__ushort_as_half(sbit));
    auto           word = [&](int i) -> uint32_t {  // i-th 32-bit word of the block's quants
      const int o = off + 2 + 4 * i;
      return (o & 2) ? __byte_perm(raw[o >> 2], raw[(o >> 2) + 1], 0x5432) : raw[o >> 2];
    };
    if constexpr (WT == kQ4) {
      uint32_t lo[8], hi[8];  // fp16 pairs in element order: lo = elements 0..15, hi = 16..31
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        // bytes (B0, B1, B2, B3) -> (B0, B2, B1, B3): the unpack then yields {B0,B1} and {B2,B3}
        uint32_t u[4];
        q4_0_unpack_word(__byte_perm(word(i), 0u, 0x3120), u);
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
      uint32_t v[16];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        uint32_t u[2];
        q8_0_unpack_word(word(i), u);
        v[2 * i]     = h2_as_u32(__hmul2(u32_as_h2(u[0]), d2));
        v[2 * i + 1] = h2_as_u32(__hmul2(u32_as_h2(u[1]), d2));
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        out[4 * h + c] = make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
      }
    }
  }
}

// ---------------------------------------------------------------- the kernel

template <int WT, int BN>
__global__ void __launch_bounds__(kThreads, 1)
  gemm_tcgen05_kernel(const GemmArgs p, const __grid_constant__ CUtensorMap xmap,
                      const __grid_constant__ CUtensorMap wmap) {
  using C = GCfg<WT, BN>;
  static_assert(BN % 32 == 0 && BN <= 256 && 2 * BN <= kTmemCols, "tile width");
  static_assert(sizeof(GSmemBar) <= 512, "barrier block");
  constexpr int      kNA       = C::NA;
  constexpr int      A_BYTES   = C::A_BYTES;
  constexpr int      B_BYTES   = C::B_BYTES;
  constexpr int      RAW_BYTES = C::RAW_BYTES;
  constexpr uint32_t IDESC     = instr_desc_f16(BN);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // swizzled operand tiles need 1024-byte alignment in the shared address space
  uint8_t  *sA   = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t  *sB   = sA + kNA * A_BYTES;
  uint8_t  *sRaw = sB + kNB * B_BYTES;
  GSmemBar *bar  = reinterpret_cast<GSmemBar *>(sRaw + ((C::NR * RAW_BYTES + 127) & ~127));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int *abort_flag = &bar->abort_flag;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kNA; ++i) {
      mbar_init(&bar->a_full[i], 1);
      mbar_init(&bar->a_empty[i], 1);
    }
    for (int i = 0; i < kNB; ++i) {
      mbar_init(&bar->b_full[i], kDeqWarps * 32);
      mbar_init(&bar->b_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar->raw_full[i], 1);
      mbar_init(&bar->raw_empty[i], kDeqWarps);
      mbar_init(&bar->acc_full[i], 1);
      mbar_init(&bar->acc_empty[i], 4);
    }
    bar->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc(&bar->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bar->tmem_base;

  const int m_tiles = (p.M + kBM - 1) / kBM;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int tiles   = m_tiles * n_tiles;
  const int k_raws  = p.K / kKPerRaw;

  if (warp == 0) {
    // ---------------- TMA producer
    if (lane == 0) {
      tma_prefetch_descriptor(&xmap);
      tma_prefetch_descriptor(&wmap);
      const uint64_t pol_w = l2_policy_evict_last();   // a weight panel is re-read by the other token tiles
      const uint64_t pol_x = l2_policy_evict_last();
      Ring           ra(kNA), rr(C::NR);
      bool           ok = true;
      for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
        const int n0 = (t / m_tiles) * BN, m0 = (t % m_tiles) * kBM;
        for (int rs = 0; rs < k_raws && ok; ++rs) {
          ok = wait_or_abort(&bar->raw_empty[rr.slot], rr.phase ^ 1, abort_flag, p.err, kGemmErrProducer);
          if (!ok) {
            break;
          }
          mbar_arrive_expect_tx(&bar->raw_full[rr.slot], RAW_BYTES);
          tma_load_2d(sRaw + rr.slot * RAW_BYTES, &wmap, rs * (C::RB / 8), n0, &bar->raw_full[rr.slot], pol_w);
          rr.next();
          for (int q = 0; q < kKPerRaw / kBK; ++q) {
            ok = wait_or_abort(&bar->a_empty[ra.slot], ra.phase ^ 1, abort_flag, p.err, kGemmErrProducer);
            if (!ok) {
              break;
            }
            mbar_arrive_expect_tx(&bar->a_full[ra.slot], A_BYTES);
            tma_load_2d(sA + ra.slot * A_BYTES, &xmap, (rs * (kKPerRaw / kBK) + q) * kBK, m0, &bar->a_full[ra.slot],
                        pol_x);
            ra.next();
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer
    if (lane == 0) {
      Ring ra(kNA), rb(kNB);
      int  it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++it) {
        const int buf = it & 1, use = it >> 1;
        ok = wait_or_abort(&bar->acc_empty[buf], (use & 1) ^ 1, abort_flag, p.err, kGemmErrMma);
        if (!ok) {
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t) buf * BN;
        const int      k_steps = p.K / kBK;
        for (int kb = 0; kb < k_steps; ++kb) {
          ok = wait_or_abort(&bar->a_full[ra.slot], ra.phase, abort_flag, p.err, kGemmErrMma) &&
               wait_or_abort(&bar->b_full[rb.slot], rb.phase, abort_flag, p.err, kGemmErrMma);
          if (!ok) {
            break;
          }
          tc_fence_after();
          const uint64_t adesc = smem_desc_sw128(sA + ra.slot * A_BYTES);
          const uint64_t bdesc = smem_desc_sw128(sB + rb.slot * B_BYTES);
#pragma unroll
          for (int s = 0; s < kBK / 16; ++s) {
            // 16 fp16 = 32 bytes along K inside the swizzled row: +2 in the descriptor's 16-byte units
            umma_f16(d_tmem, adesc + 2 * s, bdesc + 2 * s, IDESC, (kb | s) ? 1u : 0u);
          }
          umma_commit(&bar->a_empty[ra.slot]);
          umma_commit(&bar->b_empty[rb.slot]);
          ra.next();
          rb.next();
        }
        if (ok) {
          umma_commit(&bar->acc_full[buf]);
        }
      }
    }
  } else if (warp >= kEpiWarp0 && warp < kEpiWarp0 + 4) {
    // ---------------- epilogue: TMEM -> registers -> y
    const int q4 = warp & 3;  // a warp may only touch TMEM lanes 32 * (warp % 4) .. + 31
    int       it = 0;
    bool      ok = true;
    for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++it) {
      const int buf = it & 1, use = it >> 1;
      const int n0 = (t / m_tiles) * BN, m0 = (t % m_tiles) * kBM;
      ok = wait_or_abort(&bar->acc_full[buf], use & 1, abort_flag, p.err, kGemmErrEpilogue);
      if (!ok) {
        break;
      }
      tc_fence_after();
      const int      row   = m0 + q4 * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t) (q4 * 32) << 16) + (uint32_t) buf * BN;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        float v[32];
        tmem_ld32(taddr + c0, v);
        if (row < p.M && n0 + c0 < p.N) {  // N is a multiple of 32: a 32-column group is in or out
          float4 *dst = reinterpret_cast<float4 *>(p.y + (long long) row * p.N + n0 + c0);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bar->acc_empty[buf]);
      }
    }
  } else if (warp >= kDeqWarp0) {
    // ---------------- dequantisation: thread r owns weight row r of the tile
    const int r = (warp - kDeqWarp0) * 32 + lane;
    Ring      rr(C::NR), rb(kNB);
    bool      ok = true;
    {
      for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
        for (int rs = 0; rs < k_raws && ok; ++rs) {
          ok = wait_or_abort(&bar->raw_full[rr.slot], rr.phase, abort_flag, p.err, kGemmErrDequant);
          if (!ok) {
            break;
          }
          // The row's 144 / 272 raw bytes go to registers with 16-byte loads, LAST chunk first.  The
          // stage is handed back to the TMA producer as soon as possible, but only after the loads
          // have RETURNED: issuing the release right behind the loads was observed to let the next
          // TMA copy overwrite the chunk loaded last before it was read (an mbarrier arrive does not
          // wait for this thread's outstanding shared-memory loads).  Chunk 0 is therefore loaded
          // last and consumed first (the first K step needs it), loads of one thread return in
          // order, and the release follows that first use.
          uint32_t raw[C::RW * 4 + 1];
          if (r < BN) {
            const uint32_t src = smem_u32(sRaw + rr.slot * RAW_BYTES + r * C::RB);
#pragma unroll
            for (int i = C::RW - 1; i >= 0; --i) {
              asm volatile("ld.volatile.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(raw[4 * i]), "=r"(raw[4 * i + 1]), "=r"(raw[4 * i + 2]), "=r"(raw[4 * i + 3])
                           : "r"(src + 16 * i)
                           : "memory");
            }
          }
          raw[C::RW * 4]     = 0;  // the word past the end is only ever the unused half of a byte_perm
          const int raw_slot = rr.slot;
          rr.next();
          // The fp16 values of a K step are computed BEFORE waiting for its operand stage to be
          // free, so the arithmetic overlaps the tensor core's work on the previous steps.
          uint4 out[8];
          if (r < BN) {
            dequant_two_blocks<WT>(raw, 0, out);
          }
          // `out` was computed from chunk 0, the load issued last: every raw load has returned
          asm volatile("fence.acq_rel.cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(&bar->raw_empty[raw_slot]);
          }
#pragma unroll
          for (int q = 0; q < kKPerRaw / kBK; ++q) {
            ok = wait_or_abort(&bar->b_empty[rb.slot], rb.phase ^ 1, abort_flag, p.err, kGemmErrDequant);
            if (!ok) {
              break;
            }
            if (r < BN) {
              uint8_t *row = sB + rb.slot * B_BYTES + r * 128;
#pragma unroll
              for (int c = 0; c < 8; ++c) {
                *reinterpret_cast<uint4 *>(row + ((c ^ (r & 7)) << 4)) = out[c];
              }
            }
            // every thread orders its own generic-proxy stores before the tensor core's async-proxy
            // reads, then arrives itself
            fence_async_smem();
            mbar_arrive(&bar->b_full[rb.slot]);
            rb.next();
            if (q + 1 < kKPerRaw / kBK && r < BN) {
              dequant_two_blocks<WT>(raw, q + 1, out);
            }
          }
        }
      }
    }
  }

  // ---------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
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

template <int WT, int BN>
cudaError_t launch(const GemmArgs &a, int sm_count, cudaStream_t stream) {
  using C = GCfg<WT, BN>;
  EncodeTiledFn enc = encode_fn();
  if (!enc) {
    return cudaErrorNotSupported;
  }
  CUtensorMap xmap, wmap;
  {
    const cuuint64_t gdim[2] = { (cuuint64_t) a.K, (cuuint64_t) a.M };
    const cuuint64_t gstr[1] = { (cuuint64_t) a.K * 2 };
    const cuuint32_t box[2]  = { kBK, kBM };
    const cuuint32_t es[2]   = { 1, 1 };
    if (enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(a.x), gdim, gstr, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      return cudaErrorInvalidValue;
    }
  }
  {
    const cuuint64_t row_bytes = (cuuint64_t) (a.K / 32) * C::BB;
    const cuuint64_t gdim[2]   = { row_bytes / 8, (cuuint64_t) a.N };
    const cuuint64_t gstr[1]   = { row_bytes };
    const cuuint32_t box[2]    = { C::RB / 8, BN };
    const cuuint32_t es[2]     = { 1, 1 };
    if (enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint8_t *>(a.w), gdim, gstr, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      return cudaErrorInvalidValue;
    }
  }
  const size_t smem = (size_t) C::NA * C::A_BYTES + C::FIXED;
  auto         kern = gemm_tcgen05_kernel<WT, BN>;
  cudaError_t  e    = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
  if (e != cudaSuccess) {
    return e;
  }
  const int m_tiles = (a.M + kBM - 1) / kBM, n_tiles = (a.N + BN - 1) / BN;
  int       grid    = m_tiles * n_tiles;
  if (grid > sm_count) {
    grid = sm_count;
  }
  kern<<<grid, kThreads, smem, stream>>>(a, xmap, wmap);
  return cudaGetLastError();
}

}  // namespace

cudaError_t gemm_tcgen05_launch(const GemmArgs &args, int wt, int sm_count, cudaStream_t stream) {
  // 224-column tiles give 256 tiles for N = 14336, M = 512 (1.73 waves) where 256 columns give 224
  // tiles (1.51 waves, the second half empty); otherwise the widest tile.
  const int  m_tiles = (args.M + kBM - 1) / kBM;
  const auto waves   = [&](int bn) {
    const long tiles = (long) m_tiles * ((args.N + bn - 1) / bn);
    const long full  = (tiles + sm_count - 1) / sm_count;
    return (double) tiles * bn / ((double) full * sm_count * bn) * (bn / 256.0 * 0.1 + 0.9);
  };
  const bool use224 = g_opt_gemm_tile_n ? g_opt_gemm_tile_n == 224 : waves(224) > waves(256);
  if (wt == kQ4) {
    return use224 ? launch<kQ4, 224>(args, sm_count, stream) : launch<kQ4, 256>(args, sm_count, stream);
  }
  // Q8_0: the 272-byte raw rows leave room for only three activation stages beside a 256-row tile
  const bool q8_224 = g_opt_gemm_tile_n ? g_opt_gemm_tile_n == 224 : true;
  return q8_224 ? launch<kQ8, 224>(args, sm_count, stream) : launch<kQ8, 256>(args, sm_count, stream);
}

}  // namespace htp
