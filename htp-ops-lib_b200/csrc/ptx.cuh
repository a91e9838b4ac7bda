// Thin inline-PTX wrappers used by the sm_100a kernels: mbarrier, bulk async copies,
// warp-level MMA, programmatic dependent launch.  Every wait is bounded: a wait that runs out
// returns false and the caller records an error code instead of spinning forever.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace htp {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- mbarrier

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
    "{\n\t.reg .pred p;\n\t"
    "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
    "selp.u32 %0, 1, 0, p;\n\t}"
    : "=r"(ok)
    : "r"(smem_u32(bar)), "r"(parity)
    : "memory");
  return ok != 0;
}

// Bounded wait.  try_wait itself blocks for a hardware-defined slice, so the cap below is
// far beyond any legitimate latency (seconds) yet finite.
constexpr uint32_t kWaitCap = 1u << 20;

__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
  for (uint32_t i = 0; i < kWaitCap; ++i) {
    if (mbar_try_wait(bar, parity)) {
      return true;
    }
    if (i >= 4) {
      __nanosleep(128);  // a failed try_wait returns at once: do not spin at full speed
    }
  }
  return false;
}

// ---------------------------------------------------------------- bulk async copy (no multicast)

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}

__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}

// global -> this CTA's shared memory; src, dst 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar,
                                         uint64_t policy) {
  asm volatile(
    "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
      smem_u32(dst_smem)),
    "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
    : "memory");
}

// 2-D tiled tensor copy global -> this CTA's shared memory through a tensor map (no multicast).
// x is the coordinate along the innermost dimension in ELEMENTS of the map's data type; x times
// the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void *dst_smem, const void *tmap, int x, int y, uint64_t *bar,
                                            uint64_t policy) {
  asm volatile(
    "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
    "[%0], [%1, {%2, %3}], [%4], %5;" ::"r"(smem_u32(dst_smem)),
    "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
    : "memory");
}

__device__ __forceinline__ void tma_prefetch_descriptor(const void *tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---------------------------------------------------------------- programmatic dependent launch

__device__ __forceinline__ void pdl_wait_prior_grids() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------- warp MMA m16n8k16 f16 x f16 -> f32

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
    "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
    : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
    : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// same, with a zero accumulator input: c = a * b
__device__ __forceinline__ void mma_16816_zero(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
    "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
    : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
    : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Barrier over `threads` threads that also ANDs a flag: every participant gets true only if every
// participant passed true.  Lets a group leave a loop together when one member has given up a wait.
__device__ __forceinline__ bool named_bar_and(int id, int threads, bool flag) {
  uint32_t out;
  asm volatile(
    "{\n\t.reg .pred p, q;\n\t"
    "setp.ne.u32 q, %3, 0;\n\t"
    "bar.red.and.pred p, %1, %2, q;\n\t"
    "selp.u32 %0, 1, 0, p;\n\t}"
    : "=r"(out)
    : "r"(id), "r"(threads), "r"((uint32_t) flag)
    : "memory");
  return out != 0;
}

}  // namespace htp
