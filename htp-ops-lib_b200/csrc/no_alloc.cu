// htp_b200_mul_mat_static_scratch: the decode mat-vec for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc once they are running: an inference server
// that hands the whole of device memory to its own pools at start-up (a later cudaMalloc fails or
// fragments the pool), or a latency-critical decode loop that cannot afford the device-wide
// synchronisation an allocation implies.  htp_b200_mul_mat allocates a small scratch area the
// first time it sees a (device, stream) pair; this entry point never does.  Its scratch is the
// file-scope device array below, which every GPU that loads the library holds until the process
// exits (kStaticScratchBytes, about 0.4 MB).
//
// Rules that follow from sharing one array:
//   * Every call on a device uses the same array, and the array keeps what the previous call left
//     in it.  The part that must start at zero (the arrival counters and the error word) is
//     cleared on the caller's stream at the start of every call.
//   * Two calls that overlap on the GPU (different streams, or different threads) race on the
//     array.  Calls must be ordered, for example by issuing them on one stream.
//   * The first call on a device looks the array's device address up (cudaGetSymbolAddress).  Make
//     that first call during set-up, before any stream capture is begun.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <mutex>

#include "device_ctx.h"
#include "gemv_mma.h"
#include "htp_ops_b200.h"

namespace {

constexpr int    kStaticMaxGrid      = 192;  // CTAs the scratch has room for (a B200 has 148 SMs)
constexpr size_t kStaticPartialBytes = (size_t) kStaticMaxGrid * 2 * 256 * sizeof(float);
constexpr size_t kStaticCounterBytes = (size_t) kStaticMaxGrid * sizeof(unsigned);
constexpr size_t kStaticScratchBytes = kStaticPartialBytes + kStaticCounterBytes + 256;

// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int  kMaxDevices = 64;
std::mutex     g_mu;
unsigned char *g_scratch_addr[kMaxDevices];  // device address of g_static_scratch, per device
int            g_sm_count[kMaxDevices];
int            g_max_smem[kMaxDevices];

// Once per device, with that device current: resolve the array's device address.
unsigned char *static_scratch_for_current_device(int *sm_count, int *max_smem) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_scratch_addr[dev]) {
    unsigned char *ptr = nullptr;
    if (cudaGetSymbolAddress((void **) &ptr, g_static_scratch) != cudaSuccess || !ptr ||
        cudaDeviceGetAttribute(&g_sm_count[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&g_max_smem[dev], cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) {
      cudaGetLastError();
      fprintf(stderr, "htp_b200_mul_mat_static_scratch: cannot resolve the static scratch on device %d\n", dev);
      return nullptr;
    }
    g_scratch_addr[dev] = ptr;
  }
  *sm_count = g_sm_count[dev];
  *max_smem = g_max_smem[dev];
  return g_scratch_addr[dev];
}

}  // namespace

extern "C" int htp_b200_mul_mat_static_scratch(void *dst, const void *activation, const void *weight, int m, int k,
                                                int n, int weight_type, int act_type, void *stream) {
  using namespace htp;
  // the same argument checks as htp_b200_mul_mat
  if (!dst || !activation || !weight || m <= 0 || n <= 0 || k <= 0 || k % 32 != 0 || n % 32 != 0) {
    return -1;
  }
  if (((uintptr_t) dst | (uintptr_t) activation | (uintptr_t) weight) & 127u) {
    return -1;
  }
  const int wt = weight_type == 2 ? 0 : (weight_type == 8 ? 1 : (weight_type == 20 ? 2 : -1));  // Q4_0, Q8_0, IQ4_NL
  if (wt < 0 || (act_type != HTP_B200_ACT_F32 && act_type != HTP_B200_ACT_F16)) {
    return -1;
  }
  // limits of this variant
  if (m > 8 || k % 256 != 0) {
    fprintf(stderr,
            "htp_b200_mul_mat_static_scratch: m = %d, k = %d is outside this entry point's range "
            "(m <= 8 and k a multiple of 256); use htp_b200_mul_mat\n", m, k);
    return -3;
  }
  int            sm_count = 0, max_smem = 0;
  unsigned char *scratch = static_scratch_for_current_device(&sm_count, &max_smem);
  if (!scratch) {
    return -2;
  }
  const bool a16     = act_type == HTP_B200_ACT_F16;
  const int  bb      = wt == 1 ? 34 : 18;
  const int  kblocks = k / 32;
  // the same plan as htp_b200_mul_mat (token padding, stage geometry, ring depth) - but a K range that
  // would need accumulating launches is refused here
  GemvPlan pl;
  if (!gemv_plan(max_smem, wt, a16, m, kblocks, &pl) || pl.nchunks > 1) {
    fprintf(stderr,
            "htp_b200_mul_mat_static_scratch: k = %d with m = %d needs more activation fragments than one launch "
            "holds in shared memory; use htp_b200_mul_mat (which splits K)\n", k, m);
    return -3;
  }
  const int    mpad  = pl.mpad;
  const int    stage = pl.stage_bytes;
  const int    nst   = pl.n_stages;
  const size_t frag  = gemv_frag_bytes(wt, a16, mpad, kblocks);
  GemvArgs a        = {};
  a.y               = static_cast<float *>(dst);
  a.x               = activation;
  a.w               = static_cast<const uint8_t *>(weight);
  a.w_row_bytes     = (long long) kblocks * bb;
  a.w_k_off_bytes   = 0;
  a.x_k_off         = 0;
  a.x_stride        = k;
  a.M               = m;
  a.N               = n;
  a.kblocks         = kblocks;
  a.accumulate      = 0;
  a.stages_per_tile = (kblocks + pl.stage_blocks - 1) / pl.stage_blocks;
  a.total_items     = (long long) (n / kGemvTileRows) * a.stages_per_tile;
  long long grid    = sm_count < kStaticMaxGrid ? sm_count : kStaticMaxGrid;
  if (grid > a.total_items) {
    grid = a.total_items;
  }
  // the same work split as htp_b200_mul_mat: one whole tile per CTA when there are no more tiles than SMs
  if (n / kGemvTileRows <= grid && g_opt_gemv_whole_tiles) {
    grid = n / kGemvTileRows;
  }
  const long long per_cta = (a.total_items + grid - 1) / grid;
  a.n_stages              = nst > per_cta ? (int) (per_cta < 2 ? 2 : per_cta) : nst;
  a.partials              = reinterpret_cast<float *>(scratch);
  a.counters              = reinterpret_cast<unsigned *>(scratch + kStaticPartialBytes);
  a.err                   = reinterpret_cast<int *>(scratch + kStaticPartialBytes + kStaticCounterBytes);
  cudaStream_t st         = static_cast<cudaStream_t>(stream);
  // the counters and the error word must start at zero; a kernel that gave up may have left some
  if (cudaMemsetAsync(a.counters, 0, kStaticCounterBytes + 256, st) != cudaSuccess) {
    cudaGetLastError();
    return -2;
  }
  const size_t smem = (size_t) gemv_header_bytes(mpad) + frag + (size_t) a.n_stages * stage;
  // plain stream order (no programmatic dependent launch): the memset above must be complete
  if (gemv_mma_launch(a, wt, a16, mpad, (int) grid, smem, st, false) != cudaSuccess) {
    cudaGetLastError();
    return -2;
  }
  count_launch();
  return 0;
}
