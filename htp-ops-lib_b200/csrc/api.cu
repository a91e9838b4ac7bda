// Compute entry points (include/htp_ops_b200.h): argument checks in the reference's order
// (src/dsp/ops/mat_mul.c:878-892), kernel selection, launch.
#include "htp_ops_b200.h"

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

#include "aux_kernels.h"
#include "device_ctx.h"
#include "gemm_tcgen05.h"
#include "gemv_mma.h"
#include "tiled_weights.h"

namespace htp {

int g_opt_pdl           = getenv("HTP_OPS_NO_PDL") ? 0 : 1;  // programmatic dependent launch
int g_opt_force_generic = 0;
// Matmuls with at least this many tokens go to the tensor-core GEMM.  fp32 activations only from
// kGemmMinMF32 tokens on: up to there two passes of the decode kernel keep them exact.
int           g_opt_gemm_min_m = 9;
constexpr int kGemmMinMF32     = 17;
// fp32 activations reach the GEMM as fp16 copies (as in the reference, mat_mul.c:89-128).  1 = keep
// fp32-activation matmuls of any token count on the decode kernel (exact weights, fixed-point
// activations: 1e-5 instead of 1e-3, at one pass over the weights per eight tokens).
int g_opt_a32_exact      = 0;
int g_opt_gemv_whole_tiles = getenv("HTP_OPS_NO_WHOLE_TILES") ? 0 : 1;  // small mat-vecs: one whole tile per CTA
// Cut the GEMM's work into equal K ranges when the tile count is uneven.  Off by default: on the
// shapes measured (112 to 4008 tiles on 74 CTA pairs) the whole-tile schedule was 1-9 % faster -
// the SMs left idle in the last wave let the busy ones clock higher, and the split adds an
// epilogue that nothing overlaps.
int g_opt_gemm_split     = getenv("HTP_OPS_GEMM_SPLIT") ? 1 : 0;
// Op indices 2, 3 and 4 of the dispatcher read the reference's permuted super-blocks (1) instead of
// standard ggml blocks (0).
int g_opt_permuted_weights = 0;
int g_opt_gemm_tile_n    = 0;   // tokens per GEMM tile: 0 = by M, else 128 or 256

namespace {
std::mutex                                            g_mu;
std::map<int, DeviceCtx>                              g_devices;
std::map<std::pair<int, cudaStream_t>, StreamScratch> g_scratch;
std::atomic<uint64_t>                                 g_launches{ 0 };
}  // namespace

void count_launch(int n) {
  g_launches.fetch_add((uint64_t) n, std::memory_order_relaxed);
}

DeviceCtx *current_device_ctx() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  auto                        it = g_devices.find(dev);
  if (it != g_devices.end()) {
    return &it->second;
  }
  DeviceCtx c;
  c.device = dev;
  if (cudaDeviceGetAttribute(&c.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&c.max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return &(g_devices[dev] = c);
}

StreamScratch *stream_scratch(DeviceCtx *ctx, cudaStream_t stream) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto                        key = std::make_pair(ctx->device, stream);
  auto                        it  = g_scratch.find(key);
  if (it != g_scratch.end()) {
    return &it->second;
  }
  StreamScratch s;
  const size_t  pbytes = (size_t) kGemvMaxGrid * 2 * 256 * sizeof(float);
  const size_t  cbytes = (size_t) kGemvMaxGrid * sizeof(unsigned);
  uint8_t      *base   = nullptr;
  if (cudaMalloc(&base, pbytes + cbytes + 256) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  // (the memset runs on the default stream, which non-blocking streams do not wait for: finish it
  // before any kernel can use the area)
  if (cudaMemset(base, 0, pbytes + cbytes + 256) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    cudaGetLastError();
    cudaFree(base);
    return nullptr;
  }
  s.partials = reinterpret_cast<float *>(base);
  s.counters = reinterpret_cast<unsigned *>(base + pbytes);
  s.err      = reinterpret_cast<int *>(base + pbytes + cbytes);
  if (cudaHostAlloc(reinterpret_cast<void **>(&s.err_host), 64, cudaHostAllocDefault) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(base);
    return nullptr;
  }
  *s.err_host = 0;
  return &(g_scratch[key] = s);
}

// Split-tile scratch of the prefill GEMM for this stream (about 19 MB, allocated on the first GEMM
// of the stream).  nullptr when it cannot be had: the GEMM then runs without splitting tiles.
float *gemm_scratch(DeviceCtx *ctx, StreamScratch *sc) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (sc->gemm_part) {
    return sc->gemm_part;
  }
  const size_t bytes = gemm_scratch_bytes(ctx->sm_count);
  void        *base  = nullptr;
  if (cudaMalloc(&base, bytes) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  if (cudaMemset(base, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    cudaGetLastError();
    cudaFree(base);
    return nullptr;
  }
  sc->gemm_part = static_cast<float *>(base);
  return sc->gemm_part;
}

// Room for m x k fp16 activations and (after them) m per-token scales on this stream; grown when a
// larger matmul arrives (the stream is drained first: earlier GEMMs may still read the old area).
uint8_t *act16_scratch(StreamScratch *sc, cudaStream_t st, int m, int k, float **scales) {
  std::lock_guard<std::mutex> lk(g_mu);
  const size_t mpad = ((size_t) m + 255) & ~(size_t) 255;
  const size_t xb   = (mpad * (size_t) k * 2 + 255) & ~(size_t) 255;
  const size_t need = xb + mpad * sizeof(float);
  if (need > sc->act16_bytes) {
    if (sc->act16) {
      cudaStreamSynchronize(st);
      cudaFree(sc->act16);
      sc->act16 = nullptr, sc->act16_bytes = 0;
    }
    const size_t bytes = need + need / 2;
    void        *base  = nullptr;
    if (cudaMalloc(&base, bytes) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    sc->act16 = static_cast<uint8_t *>(base), sc->act16_bytes = bytes;
  }
  *scales = reinterpret_cast<float *>(sc->act16 + xb);
  return sc->act16;
}

// Room for the K-range slabs of one batch on this stream, grown when a larger batch arrives.
float *kslab_scratch(StreamScratch *sc, cudaStream_t st, size_t need) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (need > sc->kslab_bytes) {
    if (sc->kslab) {
      cudaStreamSynchronize(st);
      cudaFree(sc->kslab);
      sc->kslab = nullptr, sc->kslab_bytes = 0;
    }
    const size_t bytes = need + need / 2;
    void        *base  = nullptr;
    if (cudaMalloc(&base, bytes) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    sc->kslab = static_cast<uint8_t *>(base), sc->kslab_bytes = bytes;
  }
  return reinterpret_cast<float *>(sc->kslab);
}

void release_all_scratch() {
  std::lock_guard<std::mutex> lk(g_mu);
  int                         cur = -1;
  cudaGetDevice(&cur);
  for (auto &kv : g_scratch) {
    cudaSetDevice(kv.first.first);
    cudaFree(kv.second.partials);
    cudaFree(kv.second.gemm_part);
    cudaFree(kv.second.act16);
    cudaFree(kv.second.kslab);
    cudaFreeHost(kv.second.err_host);
  }
  g_scratch.clear();
  if (cur >= 0) {
    cudaSetDevice(cur);
  }
}

namespace {

inline bool aligned128(const void *p) {
  return (reinterpret_cast<uintptr_t>(p) & 127u) == 0;
}

// Tile-order formats (tiled_weights.h) behind their weight_type codes, -1 for the row-major ones.
inline int tile_fmt_index(int weight_type) {
  switch (weight_type) {
    case HTP_B200_WT_F16_TILED: return kTileF16;
    case HTP_B200_WT_PERMUTED | 2: return kTileQ4;
    case HTP_B200_WT_PERMUTED | 8: return kTileQ8;
    case HTP_B200_WT_PERMUTED | 20: return kTileIQ4;
    default: return -1;
  }
}

inline int wt_index(int weight_type) {
  return weight_type == 2 ? 0 : (weight_type == 8 ? 1 : (weight_type == 20 ? 2 : -1));  // kQ4, kQ8, kIQ4
}

// Decode path: M <= 8 rows of activations per launch, K split into launches whose activation
// fragments fit in shared memory next to at least three pipeline stages.
// Placement of the output as a column band of several matrices (see GemvArgs); nullptr = plain.
struct OutBand {
  int          n_dst;
  long long    ld, col0;
  float *const *more;  // n_dst - 1 further destinations
  unsigned *const *flags = nullptr;  // optional completion flags, one per destination
  unsigned     epoch     = 0;
  const unsigned *wait_flags = nullptr;  // optional: this GPU's flag array, waited for inside the launch
};

int run_gemv(DeviceCtx *ctx, float *dst, const void *act, const uint8_t *w, int m, int k, int n, int wt, bool a16,
             cudaStream_t stream, bool pdl, const OutBand *band = nullptr) {
  StreamScratch *sc = stream_scratch(ctx, stream);
  if (!sc) {
    return -2;
  }
  const int bb     = wt == 1 ? 34 : 18;
  const int kb_all = k / 32;
  const int asz    = a16 ? 2 : 4;

  // Eight tokens per launch (one or two on their own narrower paths); more tokens re-read the weights
  // once per slice of eight.
  const int slice = 8;
  for (int m0 = 0; m0 < m; m0 += slice) {
    const int mm = (m - m0) < slice ? (m - m0) : slice;
    GemvPlan  pl;
    if (!gemv_plan(ctx->max_smem, wt, a16, mm, kb_all, &pl)) {
      return -2;
    }
    if (band && pl.nchunks > 1) {
      return -1;  // K cut into ranges: not offered with several destinations
    }
    if (pl.nchunks > 1) {
      // the ranges run as entries of ONE persistent launch, each into a slab of its own, and a small
      // kernel adds the slabs (the batched form, with one operator)
      const MatMulDesc one = { dst + (size_t) m0 * n, static_cast<const uint8_t *>(act) + (size_t) m0 * k * asz, w, k, n };
      const int        rc  = mul_mat_batch_checked(&one, 1, mm, wt == 0 ? 2 : (wt == 1 ? 8 : 20),
                                                   a16 ? HTP_B200_ACT_F16 : HTP_B200_ACT_F32, stream, pdl);
      if (rc != 0) {
        return rc;
      }
      continue;
    }
    if (band && band->flags && m > slice) {
      return -1;  // the completion signal belongs to ONE launch
    }
    const int periods = kb_all / 8;
    for (int c = 0; c < pl.nchunks; ++c) {
      const int p0  = c * pl.chunk_periods;
      const int pn  = (periods - p0) < pl.chunk_periods ? (periods - p0) : pl.chunk_periods;
      GemvArgs  a   = {};
      a.y           = dst + (size_t) m0 * (band ? band->ld : n);
      if (band) {
        a.n_dst = band->n_dst, a.y_ld = band->ld, a.y_col0 = band->col0;
        for (int d = 1; d < band->n_dst; ++d) {
          a.y_more[d - 1] = band->more[d - 1] + (size_t) m0 * band->ld;
        }
        if (band->flags) {
          a.done_counter = reinterpret_cast<unsigned *>(sc->err) + 4;  // spare zeroed word of the scratch
          a.epoch        = band->epoch;
          for (int d = 0; d < band->n_dst; ++d) {
            a.sig_flags[d] = band->flags[d];
          }
          a.wait_flags = band->wait_flags;
          a.n_wait     = band->n_dst;
        }
      }
      a.x           = static_cast<const uint8_t *>(act) + (size_t) m0 * k * asz;
      a.w           = w;
      a.w_row_bytes = (long long) kb_all * bb;
      a.w_k_off_bytes = (long long) p0 * 8 * bb;
      a.x_k_off       = p0 * 256;
      a.x_stride      = k;
      a.M             = mm;
      a.N             = n;
      a.kblocks       = pn * 8;
      a.accumulate    = c > 0;
      a.stages_per_tile = (a.kblocks + pl.stage_blocks - 1) / pl.stage_blocks;
      a.total_items     = (long long) (n / kGemvTileRows) * a.stages_per_tile;
      const size_t frag = gemv_frag_bytes(wt, a16, pl.mpad, a.kblocks);
      // ring depth: never more stages than the busiest CTA has items
      long long grid = ctx->sm_count < kGemvMaxGrid ? ctx->sm_count : kGemvMaxGrid;
      if (grid > a.total_items) {
        grid = a.total_items;
      }
      // A matrix with no more tiles than SMs: one whole tile per CTA.  Equal item ranges would cut
      // nearly every tile in two, and the exchange of partial sums through scratch (stores, fences,
      // an atomic, a re-read by the last arriver) costs more than the few idle SMs.
      const long long tiles = n / kGemvTileRows;
      if (tiles <= grid && g_opt_gemv_whole_tiles) {
        grid = tiles;
      }
      const long long per_cta = (a.total_items + grid - 1) / grid;
      a.n_stages              = pl.n_stages;
      if (a.n_stages > per_cta) {
        a.n_stages = (int) (per_cta < 2 ? 2 : per_cta);
      }
      a.partials = sc->partials;
      a.counters = sc->counters;
      a.err      = sc->err;
      const size_t smem = (size_t) gemv_header_bytes(pl.mpad) + frag + (size_t) a.n_stages * pl.stage_bytes;
      if (gemv_mma_launch(a, wt, a16, pl.mpad, (int) grid, smem, stream, pdl) != cudaSuccess) {
        cudaGetLastError();
        return -2;
      }
      count_launch();
    }
  }
  return 0;
}

}  // namespace
}  // namespace htp

using namespace htp;

namespace htp {

int mul_mat_checked(void *dst, const void *activation, const void *weight, int m, int k, int n, int weight_type,
                    int act_type, cudaStream_t st, bool allow_pdl) {
  if (!dst || !activation || !weight || m <= 0 || n <= 0 || k <= 0) {
    return -1;
  }
  if (k % 32 != 0 || n % 32 != 0) {
    return -1;
  }
  if (!aligned128(dst) || !aligned128(activation) || !aligned128(weight)) {
    return -1;
  }
  const int wt   = wt_index(weight_type);
  const int tfmt = tile_fmt_index(weight_type);
  if ((wt < 0 && tfmt < 0) || (act_type != HTP_B200_ACT_F32 && act_type != HTP_B200_ACT_F16)) {
    return -1;
  }
  DeviceCtx *ctx = current_device_ctx();
  if (!ctx) {
    return -2;
  }
  const bool a16 = act_type == HTP_B200_ACT_F16;
  if (tfmt == kTileF16 && k % 128 == 0 && m >= g_opt_gemm_min_m && (a16 || (!g_opt_a32_exact && m >= kGemmMinMF32))) {
    // fp16 weights in the reference's tile order, many tokens: the tensor-core GEMM reads the tiles
    // as they lie (its "unpack" is a copy); fp32 activations go in as per-token scaled fp16 copies
    StreamScratch *sc = stream_scratch(ctx, st);
    if (!sc) {
      return -2;
    }
    GemmArgs a = {};
    a.y = static_cast<float *>(dst), a.x = activation, a.w = static_cast<const uint8_t *>(weight);
    a.M = m, a.N = n, a.K = k, a.err = sc->err;
    if (!a16) {
      float   *scales = nullptr;
      uint8_t *x16    = act16_scratch(sc, st, m, k, &scales);
      if (!x16 || act_f32_to_f16_launch(x16, scales, static_cast<const float *>(activation), m, k, st) != cudaSuccess) {
        cudaGetLastError();
        return -2;
      }
      count_launch();
      a.x = x16, a.tok_scale = scales;
    }
    if (gemm_tcgen05_launch(a, kGemmWtF16Tiled, ctx->sm_count, st) != cudaSuccess) {
      cudaGetLastError();
      return -2;
    }
    count_launch();
    return 0;
  }
  if (tfmt > kTileF16 && k % 128 == 0 && m >= g_opt_gemm_min_m && (a16 || (!g_opt_a32_exact && m >= kGemmMinMF32))) {
    // the reference's permuted super-blocks, many tokens: the same GEMM, its unpack reading the
    // super-blocks as they lie (value * scale rounded to fp16 once, as the reference does,
    // src/dsp/ops/mat_mul.c:396-405, 490-506)
    StreamScratch *sc = stream_scratch(ctx, st);
    if (!sc) {
      return -2;
    }
    GemmArgs a = {};
    a.y = static_cast<float *>(dst), a.x = activation, a.w = static_cast<const uint8_t *>(weight);
    a.M = m, a.N = n, a.K = k, a.err = sc->err;
    if (!a16) {
      float   *scales = nullptr;
      uint8_t *x16    = act16_scratch(sc, st, m, k, &scales);
      if (!x16 || act_f32_to_f16_launch(x16, scales, static_cast<const float *>(activation), m, k, st) != cudaSuccess) {
        cudaGetLastError();
        return -2;
      }
      count_launch();
      a.x = x16, a.tok_scale = scales;
    }
    const int gwt = tfmt == kTileQ4 ? kGemmWtPermQ4 : (tfmt == kTileQ8 ? kGemmWtPermQ8 : kGemmWtPermIQ4);
    if (gemm_tcgen05_launch(a, gwt, ctx->sm_count, st) != cudaSuccess) {
      cudaGetLastError();
      return -2;
    }
    count_launch();
    return 0;
  }
  if (tfmt >= 0) {
    // weights in the reference's tile order: streamed in place by the tile-order kernel
    if (tiled_mul_mat_launch(static_cast<float *>(dst), activation, static_cast<const uint8_t *>(weight), m, k, n,
                             tfmt, a16, st) != cudaSuccess) {
      cudaGetLastError();
      return -2;
    }
    count_launch();
    return 0;
  }
  if (g_opt_force_generic || k % 256 != 0) {
    if (mul_mat_generic_launch(static_cast<float *>(dst), activation, static_cast<const uint8_t *>(weight), m, k, n,
                               wt, a16, st) != cudaSuccess) {
      return -2;
    }
    count_launch();
    return 0;
  }
  if (m >= g_opt_gemm_min_m && (a16 || (!g_opt_a32_exact && m >= kGemmMinMF32))) {
    // prefill: tensor-core GEMM; fp32 activations go in as per-token scaled fp16 copies
    StreamScratch *sc = stream_scratch(ctx, st);
    if (!sc) {
      return -2;
    }
    GemmArgs a = {};
    a.y = static_cast<float *>(dst), a.x = activation, a.w = static_cast<const uint8_t *>(weight);
    a.M = m, a.N = n, a.K = k, a.err = sc->err;
    if (!a16) {
      float   *scales = nullptr;
      uint8_t *x16    = act16_scratch(sc, st, m, k, &scales);
      if (!x16 || act_f32_to_f16_launch(x16, scales, static_cast<const float *>(activation), m, k, st) != cudaSuccess) {
        cudaGetLastError();
        return -2;
      }
      count_launch();
      a.x = x16, a.tok_scale = scales;
    }
    a.part = g_opt_gemm_split ? gemm_scratch(ctx, sc) : nullptr;
    if (gemm_tcgen05_launch(a, wt, ctx->sm_count, st) != cudaSuccess) {
      cudaGetLastError();
      return -2;
    }
    count_launch();
    return 0;
  }
  return run_gemv(ctx, static_cast<float *>(dst), activation, static_cast<const uint8_t *>(weight), m, k, n, wt, a16,
                  st, allow_pdl && g_opt_pdl != 0);
}


bool mul_mat_batchable(int m, int k, int n, int weight_type, int act_type) {
  const int wt = wt_index(weight_type);
  if (wt < 0 || m <= 0 || m > 8 || k <= 0 || n <= 0 || k % 256 != 0 || n % 32 != 0 || g_opt_force_generic) {
    return false;
  }
  const bool a16 = act_type == HTP_B200_ACT_F16;
  GemvPlan   pl;
  return gemv_plan(kGemvSmemBudget, wt, a16, m, k / 32, &pl);
}

// Operators are laid end to end in persistent launches of up to kGemvBatchMaxOps entries.  An operator
// whose activation fragments do not fit one launch is entered once per K range; each range writes a
// slab of its own in stream scratch, and one small kernel afterwards adds the slabs into the output in
// range order (deterministic, no atomics, no launches that wait for each other's outputs).
int mul_mat_batch_checked(const MatMulDesc *d, int n_ops, int m, int weight_type, int act_type, cudaStream_t st,
                          bool allow_pdl) {
  const int wt = wt_index(weight_type);
  if (!d || n_ops <= 0 || wt < 0 || (act_type != HTP_B200_ACT_F32 && act_type != HTP_B200_ACT_F16)) {
    return -1;
  }
  for (int i = 0; i < n_ops; ++i) {
    if (!d[i].y || !d[i].x || !d[i].w || !aligned128(d[i].y) || !aligned128(d[i].x) || !aligned128(d[i].w) ||
        !mul_mat_batchable(m, d[i].k, d[i].n, weight_type, act_type)) {
      return -1;
    }
  }
  DeviceCtx *ctx = current_device_ctx();
  if (!ctx) {
    return -2;
  }
  StreamScratch *sc = stream_scratch(ctx, st);
  if (!sc) {
    return -2;
  }
  const bool a16    = act_type == HTP_B200_ACT_F16;
  const int  bb     = wt == 1 ? 34 : 18;
  const int  budget = ctx->max_smem < kGemvSmemBudget ? ctx->max_smem : kGemvSmemBudget;
  std::vector<GemvPlan> plans((size_t) n_ops);
  size_t                slab_floats = 0;
  for (int i = 0; i < n_ops; ++i) {
    if (!gemv_plan(budget, wt, a16, m, d[i].k / 32, &plans[i])) {
      return -2;
    }
    if (plans[i].nchunks > 1) {
      slab_floats += (size_t) plans[i].nchunks * m * d[i].n;
    }
  }
  float *slabs = nullptr;
  if (slab_floats && !(slabs = kslab_scratch(sc, st, slab_floats * sizeof(float)))) {
    return -2;
  }
  const int mpad  = plans[0].mpad;
  const int stage = plans[0].stage_bytes;
  const int sb    = plans[0].stage_blocks;
  static thread_local GemvBatchArgs args;  // ~25 KB of kernel parameters, reused between launches
  static thread_local KSumArgs      sums;
  sums.n_ops = 0;
  auto flush_sums = [&]() -> bool {
    if (sums.n_ops == 0) {
      return true;
    }
    if (k_range_sum_launch(sums, st) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    count_launch();
    sums.n_ops = 0;
    return true;
  };
  int       cnt   = 0;
  long long items = 0;
  size_t    frag  = 0;
  auto launch_entries = [&]() -> bool {
    if (cnt == 0) {
      return true;
    }
    args.total_items = items;
    args.partials    = sc->partials;
    args.counters    = sc->counters;
    args.err         = sc->err;
    args.n_ops       = cnt;
    args.M           = m;
    args.frag_bytes  = (int) frag;
    long long grid   = ctx->sm_count < kGemvMaxGrid ? ctx->sm_count : kGemvMaxGrid;
    if (grid > items) {
      grid = items;
    }
    int nst = (int) (((long) budget - gemv_header_bytes(mpad) - (long) frag) / stage);
    nst     = nst > kGemvMaxStages ? kGemvMaxStages : nst;
    const long long per_cta = (items + grid - 1) / grid;
    if (nst > per_cta) {
      nst = (int) (per_cta < 2 ? 2 : per_cta);
    }
    if (nst < 2) {
      return false;
    }
    args.n_stages     = nst;
    const size_t smem = (size_t) gemv_header_bytes(mpad) + frag + (size_t) nst * stage;
    if (gemv_mma_batch_launch(args, wt, a16, mpad, (int) grid, smem, st, allow_pdl && g_opt_pdl != 0) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    count_launch();
    cnt = 0, items = 0, frag = 0;
    return true;
  };
  size_t slab_at = 0;
  for (int i = 0; i < n_ops; ++i) {
    const MatMulDesc &q       = d[i];
    const int         kb_all  = q.k / 32;
    const int         periods = kb_all / 8;
    const int         nch     = plans[i].nchunks;
    float            *slab    = nch > 1 ? slabs + slab_at : nullptr;
    for (int c = 0; c < nch; ++c) {
      if (cnt == kGemvBatchMaxOps && !launch_entries()) {
        return -2;
      }
      GemvBatchOp &op = args.ops[cnt++];
      const int    p0 = c * plans[i].chunk_periods;
      const int    pn = (periods - p0) < plans[i].chunk_periods ? (periods - p0) : plans[i].chunk_periods;
      const int    kb = pn * 8;
      if (gemv_weight_map(op.wmap, q.w + (size_t) p0 * 8 * bb, (long long) kb_all * bb, kb, q.n, wt) != cudaSuccess) {
        cudaGetLastError();
        return -2;
      }
      op.y               = slab ? slab + (size_t) c * m * q.n : q.y;
      op.x               = q.x;
      op.item_begin      = items;
      op.N               = q.n;
      op.kblocks         = kb;
      op.x_stride        = q.k;
      op.x_k_off         = p0 * 256;
      op.accumulate      = 0;
      op.stages_per_tile = (kb + sb - 1) / sb;
      items += (long long) (q.n / kGemvTileRows) * op.stages_per_tile;
      const size_t f = gemv_frag_bytes(wt, a16, mpad, kb);
      frag           = f > frag ? f : frag;
    }
    if (slab) {
      slab_at += (size_t) nch * m * q.n;
      if (sums.n_ops == kKSumMaxOps) {
        // the sums read what the entries collected so far write: issue those first
        if (!launch_entries() || !flush_sums()) {
          return -2;
        }
      }
      sums.ops[sums.n_ops++] = KSumOp{ q.y, slab, (long long) m * q.n, nch };
    }
  }
  if (!launch_entries() || !flush_sums()) {
    return -2;
  }
  return 0;
}

}  // namespace htp

extern "C" {

int htp_b200_mul_mat(void *dst, const void *activation, const void *weight, int m, int k, int n, int weight_type,
                     int act_type, void *stream) {
  return mul_mat_checked(dst, activation, weight, m, k, n, weight_type, act_type, static_cast<cudaStream_t>(stream),
                         true);
}

int htp_b200_mul_mat_batch(int n_ops, void *const *dst, const void *const *activation, const void *const *weight,
                           const int *k, const int *n, int m, int weight_type, int act_type, void *stream) {
  if (n_ops <= 0 || !dst || !activation || !weight || !k || !n) {
    return -1;
  }
  std::vector<MatMulDesc> d((size_t) n_ops);
  for (int i = 0; i < n_ops; ++i) {
    d[i] = MatMulDesc{ static_cast<float *>(dst[i]), activation[i], static_cast<const uint8_t *>(weight[i]), k[i],
                       n[i] };
    if (!mul_mat_batchable(m, k[i], n[i], weight_type, act_type)) {
      return -1;
    }
  }
  return mul_mat_batch_checked(d.data(), n_ops, m, weight_type, act_type, static_cast<cudaStream_t>(stream), true);
}

int htp_b200_decode_plan(int m, int k, int weight_type, int act_type, int *k_ranges, int *range_k, int *stages) {
  const int wt = wt_index(weight_type);
  if (wt < 0 || m < 1 || m > 8 || k <= 0 || k % 256 != 0 || (act_type != HTP_B200_ACT_F32 && act_type != HTP_B200_ACT_F16)) {
    return -1;
  }
  GemvPlan pl;
  if (!gemv_plan(kGemvSmemBudget, wt, act_type == HTP_B200_ACT_F16, m, k / 32, &pl)) {
    return -1;
  }
  if (k_ranges) {
    *k_ranges = pl.nchunks;
  }
  if (range_k) {
    *range_k = pl.chunk_periods * 256;
  }
  if (stages) {
    *stages = pl.n_stages;
  }
  return 0;
}

int htp_b200_block_sums(const void *weight, int32_t *s, int32_t *t, int64_t n_blocks, int weight_type, void *stream) {
  const int wt   = wt_index(weight_type);
  const int tfmt = tile_fmt_index(weight_type);
  if (tfmt > kTileF16) {
    // permuted super-blocks: a "block" is a scale group (32 slots), eight per super-block
    if (!weight || !s || !t || n_blocks < 0 || n_blocks % 8 != 0 || (reinterpret_cast<uintptr_t>(weight) & 15u)) {
      return -1;
    }
    if (!current_device_ctx()) {
      return -2;
    }
    if (tiled_group_sums_launch(static_cast<const uint8_t *>(weight), s, t, n_blocks / 8, tfmt,
                                static_cast<cudaStream_t>(stream)) != cudaSuccess) {
      cudaGetLastError();
      return -2;
    }
    if (n_blocks > 0) {
      count_launch();
    }
    return 0;
  }
  if (!weight || !s || !t || n_blocks < 0 || wt < 0 || (reinterpret_cast<uintptr_t>(weight) & 1u)) {
    return -1;
  }
  if (!current_device_ctx()) {
    return -2;
  }
  if (block_sums_launch(static_cast<const uint8_t *>(weight), s, t, n_blocks, wt, static_cast<cudaStream_t>(stream)) !=
      cudaSuccess) {
    return -2;
  }
  if (n_blocks > 0) {
    count_launch();
  }
  return 0;
}

static int mul_mat_multi_dst_impl(void *const *dsts, int n_dst, int64_t dst_ld, int64_t dst_col0, const void *activation,
                                  const void *weight, int m, int k, int n, int weight_type, int act_type,
                                  unsigned *const *flags, unsigned epoch, void *stream,
                                  const unsigned *wait_flags = nullptr);

int htp_b200_mul_mat_multi_dst(void *const *dsts, int n_dst, int64_t dst_ld, int64_t dst_col0, const void *activation,
                               const void *weight, int m, int k, int n, int weight_type, int act_type, void *stream) {
  return mul_mat_multi_dst_impl(dsts, n_dst, dst_ld, dst_col0, activation, weight, m, k, n, weight_type, act_type, nullptr,
                                0, stream);
}

int htp_b200_mul_mat_multi_dst_signal(void *const *dsts, int n_dst, int64_t dst_ld, int64_t dst_col0,
                                      const void *activation, const void *weight, int m, int k, int n, int weight_type,
                                      int act_type, uint32_t *const *flags, uint32_t epoch, void *stream) {
  if (!flags || m > 8) {
    return -1;
  }
  for (int d = 0; d < n_dst && d < kGemmMaxDst; ++d) {
    if (!flags[d] || (reinterpret_cast<uintptr_t>(flags[d]) & 3u)) {
      return -1;
    }
  }
  return mul_mat_multi_dst_impl(dsts, n_dst, dst_ld, dst_col0, activation, weight, m, k, n, weight_type, act_type, flags,
                                epoch, stream);
}

int htp_b200_mul_mat_gather_step(void *const *dsts, int n_dst, int64_t dst_ld, int64_t dst_col0, const void *activation,
                                 const void *weight, int m, int k, int n, int weight_type, int act_type,
                                 uint32_t *const *flags, const uint32_t *local_flags, uint32_t epoch, void *stream) {
  if (!flags || !local_flags || m > 8 || (reinterpret_cast<uintptr_t>(local_flags) & 3u)) {
    return -1;
  }
  for (int d = 0; d < n_dst && d < kGemmMaxDst; ++d) {
    if (!flags[d] || (reinterpret_cast<uintptr_t>(flags[d]) & 3u)) {
      return -1;
    }
  }
  // one launch: the mat-vec signals, and its last CTA waits for the peers' flags
  return mul_mat_multi_dst_impl(dsts, n_dst, dst_ld, dst_col0, activation, weight, m, k, n, weight_type, act_type, flags,
                                epoch, stream, local_flags);
}

int htp_b200_wait_flags(const uint32_t *flags, int n, uint32_t epoch, void *stream) {
  if (!flags || n < 1 || n > 32 || (reinterpret_cast<uintptr_t>(flags) & 3u)) {
    return -1;
  }
  DeviceCtx *ctx = current_device_ctx();
  if (!ctx) {
    return -2;
  }
  cudaStream_t   st = static_cast<cudaStream_t>(stream);
  StreamScratch *sc = stream_scratch(ctx, st);
  if (!sc || flags_wait_launch(flags, n, epoch, sc->err, st) != cudaSuccess) {
    cudaGetLastError();
    return -2;
  }
  count_launch();
  return 0;
}

static int mul_mat_multi_dst_impl(void *const *dsts, int n_dst, int64_t dst_ld, int64_t dst_col0, const void *activation,
                                  const void *weight, int m, int k, int n, int weight_type, int act_type,
                                  unsigned *const *flags, unsigned epoch, void *stream, const unsigned *wait_flags) {
  if (!dsts || n_dst < 1 || n_dst > kGemmMaxDst || !activation || !weight || m <= 0 || n <= 0 || k <= 0) {
    return -1;
  }
  const int  wt     = wt_index(weight_type);
  const bool a16    = act_type == HTP_B200_ACT_F16;
  const bool decode = m <= 8;
  // the decode kernel (m <= 8) or the tensor-core GEMM (fp16 activations, m >= gemm_min_m); both want
  // 16-byte aligned weight rows
  if (wt < 0 || (act_type != HTP_B200_ACT_F32 && !a16) || k % 256 != 0 || n % 32 != 0 ||
      (!decode && (!a16 || m < g_opt_gemm_min_m))) {
    return -1;
  }
  if (dst_ld < n || dst_ld % 32 != 0 || dst_col0 < 0 || dst_col0 % 32 != 0 || dst_col0 + n > dst_ld) {
    return -1;
  }
  if (!aligned128(activation) || !aligned128(weight)) {
    return -1;
  }
  for (int d = 0; d < n_dst; ++d) {
    if (!dsts[d] || !aligned128(dsts[d])) {
      return -1;
    }
  }
  DeviceCtx *ctx = current_device_ctx();
  if (!ctx) {
    return -2;
  }
  cudaStream_t   st = static_cast<cudaStream_t>(stream);
  StreamScratch *sc = stream_scratch(ctx, st);
  if (!sc) {
    return -2;
  }
  if (decode) {
    float *more[kGemmMaxDst - 1] = {};
    for (int d = 1; d < n_dst; ++d) {
      more[d - 1] = static_cast<float *>(dsts[d]);
    }
    OutBand band = { n_dst, dst_ld, dst_col0, more };
    band.flags      = flags;
    band.epoch      = epoch;
    band.wait_flags = wait_flags;
    return run_gemv(ctx, static_cast<float *>(dsts[0]), activation, static_cast<const uint8_t *>(weight), m, k, n, wt,
                    a16, st, g_opt_pdl != 0, &band);
  }
  GemmArgs a = {};
  a.y = static_cast<float *>(dsts[0]), a.x = activation, a.w = static_cast<const uint8_t *>(weight);
  a.M = m, a.N = n, a.K = k, a.err = sc->err;
  a.n_dst = n_dst, a.y_ld = dst_ld, a.y_col0 = dst_col0;
  for (int d = 1; d < n_dst; ++d) {
    a.y_more[d - 1] = static_cast<float *>(dsts[d]);
  }
  if (gemm_tcgen05_launch(a, wt, ctx->sm_count, st) != cudaSuccess) {
    cudaGetLastError();
    return -2;
  }
  count_launch();
  return 0;
}

int htp_b200_rms_norm_f32(float *dst, const float *src, int ne0, int ne1, void *stream) {
  // argument rules of the reference: src/dsp/ops/rms_norm.c:69-74
  if (!dst || !src || ne0 <= 0 || ne1 <= 0) {
    return -1;
  }
  if ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 127u) {
    return -1;
  }
  if (!current_device_ctx()) {
    return -2;
  }
  if (rms_norm_f32_launch(dst, src, ne0, ne1, static_cast<cudaStream_t>(stream)) != cudaSuccess) {
    return -2;
  }
  count_launch();
  return 0;
}

size_t htp_b200_weight_bytes(int weight_type, int64_t k, int64_t n) {
  const int tfmt = tile_fmt_index(weight_type);
  if (tfmt >= 0) {
    if (k <= 0 || n <= 0 || k % 32 != 0 || n % 32 != 0) {
      return 0;
    }
    return (size_t) (n / 32) * (size_t) (k / 32) * (size_t) tile_bytes(tfmt);
  }
  const int wt = wt_index(weight_type);
  if (wt < 0 || k <= 0 || n <= 0 || k % 32 != 0) {
    return 0;
  }
  return (size_t) n * (size_t) (k / 32) * (wt == 1 ? 34u : 18u);
}

int htp_b200_stream_status(void *stream) {
  DeviceCtx *ctx = current_device_ctx();
  if (!ctx) {
    return -2;
  }
  cudaStream_t   st = static_cast<cudaStream_t>(stream);
  StreamScratch *sc = stream_scratch(ctx, st);
  if (!sc) {
    return -2;
  }
  // the error word travels to pinned host memory behind the work it reports on: ONE wait, no
  // blocking copy afterwards
  if (cudaMemcpyAsync(sc->err_host, sc->err, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
      cudaStreamSynchronize(st) != cudaSuccess) {
    return -2;
  }
  const int code = *static_cast<volatile int *>(sc->err_host);
  if (code != 0) {
    cudaMemsetAsync(sc->err, 0, 32, st);  // the error word and the launch-completion counter behind it
    // a kernel that gave up may have left arrival counters behind
    cudaMemsetAsync(sc->counters, 0, (size_t) kGemvMaxGrid * sizeof(unsigned), st);
    cudaStreamSynchronize(st);
  }
  return code;
}

int htp_b200_set_option(const char *name, int value) {
  if (!name) {
    return -1;
  }
  int *slot = nullptr;
  if (!strcmp(name, "pdl")) {
    slot = &g_opt_pdl;
  } else if (!strcmp(name, "force_generic")) {
    slot = &g_opt_force_generic;
  } else if (!strcmp(name, "gemm_min_m")) {
    slot = &g_opt_gemm_min_m;
  } else if (!strcmp(name, "gemm_tile_n")) {
    if (value != 0 && value != 128 && value != 256) {
      return -1;
    }
    slot = &g_opt_gemm_tile_n;
  } else if (!strcmp(name, "gemm_split")) {
    slot = &g_opt_gemm_split;
  } else if (!strcmp(name, "permuted_weights")) {
    slot = &g_opt_permuted_weights;
  } else if (!strcmp(name, "a32_exact")) {
    slot = &g_opt_a32_exact;
  }
  if (!slot) {
    return -1;
  }
  const int old = *slot;
  *slot         = value;
  return old;
}

uint64_t htp_b200_launch_count(void) {
  return g_launches.load(std::memory_order_relaxed);
}

const char *htp_b200_version(void) {
  return "htp-ops-lib_b200 0.1 (sm_100a)";
}

}  // extern "C"
