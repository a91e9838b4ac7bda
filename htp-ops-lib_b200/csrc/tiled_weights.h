// Launcher of the matmul over weights stored in the reference's 32 x 32 tile order
// (tiled_weights.cu): fp16 tiles and the permuted Q4_0 / Q8_0 / IQ4_NL super-blocks.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace htp {

// Weight formats in tile order.  Tile (n / 32, k / 32) is tile number (n / 32) * (K / 32) + k / 32.
constexpr int kTileF16 = 0;  // 1024 fp16 per tile (2048 B)
constexpr int kTileQ4  = 1;  // four 144-byte super-blocks per tile (576 B), value = nibble - 8
constexpr int kTileQ8  = 2;  // four 272-byte super-blocks per tile (1088 B), value = signed byte
constexpr int kTileIQ4 = 3;  // as kTileQ4, value from the IQ4_NL table

// Bytes of one 32 x 32 tile, 0 for an unknown format.
__host__ __device__ constexpr int tile_bytes(int fmt) {
  return fmt == kTileF16 ? 2048 : (fmt == kTileQ8 ? 1088 : ((fmt == kTileQ4 || fmt == kTileIQ4) ? 576 : 0));
}

// y[M][N] (fp32) = x[M][K] . W, W[k][n] read from tile order.  K % 32 == 0, N % 32 == 0, x and w
// 16-byte aligned.  Any M: tokens are taken four at a time (grid.y), each group re-reading W.
cudaError_t tiled_mul_mat_launch(float *y, const void *x, const uint8_t *w, int M, int K, int N, int fmt, bool a16,
                                 cudaStream_t stream);

// Integer probe of the super-block decode (formats kTileQ4, kTileQ8, kTileIQ4): per scale group g of
// every super-block (8 groups of 32 consecutive slots each) s[8 * sb + g] = sum_j q_j and
// t[8 * sb + g] = sum_j (j + 1) q_j, j the slot's index within its group.
cudaError_t tiled_group_sums_launch(const uint8_t *w, int32_t *s, int32_t *t, long long n_super_blocks, int fmt,
                                    cudaStream_t stream);

}  // namespace htp
