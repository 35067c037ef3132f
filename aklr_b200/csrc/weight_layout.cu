// Load-time conversion of FP8 expert weights to the tile-contiguous layout the grouped GEMMs can take
// instead of the checkpoint's row-major one: [matrix][rows/128][cols/128][128 rows][128 bytes].  Every
// 128 x 128-byte box a TMA load fetches is then one contiguous 16 KB run of HBM.  The reference names
// such engine-side layouts as variants detected by a tensor attribute (its `Preshuffle` layout and
// `is_shuffled`, aklr/core/contract/semantics/_layouts.py:103-121,
// aklr/plugins/sglang/models/deepseek_v2/contract.py:181-185); this is the sm_100a counterpart.  Runs once
// per checkpoint, outside any layer call: one CTA per tile, 16-byte loads along a row, 16-byte stores.
#include "common.cuh"
#include "kernels.h"

namespace aklr {

__global__ void __launch_bounds__(256) tile_weights_fp8_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                               int row_tiles, int col_tiles, int64_t n_tiles) {
  const int cols16 = col_tiles * 8;  // 16-byte vectors per source row
  for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int ct = static_cast<int>(tile % col_tiles);
    const int64_t rt_all = tile / col_tiles;  // matrix * row_tiles + row tile
    const int64_t src_row0 = rt_all * 128;    // rows of all matrices are stacked
    for (int i = threadIdx.x; i < 128 * 8; i += blockDim.x) {
      const int r = i >> 3, v = i & 7;
      dst[tile * 1024 + i] = src[(src_row0 + r) * cols16 + ct * 8 + v];
    }
  }
  (void)row_tiles;
}

int launch_tile_weights_fp8(const void* src, void* dst, int64_t matrices, int rows, int cols, cudaStream_t stream) {
  if (rows % 128 != 0 || cols % 128 != 0 || rows < 128 || cols < 128 || matrices < 1) return AKLR_ERR_UNSUPPORTED_SHAPE;
  if (reinterpret_cast<uintptr_t>(src) % 16 != 0 || reinterpret_cast<uintptr_t>(dst) % 16 != 0) return AKLR_ERR_BAD_ARGUMENT;
  const int64_t n_tiles = matrices * (rows / 128) * (cols / 128);
  if (n_tiles * 128 >= (int64_t{1} << 31)) return AKLR_ERR_TOO_LARGE;  // a TMA coordinate is a 32-bit row index
  const int grid = static_cast<int>(n_tiles < 148 * 16 ? n_tiles : 148 * 16);
  tile_weights_fp8_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst), rows / 128,
                                                    cols / 128, n_tiles);
  return cudaGetLastError() == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

}  // namespace aklr
