// Expert-parallel plumbing kernels, sm_100a.  Tokens stay on their home rank; a route to an
// expert of another rank travels as the FP8 row + its scales (NCCL all-to-all, issued by the host
// code), is computed there, and comes back as a weighted bf16 row.  Ownership follows the
// reference's statement: global expert e is local expert e % n_local of rank e / n_local
// (aklr/ops/mega_moe/reference.py:25,38).
#include "common.cuh"
#include "kernels.h"

namespace aklr {

// Per sent route: its expert id on the destination rank, its weight, and the inverse map
// route -> position in the send order (the home-side combine reads rows back through it).
__global__ void __launch_bounds__(256) ep_meta_kernel(EpMetaParams p) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= p.n_send) return;
  const int rid = p.sorted_ids[i];
  if (rid < 0 || rid >= p.n_routes) return;
  p.send_expert[i] = p.topk_ids[rid] % p.experts_per_rank;
  p.send_weight[i] = p.topk_weights[rid];
  p.position_of_route[rid] = i;
}

int launch_ep_meta(const EpMetaParams& p, cudaStream_t stream) {
  if (p.n_send == 0) return AKLR_OK;
  ep_meta_kernel<<<(p.n_send + 255) / 256, 256, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

// out[t] = bf16( sum_k rows[position(t,k)] + shared[t] ), float32 sum in slot order, shared last:
// the order of the single-GPU combine, so both give the same bits.
__global__ void __launch_bounds__(256) ep_combine_kernel(EpCombineParams p) {
  const int vec_per_row = p.hidden >> 3;
  const int64_t total = static_cast<int64_t>(p.n_tokens) * vec_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int token = static_cast<int>(i / vec_per_row);
    const int v = static_cast<int>(i - static_cast<int64_t>(token) * vec_per_row);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    auto add = [&](const void* base, size_t row) {
      const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + row * p.hidden + v * 8);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        acc[2 * q] += __uint_as_float(w[q] << 16);
        acc[2 * q + 1] += __uint_as_float(w[q] & 0xFFFF0000u);
      }
    };
    for (int s = 0; s < p.topk; ++s) {
      const int pos = p.position_of_route[token * p.topk + s];
      if (pos >= 0) add(p.rows, static_cast<size_t>(pos));
    }
    if (p.shared_rows) add(p.shared_rows, static_cast<size_t>(token));
    uint4 packed;
    uint32_t* o = reinterpret_cast<uint32_t*>(&packed);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const __nv_bfloat162 two = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
      o[q] = *reinterpret_cast<const uint32_t*>(&two);
    }
    *reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.out) + static_cast<size_t>(token) * p.hidden + v * 8) = packed;
  }
}

int launch_ep_combine(const EpCombineParams& p, cudaStream_t stream) {
  if (p.hidden % 8 != 0) return AKLR_ERR_UNSUPPORTED_SHAPE;
  if (p.n_tokens == 0) return AKLR_OK;
  const int64_t total = static_cast<int64_t>(p.n_tokens) * (p.hidden / 8);
  const int64_t blocks = (total + 255) / 256;
  const int grid = static_cast<int>(blocks < 148 * 8 ? blocks : 148 * 8);
  ep_combine_kernel<<<grid, 256, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

}  // namespace aklr
