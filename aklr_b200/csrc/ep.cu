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

// ---- one row per (token, destination rank) ------------------------------------------------------
// A token whose routes name several experts of one rank sends that rank ONE row; the rank runs all of
// them and returns one row, their weighted sum.  first_rank[t, s] = rank of slot s when no earlier slot
// of the token goes to the same rank, else -1: sorting these "pairs" by rank (moe_align, block 1) gives
// the send order.  position_of_route starts at -1 everywhere; pack fills in the sent slots.
__global__ void __launch_bounds__(256) ep_first_slots_kernel(EpPlanParams p) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= p.n_tokens) return;
  const int32_t* ids = p.topk_ids + static_cast<size_t>(t) * p.topk;
  for (int s = 0; s < p.topk; ++s) {
    const int e = ids[s];
    int rank = e >= 0 ? e / p.experts_per_rank : -1;
    for (int q = 0; q < s && rank >= 0; ++q)
      if (ids[q] >= 0 && ids[q] / p.experts_per_rank == rank) rank = -1;
    p.first_rank[static_cast<size_t>(t) * p.topk + s] = rank;
    p.position_of_route[static_cast<size_t>(t) * p.topk + s] = -1;
  }
}

int launch_ep_first_slots(const EpPlanParams& p, cudaStream_t stream) {
  if (p.n_tokens == 0) return AKLR_OK;
  if (p.topk < 1 || p.topk > 32 || p.experts_per_rank < 1) return AKLR_ERR_BAD_ARGUMENT;
  ep_first_slots_kernel<<<(p.n_tokens + 255) / 256, 256, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

// Send row i = token t's quantised row, its scales, and for each of the token's slots the expert id local
// to the destination rank (or -1 when the slot goes elsewhere) with its weight: one buffer, one all-to-all.
// Row layout: [hidden codes][scale_bytes scales][topk int32 ids][topk float weights], padded to row_bytes.
__global__ void __launch_bounds__(256) ep_pack_kernel(EpPackParams p) {
  const int vec_per_row = p.hidden >> 4;
  const int scale_words = p.scale_bytes >> 2;
  const int n_send = p.n_send_device ? min(__ldg(p.n_send_device), p.n_send) : p.n_send;
  for (int i = blockIdx.x; i < n_send; i += gridDim.x) {
    const int rid = p.sorted_ids[i];
    if (rid < 0 || rid >= p.n_tokens * p.topk) continue;
    const int t = rid / p.topk;
    uint8_t* dst = p.packed + static_cast<size_t>(i) * p.row_bytes;
    const uint4* src = reinterpret_cast<const uint4*>(p.tokens_q + static_cast<size_t>(t) * p.hidden);
    for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) reinterpret_cast<uint4*>(dst)[v] = __ldg(src + v);
    const uint32_t* ssrc = reinterpret_cast<const uint32_t*>(p.tokens_scale + static_cast<size_t>(t) * p.scale_bytes);
    for (int v = threadIdx.x; v < scale_words; v += blockDim.x)
      reinterpret_cast<uint32_t*>(dst + p.hidden)[v] = __ldg(ssrc + v);
    if (threadIdx.x < p.topk) {
      const int s = threadIdx.x;
      const int rank = p.topk_ids[rid] / p.experts_per_rank;
      const int e = p.topk_ids[static_cast<size_t>(t) * p.topk + s];
      const bool here = e >= 0 && e / p.experts_per_rank == rank;
      int32_t* meta = reinterpret_cast<int32_t*>(dst + p.hidden + p.scale_bytes);
      meta[s] = here ? e % p.experts_per_rank : -1;
      reinterpret_cast<float*>(meta + p.topk)[s] = here ? p.topk_weights[static_cast<size_t>(t) * p.topk + s] : 0.0f;
    }
    if (threadIdx.x == 0) p.position_of_route[rid] = i;
  }
}

int launch_ep_pack(const EpPackParams& p, cudaStream_t stream) {
  if (p.n_send == 0) return AKLR_OK;
  if (p.hidden % 16 != 0 || p.scale_bytes % 4 != 0 || p.row_bytes % 16 != 0 || p.topk < 1 || p.topk > 32 ||
      p.row_bytes < p.hidden + p.scale_bytes + 8 * p.topk)
    return AKLR_ERR_BAD_ARGUMENT;
  const int grid = p.n_send < 148 * 16 ? p.n_send : 148 * 16;
  ep_pack_kernel<<<grid, 256, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

// Receiver: the ids and weights of the rows received, as the [rows, topk] tables the expert call takes.
__global__ void __launch_bounds__(256) ep_unpack_meta_kernel(const uint8_t* packed, int n_rows, int row_bytes, int meta_offset,
                                                             int topk, int32_t* ids, float* weights) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_rows * topk) return;
  const int row = i / topk, s = i - row * topk;
  const int32_t* meta = reinterpret_cast<const int32_t*>(packed + static_cast<size_t>(row) * row_bytes + meta_offset);
  ids[i] = meta[s];
  weights[i] = reinterpret_cast<const float*>(meta + topk)[s];
}

int launch_ep_unpack_meta(const uint8_t* packed, int n_rows, int row_bytes, int meta_offset, int topk, int32_t* ids,
                          float* weights, cudaStream_t stream) {
  if (n_rows == 0) return AKLR_OK;
  if (meta_offset % 4 != 0 || row_bytes % 4 != 0 || topk < 1) return AKLR_ERR_BAD_ARGUMENT;
  ep_unpack_meta_kernel<<<(n_rows * topk + 255) / 256, 256, 0, stream>>>(packed, n_rows, row_bytes, meta_offset, topk, ids, weights);
  return cudaGetLastError() == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

// The split sizes of the uneven all-to-all have to reach the host.  A device-to-host copy would queue on
// the copy engine behind whatever large copy a serving loop has in flight there (a step's output going
// back to the host: milliseconds); stores from an SM into mapped pinned host memory do not.
__global__ void ep_counts_to_host_kernel(const int32_t* send_counts, const int32_t* recv_counts, int world,
                                         int32_t* host_mapped) {
  const int i = threadIdx.x;
  if (i < world) {
    volatile int32_t* out = host_mapped;
    out[i] = send_counts[i];
    out[world + i] = recv_counts[i];
  }
  __threadfence_system();
}

int launch_ep_counts_to_host(const int32_t* send_counts, const int32_t* recv_counts, int world, int32_t* host_mapped,
                             cudaStream_t stream) {
  if (world < 1 || world > 1024) return AKLR_ERR_BAD_ARGUMENT;
  ep_counts_to_host_kernel<<<1, (world + 31) / 32 * 32, 0, stream>>>(send_counts, recv_counts, world, host_mapped);
  return cudaGetLastError() == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

// out[t] = bf16( sum_k rows[position(t,k)] + shared[t] ), float32 sum in slot order, shared last:
// the order of the single-GPU combine, so both give the same bits.
__global__ void __launch_bounds__(256) ep_combine_kernel(EpCombineParams p) {
  const int vec_per_row = p.hidden >> 3;
  const int64_t total = static_cast<int64_t>(p.n_tokens) * vec_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int token = static_cast<int>(static_cast<uint32_t>(i) / static_cast<uint32_t>(vec_per_row));  // total < 2^31: checked at launch
    const int v = static_cast<int>(static_cast<uint32_t>(i) - static_cast<uint32_t>(token) * static_cast<uint32_t>(vec_per_row));
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
  if (total >= (int64_t{1} << 31)) return AKLR_ERR_TOO_LARGE;
  const int64_t blocks = (total + 255) / 256;
  const int grid = static_cast<int>(blocks < 148 * 8 ? blocks : 148 * 8);
  ep_combine_kernel<<<grid, 256, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

}  // namespace aklr
