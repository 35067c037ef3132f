// Per-token-group FP8 activation quantisation, sm_100a.  All three kernels are HBM-bound
// element-wise passes: 16-byte loads (8 bf16 per lane), shuffle reductions inside the lanes of
// one group, 8-byte stores.
//
//  * gather_quant_fp8: the MoE layer's scheme -- scale = max(amax/448, FLT_MIN), code =
//    e4m3(x / scale), both true divisions, as the reference's _fp8_input does
//    (aklr/plugins/sglang/models/qwen3_moe/reference.py:44-54); rows are gathered through the
//    sorted route table so the grouped GEMM reads expert-contiguous rows.
//  * per_group_quant_fp8: the standalone op -- scale = max(amax,1e-10)*(1/448), code =
//    e4m3(clamp(x * (1/scale))), scales stored group-major (aklr/ops/quant/reference.py:9-28).
//  * per_group_quant_mxfp8: 1 x 32 groups, power-of-two scale rounded up, e8m0 exponent bytes
//    (aklr/ops/quant/reference.py:31-48).
#include <cfloat>

#include "common.cuh"
#include "kernels.h"
#include "quant_rows.cuh"

namespace aklr {

__global__ void __launch_bounds__(256) gather_quant_fp8_kernel(GatherQuantParams p) {
  griddep_wait();
  griddep_launch();
  gather_quant_fp8_groups(p, (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4,
                          (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 4);
}

// Rows already quantised elsewhere (each token once, or by the sender of an expert-parallel
// dispatch): copy row rid's codes and scales into the expert-sorted table.  One warp per destination row, no
// block-wide barrier: a lane issues all of its 16-byte loads of the row (hidden / 512 of them, 14 at 7168) before
// its first store, so a warp keeps a whole row in flight.
constexpr int kGatherMaxVecPerLane = 16;  // hidden <= 8192 in one pass; wider rows take further passes

__global__ void __launch_bounds__(256) gather_rows_fp8_kernel(GatherQuantParams p) {
  griddep_wait();
  griddep_launch();
  const int lane = threadIdx.x & 31;
  const int vec_per_row = p.hidden >> 4;
  const int groups_per_row = p.hidden >> 7;
  const size_t q_pitch = p.q_in_stride ? p.q_in_stride : p.hidden;
  const size_t s_pitch = p.scales_in_stride ? p.scales_in_stride : groups_per_row * sizeof(float);
  const int n_rows = p.num_rows ? min(*p.num_rows, p.n_rows) : p.n_rows;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < n_rows; row += warps) {
    const int rid = p.sorted_ids[row];  // the same address for the whole warp: one broadcast load
    if (rid < 0) {
      // Padding rows are never read back, but the tensor core multiplies them all the same, and what it draws
      // depends on the operands: with zero rows in place of stale codes the part holds a higher clock under the
      // token-major GEMM (an N = 256 MMA stream alone: 1600 MHz on random operands, 1740 with half the rows zero).
      if (p.zero_padding)
        for (int v = lane; v < vec_per_row; v += 32)
          reinterpret_cast<uint4*>(p.q + static_cast<size_t>(row) * p.hidden)[v] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const int src = rid / p.routes_per_token;
    const uint4* from = reinterpret_cast<const uint4*>(p.q_in + static_cast<size_t>(src) * q_pitch);
    uint4* to = reinterpret_cast<uint4*>(p.q + static_cast<size_t>(row) * p.hidden);
    for (int v0 = 0; v0 < vec_per_row; v0 += 32 * kGatherMaxVecPerLane) {
      uint4 val[kGatherMaxVecPerLane];
#pragma unroll
      for (int u = 0; u < kGatherMaxVecPerLane; ++u) {
        const int v = v0 + u * 32 + lane;
        if (v < vec_per_row) val[u] = __ldg(from + v);
      }
#pragma unroll
      for (int u = 0; u < kGatherMaxVecPerLane; ++u) {
        const int v = v0 + u * 32 + lane;
        if (v < vec_per_row) to[v] = val[u];
      }
    }
    const float* scales_from = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(p.scales_in) + static_cast<size_t>(src) * s_pitch);
    float* scales_to = p.scales + static_cast<size_t>(row / p.block_m) * groups_per_row * p.block_m + row % p.block_m;
    for (int grp = lane; grp < groups_per_row; grp += 32) scales_to[static_cast<size_t>(grp) * p.block_m] = __ldg(scales_from + grp);
  }
}

int launch_gather_rows_fp8(const GatherQuantParams& p, cudaStream_t stream) {
  if (p.hidden % 128 != 0 || p.block_m < 1) return AKLR_ERR_UNSUPPORTED_SHAPE;
  if (p.n_rows == 0) return AKLR_OK;
  const int64_t blocks = (static_cast<int64_t>(p.n_rows) + 7) / 8;  // eight warps = eight rows per CTA and pass
  const int grid = static_cast<int>(blocks < 148 * 16 ? blocks : 148 * 16);
  return launch_kernel(gather_rows_fp8_kernel, dim3(grid), dim3(256), 0, stream, 1, p) == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

int launch_gather_quant_fp8(const GatherQuantParams& p, cudaStream_t stream) {
  if (p.hidden % 128 != 0) return AKLR_ERR_UNSUPPORTED_SHAPE;
  if (p.n_rows == 0) return AKLR_OK;
  const int64_t groups = static_cast<int64_t>(p.n_rows) * (p.hidden / 128);
  if (groups >= (int64_t{1} << 31)) return AKLR_ERR_TOO_LARGE;
  const int64_t blocks = (groups * 16 + 255) / 256;
  const int grid = static_cast<int>(blocks < 148 * 16 ? blocks : 148 * 16);
  return launch_kernel(gather_quant_fp8_kernel, dim3(grid), dim3(256), 0, stream, 1, p) == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

__global__ void __launch_bounds__(256)
per_group_quant_fp8_kernel(const uint16_t* __restrict__ x, uint8_t* __restrict__ q,
                           float* __restrict__ scales, int rows, int hidden) {
  const int groups_per_row = hidden >> 7;
  const int64_t total = static_cast<int64_t>(rows) * groups_per_row;
  const int sub = threadIdx.x & 15;
  const uint32_t group_mask = 0xFFFFu << (threadIdx.x & 16);  // the lanes of this half-warp
  const int64_t half_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 4;
  // kOpGroupsInFlight groups per half-warp and pass (more than one measured slower: occupancy hides the latency already)
  for (int64_t g0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4; g0 < total;
       g0 += half_warps * kOpGroupsInFlight) {
    uint4 raw[kOpGroupsInFlight];
#pragma unroll
    for (int u = 0; u < kOpGroupsInFlight; ++u) {
      const int64_t g = g0 + u * half_warps;
      if (g < total) raw[u] = *reinterpret_cast<const uint4*>(x + g * 128 + sub * 8);  // groups of a row follow one another
    }
#pragma unroll
    for (int u = 0; u < kOpGroupsInFlight; ++u) {
      const int64_t g = g0 + u * half_warps;
      if (g >= total) continue;
      float v[8];
      unpack8(raw[u], v);
      float m = amax8(v);
#pragma unroll
      for (int off = 8; off >= 1; off >>= 1) m = fmaxf(m, __shfl_xor_sync(group_mask, m, off, 16));
      const float scale = __fmul_rn(fmaxf(m, 1e-10f), 1.0f / 448.0f);
      const float recip = __fdiv_rn(1.0f, scale);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = fminf(fmaxf(__fmul_rn(v[i], recip), -448.0f), 448.0f);
      *reinterpret_cast<uint2*>(q + g * 128 + sub * 8) = pack8_e4m3(v);
      if (sub == 0) {
        const uint32_t row = static_cast<uint32_t>(g) / static_cast<uint32_t>(groups_per_row);  // g < 2^31: checked at launch
        const uint32_t grp = static_cast<uint32_t>(g) - row * static_cast<uint32_t>(groups_per_row);
        scales[static_cast<size_t>(grp) * rows + row] = scale;
      }
    }
  }
}

int launch_per_group_quant_fp8(const void* x, uint8_t* q, float* scales, int rows, int hidden,
                               cudaStream_t stream) {
  if (hidden % 128 != 0) return AKLR_ERR_UNSUPPORTED_SHAPE;
  if (rows == 0) return AKLR_OK;
  const int64_t groups = static_cast<int64_t>(rows) * (hidden / 128);
  if (groups >= (int64_t{1} << 31)) return AKLR_ERR_TOO_LARGE;
  const int64_t blocks = (groups * 16 + 255) / 256;
  const int grid = static_cast<int>(blocks < 148 * 16 ? blocks : 148 * 16);
  per_group_quant_fp8_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(x), q, scales, rows, hidden);
  return cudaGetLastError() == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

// Four lanes x 8 values per 1 x 32 group.  The scale is a power of two, so dividing by it is multiplying by the
// power of two that is its reciprocal: the same real number rounded the same way, without a division.
__global__ void __launch_bounds__(256)
per_group_quant_mxfp8_kernel(const uint16_t* __restrict__ x, uint8_t* __restrict__ q,
                             uint8_t* __restrict__ scales, int64_t elements) {
  const int64_t slots = elements >> 3;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const uint32_t group_mask = 0xFu << (threadIdx.x & 28);  // the four lanes of this group
  // the four lanes of a group run the same number of iterations: slots and the stride are multiples of 4
  for (int64_t slot0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; slot0 < slots; slot0 += stride * kOpGroupsInFlight) {
    uint4 raw[kOpGroupsInFlight];
#pragma unroll
    for (int u = 0; u < kOpGroupsInFlight; ++u)
      if (slot0 + u * stride < slots) raw[u] = *reinterpret_cast<const uint4*>(x + (slot0 + u * stride) * 8);
#pragma unroll
    for (int u = 0; u < kOpGroupsInFlight; ++u) {
      const int64_t slot = slot0 + u * stride;
      if (slot >= slots) continue;
      float v[8];
      unpack8(raw[u], v);
      float m = amax8(v);
      m = fmaxf(m, __shfl_xor_sync(group_mask, m, 2, 4));
      m = fmaxf(m, __shfl_xor_sync(group_mask, m, 1, 4));
      const uint32_t bits = __float_as_uint(__fmul_rn(fmaxf(m, 1e-10f), 1.0f / 448.0f));
      const uint32_t exponent = (bits >> 23) + ((bits & 0x7FFFFFu) != 0u ? 1u : 0u);  // 2^(exponent-127), 94 .. 255 here
      // 2^(127-exponent): a normal number down to exponent 253, below that two exact factors
      const float r1 = __uint_as_float((exponent <= 253u ? 254u - exponent : 1u) << 23);
      const float r2 = exponent <= 253u ? 1.0f : __uint_as_float((255u - exponent) << 23);  // 2^-1 or 2^-2 past 2^-126
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = fminf(fmaxf(__fmul_rn(__fmul_rn(v[i], r1), r2), -448.0f), 448.0f);
      *reinterpret_cast<uint2*>(q + slot * 8) = pack8_e4m3(v);
      if ((slot & 3) == 0) scales[slot >> 2] = static_cast<uint8_t>(exponent);
    }
  }
}

int launch_per_group_quant_mxfp8(const void* x, uint8_t* q, uint8_t* scales, int rows, int hidden,
                                 cudaStream_t stream) {
  if (hidden % 32 != 0) return AKLR_ERR_UNSUPPORTED_SHAPE;
  if (rows == 0) return AKLR_OK;
  const int64_t elements = static_cast<int64_t>(rows) * hidden;
  const int64_t blocks = (elements / 8 + 255) / 256;
  const int grid = static_cast<int>(blocks < 148 * 16 ? blocks : 148 * 16);
  per_group_quant_mxfp8_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(x), q, scales, elements);
  return cudaGetLastError() == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

// Self-test of ExactDivider against the division it replaces: counts the pairs where they differ.
__global__ void __launch_bounds__(256)
exact_divide_selftest_kernel(const float* __restrict__ x, const float* __restrict__ scale, int64_t n, int32_t* mismatches) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int bad = 0;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const ExactDivider divide(scale[i]);
    bad += __float_as_uint(divide(x[i])) != __float_as_uint(__fdiv_rn(x[i], scale[i]));
  }
  if (bad) atomicAdd(mismatches, bad);
}

int launch_exact_divide_selftest(const float* x, const float* scale, int64_t n, int32_t* mismatches, cudaStream_t stream) {
  if (n <= 0) return AKLR_OK;
  const int64_t blocks = (n + 255) / 256;
  exact_divide_selftest_kernel<<<static_cast<int>(blocks < 148 * 8 ? blocks : 148 * 8), 256, 0, stream>>>(x, scale, n, mismatches);
  return cudaGetLastError() == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

}  // namespace aklr
