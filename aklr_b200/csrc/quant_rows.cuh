// The FP8 activation quantisation of one 1 x 128 group, shared by the stand-alone kernels and the
// fused decode prologue: scale = max(amax/448, FLT_MIN), code = e4m3(x / scale), both true
// divisions, as the reference's _fp8_input does
// (aklr/plugins/sglang/models/qwen3_moe/reference.py:44-54).
#pragma once
#include <cfloat>

#include "common.cuh"
#include "kernels.h"

namespace aklr {

__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

__device__ __forceinline__ float amax8(const float (&v)[8]) {
  float m = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
  return m;
}

__device__ __forceinline__ uint2 pack8_e4m3(const float (&v)[8]) {
  uint2 out;
  out.x = cvt_e4m3x2(v[0], v[1]) | (static_cast<uint32_t>(cvt_e4m3x2(v[2], v[3])) << 16);
  out.y = cvt_e4m3x2(v[4], v[5]) | (static_cast<uint32_t>(cvt_e4m3x2(v[6], v[7])) << 16);
  return out;
}

// One half-warp (16 lanes x 8 values) per 1 x 128 group: this half-warp takes groups ``first``,
// ``first + stride``, ... of the row table (the caller's grid-stride, or one CTA's share).
__device__ __forceinline__ void gather_quant_fp8_groups(const GatherQuantParams& p, int64_t first, int64_t stride) {
  const int groups_per_row = p.hidden >> 7;
  const int n_rows = p.num_rows ? min(*p.num_rows, p.n_rows) : p.n_rows;
  const int64_t total = static_cast<int64_t>(n_rows) * groups_per_row;
  const int sub = threadIdx.x & 15;
  const uint32_t group_mask = 0xFFFFu << (threadIdx.x & 16);  // the lanes of this half-warp
  for (int64_t g = first; g < total; g += stride) {
    const int row = static_cast<int>(g / groups_per_row);
    const int grp = static_cast<int>(g - static_cast<int64_t>(row) * groups_per_row);
    int token = row;
    if (p.sorted_ids) {
      const int rid = p.sorted_ids[row];
      token = rid < 0 ? -1 : rid / p.routes_per_token;
    }
    if (token < 0) continue;  // padding rows are never read back
    const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.x) +
                                                      static_cast<size_t>(token) * p.hidden + grp * 128 + sub * 8);
    float v[8];
    unpack8(raw, v);
    float m = amax8(v);
#pragma unroll
    for (int off = 8; off >= 1; off >>= 1) m = fmaxf(m, __shfl_xor_sync(group_mask, m, off, 16));
    const float scale = fmaxf(__fdiv_rn(m, 448.0f), FLT_MIN);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __fdiv_rn(v[i], scale);
    *reinterpret_cast<uint2*>(p.q + static_cast<size_t>(row) * p.hidden + grp * 128 + sub * 8) = pack8_e4m3(v);
    if (sub == 0) {
      if (p.block_m > 0)  // [block][group][row in block]: what the grouped GEMM stages per tile
        p.scales[(static_cast<size_t>(row / p.block_m) * groups_per_row + grp) * p.block_m + row % p.block_m] = scale;
      else
        p.scales[static_cast<size_t>(row) * groups_per_row + grp] = scale;
    }
  }
}

}  // namespace aklr
