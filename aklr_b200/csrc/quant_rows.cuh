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

// x / scale rounded to nearest, as the reference's true division gives it, without eight IEEE divisions per
// lane: with y = RN(1/scale), q = RN(x*y), r = x - q*scale (exact in one fma) the quotient RN(q + r*y) is the
// correctly rounded x/scale whenever nothing under- or overflows on the way and scale's significand is not all
// ones (Markstein's theorem).  |x/scale| <= 448 here; the groups where the shortcut is not proven -- an all-ones
// significand, or a scale so small that its reciprocal or the residual leaves the normal range -- take the
// division itself (uniform over a group's lanes, rare).
struct ExactDivider {
  float scale, recip;
  bool slow;
  __device__ __forceinline__ explicit ExactDivider(float s) {
    scale = s;
    recip = __fdiv_rn(1.0f, s);  // correctly rounded
    const uint32_t bits = __float_as_uint(s);
    slow = (bits & 0x7FFFFFu) == 0x7FFFFFu || s < 1.0e-30f || s > 1.0e30f;
  }
  __device__ __forceinline__ float operator()(float x) const {
    if (slow) return __fdiv_rn(x, scale);
    const float q = __fmul_rn(x, recip);
    return __fmaf_rn(__fmaf_rn(-q, scale, x), recip, q);
  }
};

// One half-warp (16 lanes x 8 values) per 1 x 128 group: this half-warp takes groups ``first``,
// ``first + stride``, ... of the row table (the caller's grid-stride, or one CTA's share), kGroupsInFlight of
// them at a time.
constexpr int kGroupsInFlight = 1;  // measured on the layer's quantiser: 1 -> 0.121 ms, 2 -> 0.125, 4 -> 0.133 (T = 4096)
constexpr int kOpGroupsInFlight = 1;  // the standalone quantisers: 1 -> 75.8 us, 2 and 4 -> 81.9 us (16384 x 7168)

__device__ __forceinline__ void gather_quant_fp8_groups(const GatherQuantParams& p, int64_t first, int64_t stride) {
  const int groups_per_row = p.hidden >> 7;
  const int n_rows = p.num_rows ? min(*p.num_rows, p.n_rows) : p.n_rows;
  const int64_t total = static_cast<int64_t>(n_rows) * groups_per_row;
  const int sub = threadIdx.x & 15;
  const uint32_t group_mask = 0xFFFFu << (threadIdx.x & 16);  // the lanes of this half-warp
  for (int64_t g0 = first; g0 < total; g0 += stride * kGroupsInFlight) {
    uint4 raw[kGroupsInFlight];
    int row[kGroupsInFlight], grp[kGroupsInFlight];
    bool live[kGroupsInFlight];
#pragma unroll
    for (int u = 0; u < kGroupsInFlight; ++u) {
      const int64_t g = g0 + u * stride;
      live[u] = g < total;
      row[u] = grp[u] = 0;
      if (live[u]) {
        // 32-bit division: a 64-bit one is a subroutine of a hundred instructions, per group and lane
        row[u] = static_cast<int>(static_cast<uint32_t>(g) / static_cast<uint32_t>(groups_per_row));
        grp[u] = static_cast<int>(static_cast<uint32_t>(g) - static_cast<uint32_t>(row[u]) * static_cast<uint32_t>(groups_per_row));
        int token = row[u];
        if (p.sorted_ids) {
          const int rid = p.sorted_ids[row[u]];
          token = rid < 0 ? -1 : rid / p.routes_per_token;
        }
        live[u] = token >= 0;  // padding rows are never read back
        if (!live[u] && p.zero_padding)  // but multiplied: zero codes cost the tensor core least
          *reinterpret_cast<uint2*>(p.q + static_cast<size_t>(row[u]) * p.hidden + grp[u] * 128 + sub * 8) = make_uint2(0u, 0u);
        if (live[u])
          raw[u] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.x) +
                                                   static_cast<size_t>(token) * p.hidden + grp[u] * 128 + sub * 8);
      }
    }
#pragma unroll
    for (int u = 0; u < kGroupsInFlight; ++u) {
      if (!live[u]) continue;  // uniform over the half-warp: all of its lanes work on the same group
      float v[8];
      unpack8(raw[u], v);
      float m = amax8(v);
#pragma unroll
      for (int off = 8; off >= 1; off >>= 1) m = fmaxf(m, __shfl_xor_sync(group_mask, m, off, 16));
      const float scale = fmaxf(__fdiv_rn(m, 448.0f), FLT_MIN);
      const ExactDivider divide(scale);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = divide(v[i]);
      *reinterpret_cast<uint2*>(p.q + static_cast<size_t>(row[u]) * p.hidden + grp[u] * 128 + sub * 8) = pack8_e4m3(v);
      if (sub == 0) {
        if (p.block_m > 0)  // [block][group][row in block]: what the grouped GEMM stages per tile
          p.scales[(static_cast<size_t>(row[u] / p.block_m) * groups_per_row + grp[u]) * p.block_m + row[u] % p.block_m] = scale;
        else
          p.scales[static_cast<size_t>(row[u]) * groups_per_row + grp[u]] = scale;
      }
    }
  }
}

}  // namespace aklr
