// Top-k weighted combine (unpermute) and the router projection, sm_100a.
//
// combine: out[t] = bf16( sum over the token's routes of its per-route row ), summed in float32
// in slot order; the rows already carry the route weight (the down projection applies it).
// Routes to experts this rank does not hold add nothing, as in the reference's expert_mask /
// expert_offset statements (aklr/ops/fused_moe/reference.py:78-84).  HBM-bound: 16-byte loads.
//
// router: logits = bf16( x @ W^T ) with float32 accumulation, the rounding point of the
// reference's _router_logits (aklr/plugins/sglang/models/qwen3_moe/reference.py:24-31).
#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace aklr {

__global__ void __launch_bounds__(256) combine_kernel(CombineParams p) {
  griddep_wait();
  griddep_launch();
  const int vec_per_row = p.hidden >> 3;  // 8 bf16 per 16-byte vector
  const int64_t total = static_cast<int64_t>(p.n_tokens) * vec_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    // 32-bit division (the total is far below 2^31): the 64-bit one is a subroutine
    const int token = static_cast<int>(static_cast<uint32_t>(i) / static_cast<uint32_t>(vec_per_row));
    const int v = static_cast<int>(static_cast<uint32_t>(i) - static_cast<uint32_t>(token) * static_cast<uint32_t>(vec_per_row));
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const bool received = !p.num_local_tokens || token < __ldg(p.num_local_tokens);
    // Slots are summed in order, but their loads do not wait for one another: ids of a batch of
    // slots first, then all of its rows, then the additions (a decode call is one latency chain).
    constexpr int kBatchSlots = 9;
    for (int s0 = 0; s0 < p.routes_per_token; s0 += kBatchSlots) {
      bool live[kBatchSlots];
      uint4 raw[kBatchSlots];
#pragma unroll
      for (int d = 0; d < kBatchSlots; ++d) {
        const int s = s0 + d;
        live[d] = false;
        if (s < p.routes_per_token) {
          const int e = __ldg(p.topk_ids + token * p.routes_per_token + s);
          live[d] = received && e >= 0 && e < p.n_experts_global && (!p.expert_map || __ldg(p.expert_map + e) >= 0);
        }
      }
#pragma unroll
      for (int d = 0; d < kBatchSlots; ++d)
        if (live[d])
          raw[d] = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.rows) +
                                                   static_cast<size_t>(token * p.routes_per_token + s0 + d) * p.hidden + v * 8);
#pragma unroll
      for (int d = 0; d < kBatchSlots; ++d) {
        if (!live[d]) continue;
        const uint32_t w[4] = {raw[d].x, raw[d].y, raw[d].z, raw[d].w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          acc[2 * q] += __uint_as_float(w[q] << 16);
          acc[2 * q + 1] += __uint_as_float(w[q] & 0xFFFF0000u);
        }
      }
    }
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

int launch_combine(const CombineParams& p, cudaStream_t stream) {
  if (p.hidden % 8 != 0) return AKLR_ERR_UNSUPPORTED_SHAPE;
  if (p.n_tokens == 0) return AKLR_OK;
  const int64_t total = static_cast<int64_t>(p.n_tokens) * (p.hidden / 8);
  if (total >= (int64_t{1} << 31)) return AKLR_ERR_TOO_LARGE;
  const int64_t blocks = (total + 255) / 256;
  const int grid = static_cast<int>(blocks < 148 * 8 ? blocks : 148 * 8);
  return launch_kernel(combine_kernel, dim3(grid), dim3(256), 0, stream, 1, p) == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

// One warp per (token, kRouterExperts experts): lanes stride the hidden dimension with 16-byte loads.
template <int kRouterExperts>
__global__ void __launch_bounds__(256)
router_gemm_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w, uint16_t* __restrict__ logits,
                   int n_tokens, int hidden, int n_routed) {
  const int lane = threadIdx.x & 31;
  const int groups = (n_routed + kRouterExperts - 1) / kRouterExperts;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= static_cast<int64_t>(n_tokens) * groups) return;
  const int token = static_cast<int>(item / groups);
  const int e0 = static_cast<int>(item - static_cast<int64_t>(token) * groups) * kRouterExperts;
  float acc[kRouterExperts];
#pragma unroll
  for (int j = 0; j < kRouterExperts; ++j) acc[j] = 0.0f;
  for (int h = lane * 8; h < hidden; h += 256) {
    const uint4 xr = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(token) * hidden + h);
    const uint32_t xw[4] = {xr.x, xr.y, xr.z, xr.w};
#pragma unroll
    for (int j = 0; j < kRouterExperts; ++j) {
      if (e0 + j < n_routed) {
        const uint4 wr = *reinterpret_cast<const uint4*>(w + static_cast<size_t>(e0 + j) * hidden + h);
        const uint32_t ww[4] = {wr.x, wr.y, wr.z, wr.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          acc[j] = fmaf(__uint_as_float(xw[q] << 16), __uint_as_float(ww[q] << 16), acc[j]);
          acc[j] = fmaf(__uint_as_float(xw[q] & 0xFFFF0000u), __uint_as_float(ww[q] & 0xFFFF0000u), acc[j]);
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < kRouterExperts; ++j) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) acc[j] += __shfl_xor_sync(0xFFFFFFFFu, acc[j], off);
  }
  if (lane < kRouterExperts && e0 + lane < n_routed) {
    float v = acc[0];
#pragma unroll
    for (int j = 1; j < kRouterExperts; ++j)
      if (lane == j) v = acc[j];
    const __nv_bfloat16 r = __float2bfloat16_rn(v);
    logits[static_cast<size_t>(token) * n_routed + e0 + lane] = *reinterpret_cast<const uint16_t*>(&r);
  }
}

// Qwen2-MoE's gated shared expert (aklr/plugins/sglang/models/qwen2_moe/reference.py:84-90): the
// routing table gets one more slot per token, expert ``shared_slot`` at weight
// sigmoid(x . shared_gate).  ``ids_in`` / ``weights_in`` [T, K] given: copied into the first K
// slots of the [T, K+1] tables; null: those slots are already in place.  One warp per token.
__global__ void __launch_bounds__(256)
shared_gate_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ gate, const int32_t* __restrict__ ids_in,
                   const float* __restrict__ weights_in, int32_t* __restrict__ ids, float* __restrict__ weights,
                   int n_tokens, int hidden, int topk, int shared_slot) {
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (token >= n_tokens) return;
  float acc = 0.0f;
  for (int h = lane * 8; h < hidden; h += 256) {
    const uint4 xr = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(token) * hidden + h);
    const uint4 gr = *reinterpret_cast<const uint4*>(gate + h);
    const uint32_t xw[4] = {xr.x, xr.y, xr.z, xr.w}, gw[4] = {gr.x, gr.y, gr.z, gr.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      acc = fmaf(__uint_as_float(xw[q] << 16), __uint_as_float(gw[q] << 16), acc);
      acc = fmaf(__uint_as_float(xw[q] & 0xFFFF0000u), __uint_as_float(gw[q] & 0xFFFF0000u), acc);
    }
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, off);
  const size_t row = static_cast<size_t>(token) * (topk + 1);
  if (ids_in && lane < topk) {
    ids[row + lane] = ids_in[static_cast<size_t>(token) * topk + lane];
    weights[row + lane] = weights_in[static_cast<size_t>(token) * topk + lane];
  }
  if (lane == 0) {
    ids[row + topk] = shared_slot;
    weights[row + topk] = __fdiv_rn(1.0f, 1.0f + expf(-acc));
  }
}

int launch_shared_gate(const void* x, const void* gate, const int32_t* ids_in, const float* weights_in, int32_t* ids,
                       float* weights, int n_tokens, int hidden, int topk, int shared_slot, cudaStream_t stream) {
  if (hidden % 8 != 0 || topk < 1 || topk > 31) return AKLR_ERR_UNSUPPORTED_SHAPE;
  if (n_tokens == 0) return AKLR_OK;
  shared_gate_kernel<<<(n_tokens + 7) / 8, 256, 0, stream>>>(static_cast<const uint16_t*>(x), static_cast<const uint16_t*>(gate),
                                                          ids_in, weights_in, ids, weights, n_tokens, hidden, topk, shared_slot);
  return cudaGetLastError() == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

// A shared expert kept apart from the routed ones in bf16 (qwen2_moe_mxfp4_moe,
// aklr/plugins/sglang/models/qwen2_moe/reference.py:160-185): its two projections are dense bf16
// GEMMs the caller runs; these are the two steps around them.
//  * silu_mul: h[t, i] = bf16( silu(gate_up[t, i]) * gate_up[t, I + i] ), 8 values per thread;
//  * add_gated_rows: out[t] = bf16( out[t] + sigmoid(x[t] . gate) * rows[t] ), one warp per token.
__global__ void __launch_bounds__(256)
silu_mul_bf16_kernel(const uint16_t* __restrict__ gate_up, uint16_t* __restrict__ out, int64_t n_vectors, int vec_per_row) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vectors; i += stride) {
    const int64_t row = static_cast<uint32_t>(i) / static_cast<uint32_t>(vec_per_row);  // n_vectors < 2^31: checked at launch
    const int64_t v = i - row * vec_per_row;
    const uint4 g = *reinterpret_cast<const uint4*>(gate_up + (row * 2 * vec_per_row + v) * 8);
    const uint4 u = *reinterpret_cast<const uint4*>(gate_up + (row * 2 * vec_per_row + vec_per_row + v) * 8);
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t r[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float g0 = __uint_as_float(gw[q] << 16), g1 = __uint_as_float(gw[q] & 0xFFFF0000u);
      const float u0 = __uint_as_float(uw[q] << 16), u1 = __uint_as_float(uw[q] & 0xFFFF0000u);
      const __nv_bfloat162 pair = __floats2bfloat162_rn(__fdiv_rn(g0, 1.0f + expf(-g0)) * u0, __fdiv_rn(g1, 1.0f + expf(-g1)) * u1);
      r[q] = *reinterpret_cast<const uint32_t*>(&pair);
    }
    *reinterpret_cast<uint4*>(out + i * 8) = make_uint4(r[0], r[1], r[2], r[3]);
  }
}

__global__ void __launch_bounds__(256)
add_gated_rows_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ gate, const uint16_t* __restrict__ rows,
                      uint16_t* __restrict__ out, int n_tokens, int hidden) {
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (token >= n_tokens) return;
  const size_t base = static_cast<size_t>(token) * hidden;
  float acc = 0.0f;
  for (int h = lane * 8; h < hidden; h += 256) {
    const uint4 xr = *reinterpret_cast<const uint4*>(x + base + h);
    const uint4 gr = *reinterpret_cast<const uint4*>(gate + h);
    const uint32_t xw[4] = {xr.x, xr.y, xr.z, xr.w}, gw[4] = {gr.x, gr.y, gr.z, gr.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      acc = fmaf(__uint_as_float(xw[q] << 16), __uint_as_float(gw[q] << 16), acc);
      acc = fmaf(__uint_as_float(xw[q] & 0xFFFF0000u), __uint_as_float(gw[q] & 0xFFFF0000u), acc);
    }
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, off);
  const float weight = __fdiv_rn(1.0f, 1.0f + expf(-acc));
  for (int h = lane * 8; h < hidden; h += 256) {
    const uint4 rr = *reinterpret_cast<const uint4*>(rows + base + h);
    const uint4 orr = *reinterpret_cast<const uint4*>(out + base + h);
    const uint32_t rw[4] = {rr.x, rr.y, rr.z, rr.w}, ow[4] = {orr.x, orr.y, orr.z, orr.w};
    uint32_t res[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float lo = fmaf(weight, __uint_as_float(rw[q] << 16), __uint_as_float(ow[q] << 16));
      const float hi = fmaf(weight, __uint_as_float(rw[q] & 0xFFFF0000u), __uint_as_float(ow[q] & 0xFFFF0000u));
      const __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
      res[q] = *reinterpret_cast<const uint32_t*>(&pair);
    }
    *reinterpret_cast<uint4*>(out + base + h) = make_uint4(res[0], res[1], res[2], res[3]);
  }
}

int launch_silu_mul_bf16(const void* gate_up, void* out, int n_tokens, int inter, cudaStream_t stream) {
  if (inter % 8 != 0 || inter < 8) return AKLR_ERR_UNSUPPORTED_SHAPE;
  if (n_tokens == 0) return AKLR_OK;
  const int vec_per_row = inter / 8;
  const int64_t n_vectors = static_cast<int64_t>(n_tokens) * vec_per_row;
  if (n_vectors >= (int64_t{1} << 31)) return AKLR_ERR_TOO_LARGE;
  const int grid = static_cast<int>(std::min<int64_t>((n_vectors + 255) / 256, 148 * 8));
  silu_mul_bf16_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(gate_up), static_cast<uint16_t*>(out), n_vectors, vec_per_row);
  return cudaGetLastError() == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

int launch_add_gated_rows(const void* x, const void* gate, const void* rows, void* out, int n_tokens, int hidden,
                          cudaStream_t stream) {
  if (hidden % 8 != 0) return AKLR_ERR_UNSUPPORTED_SHAPE;
  if (n_tokens == 0) return AKLR_OK;
  add_gated_rows_kernel<<<(n_tokens + 7) / 8, 256, 0, stream>>>(static_cast<const uint16_t*>(x), static_cast<const uint16_t*>(gate),
                                                             static_cast<const uint16_t*>(rows), static_cast<uint16_t*>(out), n_tokens, hidden);
  return cudaGetLastError() == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

// Router with float32 weights and float32 logits (MiniMax-M2's gate:
// aklr/plugins/sglang/models/minimax_m2/reference.py:43-50 takes x @ router^T in float32, nothing
// rounded).  CUDA cores, float32 FMAs in k order.
//  * few tokens: one warp per (token, expert) dot product, so the weight is read by many SMs;
//  * else a 64 x 64 tile per CTA, 16 k per step through shared memory, 4 x 4 outputs per thread.
__global__ void __launch_bounds__(256)
router_dot_f32_kernel(const uint16_t* __restrict__ x, const float* __restrict__ w, float* __restrict__ logits,
                      int n_tokens, int hidden, int n_routed) {
  const int lane = threadIdx.x & 31;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= static_cast<int64_t>(n_tokens) * n_routed) return;
  const int token = static_cast<int>(item / n_routed), e = static_cast<int>(item - static_cast<int64_t>(token) * n_routed);
  float acc = 0.0f;
  for (int h = lane * 4; h < hidden; h += 128) {
    const uint2 xr = *reinterpret_cast<const uint2*>(x + static_cast<size_t>(token) * hidden + h);
    const float4 wr = *reinterpret_cast<const float4*>(w + static_cast<size_t>(e) * hidden + h);
    acc = fmaf(__uint_as_float(xr.x << 16), wr.x, acc);
    acc = fmaf(__uint_as_float(xr.x & 0xFFFF0000u), wr.y, acc);
    acc = fmaf(__uint_as_float(xr.y << 16), wr.z, acc);
    acc = fmaf(__uint_as_float(xr.y & 0xFFFF0000u), wr.w, acc);
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, off);
  if (lane == 0) logits[static_cast<size_t>(token) * n_routed + e] = acc;
}

__global__ void __launch_bounds__(256)
router_tile_f32_kernel(const uint16_t* __restrict__ x, const float* __restrict__ w, float* __restrict__ logits,
                       int n_tokens, int hidden, int n_routed) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int token0 = blockIdx.x * BM, e0 = blockIdx.y * BN;
  const int lrow = tid >> 2, lk = (tid & 3) * 4;  // this thread stages 4 k of one row of each tile
  float acc[4][4] = {};
  for (int k0 = 0; k0 < hidden; k0 += BK) {
    uint2 xr = make_uint2(0u, 0u);
    float4 wr = make_float4(0.f, 0.f, 0.f, 0.f);
    if (token0 + lrow < n_tokens) xr = *reinterpret_cast<const uint2*>(x + static_cast<size_t>(token0 + lrow) * hidden + k0 + lk);
    if (e0 + lrow < n_routed) wr = *reinterpret_cast<const float4*>(w + static_cast<size_t>(e0 + lrow) * hidden + k0 + lk);
    __syncthreads();  // the previous step is done with the tiles
    xs[lk + 0][lrow] = __uint_as_float(xr.x << 16);
    xs[lk + 1][lrow] = __uint_as_float(xr.x & 0xFFFF0000u);
    xs[lk + 2][lrow] = __uint_as_float(xr.y << 16);
    xs[lk + 3][lrow] = __uint_as_float(xr.y & 0xFFFF0000u);
    ws[lk + 0][lrow] = wr.x;
    ws[lk + 1][lrow] = wr.y;
    ws[lk + 2][lrow] = wr.z;
    ws[lk + 3][lrow] = wr.w;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 a = *reinterpret_cast<const float4*>(&xs[k][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&ws[k][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int token = token0 + ty * 4 + i;
    if (token >= n_tokens) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int e = e0 + tx * 4 + j;
      if (e < n_routed) logits[static_cast<size_t>(token) * n_routed + e] = acc[i][j];
    }
  }
}

int launch_router_gemm_f32(const void* x, const float* w, float* logits, int n_tokens, int hidden, int n_routed,
                           cudaStream_t stream) {
  if (hidden % 128 != 0) return AKLR_ERR_UNSUPPORTED_SHAPE;
  if (n_tokens == 0 || n_routed == 0) return AKLR_OK;
  auto* xp = static_cast<const uint16_t*>(x);
  if (n_tokens <= 16) {
    const int64_t blocks = (static_cast<int64_t>(n_tokens) * n_routed + 7) / 8;
    router_dot_f32_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(xp, w, logits, n_tokens, hidden, n_routed);
  } else {
    const dim3 grid((n_tokens + 63) / 64, (n_routed + 63) / 64);
    router_tile_f32_kernel<<<grid, 256, 0, stream>>>(xp, w, logits, n_tokens, hidden, n_routed);
  }
  return cudaGetLastError() == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

int launch_router_gemm(const void* x, const void* w, void* logits, int n_tokens, int hidden, int n_routed,
                       cudaStream_t stream) {
  if (hidden % 8 != 0) return AKLR_ERR_UNSUPPORTED_SHAPE;
  if (n_tokens == 0) return AKLR_OK;
  // few tokens: one expert per warp so the router weight is streamed by many SMs
  const int per_warp = n_tokens <= 16 ? 1 : 8;
  const int groups = (n_routed + per_warp - 1) / per_warp;
  const int64_t items = static_cast<int64_t>(n_tokens) * groups;
  const int64_t blocks = (items + 7) / 8;
  if (blocks > 0x7FFFFFFF) return AKLR_ERR_TOO_LARGE;
  auto* xp = static_cast<const uint16_t*>(x);
  auto* wp = static_cast<const uint16_t*>(w);
  auto* lp = static_cast<uint16_t*>(logits);
  if (per_warp == 1)
    router_gemm_kernel<1><<<static_cast<int>(blocks), 256, 0, stream>>>(xp, wp, lp, n_tokens, hidden, n_routed);
  else
    router_gemm_kernel<8><<<static_cast<int>(blocks), 256, 0, stream>>>(xp, wp, lp, n_tokens, hidden, n_routed);
  return cudaGetLastError() == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

}  // namespace aklr
