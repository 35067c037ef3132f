// Router projection on the tensor cores, sm_100a: logits[T, E] = bf16( x[T, H] . W[E, H]^T ) with
// float32 accumulation in TMEM, the rounding point of the reference's _router_logits
// (aklr/plugins/sglang/models/qwen3_moe/reference.py:24-31).  One CTA per 128 tokens x up to 256
// experts: TMA (SWIZZLE_128B, 64 bf16 = 128 bytes of K per stage) feeds tcgen05.mma kind::f16
// (M128, N = experts rounded up to 16, K16); rows and experts past the end are zero-filled by the
// TMA.  192 threads: warp 0 TMA, warp 1 MMA + TMEM, warps 2..5 epilogue (one TMEM lane quarter each).
#include "common.cuh"
#include "kernels.h"

namespace aklr {

namespace {

constexpr int kThreads = 192;
constexpr int kStages = 4;
constexpr int kABytes = 128 * 128;

struct RouterParams {
  CUtensorMap map_x;  // bf16 [T, H], box 64 x 128
  CUtensorMap map_w;  // bf16 [E, H], box 64 x n_tile
  uint16_t* logits;   // bf16 [T, E]
  int32_t* status;    // optional [2]
  int32_t* host_status;  // the device's host-visible copy of a failure (or null)
  int n_tokens, hidden, n_routed, n_tile;
};

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

__global__ void __launch_bounds__(kThreads, 1) router_gemm_tc_kernel(const __grid_constant__ RouterParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stage_bytes = kABytes + p.n_tile * 128;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * stage_bytes);
  uint64_t* empty = full + kStages;
  uint64_t* acc_full = empty + kStages;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(acc_full + 1);
  // everything lives in the dynamic allocation: a static __shared__ variable on top of the 227 KB
  // opt-in would exceed the per-CTA limit
  int* abort_word = reinterpret_cast<int*>(tmem_ptr + 1);
  int* local_status = abort_word + 1;
  volatile int* abort_flag = abort_word;
  int* status = p.status ? p.status : local_status;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_steps = p.hidden >> 6;
  const int tok0 = blockIdx.x * 128, exp0 = blockIdx.y * p.n_tile;
  uint32_t tmem_cols = 32;
  while (tmem_cols < static_cast<uint32_t>(p.n_tile)) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_word = 0;
    local_status[0] = local_status[1] = 0;
    fence_mbar_init();
    tma_prefetch_desc(&p.map_x);
    tma_prefetch_desc(&p.map_w);
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr;

  if (warp == 0) {
    if (lane == 0) {
      for (int it = 0; it < k_steps; ++it) {
        const int s = it % kStages;
        if (!mbar_wait(&empty[s], ((it / kStages) & 1) ^ 1, abort_flag, status, 31)) break;
        uint8_t* st = smem + s * stage_bytes;
        mbar_expect_tx(&full[s], stage_bytes);
        tma_load_2d(st, &p.map_x, &full[s], it * 64, tok0);
        tma_load_2d(st + kABytes, &p.map_w, &full[s], it * 64, exp0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // kind::f16: f32 accumulator, bf16 A and B, K-major, M 128, N n_tile
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(p.n_tile >> 3) << 17) |
                             (static_cast<uint32_t>(128 >> 4) << 24);
      bool ok = true;
      for (int it = 0; it < k_steps; ++it) {
        const int s = it % kStages;
        if (!mbar_wait(&full[s], (it / kStages) & 1, abort_flag, status, 32)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t a0 = smem_u32(smem + s * stage_bytes);
        const uint64_t da = umma_desc_sw128(a0), db = umma_desc_sw128(a0 + kABytes);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (it > 0 || k > 0) ? 1u : 0u);
        tc_commit(&empty[s]);
      }
      if (ok) tc_commit(acc_full);
    }
  } else {
    const int quarter = warp & 3;
    const int token = tok0 + quarter * 32 + lane;
    const bool got = mbar_wait(acc_full, 0, abort_flag, status, 33);
    tc_fence_after_sync();
    const uint32_t t0 = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    for (int c = 0; c < p.n_tile; c += 16) {
      uint32_t r[16];
      AKLR_TMEM_LD_16(t0 + c, r);
      tc_wait_ld();
      if (got && token < p.n_tokens) {
        uint16_t* dst = p.logits + static_cast<size_t>(token) * p.n_routed + exp0 + c;
        if (exp0 + c + 16 <= p.n_routed && (p.n_routed & 7) == 0) {
          uint32_t o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const __nv_bfloat162 two = __floats2bfloat162_rn(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
            o[i] = *reinterpret_cast<const uint32_t*>(&two);
          }
          *reinterpret_cast<uint4*>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4*>(dst + 8) = make_uint4(o[4], o[5], o[6], o[7]);
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (exp0 + c + i < p.n_routed) {
              const __nv_bfloat16 v = __float2bfloat16_rn(__uint_as_float(r[i]));
              dst[i] = *reinterpret_cast<const uint16_t*>(&v);
            }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) publish_wait_failure(status, p.host_status);
    const uint64_t start = global_timer_ns();
    while (global_timer_ns() - start < 200000ull) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

}  // namespace

int launch_router_gemm_tc(const CUtensorMap& map_x, const CUtensorMap& map_w, void* logits, int n_tokens, int hidden,
                          int n_routed, int n_tile, int32_t* host_status, cudaStream_t stream) {
  if (hidden % 64 != 0 || n_tile % 16 != 0 || n_tile < 16 || n_tile > 256) return AKLR_ERR_UNSUPPORTED_SHAPE;
  RouterParams p{};
  p.map_x = map_x;
  p.map_w = map_w;
  p.logits = static_cast<uint16_t*>(logits);
  p.status = nullptr;
  p.host_status = host_status;
  p.n_tokens = n_tokens;
  p.hidden = hidden;
  p.n_routed = n_routed;
  p.n_tile = n_tile;
  const size_t smem = static_cast<size_t>(kStages) * (kABytes + n_tile * 128) + (2 * kStages + 1) * 8 + 32 + 1024;
  if (ensure_max_dynamic_smem(reinterpret_cast<const void*>(router_gemm_tc_kernel)) != AKLR_OK) return AKLR_ERR_CUDA;
  const dim3 grid((n_tokens + 127) / 128, (n_routed + n_tile - 1) / n_tile);
  router_gemm_tc_kernel<<<grid, kThreads, smem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

}  // namespace aklr
