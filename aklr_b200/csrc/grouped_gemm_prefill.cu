// Token-major grouped FP8 GEMM for full blocks (block_m = 128): the prefill path, sm_100a.
//
// Same arithmetic as grouped_gemm.cu (128x128 weight block scales and 1x128 activation scales
// applied per K-block of 128 in float32, SiLU*mul + 1x128 requant after gate_up, route weight after
// down; aklr/plugins/sglang/models/deepseek_v2/reference.py:146-183), the other orientation:
// the block's 128 TOKENS are the MMA's M side (one token per TMEM lane = one token per epilogue
// thread), 256 weight rows are the N side -- gate rows j*128.. and up rows I + j*128.. for gate_up,
// 256 consecutive output channels for down.  One tcgen05.mma M128 N256 K32 per 32 K bytes runs
// the tensor core at its full rate, and the per-K-block scale becomes a per-thread scalar
// (activation scale of the thread's token x the weight block scale), so folding a partial into the
// float32 accumulators is exactly one FMA per element with both operands in registers.
//
// Per thread the epilogue also becomes local: a token's 64 (gate_up) or 128 (down) channels sit in
// one thread, which writes them as whole 16-byte vectors of its own output row.
//
// Warp roles (64 + 128*kCS threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, the rest
// epilogue (TMEM lane quarter = warp % 4, column split = (warp-2)/4).  Measured on B200: a warp
// drains TMEM at about one column per 4.3 cycles when the tensor core is idle and one per 8 cycles
// while MMAs run, whatever the tcgen05.ld width, and more warps per lane quarter add up; with this
// tile the drain (256 columns per quarter per K-block) costs about as much as the MMAs, so 8 and 16
// epilogue warps, and one N=256 or two N=128 MMA groups per K-block, all land within 10%.  Persistent CTAs, TMA
// SWIZZLE_128B ring, two 256-column TMEM partial buffers, no cluster, no multicast, bounded waits.
#include <cfloat>

#include "common.cuh"
#include "kernels.h"

namespace aklr {

#ifdef AKLR_GEMM_TIMING
// Development aid, compiled only on request: cycle counts per role of CTA 0.
// [1] mma wait-full [2] mma wait-tmem-empty [3] mma issue [4] epi wait [5] epi ld+fma [6] setup [7] final [8] kblocks
__device__ long long g_prefill_timing[2][16];
#define PT(slot, expr)                                         \
  do {                                                         \
    const long long t_begin_ = clock64();                      \
    expr;                                                      \
    if (blockIdx.x == 0) tacc[slot] += clock64() - t_begin_;   \
  } while (0)
#else
#define PT(slot, expr) \
  do {                 \
    expr;              \
  } while (0)
#endif

namespace {

constexpr int kCS = 2;                   // column splits: epilogue warps = 4 lane quarters x kCS
constexpr int kEpiWarps = 4 * kCS;
constexpr int kEpi = 32 * kEpiWarps;
constexpr int kThreads = 64 + kEpi;
constexpr int kBM = 128;                 // tokens per block
constexpr int kBN = 256;                 // weight rows per tile
constexpr int kABytes = kBM * 128;       // token tile of one K-block
constexpr int kBBytes = kBN * 128;       // weight tile of one K-block
constexpr int kStageBytes = kABytes + kBBytes;
constexpr bool kSplitGroups = false;     // true: two N=128 MMA groups per K-block instead of one N=256

struct PrefillLayout {
  int off_xs, off_ws, off_rid, off_wgt, off_wmax, off_bars, total;
};

__host__ __device__ inline PrefillLayout prefill_layout(int k, int stages) {
  PrefillLayout l;
  const int kb = k / 128;
  l.off_xs = stages * kStageBytes;            // float[kb][128] activation scales of the block
  l.off_ws = l.off_xs + kb * kBM * 4;         // float[2][kb] weight block scales of the two halves
  l.off_rid = l.off_ws + ((2 * kb * 4 + 15) & ~15);
  l.off_wgt = l.off_rid + kBM * 4;            // float[128] route weights
  l.off_wmax = l.off_wgt + kBM * 4;           // float[kCS][128] amax per column split
  l.off_bars = l.off_wmax + kCS * kBM * 4;
  l.total = l.off_bars + (2 * stages + 8) * 8 + 16;
  return l;
}

// Two float32 FMAs in one instruction (sm_100 packed f32x2): halves the issue slots of the fold.
__device__ __forceinline__ uint64_t pack_f32x2(uint32_t lo, uint32_t hi) {
  uint64_t v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(lo), "r"(hi));
  return v;
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ float lo_f32(uint64_t v) { return __uint_as_float(static_cast<uint32_t>(v)); }
__device__ __forceinline__ float hi_f32(uint64_t v) { return __uint_as_float(static_cast<uint32_t>(v >> 32)); }

__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kEpi) : "memory"); }
__device__ __forceinline__ bool epi_any(int flag) {
  uint32_t any;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.or.pred p, 1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(any)
      : "r"(flag), "n"(kEpi)
      : "memory");
  return any != 0;
}

template <bool GATE_UP>
__global__ void __launch_bounds__(kThreads, 1) grouped_gemm_prefill_kernel(const __grid_constant__ GroupedGemmParams p) {
  constexpr int NH = kBN / kCS;   // accumulator columns per epilogue thread
  constexpr int CH = 8;     // columns per tcgen05.ld

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int KB = p.k >> 7;
  const int S = p.stages;
  const PrefillLayout L = prefill_layout(p.k, S);
  float* xs_s = reinterpret_cast<float*>(smem + L.off_xs);
  float* ws_s = reinterpret_cast<float*>(smem + L.off_ws);
  int* rid_s = reinterpret_cast<int*>(smem + L.off_rid);
  float* wgt_s = reinterpret_cast<float*>(smem + L.off_wgt);
  float* wmax = reinterpret_cast<float*>(smem + L.off_wmax);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.off_bars);
  uint64_t* empty = full + S;
  uint64_t* tmem_full = empty + S;
  uint64_t* tmem_empty = tmem_full + 4;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(tmem_empty + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int nb = *p.num_blocks;
  if (nb > p.max_blocks) nb = p.max_blocks;
  // gate_up: one tile per 128 intermediate channels (128 gate + 128 up rows); down: per 256 channels
  const int tiles_per_block = GATE_UP ? (p.out_dim >> 7) : (p.out_dim >> 8);
  const int total_tiles = nb * tiles_per_block;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 4; ++i) {  // buffer = (K-block parity) * 2 + column group
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], GATE_UP ? kEpiWarps : kEpiWarps / 2);  // the warps that read the group
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&p.map_w);
    tma_prefetch_desc(&p.map_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr;

  if (warp == 0) {
    // ------------------------------- TMA producer ------------------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int b = t / tiles_per_block, j = t - b * tiles_per_block;
        const int e = p.block_expert[b];
        const int w_row = e * p.rows_per_expert + (GATE_UP ? j * 128 : j * 256);
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 11)) { ok = false; break; }
          uint8_t* st = smem + s * kStageBytes;
          mbar_expect_tx(&full[s], kStageBytes);
          tma_load_2d(st, &p.map_x, &full[s], kb * 128, b * kBM);
          if (GATE_UP) {  // gate rows, then the matching up rows: one 256-row K-major operand
            tma_load_2d(st + kABytes, &p.map_w, &full[s], kb * 128, w_row);
            tma_load_2d(st + kABytes + kBBytes / 2, &p.map_w, &full[s], kb * 128, w_row + p.out_dim);
          } else {
            tma_load_2d(st + kABytes, &p.map_w, &full[s], kb * 128, w_row);  // box of 256 rows
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer --------------------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
#ifdef AKLR_GEMM_TIMING
      long long tacc[16] = {0};
#endif
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          const int buf = it & 1;
          const uint32_t bph = (it >> 1) & 1;
          bool got;
          PT(1, got = mbar_wait(&full[s], ph, abort_flag, p.status, 12));
          if (!got) { ok = false; break; }
          const uint32_t a0 = smem_u32(smem + s * kStageBytes);
          const uint64_t da = umma_desc_sw128(a0);
          // Two column groups of 128 weight rows, each into its own TMEM buffer with its own
          // hand-off: the epilogue starts on the first while the second is still being computed,
          // and four buffers in flight hide the commit -> wake-up latency.
          if (kSplitGroups) {
#pragma unroll
            for (int g = 0; g < 2; ++g) {
              const int tb = buf * 2 + g;
              PT(2, got = mbar_wait(&tmem_empty[tb], bph ^ 1, abort_flag, p.status, 13));
              if (!got) { ok = false; break; }
#ifdef AKLR_GEMM_TIMING
              const long long t_issue = clock64();
#endif
              tc_fence_after_sync();
              const uint64_t db = umma_desc_sw128(a0 + kABytes + g * (kBBytes / 2));
              const uint32_t d = tmem_base + tb * 128;
#pragma unroll
              for (int k = 0; k < 4; ++k) umma_f8f6f4(d, da + 2 * k, db + 2 * k, umma_idesc_e4m3(128), k > 0);
              tc_commit(&tmem_full[tb]);
#ifdef AKLR_GEMM_TIMING
              tacc[3] += clock64() - t_issue;
#endif
            }
          } else {  // one N=256 MMA per 32 K bytes over both groups' buffers (adjacent TMEM columns)
            PT(2, got = mbar_wait(&tmem_empty[buf * 2], bph ^ 1, abort_flag, p.status, 13));
            if (!got) { ok = false; break; }
            PT(2, got = mbar_wait(&tmem_empty[buf * 2 + 1], bph ^ 1, abort_flag, p.status, 13));
            if (!got) { ok = false; break; }
#ifdef AKLR_GEMM_TIMING
            const long long t_issue = clock64();
#endif
            tc_fence_after_sync();
            const uint64_t db = umma_desc_sw128(a0 + kABytes);
            const uint32_t d = tmem_base + buf * 256;
#pragma unroll
            for (int k = 0; k < 4; ++k) umma_f8f6f4(d, da + 2 * k, db + 2 * k, umma_idesc_e4m3(256), k > 0);
            tc_commit(&tmem_full[buf * 2]);
            tc_commit(&tmem_full[buf * 2 + 1]);
#ifdef AKLR_GEMM_TIMING
            tacc[3] += clock64() - t_issue;
#endif
          }
          if (!ok) break;
          tc_commit(&empty[s]);
        }
      }
#ifdef AKLR_GEMM_TIMING
      if (blockIdx.x == 0) {
        for (int i = 1; i <= 3; ++i) g_prefill_timing[GATE_UP][i] = tacc[i];
        g_prefill_timing[GATE_UP][8] = it;
      }
#endif
    }
  } else {
    // ------------------------------- epilogue warps ----------------------------------------
    const int quarter = warp & 3;
    const int cs = (warp - 2) >> 2;       // which column split this warp folds
    const int et = threadIdx.x - 64;
    const int row = quarter * 32 + lane;  // token inside the block = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int IB = p.out_dim >> 7;
    uint32_t it = 0;
    bool bad = false;
#ifdef AKLR_GEMM_TIMING
    long long tacc[16] = {0};
    long long t_mark = clock64();
#endif
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
#ifdef AKLR_GEMM_TIMING
      tacc[7] += clock64() - t_mark;
      t_mark = clock64();
#endif
      if (epi_any(*abort_flag)) break;
      const int b = t / tiles_per_block, j = t - b * tiles_per_block;
      const int e = p.block_expert[b];
      {
        const float* xs = p.x_scale + static_cast<size_t>(b) * KB * kBM;
        for (int i = et; i < KB * kBM; i += kEpi) xs_s[i] = __ldg(xs + i);
        // weight block scales of the tile's two 128-row halves
        const int rb0 = GATE_UP ? j : 2 * j;
        const int rb1 = GATE_UP ? IB + j : 2 * j + 1;
        const float* wsb = p.w_scale + static_cast<size_t>(e) * (p.rows_per_expert >> 7) * KB;
        for (int i = et; i < KB; i += kEpi) {
          ws_s[i] = __ldg(wsb + static_cast<size_t>(rb0) * KB + i);
          ws_s[KB + i] = __ldg(wsb + static_cast<size_t>(rb1) * KB + i);
        }
        if (et < kBM) {
          const int rid = p.sorted_ids[b * kBM + et];
          rid_s[et] = rid;
          if (!GATE_UP) wgt_s[et] = rid >= 0 ? p.topk_weights[rid] : 0.0f;
        }
      }
      epi_sync();

      // gate_up: first NH/2 accumulators gate channels cs*NH/2.., then the matching up channels
      // down:    NH output channels cs*NH..
#ifdef AKLR_GEMM_TIMING
      tacc[6] += clock64() - t_mark;
#endif
      uint64_t acc2[NH / 2];  // pairs of float32 accumulators
#pragma unroll
      for (int i = 0; i < NH / 2; ++i) acc2[i] = 0ull;

      for (int kb = 0; kb < KB; ++kb, ++it) {
        const int buf = it & 1;
        const uint32_t bph = (it >> 1) & 1;
        const float sx = xs_s[kb * kBM + row];
        // gate_up: group 0 = gate columns, group 1 = up columns, this warp's NH/2 of each.
        // down: this warp's NH channels lie in one group.
        constexpr int GROUPS = GATE_UP ? 2 : 1;
        constexpr int GC = NH / GROUPS;  // columns this thread takes from one group
#ifdef AKLR_GEMM_TIMING
        long long t_work = clock64();
#endif
#pragma unroll
        for (int gi = 0; gi < GROUPS; ++gi) {
          const int g = GATE_UP ? gi : (cs * NH) / 128;
          const int tb = buf * 2 + g;
          bool got;
#ifdef AKLR_GEMM_TIMING
          if (blockIdx.x == 0) tacc[5] += clock64() - t_work;
#endif
          PT(4, got = mbar_wait(&tmem_full[tb], bph, abort_flag, p.status, 14));
#ifdef AKLR_GEMM_TIMING
          t_work = clock64();
#endif
          if (!got) bad = true;
          tc_fence_after_sync();
          const float f = sx * ws_s[g * KB + kb];
          const uint64_t f2 = pack_f32x2(__float_as_uint(f), __float_as_uint(f));
          const uint32_t t0 = tmem_base + lane_addr + tb * 128 + (GATE_UP ? cs * GC : (cs * NH) % 128);
          uint32_t r[2][CH];
          AKLR_TMEM_LD_8(t0, r[0]);
#pragma unroll
          for (int k = 0; k < GC / CH; ++k) {
            tc_wait_ld();
            if (k + 1 < GC / CH) {
              AKLR_TMEM_LD_8(t0 + (k + 1) * CH, r[(k + 1) & 1]);
            } else {
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(&tmem_empty[tb]);
            }
#pragma unroll
            for (int i = 0; i < CH; i += 2) {
              const int at = (gi * GC + k * CH + i) / 2;
              acc2[at] = fma_f32x2(pack_f32x2(r[k & 1][i], r[k & 1][i + 1]), f2, acc2[at]);
            }
          }
        }
#ifdef AKLR_GEMM_TIMING
        if (blockIdx.x == 0) tacc[5] += clock64() - t_work;
#endif
      }
#ifdef AKLR_GEMM_TIMING
      t_mark = clock64();
#endif

      float acc[NH];
#pragma unroll
      for (int i = 0; i < NH / 2; ++i) {
        acc[2 * i] = lo_f32(acc2[i]);
        acc[2 * i + 1] = hi_f32(acc2[i]);
      }
      const int rid = rid_s[row];
      if (GATE_UP) {
        constexpr int HC = NH / 2;  // h channels of this thread
        float m = 0.0f;
#pragma unroll
        for (int i = 0; i < HC; ++i) {
          const float g = acc[i];
          const float h = __fdividef(g, 1.0f + __expf(-g)) * acc[HC + i];
          acc[i] = __bfloat162float(__float2bfloat16_rn(h));
          m = fmaxf(m, fabsf(acc[i]));
        }
        wmax[cs * kBM + row] = m;
        epi_sync();
#pragma unroll
        for (int c = 0; c < kCS; ++c) m = fmaxf(m, wmax[c * kBM + row]);
        const float scale = fmaxf(__fdiv_rn(m, 448.0f), FLT_MIN);
        const float inv = __fdiv_rn(1.0f, scale);
        if (rid >= 0 && !bad) {
          if (cs == 0) p.out_scale[(static_cast<size_t>(b) * IB + j) * kBM + row] = scale;
          uint8_t* dst = p.out_q + static_cast<size_t>(b * kBM + row) * p.out_dim + j * 128 + cs * HC;
#pragma unroll
          for (int v = 0; v < HC / 16; ++v) {
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int i = v * 16 + q * 4;
              w[q] = cvt_e4m3x2(acc[i] * inv, acc[i + 1] * inv) |
                     (static_cast<uint32_t>(cvt_e4m3x2(acc[i + 2] * inv, acc[i + 3] * inv)) << 16);
            }
            *reinterpret_cast<uint4*>(dst + v * 16) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      } else if (rid >= 0 && !bad) {
        const float w = wgt_s[row];
        uint8_t* dst = static_cast<uint8_t*>(p.out_rows) +
                       (static_cast<size_t>(rid) * p.out_dim + j * 256 + cs * NH) * 2;
#pragma unroll
        for (int v = 0; v < NH / 8; ++v) {
          uint32_t o[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const __nv_bfloat162 two = __floats2bfloat162_rn(acc[v * 8 + 2 * q] * w, acc[v * 8 + 2 * q + 1] * w);
            o[q] = *reinterpret_cast<const uint32_t*>(&two);
          }
          *reinterpret_cast<uint4*>(dst + v * 16) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
    }
#ifdef AKLR_GEMM_TIMING
    if (blockIdx.x == 0 && warp == 2 && lane == 0)
      for (int i = 4; i <= 7; ++i) g_prefill_timing[GATE_UP][i] = tacc[i];
#endif
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {  // a wait gave up: let copies in flight land before shared memory is released
    const uint64_t start = global_timer_ns();
    while (global_timer_ns() - start < 200000ull) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace

#ifdef AKLR_GEMM_TIMING
extern "C" int aklr_debug_read_prefill_timing(long long* host32) {
  return cudaMemcpyFromSymbol(host32, g_prefill_timing, sizeof(g_prefill_timing)) == cudaSuccess ? 0 : -3;
}
#endif

bool grouped_gemm_is_token_major(bool gate_up, int block_m, int out_dim) {
  return block_m == 128 && (gate_up || out_dim % 256 == 0);
}

int grouped_gemm_prefill_pick_stages(int k) {
  for (int s = 6; s >= 2; --s)
    if (prefill_layout(k, s).total + 1024 <= 227 * 1024) return s;
  return 0;
}

int launch_grouped_gemm_prefill(const GroupedGemmParams& p, bool gate_up, int sm_count, cudaStream_t stream) {
  if (p.k % 128 != 0 || p.block_m != 128 || p.max_blocks < 1 || p.stages < 2) return AKLR_ERR_UNSUPPORTED_SHAPE;
  if (gate_up ? (p.out_dim % 128 != 0) : (p.out_dim % 256 != 0)) return AKLR_ERR_UNSUPPORTED_SHAPE;
  const size_t smem = static_cast<size_t>(prefill_layout(p.k, p.stages).total) + 1024;
  if (smem > 227 * 1024) return AKLR_ERR_UNSUPPORTED_SHAPE;
  const long long tiles = static_cast<long long>(p.max_blocks) * (gate_up ? p.out_dim / 128 : p.out_dim / 256);
  const int grid = static_cast<int>(tiles < sm_count ? tiles : sm_count);
  auto run = [&](auto kernel) {
    if (ensure_max_dynamic_smem(reinterpret_cast<const void*>(kernel)) != AKLR_OK) return AKLR_ERR_CUDA;
    kernel<<<grid, kThreads, smem, stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
  };
  return gate_up ? run(grouped_gemm_prefill_kernel<true>) : run(grouped_gemm_prefill_kernel<false>);
}

}  // namespace aklr
