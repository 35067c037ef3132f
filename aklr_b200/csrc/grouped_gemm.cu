// Grouped FP8 GEMMs of the fused-MoE layer on tcgen05 (sm_100a): gate_up (+ SiLU*mul + 1x128
// FP8 requant) and down (+ route weight), both with 128x128 weight block scales and 1x128
// activation scales applied in float32 exactly where the reference's dequantised matmul has them
// (aklr/plugins/sglang/models/deepseek_v2/reference.py:146-183,
//  aklr/plugins/sglang/models/qwen3_moe/reference.py:57-88).
//
// Orientation ("swap-AB"): the WEIGHT tile is the MMA's M side (128 output channels = 128 TMEM
// lanes), the block's tokens are the N side (block_m = 16..128 columns).  A decode batch with a
// handful of rows per expert therefore streams each weight byte from HBM exactly once and spends
// tensor work only on 16 token columns, and a weight block scale is one scalar per (tile, K-block)
// while the activation scale varies along the columns.
//
// Per K-block of 128 the MMA warp issues 4 (x2 for gate and up) tcgen05.mma of K=32 into one of
// two TMEM partial buffers; the epilogue warps drain the partial with tcgen05.ld and fold it into
// float32 register accumulators times (weight scale x activation scale) -- the tensor core has no
// 128-granular float scale input.  Persistent CTAs (one per SM) walk the (block, channel-tile)
// list; TMA (SWIZZLE_128B) feeds a ring of shared-memory stages.  No cluster, no multicast.
//
// Warp roles (320 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..9
// epilogue (TMEM lane quarter = warp % 4, column half = (warp-2)/4).
#include <cfloat>
#include <cstdlib>
#include <map>
#include <mutex>
#include <utility>

#include "common.cuh"
#include "kernels.h"

namespace aklr {

constexpr int kGemmThreads = 320;
constexpr int kEpiThreads = 256;
constexpr int kWTileBytes = 128 * 128;  // 128 channels x 128 K bytes

struct GemmSmemLayout {
  int stage_bytes, misc_bytes, total_bytes;
  int off_misc, off_rid, off_wmax, off_wscale, off_bars;
};

__host__ __device__ inline GemmSmemLayout gemm_layout(bool gate_up, int block_m, int k, int stages, bool wide = false) {
  GemmSmemLayout l;
  const int kb = k / 128;
  const int w_tiles = (gate_up || wide) ? 2 : 1;  // weight tiles per stage: gate + up, or two neighbouring down tiles
  l.stage_bytes = w_tiles * kWTileBytes + block_m * 128;
  const int scale_bytes = w_tiles * kb * block_m * 4;  // combined scale table(s)
  const int out_bytes = block_m * 128 * (gate_up ? 1 : 2);
  l.misc_bytes = ((scale_bytes > out_bytes ? scale_bytes : out_bytes) + 127) & ~127;
  l.off_misc = stages * l.stage_bytes;
  l.off_rid = l.off_misc + l.misc_bytes;       // int[block_m]
  l.off_wmax = l.off_rid + block_m * 4;        // float[4][block_m]
  l.off_wscale = l.off_wmax + 4 * block_m * 4; // float[block_m]: per-column requant inverse / route weight
  l.off_bars = (l.off_wscale + block_m * 4 + 15) & ~15;  // barriers, tmem ptr, abort flag
  l.total_bytes = l.off_bars + (2 * stages + 4) * 8 + 16;
  return l;
}

size_t grouped_gemm_smem_bytes(bool gate_up, int block_m, int k, int stages, bool wide) {
  return static_cast<size_t>(gemm_layout(gate_up, block_m, k, stages, wide).total_bytes) + 1024;  // alignment slack
}

int grouped_gemm_pick_stages(bool gate_up, int block_m, int k, bool wide) {
  for (int s = 8; s >= 2; --s)
    if (grouped_gemm_smem_bytes(gate_up, block_m, k, s, wide) <= 227 * 1024) return s;
  return 0;
}

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ bool epi_bar_any(int flag) {
  uint32_t any;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.or.pred p, 1, 256, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(any)
      : "r"(flag)
      : "memory");
  return any != 0;
}

// WIDE (down projection only): a tile is 256 output channels, two weight tiles per stage sharing the token tile as
// gate and up do.  A decode block's K-block then moves 32 KB of weights instead of 16 KB per hand-off, which is what
// lets the down projection stream at the rate of gate_up.
template <int BM, bool GATE_UP, bool WIDE = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_kernel(const __grid_constant__ GroupedGemmParams p) {
  static_assert(!(GATE_UP && WIDE), "wide tiles are for the down projection");
  constexpr bool TWO = GATE_UP || WIDE;             // two weight tiles per stage and two accumulator tiles
  constexpr int kTileShift = WIDE ? 8 : 7;          // output channels per tile: 256 or 128
  constexpr int NH = BM / 2;                        // columns per epilogue warp
  constexpr int CH = (NH >= 16 && !(GATE_UP && BM >= 64)) ? 16 : 8;  // columns per tcgen05.ld (register budget: 168 per thread)
  constexpr int BUF_COLS = (TWO ? 2 : 1) * BM;      // TMEM columns of one partial buffer
  constexpr int TMEM_COLS = 2 * BUF_COLS < 32 ? 32 : 2 * BUF_COLS;
  constexpr uint32_t IDESC = umma_idesc_e4m3(BM);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int KB = p.k >> 7;
  const int S = p.stages;
  const GemmSmemLayout L = gemm_layout(GATE_UP, BM, p.k, S, WIDE);
  float* ftab = reinterpret_cast<float*>(smem + L.off_misc);  // [tiles][KB][BM] combined scales ...
  uint8_t* out_tile = smem + L.off_misc;                      // ... aliased by the output tile
  int* rid_s = reinterpret_cast<int*>(smem + L.off_rid);
  float* wmax = reinterpret_cast<float*>(smem + L.off_wmax);
  float* colscale = reinterpret_cast<float*>(smem + L.off_wscale);  // [BM]
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.off_bars);
  uint64_t* empty = full + S;
  uint64_t* tmem_empty = empty + S;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_empty[i], kEpiThreads / 32);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&p.map_w);
    tma_prefetch_desc(&p.map_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr;
  // The weight boxes of this CTA's first tile go on their way BEFORE the wait: weights are not written by any kernel,
  // and the block table that says which expert's they are comes from the sort, which ran before the kernel before
  // this one -- every kernel of the library signals its dependents only after its own wait, so whatever preceded
  // the previous kernel is complete when this one starts.  The activation boxes of those stages follow the wait.
  int early = 0;  // K-blocks of the first tile whose weight loads are already in flight (producer thread only)
  if (warp == 0 && lane == 0) {
    int nb0 = *p.num_blocks;
    if (nb0 > p.max_blocks) nb0 = p.max_blocks;
    const int tiles_per_block0 = p.out_dim >> kTileShift;
    if (static_cast<int>(blockIdx.x) < nb0 * tiles_per_block0) {
      const int b = blockIdx.x / tiles_per_block0, j = blockIdx.x - b * tiles_per_block0;
      const int w_row = p.block_expert[b] * p.rows_per_expert + (j << kTileShift);
      early = KB < S ? KB : S;
      for (int kb = 0; kb < early; ++kb) {
        uint8_t* st = smem + kb * L.stage_bytes;
        mbar_expect_tx(&full[kb], L.stage_bytes);  // the activation box's bytes too: it comes after the wait
        int wx, wy;
        weight_box(p.w_tiled != 0, KB, w_row, kb, &wx, &wy);
        tma_load_2d(st, &p.map_w, &full[kb], wx, wy);
        if (TWO) {
          weight_box(p.w_tiled != 0, KB, w_row + (GATE_UP ? p.out_dim : 128), kb, &wx, &wy);
          tma_load_2d(st + kWTileBytes, &p.map_w, &full[kb], wx, wy);
        }
      }
    }
  }
  griddep_wait();    // everything below reads what earlier kernels of the call wrote
  griddep_launch();  // after the wait: a dependent that starts knows every kernel before this one is complete
  int nb = *p.num_blocks;
  if (nb > p.max_blocks) nb = p.max_blocks;
  const int tiles_per_block = p.out_dim >> kTileShift;
  const int total_tiles = nb * tiles_per_block;

  if (warp == 0) {
    // ------------------------------- TMA producer ------------------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      int s = 0;  // ring position and the parity of its current use
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int b = t / tiles_per_block, j = t - b * tiles_per_block;
        const int e = p.block_expert[b];
        const int w_row = e * p.rows_per_expert + (j << kTileShift);
        for (int kb = 0; kb < KB; ++kb, ++it) {
          uint8_t* st = smem + s * L.stage_bytes;
          if (static_cast<int>(it) >= early) {  // else: stage free from the start, bytes announced and weights under way
            bool got;
            got = mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 1);
            if (!got) { ok = false; break; }
            mbar_expect_tx(&full[s], L.stage_bytes);
            int wx, wy;
            weight_box(p.w_tiled != 0, KB, w_row, kb, &wx, &wy);
            tma_load_2d(st, &p.map_w, &full[s], wx, wy);
            if (TWO) {
              weight_box(p.w_tiled != 0, KB, w_row + (GATE_UP ? p.out_dim : 128), kb, &wx, &wy);
              tma_load_2d(st + kWTileBytes, &p.map_w, &full[s], wx, wy);
            }
          }
          tma_load_2d(st + (TWO ? 2 : 1) * kWTileBytes, &p.map_x, &full[s], kb * 128, b * BM);
          if (++s == S) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer --------------------------------------------
    if (lane == 0) {
      // A lone thread pays the full latency of every instruction: ring position, phases and
      // descriptors are carried forward, and one commit per K-block serves both the producer (stage
      // free) and the epilogue (partial complete).
      int s = 0;
      uint32_t ph = 0, buf = 0, bph = 0;
      const uint64_t desc0 = umma_desc_sw128(smem_u32(smem));
      const uint32_t stage_step = static_cast<uint32_t>(L.stage_bytes) >> 4;
      uint64_t da0 = desc0;  // first weight tile of stage s; the second one and the token tile follow
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        for (int kb = 0; kb < KB; ++kb) {
          bool got;
          got = mbar_wait(&full[s], ph, abort_flag, p.status, 2);
          if (!got) { ok = false; break; }
          got = mbar_wait(&tmem_empty[buf], bph ^ 1, abort_flag, p.status, 3);
          if (!got) { ok = false; break; }
          tc_fence_after_sync();
          const uint64_t da1 = da0 + (kWTileBytes >> 4);
          const uint64_t db = da0 + (((TWO ? 2 : 1) * kWTileBytes) >> 4);
          const uint32_t d = tmem_base + buf * BUF_COLS;
#pragma unroll
          for (int k = 0; k < 4; ++k) {  // 32 K bytes per MMA: the descriptor start moves 32 B
            umma_f8f6f4(d, da0 + 2 * k, db + 2 * k, IDESC, k > 0);
            if (TWO) umma_f8f6f4(d + BM, da1 + 2 * k, db + 2 * k, IDESC, k > 0);
          }
          tc_commit(&empty[s]);
          da0 += stage_step;
          if (++s == S) { s = 0; ph ^= 1; da0 = desc0; }
          bph ^= buf;
          buf ^= 1;
        }
      }
    }
  } else {
    // ------------------------------- epilogue warps ----------------------------------------
    const int ew = warp - 2;
    const int quarter = warp & 3;            // TMEM lanes this warp may read
    const int half = ew >> 2;                // which half of the columns
    const int et = threadIdx.x - 64;         // 0..255
    const int chan = quarter * 32 + lane;    // output channel inside the tile = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int IB = p.out_dim >> 7;           // gate_up: 128-blocks of the intermediate size
    constexpr int TILES = TWO ? 2 : 1;
    constexpr int CPT = NH / CH;             // chunks per accumulator tile
    constexpr int NC = TILES * CPT;          // chunks per K-block
    uint32_t it = 0;
    int ring = 0;  // the stage whose "empty" barrier reports MMA(it) complete, and its parity
    uint32_t ring_ph = 0;
    bool bad = false;
    constexpr int kPreBatch = 4;
    constexpr bool kPrefetch = BM <= 32;  // the decode blocks; larger ones have no registers to spare
    float pre_s[kPreBatch], pre_w0[kPreBatch], pre_w1[kPreBatch], pre_weight = 0.0f;
    int pre_rid = -1;
    bool have_pre = false;
    // experts of this CTA's current and next tile, read a tile ahead of the addresses that need them
    int e_cur = blockIdx.x < total_tiles ? p.block_expert[blockIdx.x / tiles_per_block] : 0;
    int e_ahead = blockIdx.x + gridDim.x < total_tiles ? p.block_expert[(blockIdx.x + gridDim.x) / tiles_per_block] : 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      if (epi_bar_any(*abort_flag)) break;   // also fences the aliased smem against the last tile
      const int b = t / tiles_per_block, j = t - b * tiles_per_block;
      const int e = e_cur;
      // Combined scale table of the tile, ftab[tile][kb][n] = activation scale x weight block
      // scale, so the K loop is one shared-memory float4 per four columns and one FMA per element.
      // The first batch of its inputs, the tile's route ids and (down) route weights were loaded
      // during the previous tile of this CTA (``pre_*``): a tile of a short reduction (6..16 K-blocks)
      // would otherwise spend a third of its time waiting for these dependent global loads.
      {
        // weight block scales of the tile's first 128 channels; the second set is gate_up's up rows, or the next 128 channels
        const float* ws0 = p.w_scale + (static_cast<size_t>(e) * (p.rows_per_expert >> 7) + (WIDE ? 2 * j : j)) * KB;
        const size_t second = static_cast<size_t>(GATE_UP ? IB : 1) * KB;
        const float* xs = p.x_scale + static_cast<size_t>(b) * KB * BM;  // [kb][n] of this block
        for (int base = et; base < BM * KB; base += kEpiThreads * kPreBatch) {
          float s[kPreBatch], w0[kPreBatch], w1[kPreBatch];
          const bool from_pre = have_pre && base == et;
#pragma unroll
          for (int u = 0; u < kPreBatch; ++u) {  // loads of a batch are issued together: one L2 round trip
            if (from_pre) {
              s[u] = pre_s[u], w0[u] = pre_w0[u], w1[u] = pre_w1[u];
            } else {
              const int i = base + u * kEpiThreads;
              const bool in = i < BM * KB;
              const int kb = in ? i / BM : 0;
              s[u] = in ? __ldg(xs + i) : 0.0f;
              w0[u] = __ldg(ws0 + kb);
              w1[u] = TWO ? __ldg(ws0 + second + kb) : 0.0f;
            }
          }
#pragma unroll
          for (int u = 0; u < kPreBatch; ++u) {
            const int i = base + u * kEpiThreads;
            if (i < BM * KB) {
              ftab[i] = s[u] * w0[u];
              if (TWO) ftab[BM * KB + i] = s[u] * w1[u];
            }
          }
        }
      }
      if (et < BM) {
        const int rid = have_pre ? pre_rid : p.sorted_ids[b * BM + et];
        rid_s[et] = rid;
        if (!GATE_UP) colscale[et] = have_pre ? pre_weight : (rid >= 0 ? p.topk_weights[rid] : 0.0f);
      }
      epi_bar_sync();
      {  // issue the next tile's loads; they land while this tile's K loop runs
        const int tn = t + gridDim.x;
        have_pre = kPrefetch && tn < total_tiles;
        if (have_pre) {
          const int bn = tn / tiles_per_block, jn = tn - bn * tiles_per_block;
          const int en = e_ahead;
          const float* ws0 = p.w_scale + (static_cast<size_t>(en) * (p.rows_per_expert >> 7) + (WIDE ? 2 * jn : jn)) * KB;
          const size_t second = static_cast<size_t>(GATE_UP ? IB : 1) * KB;
          const float* xs = p.x_scale + static_cast<size_t>(bn) * KB * BM;
#pragma unroll
          for (int u = 0; u < kPreBatch; ++u) {
            const int i = et + u * kEpiThreads;
            const bool in = i < BM * KB;
            const int kb = in ? i / BM : 0;
            pre_s[u] = in ? __ldg(xs + i) : 0.0f;
            pre_w0[u] = __ldg(ws0 + kb);
            pre_w1[u] = TWO ? __ldg(ws0 + second + kb) : 0.0f;
          }
          pre_rid = et < BM ? p.sorted_ids[bn * BM + et] : -1;
        }
        e_cur = e_ahead;
        const int t2 = tn + gridDim.x;
        e_ahead = t2 < total_tiles ? p.block_expert[t2 / tiles_per_block] : 0;
      }

      float acc[TILES][NH];
#pragma unroll
      for (int a = 0; a < TILES; ++a)
#pragma unroll
        for (int i = 0; i < NH; ++i) acc[a][i] = 0.0f;

      for (int kb = 0; kb < KB; ++kb, ++it) {
        const int buf = it & 1;
        bool got;
        got = mbar_wait(&empty[ring], ring_ph, abort_flag, p.status, 4);
        if (++ring == S) { ring = 0; ring_ph ^= 1; }
        if (!got) bad = true;
        tc_fence_after_sync();
        const float* fk = ftab + kb * BM + half * NH;
        const uint32_t t0 = tmem_base + lane_addr + buf * BUF_COLS + half * NH;
        // software pipeline: the load of chunk k+1 is in flight while chunk k is folded in
        uint32_t r[2][CH];
        if (CH == 16) AKLR_TMEM_LD_16(t0, r[0]); else AKLR_TMEM_LD_8(t0, r[0]);
#pragma unroll
        for (int k = 0; k < NC; ++k) {
          tc_wait_ld();
          if (k + 1 < NC) {
            const uint32_t at = t0 + ((k + 1) / CPT) * BM + ((k + 1) % CPT) * CH;
            if (CH == 16) AKLR_TMEM_LD_16(at, r[(k + 1) & 1]); else AKLR_TMEM_LD_8(at, r[(k + 1) & 1]);
          } else {  // everything is read: hand the buffer back to the MMA warp
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[buf]);
          }
          const int a = k / CPT, c = (k % CPT) * CH;
          const float* f = fk + a * (BM * KB) + c;
#pragma unroll
          for (int i = 0; i < CH; i += 4) {
            const float4 f4 = *reinterpret_cast<const float4*>(f + i);
            acc[a][c + i + 0] = fmaf(__uint_as_float(r[k & 1][i + 0]), f4.x, acc[a][c + i + 0]);
            acc[a][c + i + 1] = fmaf(__uint_as_float(r[k & 1][i + 1]), f4.y, acc[a][c + i + 1]);
            acc[a][c + i + 2] = fmaf(__uint_as_float(r[k & 1][i + 2]), f4.z, acc[a][c + i + 2]);
            acc[a][c + i + 3] = fmaf(__uint_as_float(r[k & 1][i + 3]), f4.w, acc[a][c + i + 3]);
          }
        }
      }

      // the next tile's route weights: their ids have arrived by now, and the epilogue below hides this load
      if (!GATE_UP && have_pre && et < BM) pre_weight = pre_rid >= 0 ? p.topk_weights[pre_rid] : 0.0f;
      epi_bar_sync();  // every warp is done with the scale table: the region becomes the out tile
      if (GATE_UP) {
        // h = silu(gate) * up, rounded to bf16; then 1 x 128 requant over this tile's 128 channels
#pragma unroll
        for (int i = 0; i < NH; ++i) {
          const float g = acc[0][i];
          const float h = __fdividef(g, 1.0f + __expf(-g)) * acc[TILES - 1][i];
          acc[0][i] = __bfloat162float(__float2bfloat16_rn(h));
          const float m = warp_max_nonneg(fabsf(acc[0][i]));
          if (lane == 0) wmax[quarter * BM + half * NH + i] = m;
        }
        epi_bar_sync();
        if (et < BM) {  // one thread per token column: its scale, stored for the down projection
          const float m = fmaxf(fmaxf(wmax[et], wmax[BM + et]), fmaxf(wmax[2 * BM + et], wmax[3 * BM + et]));
          const float scale = fmaxf(__fdiv_rn(m, 448.0f), FLT_MIN);
          colscale[et] = __fdiv_rn(1.0f, scale);
          if (rid_s[et] >= 0 && !bad) p.out_scale[(static_cast<size_t>(b) * IB + j) * BM + et] = scale;
        }
        epi_bar_sync();
#pragma unroll
        for (int i = 0; i < NH; ++i) {
          const int n = half * NH + i;
          out_tile[n * 128 + chan] = static_cast<uint8_t>(
              __nv_cvt_float_to_fp8(acc[0][i] * colscale[n], __NV_SATFINITE, __NV_E4M3));
        }
        epi_bar_sync();
        for (int i = et; i < BM * 8; i += kEpiThreads) {  // 16 bytes per thread, 8 per row
          const int n = i >> 3, seg = i & 7;
          if (rid_s[n] >= 0 && !bad)
            *reinterpret_cast<uint4*>(p.out_q + static_cast<size_t>(b * BM + n) * p.out_dim + j * 128 + seg * 16) =
                *reinterpret_cast<const uint4*>(out_tile + n * 128 + seg * 16);
        }
      } else {
        __nv_bfloat16* out16 = reinterpret_cast<__nv_bfloat16*>(out_tile);
#pragma unroll
        for (int a = 0; a < TILES; ++a) {  // one pass per 128 channels through the same staging tile
          if (a > 0) epi_bar_sync();       // the pass before has been written out
#pragma unroll
          for (int i = 0; i < NH; ++i) {
            const int n = half * NH + i;
            out16[n * 128 + chan] = __float2bfloat16_rn(acc[a][i] * colscale[n]);
          }
          epi_bar_sync();
          for (int i = et; i < BM * 16; i += kEpiThreads) {  // 16 bytes per thread, 16 per row
            const int n = i >> 4, seg = i & 15;
            const int rid = rid_s[n];
            if (rid >= 0 && !bad)
              *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.out_rows) +
                                        (static_cast<size_t>(rid) * p.out_dim + (j << kTileShift) + a * 128) * 2 + seg * 16) =
                  *reinterpret_cast<const uint4*>(out_tile + n * 256 + seg * 16);
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {  // a wait gave up: let copies in flight land before shared memory is released
    if (threadIdx.x == 0) publish_wait_failure(p.status, p.host_status);
    const uint64_t start = global_timer_ns();
    while (global_timer_ns() - start < 200000ull) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

bool pdl_enabled() {
  // On unless AKLR_PDL=0: a kernel's set-up, and the weight-major GEMM's first weight loads, overlap the tail of the
  // kernel before it (measured on B200 under CUDA-graph replay: one token 91.7 -> see the decode sweep).
  static const bool on = [] {
    const char* v = getenv("AKLR_PDL");
    return !(v && v[0] == '0');
  }();
  return on;
}

int ensure_max_dynamic_smem(const void* kernel) {
  static std::mutex lock;
  static std::map<std::pair<const void*, int>, bool> granted;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return AKLR_ERR_CUDA;
  std::lock_guard<std::mutex> guard(lock);
  bool& done = granted[{kernel, dev}];
  if (!done) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
      return AKLR_ERR_CUDA;
    done = true;
  }
  return AKLR_OK;
}

// The down projection of decode blocks (16 or 32 tokens) on 256-channel tiles: with 128-channel tiles a K-block hands
// over 16 KB of weights, and the hand-offs, not HBM, set its pace (4.2 TB/s at one token where gate_up, whose
// K-blocks carry 32 KB, reaches 5.8).
// Not when so few blocks are in play that 256-channel tiles would leave SMs without one (two experts of Mixtral's
// width at one token: 32 wide tiles for 148 SMs).
bool grouped_gemm_down_is_wide(int block_m, int out_dim, int max_blocks, int sm_count) {
  return (block_m == 16 || block_m == 32) && out_dim % 256 == 0 && static_cast<long long>(max_blocks) * (out_dim / 256) >= sm_count;
}

template <bool GATE_UP>
static int launch_grouped(const GroupedGemmParams& p, int sm_count, cudaStream_t stream) {
  if (p.k % 128 != 0 || p.out_dim % 128 != 0 || p.max_blocks < 1) return AKLR_ERR_UNSUPPORTED_SHAPE;
  if (p.stages < 2) return AKLR_ERR_UNSUPPORTED_SHAPE;
  const bool wide = !GATE_UP && p.wide != 0;
  if (wide && !((p.block_m == 16 || p.block_m == 32) && p.out_dim % 256 == 0)) return AKLR_ERR_UNSUPPORTED_SHAPE;
  const size_t smem = grouped_gemm_smem_bytes(GATE_UP, p.block_m, p.k, p.stages, wide);
  if (smem > 227 * 1024) return AKLR_ERR_UNSUPPORTED_SHAPE;
  const long long tiles = static_cast<long long>(p.max_blocks) * (p.out_dim / (wide ? 256 : 128));
  const int grid = static_cast<int>(tiles < sm_count ? tiles : sm_count);
  auto run = [&](auto kernel) {
    if (ensure_max_dynamic_smem(reinterpret_cast<const void*>(kernel)) != AKLR_OK) return AKLR_ERR_CUDA;
    return launch_kernel(kernel, dim3(grid), dim3(kGemmThreads), smem, stream, 1, p) == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
  };
  if constexpr (!GATE_UP) {
    if (wide) return p.block_m == 16 ? run(grouped_gemm_kernel<16, false, true>) : run(grouped_gemm_kernel<32, false, true>);
  }
  switch (p.block_m) {
    case 16: return run(grouped_gemm_kernel<16, GATE_UP>);
    case 32: return run(grouped_gemm_kernel<32, GATE_UP>);
    case 64: return run(grouped_gemm_kernel<64, GATE_UP>);
    case 128:
      // gate_up on 128-token blocks is always the token-major kernel's; a weight-major one would keep
      // 128 accumulators per thread and spill
      if constexpr (GATE_UP) return AKLR_ERR_UNSUPPORTED_SHAPE;
      else return run(grouped_gemm_kernel<128, false>);
    default: return AKLR_ERR_UNSUPPORTED_SHAPE;
  }
}


int launch_grouped_gemm_gate_up(const GroupedGemmParams& p, int sm_count, cudaStream_t stream) {
  return launch_grouped<true>(p, sm_count, stream);
}
int launch_grouped_gemm_down(const GroupedGemmParams& p, int sm_count, cudaStream_t stream) {
  return launch_grouped<false>(p, sm_count, stream);
}

}  // namespace aklr
