// Token-major grouped FP8 GEMM for full 128-token blocks with FOUR partials in flight, sm_100a.
//
// Same arithmetic, element for element, as grouped_gemm_prefill.cu (128x128 weight block scales and
// 1x128 activation scales folded per K-block of 128 in float32, SiLU*mul + 1x128 requant after
// gate_up, route weight after down; aklr/plugins/sglang/models/deepseek_v2/reference.py:146-183).
// What differs is the pipeline between the tensor core and the CUDA cores that fold its partials.
//
// The 512 TMEM columns hold two N=256 partials, so with 128 x 256 tiles the MMA of K-block k+2 waits
// for the fold of k, the fold of k+1 for its MMA, and every edge of that cycle pays a wake-up: the
// measured period is ~1.6 x the MMA time.  Here a tile is 128 tokens x 128 weight rows: the same
// TMEM holds FOUR partials, the MMA runs up to three K-blocks ahead of the fold, and an epilogue
// thread's share of a partial (64 columns) fits in registers twice over next to its 64 accumulators --
// so a thread drains a whole partial in one round trip, frees its TMEM buffer at once, and folds it
// while the loads of the next partial are already in flight.
//
// gate_up: a unit is 128 intermediate channels of a block, worked as two sub-tiles of 64 gate + 64 up
// rows one after the other by the same CTA (the requant group is 128 channels: the first sub-tile's
// gated product waits in shared memory as bf16 until the second one's amax is known).
// down: a unit is 128 output channels.
//
// Outcome on B200 (DeepSeek-V3 widths, 4096 / 16384 tokens): bit-identical outputs, gate_up 2.8 / 8.3 ms against
// 2.0 / 5.9 ms of the two-buffer kernel.  Twice the K-blocks, each with the same fixed cost: the waits on
// free TMEM buffers are gone, the period per K-block is not.  It is therefore NOT the default; a call selects
// it with AKLR_VARIANT_DEEP_PIPELINE, and it stays in the test suite as the measurement of "more buffers".
//
// Warp roles (384 threads): warp 0 TMA producer, warps 1-2 MMA issuers taking K-blocks alternately (warp 1
// owns TMEM), warp 3 idle, warps 4-11 epilogue (TMEM lane quarter = warp % 4, column half = (warp-4)/4);
// setmaxnreg 40 / 232.  Persistent CTAs, TMA SWIZZLE_128B ring, no multicast loads, every wait bounded.
#include <cfloat>

#include "common.cuh"
#include "kernels.h"

namespace aklr {

namespace {

constexpr int kCS = 2;                    // column halves: epilogue warps = 4 lane quarters x kCS
constexpr int kEpiWarps = 4 * kCS;
constexpr int kEpi = 32 * kEpiWarps;
constexpr int kFirstEpiWarp = 4;          // warps 0..3: TMA producer, two MMA issuers, one idle (one warpgroup)
constexpr int kThreads = 32 * kFirstEpiWarp + kEpi;
constexpr int kRegsLean = 40, kRegsEpi = 232;
constexpr int kBM = 128;                  // tokens per block
constexpr int kBN = 128;                  // weight rows per (sub-)tile
constexpr int kABytes = kBM * 128;        // token tile of one K-block
constexpr int kBBytes = kBN * 128;        // weight tile of one K-block
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kBufs = 4;                  // TMEM partial buffers of kBN columns
constexpr int NH = kBN / kCS;             // accumulator columns per epilogue thread
constexpr int kMinStages = kBufs;         // the "stage free" barrier doubles as "partial complete": the ring must
                                          // not wrap before the fold has seen it (MMA runs <= kBufs ahead)

struct DeepLayout {
  int off_aux, off_rid, off_wmax, off_bars, total;
};

__host__ __device__ inline DeepLayout deep_layout(bool gate_up, int stages) {
  DeepLayout l;
  l.off_aux = stages * kStageBytes;
  // gate_up: the first sub-tile's 64 gated channels per token as bf16 (128 rows x 128 bytes);
  // down: per epilogue warp 32 rows x 64 channels of bf16 output (128 bytes per row)
  l.off_rid = l.off_aux + (gate_up ? kBM * 128 : kEpiWarps * 32 * NH * 2);
  l.off_wmax = l.off_rid + kBM * 4;
  l.off_bars = l.off_wmax + kCS * kBM * 4;
  l.total = l.off_bars + (2 * stages + kBufs + 2) * 8 + 16;
  return l;
}

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

template <int P>
struct Slot {
  static constexpr int value = P;
};

template <bool GATE_UP>
__global__ void __launch_bounds__(kThreads, 1) grouped_gemm_deep_kernel(const __grid_constant__ GroupedGemmParams p) {
  constexpr int kSub = GATE_UP ? 2 : 1;  // sub-tiles per unit

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int KB = p.k >> 7;
  const int S = p.stages;
  const DeepLayout L = deep_layout(GATE_UP, S);
  int* rid_s = reinterpret_cast<int*>(smem + L.off_rid);
  float* wmax = reinterpret_cast<float*>(smem + L.off_wmax);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.off_bars);
  uint64_t* empty = full + S;
  uint64_t* tmem_empty = empty + S;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(tmem_empty + kBufs);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int worker = static_cast<int>(blockIdx.x), n_workers = static_cast<int>(gridDim.x);

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < kBufs; ++i) mbar_init(&tmem_empty[i], kEpiWarps);
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
  griddep_wait();  // everything below reads what earlier kernels of the call wrote
  griddep_launch();  // after the wait: a dependent that starts knows every kernel before this one is complete
  int nb = p.num_blocks[0];
  if (nb > p.max_blocks) nb = p.max_blocks;
  const int tiles_per_block = p.out_dim >> 7;  // units of 128 channels
  const int total_tiles = nb * tiles_per_block;

  if (warp < kFirstEpiWarp) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsLean));
    if (warp == 0) {
      // ------------------------------- TMA producer ------------------------------------------
      if (lane == 0) {
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int t = worker; t < total_tiles && ok; t += n_workers) {
          const int b = t / tiles_per_block, j = t - b * tiles_per_block;
          const int e = p.block_expert[b];
          for (int half = 0; half < kSub && ok; ++half) {
            // gate_up: gate rows j*128 + half*64 .. +64 and the up rows that match; down: rows j*128 .. +128
            const int w_row = e * p.rows_per_expert + j * 128 + (GATE_UP ? half * 64 : 0);
            for (int kb = 0; kb < KB; ++kb) {
              if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 21)) { ok = false; break; }
              uint8_t* st = smem + s * kStageBytes;
              mbar_expect_tx(&full[s], kStageBytes);
              tma_load_2d(st, &p.map_x, &full[s], kb * 128, b * kBM);
              int wx, wy;
              weight_box(p.w_tiled != 0, KB, w_row, kb, &wx, &wy);
              tma_load_2d(st + kABytes, &p.map_w, &full[s], wx, wy);  // gate_up: a box of 64 rows; down: of 128
              if (GATE_UP) {  // the up rows that match: together one 128-row K-major operand
                weight_box(p.w_tiled != 0, KB, w_row + p.out_dim, kb, &wx, &wy);
                tma_load_2d(st + kABytes + kBBytes / 2, &p.map_w, &full[s], wx, wy);
              }
              if (++s == S) { s = 0; ph ^= 1; }
            }
          }
        }
      }
    } else if (warp <= 2) {
      // ------------------------------- MMA issuers (K-blocks taken alternately) --------------
      // tcgen05.mma holds its issuing thread until the tensor pipe takes the instruction: with two
      // threads one waits on its barriers while the other is held by its MMAs.
      if (lane == 0) {
        const uint32_t first = static_cast<uint32_t>(warp - 1);
        const int my_tiles = worker < total_tiles ? (total_tiles - worker + n_workers - 1) / n_workers : 0;
        const uint32_t n_it = static_cast<uint32_t>(my_tiles) * static_cast<uint32_t>(kSub * KB);
        int s = static_cast<int>(first);
        uint32_t ph = 0;
        const uint64_t desc0 = umma_desc_sw128(smem_u32(smem));
        for (uint32_t it = first; it < n_it; it += 2) {
          if (!mbar_wait(&full[s], ph, abort_flag, p.status, 22)) break;
          const uint32_t q = it & (kBufs - 1);
          if (!mbar_wait(&tmem_empty[q], ((it / kBufs) & 1u) ^ 1u, abort_flag, p.status, 23)) break;
          tc_fence_after_sync();
          const uint64_t da = desc0 + static_cast<uint64_t>(s) * (kStageBytes >> 4);
          const uint64_t db = da + (kABytes >> 4);
          const uint32_t d = tmem_base + q * kBN;
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f8f6f4(d, da + 2 * k, db + 2 * k, umma_idesc_e4m3(kBN), k > 0);
          tc_commit(&empty[s]);  // frees the stage and tells the epilogue the partial is complete
          s += 2;
          if (s >= S) { s -= S; ph ^= 1; }
        }
      }
    }
  } else {
    // ------------------------------- epilogue warps ----------------------------------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsEpi));
    const int quarter = warp & 3;
    const int cs = (warp - kFirstEpiWarp) >> 2;  // which column half this warp folds
    const int row = quarter * 32 + lane;         // token inside the block = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int IB = p.out_dim >> 7;
    uint32_t it = 0;       // K-blocks whose loads have been issued so far
    int ring = 0;          // stage whose "empty" barrier reports MMA(it) complete
    uint32_t ring_ph = 0;
    bool bad = false;
    uint8_t* stash = smem + L.off_aux + row * 128;  // gate_up: this token's 64 bf16 of the first sub-tile

    for (int t = worker; t < total_tiles; t += n_workers) {
      if (epi_any(*abort_flag)) break;
      const int b = t / tiles_per_block, j = t - b * tiles_per_block;
      const int e = p.block_expert[b];
      // 32-bit offsets into the scale arrays (both far below 2^31 floats): the pointers stay in the parameters
      const uint32_t xs = static_cast<uint32_t>(b) * KB * kBM + row;  // [K-block][token]
      const uint32_t ws_lo = (static_cast<uint32_t>(e) * (p.rows_per_expert >> 7) + j) * KB;
      const uint32_t ws_hi = GATE_UP ? ws_lo + static_cast<uint32_t>(IB) * KB : ws_lo;
      const int rid = __ldg(p.sorted_ids + b * kBM + row);
      float route_w = 0.0f;
      // (the barrier inside epi_any above also means the previous unit's output pass is done with rid_s / wmax)
      if (!GATE_UP && cs == 0) rid_s[row] = rid;
      float m_first = 0.0f;  // gate_up: amax of the first sub-tile's channels of this thread

#pragma unroll 1
      for (int half = 0; half < kSub; ++half) {
        float sx_q[3], wl_q[3], wh_q[3];  // K-blocks kb, kb+1, kb+2
        sx_q[1] = __ldg(p.x_scale + xs);
        wl_q[1] = __ldg(p.w_scale + ws_lo);
        wh_q[1] = GATE_UP ? __ldg(p.w_scale + ws_hi) : wl_q[1];
        sx_q[2] = KB > 1 ? __ldg(p.x_scale + xs + kBM) : 0.0f;
        wl_q[2] = KB > 1 ? __ldg(p.w_scale + ws_lo + 1) : 0.0f;
        wh_q[2] = GATE_UP ? (KB > 1 ? __ldg(p.w_scale + ws_hi + 1) : 0.0f) : wl_q[2];

        // gate_up: NH/2 gate channels half*64 + cs*32.., then the matching up channels; down: NH channels cs*64..
        uint64_t acc2[NH / 2];
#pragma unroll
        for (int i = 0; i < NH / 2; ++i) acc2[i] = 0ull;
        uint32_t stg[2][NH];  // two partials' worth of this thread's columns

        // the loads of K-block `it` into stg[slot]; waits for its MMA first when `blocking`
        auto fetch = [&](auto slot, bool blocking) -> bool {
          constexpr int W = decltype(slot)::value;
          if (blocking) {
            if (!mbar_wait(&empty[ring], ring_ph, abort_flag, p.status, 24)) bad = true;
          } else if (!__all_sync(0xFFFFFFFFu, mbar_test_wait(&empty[ring], ring_ph))) {
            return false;
          }
          if (++ring == S) { ring = 0; ring_ph ^= 1; }
          __syncwarp();
          tc_fence_after_sync();
          const uint32_t base = tmem_base + lane_addr + (it & (kBufs - 1)) * kBN;
          if (GATE_UP) {
            AKLR_TMEM_LD_16(base + cs * 32, (stg[W]));
            AKLR_TMEM_LD_16(base + cs * 32 + 16, (stg[W] + 16));
            AKLR_TMEM_LD_16(base + 64 + cs * 32, (stg[W] + 32));
            AKLR_TMEM_LD_16(base + 64 + cs * 32 + 16, (stg[W] + 48));
          } else {
#pragma unroll
            for (int c = 0; c < NH; c += 16) AKLR_TMEM_LD_16(base + cs * NH + c, (stg[W] + c));
          }
          ++it;
          return true;
        };
        // K-block kb, its loads already in flight into stg[slot]
        auto step = [&](auto slot, int kb) {
          constexpr int W = decltype(slot)::value;
          sx_q[0] = sx_q[1]; sx_q[1] = sx_q[2];
          wl_q[0] = wl_q[1]; wl_q[1] = wl_q[2];
          wh_q[0] = wh_q[1]; wh_q[1] = wh_q[2];
          if (kb + 2 < KB) {
            sx_q[2] = __ldg(p.x_scale + xs + (kb + 2) * kBM);
            wl_q[2] = __ldg(p.w_scale + ws_lo + kb + 2);
            wh_q[2] = GATE_UP ? __ldg(p.w_scale + ws_hi + kb + 2) : wl_q[2];
          }
          if (!GATE_UP && kb == (KB > 2 ? 2 : KB - 1)) route_w = rid >= 0 ? __ldg(p.topk_weights + rid) : 0.0f;
          const float f_lo = sx_q[0] * wl_q[0];
          const float f_hi = sx_q[0] * wh_q[0];
          const uint64_t f2_lo = pack_f32x2(__float_as_uint(f_lo), __float_as_uint(f_lo));
          const uint64_t f2_hi = pack_f32x2(__float_as_uint(f_hi), __float_as_uint(f_hi));
          tc_wait_ld();  // the whole partial is in registers: its TMEM buffer is free again
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty[(it - 1) & (kBufs - 1)]);
          const bool more = kb + 1 < KB;
          bool fetched = false;
          if (more) fetched = fetch(Slot<W ^ 1>{}, false);
#pragma unroll
          for (int i = 0; i < NH; i += 2) {
            const uint64_t f2 = (GATE_UP && i >= NH / 2) ? f2_hi : f2_lo;
            acc2[i / 2] = fma_f32x2(pack_f32x2(stg[W][i], stg[W][i + 1]), f2, acc2[i / 2]);
          }
          if (more && !fetched) fetch(Slot<W ^ 1>{}, true);
        };

        fetch(Slot<0>{}, true);
        for (int kb = 0; kb < KB; kb += 2) {
          step(Slot<0>{}, kb);
          if (kb + 1 < KB) step(Slot<1>{}, kb + 1);
          else break;
        }
        // an odd K-block count leaves the parity of the staging slots alone: every sub-tile starts in slot 0

        float acc[NH];
#pragma unroll
        for (int i = 0; i < NH / 2; ++i) {
          acc[2 * i] = lo_f32(acc2[i]);
          acc[2 * i + 1] = hi_f32(acc2[i]);
        }
        if (GATE_UP) {
          constexpr int HC = NH / 2;  // gated channels of this thread in this sub-tile
          float m = 0.0f;
#pragma unroll
          for (int i = 0; i < HC; ++i) {
            const float g = acc[i];
            const float h = __fdividef(g, 1.0f + __expf(-g)) * acc[HC + i];
            acc[i] = __bfloat162float(__float2bfloat16_rn(h));
            m = fmaxf(m, fabsf(acc[i]));
          }
          if (half == 0) {
            // park the bf16 values (this thread reads them back itself: 16-byte chunks XOR-swizzled by row)
            m_first = m;
#pragma unroll
            for (int v = 0; v < HC / 8; ++v) {
              uint32_t w[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const __nv_bfloat162 two = __floats2bfloat162_rn(acc[v * 8 + 2 * q], acc[v * 8 + 2 * q + 1]);
                w[q] = *reinterpret_cast<const uint32_t*>(&two);
              }
              *reinterpret_cast<uint4*>(stash + (((cs * (HC / 8) + v) ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          } else {
            m = fmaxf(m, m_first);
            wmax[cs * kBM + row] = m;
            epi_sync();
#pragma unroll
            for (int c = 0; c < kCS; ++c) m = fmaxf(m, wmax[c * kBM + row]);
            const float scale = fmaxf(__fdiv_rn(m, 448.0f), FLT_MIN);
            const float inv = __fdiv_rn(1.0f, scale);
            if (rid >= 0 && !bad) {
              if (cs == 0) p.out_scale[(static_cast<size_t>(b) * IB + j) * kBM + row] = scale;
              uint8_t* dst = p.out_q + static_cast<size_t>(b * kBM + row) * p.out_dim + j * 128 + cs * HC;
              // first sub-tile: channels cs*32 .. +32 from shared memory
#pragma unroll
              for (int v = 0; v < HC / 16; ++v) {
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                  const uint4 raw = *reinterpret_cast<const uint4*>(stash + (((cs * (HC / 8) + 2 * v + q) ^ (row & 7)) << 4));
                  const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
                  w[2 * q] = cvt_e4m3x2(__uint_as_float(rw[0] << 16) * inv, __uint_as_float(rw[0] & 0xFFFF0000u) * inv) |
                             (static_cast<uint32_t>(cvt_e4m3x2(__uint_as_float(rw[1] << 16) * inv, __uint_as_float(rw[1] & 0xFFFF0000u) * inv)) << 16);
                  w[2 * q + 1] = cvt_e4m3x2(__uint_as_float(rw[2] << 16) * inv, __uint_as_float(rw[2] & 0xFFFF0000u) * inv) |
                                 (static_cast<uint32_t>(cvt_e4m3x2(__uint_as_float(rw[3] << 16) * inv, __uint_as_float(rw[3] & 0xFFFF0000u) * inv)) << 16);
                }
                *reinterpret_cast<uint4*>(dst + v * 16) = make_uint4(w[0], w[1], w[2], w[3]);
              }
              // second sub-tile: channels 64 + cs*32 .. +32 from registers
#pragma unroll
              for (int v = 0; v < HC / 16; ++v) {
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const int i = v * 16 + q * 4;
                  w[q] = cvt_e4m3x2(acc[i] * inv, acc[i + 1] * inv) |
                         (static_cast<uint32_t>(cvt_e4m3x2(acc[i + 2] * inv, acc[i + 3] * inv)) << 16);
                }
                *reinterpret_cast<uint4*>(dst + 64 + v * 16) = make_uint4(w[0], w[1], w[2], w[3]);
              }
            }
          }
        } else {
          // Each warp stages its 32 rows x 64 channels in shared memory (16-byte chunks XOR-swizzled by
          // row) and writes 128 contiguous bytes of 4 rows per instruction.
          uint8_t* stage = smem + L.off_aux + (warp - kFirstEpiWarp) * (32 * NH * 2);
          epi_sync();  // rid_s of this unit is visible
#pragma unroll
          for (int v = 0; v < NH / 8; ++v) {
            uint32_t o[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int i = v * 8 + 2 * q;
              const __nv_bfloat162 two = __floats2bfloat162_rn(acc[i] * route_w, acc[i + 1] * route_w);
              o[q] = *reinterpret_cast<const uint32_t*>(&two);
            }
            *reinterpret_cast<uint4*>(stage + lane * (NH * 2) + ((v ^ (lane & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = 4 * i + (lane >> 3), c = lane & 7;  // row of this warp's 32, 16-byte chunk
            const int rr = rid_s[quarter * 32 + r];
            const uint4 val = *reinterpret_cast<const uint4*>(stage + r * (NH * 2) + ((c ^ (r & 7)) << 4));
            if (rr >= 0 && !bad)
              *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.out_rows) +
                                        (static_cast<size_t>(rr) * p.out_dim + j * 128 + cs * NH + c * 8) * 2) = val;
          }
          __syncwarp();
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
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace

int grouped_gemm_deep_pick_stages(bool gate_up) {
  for (int s = 8; s >= kMinStages; --s)
    if (deep_layout(gate_up, s).total + 1024 <= 227 * 1024) return s;
  return 0;
}

int launch_grouped_gemm_deep(const GroupedGemmParams& p, bool gate_up, int sm_count, cudaStream_t stream) {
  if (p.k % 128 != 0 || p.block_m != 128 || p.max_blocks < 1 || p.stages < kMinStages || p.out_dim % 128 != 0)
    return AKLR_ERR_UNSUPPORTED_SHAPE;
  const size_t smem = static_cast<size_t>(deep_layout(gate_up, p.stages).total) + 1024;
  if (smem > 227 * 1024) return AKLR_ERR_UNSUPPORTED_SHAPE;
  const long long tiles = static_cast<long long>(p.max_blocks) * (p.out_dim / 128);
  const int grid = static_cast<int>(tiles < sm_count ? tiles : sm_count);
  auto run = [&](auto kernel) {
    if (ensure_max_dynamic_smem(reinterpret_cast<const void*>(kernel)) != AKLR_OK) return AKLR_ERR_CUDA;
    return launch_kernel(kernel, dim3(grid), dim3(kThreads), smem, stream, 1, p) == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
  };
  return gate_up ? run(grouped_gemm_deep_kernel<true>) : run(grouped_gemm_deep_kernel<false>);
}

}  // namespace aklr
