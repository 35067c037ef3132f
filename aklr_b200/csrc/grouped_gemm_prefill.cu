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
// A token's 64 (gate_up) or 128 (down) channels sit in one thread.  gate_up writes them as 16-byte
// vectors of its own FP8 row; down stages bf16 rows in shared memory and writes 128 contiguous
// bytes of 4 rows per instruction (direct stores would be 32 half-filled sectors each).
//
// Warp roles (384 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2-3 idle,
// warps 4-11 epilogue (TMEM lane quarter = warp % 4, column split = (warp-4)/4).  The first
// warpgroup gives its registers to the epilogue (setmaxnreg 40 / 232): 128 accumulators + 64
// staging registers per epilogue thread do not fit the 168 an even split allows.
//
// What bounds it, measured on B200 piece by piece on all 148 SMs: the four MMAs of a K-block take 512 cycles
// with nothing else running (nominal) and 665-750 next to the fold; the fold alone 333-364 (8 tcgen05.ld x32
// per warp + 128 packed FMAs per thread); a TMA ring alone delivers 48 KB per ~520 cycles; the kernel's
// period is 1100-1450.  No piece explains it: the hand-offs of the MMA <-> fold cycle each arrive late (512
// TMEM columns hold exactly two N=256 partials, and a ring stage is held until the MMAs that read it are
// done).  What helped: one commit per K-block and a lean MMA-issue loop, scales prefetched from global
// memory two K-blocks ahead instead of staged per tile, register hand-over (setmaxnreg).  What did not: weight
// tiles prefetched into L2 ahead of the ring (+1-3% at 4096 tokens, -18% at 1024 where every tile's weights
// come from HBM), per-half hand-offs (two N=128 MMA groups; 20%
// slower), 128 x 128 tiles with four partials in flight (grouped_gemm_deep.cu; 40% slower), two MMA-issuing
// threads, one polling lane per warp, issuing the next K-block's first batch early, 16 epilogue warps,
// larger or single-buffered load batches, CTA pairs (below).  Persistent CTAs, TMA SWIZZLE_128B ring,
// two 256-column TMEM partial buffers, no multicast loads, bounded waits.
#include <cfloat>
#include <map>
#include <mutex>
#include <utility>

#include "common.cuh"
#include "kernels.h"

namespace aklr {

namespace {

constexpr int kCS = 2;                   // column splits: epilogue warps = 4 lane quarters x kCS
constexpr int kEpiWarps = 4 * kCS;
constexpr int kEpi = 32 * kEpiWarps;
constexpr int kFirstEpiWarp = 4;         // warps 0..3: TMA producer, MMA issuer, two idle (one warpgroup)
constexpr int kThreads = 32 * kFirstEpiWarp + kEpi;
constexpr int kRegsLean = 40, kRegsEpi = 232;  // setmaxnreg: 128*40 + 256*232 <= 64K registers
constexpr int kBM = 128;                 // tokens per block
constexpr int kBN = 256;                 // weight rows per tile
constexpr int kABytes = kBM * 128;       // token tile of one K-block
constexpr int kBBytes = kBN * 128;       // weight tile of one K-block
__host__ __device__ constexpr int stage_bytes(bool pair) { return kABytes + (pair ? kBBytes / 2 : kBBytes); }  // a CTA of a pair holds half the weight rows
constexpr int kBatch = 32;                // TMEM columns one epilogue thread loads per round (as 4 x 8)

struct PrefillLayout {
  int off_out, off_rid, off_wmax, off_bars, total;
};

constexpr int kOutPassCols = 64;  // down: channels per thread staged per pass (128 bytes per row)

__host__ __device__ inline PrefillLayout prefill_layout(bool gate_up, bool pair, int stages) {
  PrefillLayout l;
  l.off_out = stages * stage_bytes(pair);  // down: per epilogue warp 32 rows x 128 bytes of bf16 output
  l.off_rid = l.off_out + (gate_up ? 0 : kEpiWarps * 32 * kOutPassCols * 2);
  l.off_wmax = l.off_rid + kBM * 4;  // float[kCS][128] amax per column split (gate_up)
  l.off_bars = l.off_wmax + kCS * kBM * 4;
  l.total = l.off_bars + (2 * stages + 4) * 8 + 16;
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

// PAIR: two CTAs of a cluster work on two token blocks of ONE expert with one M=256 MMA
// (cta_group::2).  Each CTA loads its own 128 tokens and HALF of the tile's 256 weight rows (the
// tensor cores read the other half from the partner's shared memory), so a K-block costs 32 KB of
// L2 -> shared-memory traffic per CTA instead of 48 KB.  The even CTA issues the MMAs; TMA bytes of
// both CTAs are counted on its "full" barrier, its commit arrives on the "empty" barrier of both,
// and both CTAs' epilogue warps arrive on its "tmem_empty" barrier.  An expert's odd last block
// runs with the odd CTA repeating the same tokens and writing nothing.
template <bool GATE_UP, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1) grouped_gemm_prefill_kernel(const __grid_constant__ GroupedGemmParams p) {
  constexpr int NH = kBN / kCS;   // accumulator columns per epilogue thread
  constexpr int kStageBytes = stage_bytes(PAIR);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int KB = p.k >> 7;
  const int S = p.stages;
  const PrefillLayout L = prefill_layout(GATE_UP, PAIR, S);
  int* rid_s = reinterpret_cast<int*>(smem + L.off_rid);
  float* wmax = reinterpret_cast<float*>(smem + L.off_wmax);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.off_bars);
  uint64_t* empty = full + S;
  uint64_t* tmem_empty = empty + S;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;  // which CTA of the pair
  // tiles are dealt to CTAs (or CTA pairs) round-robin
  const int worker = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int n_workers = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  // unit u -> this CTA's token block and whether it is a real one
  auto block_of = [&](int u, bool* live) -> int {
    if (!PAIR) { *live = true; return u; }
    const uint32_t entry = static_cast<uint32_t>(p.pair_table[u]);
    const bool second = (entry >> 31) != 0;
    *live = rank == 0 || second;
    return static_cast<int>(entry & 0x7FFFFFFFu) + (second ? static_cast<int>(rank) : 0);
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) mbar_init(&tmem_empty[i], PAIR ? 2 * kEpiWarps : kEpiWarps);  // buffer = K-block parity
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&p.map_w);
    tma_prefetch_desc(&p.map_x);
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(tmem_ptr, 512);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_ptr, 512);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // the partner's barriers exist before anything arrives on them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr;
  griddep_wait();  // everything below reads what earlier kernels of the call wrote
  griddep_launch();  // after the wait: a dependent that starts knows every kernel before this one is complete
  int nb = PAIR ? p.num_blocks[2] : p.num_blocks[0];  // units: runs of <= 2 blocks, or blocks
  if (nb > p.max_blocks) nb = p.max_blocks;
  // gate_up: one tile per 128 intermediate channels (128 gate + 128 up rows); down: per 256 channels
  const int tiles_per_block = GATE_UP ? (p.out_dim >> 7) : (p.out_dim >> 8);
  const int total_tiles = nb * tiles_per_block;

  // The accumulators of a 128 x 256 tile are 128 registers per epilogue thread, and the loads that
  // drain TMEM want 64 more in flight: the producer warpgroup hands its registers over.
  if (warp < kFirstEpiWarp) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsLean));
  if (warp == 0) {
    // ------------------------------- TMA producer ------------------------------------------
    if (lane == 0) {
      int s = 0;        // ring position and the parity of its current use
      uint32_t ph = 0;
      bool ok = true;
      const uint32_t full0 = PAIR ? mapa_shared(smem_u32(full), 0) : 0u;  // the even CTA's "full" barriers
      for (int t = worker; t < total_tiles && ok; t += n_workers) {
        const int u = t / tiles_per_block, j = t - u * tiles_per_block;
        bool live;
        const int b = block_of(u, &live);
        const int e = p.block_expert[b];
        const int w_row = e * p.rows_per_expert + (GATE_UP ? j * 128 : j * 256);
        for (int kb = 0; kb < KB; ++kb) {
          if (!mbar_wait<PAIR>(&empty[s], ph ^ 1, abort_flag, p.status, 11)) { ok = false; break; }
          uint8_t* st = smem + s * kStageBytes;
          if (PAIR) {
            if (rank == 0) mbar_expect_tx(&full[s], 2 * kStageBytes);  // both CTAs' bytes
            const uint32_t bar = full0 + s * 8;
            tma_load_2d_pair(st, &p.map_x, bar, kb * 128, b * kBM);
            // even CTA: gate rows (down: first 128 channels); odd CTA: up rows (down: the next 128)
            tma_load_2d_pair(st + kABytes, &p.map_w, bar, kb * 128,
                             w_row + static_cast<int>(rank) * (GATE_UP ? p.out_dim : 128));
          } else {
            mbar_expect_tx(&full[s], kStageBytes);
            tma_load_2d(st, &p.map_x, &full[s], kb * 128, b * kBM);
            const bool tiled = p.w_tiled != 0;
            int wx, wy;
            if (GATE_UP || tiled) {
              // gate rows, then the matching up rows: one 256-row K-major operand (tile-contiguous weights: the
              // down projection's 256 rows are two tiles that do not follow one another in memory either)
              const int second = w_row + (GATE_UP ? p.out_dim : 128);
              weight_box(tiled, KB, w_row, kb, &wx, &wy);
              tma_load_2d(st + kABytes, &p.map_w, &full[s], wx, wy);
              weight_box(tiled, KB, second, kb, &wx, &wy);
              tma_load_2d(st + kABytes + kBBytes / 2, &p.map_w, &full[s], wx, wy);
            } else {
              tma_load_2d(st + kABytes, &p.map_w, &full[s], kb * 128, w_row);  // box of 256 rows
            }
          }
          if (++s == S) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer --------------------------------------------
    if (lane == 0 && rank == 0) {
      // This thread is alone in its warp, so every instruction here costs its full latency:
      // the loop carries ring positions and descriptors forward instead of recomputing them.
      uint32_t it = 0;
      int s = 0;
      uint32_t ph = 0, buf = 0, bph = 0;
      const uint64_t desc0 = umma_desc_sw128(smem_u32(smem));
      uint64_t da = desc0;  // descriptor of stage s' token tile; the weight tile follows it
      bool ok = true;
      for (int t = worker; t < total_tiles && ok; t += n_workers) {
        for (int kb = 0; kb < KB; ++kb, ++it) {
          bool got;
          got = mbar_wait<PAIR>(&full[s], ph, abort_flag, p.status, 12);
          if (!got) { ok = false; break; }
          // One N=256 MMA per 32 K bytes into this K-block's TMEM buffer and a single commit per
          // K-block: the barrier that frees the shared-memory stage also tells the epilogue that
          // the partial is complete.  (Two N=128 groups with their own hand-offs, so that the
          // epilogue could start on the first half earlier, measured 20% slower: every extra commit
          // and barrier round costs more than the overlap gains.)
          got = mbar_wait<PAIR>(&tmem_empty[buf], bph ^ 1, abort_flag, p.status, 13);
          if (!got) { ok = false; break; }
          tc_fence_after_sync();
          const uint64_t db = da + (kABytes >> 4);
          const uint32_t d = tmem_base + buf * 256;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (PAIR) umma_f8f6f4_pair(d, da + 2 * k, db + 2 * k, umma_idesc_e4m3(256, 256), k > 0);
            else umma_f8f6f4(d, da + 2 * k, db + 2 * k, umma_idesc_e4m3(256), k > 0);
          }
          if (PAIR) tc_commit_pair(&empty[s], 3);
          else tc_commit(&empty[s]);
          da += kStageBytes >> 4;
          if (++s == S) { s = 0; ph ^= 1; da = desc0; }
          bph ^= buf;
          buf ^= 1;
        }
      }
    }
  }
  } else {
    // ------------------------------- epilogue warps ----------------------------------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsEpi));
    const int quarter = warp & 3;
    const int cs = (warp - kFirstEpiWarp) >> 2;  // which column split this warp folds
    const int row = quarter * 32 + lane;  // token inside the block = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int IB = p.out_dim >> 7;
    uint32_t it = 0;
    int ring = 0;          // shared-memory stage whose "empty" barrier reports MMA(it) complete
    uint32_t ring_ph = 0;
    bool bad = false;
    const uint32_t tmem_empty0 = PAIR ? mapa_shared(smem_u32(tmem_empty), 0) : 0u;  // in the even CTA
    for (int t = worker; t < total_tiles; t += n_workers) {
      if (epi_any(*abort_flag)) break;
      const int u = t / tiles_per_block, j = t - u * tiles_per_block;
      bool live;  // false: the odd CTA of a pair whose expert has no second block
      const int b = block_of(u, &live);
      const int e = p.block_expert[b];
      // Scales come straight from global memory (L2 hits: the quantising kernel wrote them just
      // before), two K-blocks ahead of their use; nothing is staged per tile.
      const float* xs = p.x_scale + static_cast<size_t>(b) * KB * kBM + row;  // [K-block][token]
      const float* wsb = p.w_scale + static_cast<size_t>(e) * (p.rows_per_expert >> 7) * KB;
      const float* ws_lo = wsb + static_cast<size_t>(GATE_UP ? j : 2 * j + (cs * NH) / 128) * KB;
      const float* ws_hi = GATE_UP ? wsb + static_cast<size_t>(IB + j) * KB : ws_lo;
      float sx_q[3], wl_q[3], wh_q[3];  // K-blocks kb, kb+1, kb+2
      sx_q[1] = __ldg(xs);
      wl_q[1] = __ldg(ws_lo);
      wh_q[1] = GATE_UP ? __ldg(ws_hi) : wl_q[1];
      sx_q[2] = KB > 1 ? __ldg(xs + kBM) : 0.0f;
      wl_q[2] = KB > 1 ? __ldg(ws_lo + 1) : 0.0f;
      wh_q[2] = GATE_UP ? (KB > 1 ? __ldg(ws_hi + 1) : 0.0f) : wl_q[2];
      const int rid = live ? __ldg(p.sorted_ids + b * kBM + row) : -1;
      // A block's routed rows come first, so an expert's last block often leaves whole quarters of the tile as
      // padding: a warp without a routed row hands the partials back unread.
      const bool warp_has_rows = __any_sync(0xFFFFFFFFu, rid >= 0);
      float route_w = 0.0f;
      // (the barrier inside epi_any above also means the previous tile's output pass is done with rid_s)
      if (!GATE_UP && cs == 0) rid_s[row] = rid;

      // gate_up: first NH/2 accumulators gate channels cs*NH/2.., then the matching up channels
      // down:    NH output channels cs*NH..
      uint64_t acc2[NH / 2];  // pairs of float32 accumulators
#pragma unroll
      for (int i = 0; i < NH / 2; ++i) acc2[i] = 0ull;

      // gate_up: this warp's NH/2 gate columns (weight rows 0..127 of the tile), then the matching
      // up columns (rows 128..255).  down: NH channels, all inside one 128-row scale block.
      constexpr int GC = GATE_UP ? NH / 2 : NH;  // consecutive TMEM columns before a jump
      constexpr int NB = NH / kBatch;            // load batches per K-block
      // tcgen05.ld is latency-bound per warp and tcgen05.wait::ld waits for every load in flight,
      // so the pattern is: one batch (4 x 8 columns) in flight while the previous one is folded.
      // (Issuing the next K-block's first batch before the last fold of this one measured slower.)
      uint32_t r[2][kBatch];
      auto issue = [&](int buffer, int bi) {
        const uint32_t tcol = tmem_base + lane_addr + buffer * 256 + (GATE_UP ? cs * GC : cs * NH);
        const int c = bi * kBatch;
        const uint32_t col = GATE_UP ? tcol + (c / GC) * 128 + (c % GC) : tcol + c;
#pragma unroll
        for (int q = 0; q < kBatch / 8; ++q) AKLR_TMEM_LD_8(col + q * 8, (r[bi & 1] + q * 8));
      };

      for (int kb = 0; kb < KB; ++kb, ++it) {
        const int buf = it & 1;
        sx_q[0] = sx_q[1]; sx_q[1] = sx_q[2];
        wl_q[0] = wl_q[1]; wl_q[1] = wl_q[2];
        wh_q[0] = wh_q[1]; wh_q[1] = wh_q[2];
        if (kb + 2 < KB) {
          sx_q[2] = __ldg(xs + (kb + 2) * kBM);
          wl_q[2] = __ldg(ws_lo + kb + 2);
          wh_q[2] = GATE_UP ? __ldg(ws_hi + kb + 2) : wl_q[2];
        }
        if (!GATE_UP && kb == (KB > 2 ? 2 : KB - 1)) route_w = rid >= 0 ? __ldg(p.topk_weights + rid) : 0.0f;
        const float f_lo = sx_q[0] * wl_q[0];
        const float f_hi = sx_q[0] * wh_q[0];
        const uint64_t f2_lo = pack_f32x2(__float_as_uint(f_lo), __float_as_uint(f_lo));
        const uint64_t f2_hi = pack_f32x2(__float_as_uint(f_hi), __float_as_uint(f_hi));
        bool got;
        // MMA(it) complete = the "empty" barrier of its shared-memory stage completing phase it / S
        got = mbar_wait<PAIR>(&empty[ring], ring_ph, abort_flag, p.status, 14);
        if (++ring == S) { ring = 0; ring_ph ^= 1; }
        if (!got) bad = true;
        tc_fence_after_sync();
        if (!warp_has_rows) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if (PAIR) mbar_arrive_cluster(tmem_empty0 + buf * 8);
            else mbar_arrive(&tmem_empty[buf]);
          }
          continue;
        }
        issue(buf, 0);
#pragma unroll
        for (int bi = 0; bi < NB; ++bi) {
          tc_wait_ld();
          if (bi + 1 < NB) {
            issue(buf, bi + 1);
          } else {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
              if (PAIR) mbar_arrive_cluster(tmem_empty0 + buf * 8);
              else mbar_arrive(&tmem_empty[buf]);
            }
          }
          const uint64_t f2 = (bi * kBatch) / GC == 0 ? f2_lo : f2_hi;
#pragma unroll
          for (int i = 0; i < kBatch; i += 2) {
            const int at = (bi * kBatch + i) / 2;
            acc2[at] = fma_f32x2(pack_f32x2(r[bi & 1][i], r[bi & 1][i + 1]), f2, acc2[at]);
          }
        }
      }

      float acc[NH];
#pragma unroll
      for (int i = 0; i < NH / 2; ++i) {
        acc[2 * i] = lo_f32(acc2[i]);
        acc[2 * i + 1] = hi_f32(acc2[i]);
      }
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
        if (live && !bad) {
          // padding rows get zero codes: the down projection multiplies them too, and zero operands cost it least
          if (cs == 0 && rid >= 0) p.out_scale[(static_cast<size_t>(b) * IB + j) * kBM + row] = scale;
          uint8_t* dst = p.out_q + static_cast<size_t>(b * kBM + row) * p.out_dim + j * 128 + cs * HC;
#pragma unroll
          for (int v = 0; v < HC / 16; ++v) {
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int i = v * 16 + q * 4;
              w[q] = rid < 0 ? 0u
                             : cvt_e4m3x2(acc[i] * inv, acc[i + 1] * inv) |
                                   (static_cast<uint32_t>(cvt_e4m3x2(acc[i + 2] * inv, acc[i + 3] * inv)) << 16);
            }
            *reinterpret_cast<uint4*>(dst + v * 16) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      } else {
        // A thread owns 128 channels of one token, so direct stores would write 16 bytes per lane
        // at 32 different rows (half-filled sectors, one L1 wavefront per lane).  Each warp stages
        // its 32 rows x 64 channels in shared memory (16-byte chunks XOR-swizzled by row) and
        // writes 128 contiguous bytes of 4 rows per instruction instead.
        uint8_t* stage = smem + L.off_out + (warp - kFirstEpiWarp) * (32 * kOutPassCols * 2);
        epi_sync();  // rid_s of this tile is visible
#pragma unroll
        for (int pass = 0; pass < NH / kOutPassCols; ++pass) {
#pragma unroll
          for (int v = 0; v < kOutPassCols / 8; ++v) {
            uint32_t o[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int i = pass * kOutPassCols + v * 8 + 2 * q;
              const __nv_bfloat162 two = __floats2bfloat162_rn(acc[i] * route_w, acc[i + 1] * route_w);
              o[q] = *reinterpret_cast<const uint32_t*>(&two);
            }
            *reinterpret_cast<uint4*>(stage + lane * (kOutPassCols * 2) + ((v ^ (lane & 7)) << 4)) =
                make_uint4(o[0], o[1], o[2], o[3]);
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = 4 * i + (lane >> 3), c = lane & 7;  // row of this warp's 32, 16-byte chunk
            const int rr = rid_s[quarter * 32 + r];
            const uint4 val = *reinterpret_cast<const uint4*>(stage + r * (kOutPassCols * 2) + ((c ^ (r & 7)) << 4));
            if (rr >= 0 && !bad)
              *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.out_rows) +
                                        (static_cast<size_t>(rr) * p.out_dim + j * 256 + cs * NH +
                                         pass * kOutPassCols + c * 8) * 2) = val;
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
  if (PAIR) cluster_sync_all();  // the partner is done with this CTA's shared memory and barriers
  if (warp == 1) {
    tc_fence_after_sync();
    if (PAIR) tmem_dealloc_pair(tmem_base, 512);
    else tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace


bool grouped_gemm_is_token_major(bool gate_up, int block_m, int out_dim) {
  return block_m == 128 && (gate_up || out_dim % 256 == 0);
}

int grouped_gemm_prefill_pick_stages(bool gate_up, bool pair) {
  for (int s = 8; s >= 2; --s)
    if (prefill_layout(gate_up, pair, s).total + 1024 <= 227 * 1024) return s;
  return 0;
}

namespace {
// CTA pairs that can be resident at once (a pair needs two SMs of one cluster-capable group)
template <typename Kernel>
int max_active_pairs(Kernel kernel, size_t smem) {
  static std::mutex mu;
  static std::map<std::pair<const void*, int>, int> cache;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  std::lock_guard<std::mutex> lock(mu);
  const auto key = std::make_pair(reinterpret_cast<const void*>(kernel), dev);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(2, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) n = 0;
  cache[key] = n;
  return n;
}
}  // namespace

int launch_grouped_gemm_prefill(const GroupedGemmParams& p, bool gate_up, bool pair, int sm_count, cudaStream_t stream) {
  if (p.k % 128 != 0 || p.block_m != 128 || p.max_blocks < 1 || p.stages < 2) return AKLR_ERR_UNSUPPORTED_SHAPE;
  if (gate_up ? (p.out_dim % 128 != 0) : (p.out_dim % 256 != 0)) return AKLR_ERR_UNSUPPORTED_SHAPE;
  if (pair && !p.pair_table) return AKLR_ERR_BAD_ARGUMENT;
  const size_t smem = static_cast<size_t>(prefill_layout(gate_up, pair, p.stages).total) + 1024;
  if (smem > 227 * 1024) return AKLR_ERR_UNSUPPORTED_SHAPE;
  const long long tiles = static_cast<long long>(p.max_blocks) * (gate_up ? p.out_dim / 128 : p.out_dim / 256);
  auto run = [&](auto kernel) {
    if (ensure_max_dynamic_smem(reinterpret_cast<const void*>(kernel)) != AKLR_OK) return AKLR_ERR_CUDA;
    if (!pair) {
      const int grid = static_cast<int>(tiles < sm_count ? tiles : sm_count);
      return launch_kernel(kernel, dim3(grid), dim3(kThreads), smem, stream, 1, p) == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
    }
    int pairs = max_active_pairs(kernel, smem);
    if (pairs < 1) return AKLR_ERR_CUDA;
    if (pairs > sm_count / 2) pairs = sm_count / 2;
    if (tiles < pairs) pairs = static_cast<int>(tiles);
    return launch_kernel(kernel, dim3(2 * pairs), dim3(kThreads), smem, stream, 2, p) == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
  };
  if (pair) return gate_up ? run(grouped_gemm_prefill_kernel<true, true>) : run(grouped_gemm_prefill_kernel<false, true>);
  return gate_up ? run(grouped_gemm_prefill_kernel<true, false>) : run(grouped_gemm_prefill_kernel<false, false>);
}

}  // namespace aklr
