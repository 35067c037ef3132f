// Grouped GEMMs of the MXFP4-weight / MXFP8-activation MoE layer on tcgen05 block-scaled MMA
// (sm_100a): `tcgen05.mma.kind::mxf8f6f4.block_scale`, e4m3 activations x e2m1 weights, one ue8m0
// scale per 32 K elements on both operands, applied inside the tensor core.  Arithmetic of
// aklr/ops/fused_moe/reference.py:40-127 (act_quant 8) and aklr/ops/mega_moe/reference.py:18-48:
// gate_up -> (optional clamp) -> SiLU*mul -> bf16 round -> MXFP8 requant per 1 x 32 -> down -> route
// weight.
//
// Because the scales go through the MMA, a tile's whole K reduction accumulates in TMEM and is read
// out once -- there is no per-K-block fold as in the FP8 128x128 path.
//
// Token-major tiles (128 tokens = TMEM lanes, 256 weight rows = columns; gate rows j*128.. then up
// rows I + j*128.. for gate_up, 256 output channels for down).  Operands:
//   * activations: e4m3 rows, TMA SWIZZLE_128B, 128 K bytes per K-block;
//   * weights: packed e2m1 in HBM (64 bytes per 128 K elements), loaded by a TMA map of type
//     16U4_ALIGN16B, which unpacks them in shared memory to the padded 128-byte rows the mixed
//     f8f6f4 MMA reads -- HBM traffic is 4 bits per weight;
//   * scale factors: copied shared memory -> TMEM by tcgen05.cp (32x128b.warpx4) per K-block; a
//     32-bit TMEM column holds the 4 scale bytes of a row's four K=32 steps, rows r in lane r % 32,
//     column r / 32.  Activation scales are produced in that order by the quantising kernels; weight
//     scales stay row-major in HBM ([rows, K/32] bytes, as the checkpoint stores them) and two
//     staging warps re-order one 32-bit word per row per K-block into the stage.
//
// Warp roles (384 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..9 epilogue,
// warps 10..11 stage the scale factors ahead of the MMA warp (also across tile boundaries).  Persistent CTAs, bounded waits, no cluster,
// no multicast.
#include <cfloat>
#include <cuda_fp4.h>

#include "common.cuh"
#include "kernels.h"

namespace aklr {


namespace {

constexpr int kThreads = 384;            // TMA warp, MMA warp, 8 epilogue warps, 2 scale-staging warps
constexpr int kEpi = 256;
constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kABytes = kBM * 128;
constexpr int kBBytes = kBN * 128;          // unpacked: one byte per e2m1 element in shared memory
constexpr int kSfaBytes = 512;              // 128 rows x 4 K-steps
// One pipeline stage: [activations 16 KB][second activation term 16 KB, SPLIT only][weights 32 KB]
// [activation scales 512][weight scales 1024][second term's scales 512].
__host__ __device__ constexpr int stage_bytes(bool split) { return (split ? 2 : 1) * kABytes + kBBytes + 2048; }
__host__ __device__ constexpr int stage_b_offset(bool split) { return (split ? 2 : 1) * kABytes; }
constexpr int kSfLoOffset = kSfaBytes + 1024;  // the second term's activation scales inside the 2 KB scale area
constexpr int kSfaCol = 256, kSfbCol = 260, kSfaLoCol = 268;  // TMEM columns after the 256 accumulator columns

struct MxLayout {
  int off_out, off_rid, off_wgt, off_bars, total;
};

constexpr int kOutPassCols = 32;  // down: channels per thread staged per pass (64 bytes per row)

__host__ __device__ inline MxLayout mx_layout(int stages, bool gate_up, bool split) {
  MxLayout l;
  l.off_out = stages * stage_bytes(split);  // down: per epilogue warp 32 rows x 64 bytes of bf16 output
  l.off_rid = l.off_out + (gate_up ? 0 : (kEpi / 32) * 32 * kOutPassCols * 2);
  l.off_wgt = l.off_rid + kBM * 4;
  l.off_bars = l.off_wgt + kBM * 4;
  l.total = l.off_bars + (3 * stages + 2) * 8 + 16;
  return l;
}

__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ bool epi_any(int flag) {
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

// kind::mxf8f6f4 block-scaled instruction descriptor: A e4m3, B e2m1, both K-major, ue8m0 scales,
// M = 128; sf_id picks which byte of the 32-bit scale column this K=32 step uses.
__device__ __forceinline__ uint32_t mx_idesc(int n, int sf_id) {
  return (static_cast<uint32_t>(sf_id) << 4) | (0u << 7) | (5u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (1u << 23) | (static_cast<uint32_t>(128 >> 4) << 24) | (static_cast<uint32_t>(sf_id) << 29);
}

__device__ __forceinline__ void umma_mx(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}

// 32 rows x 16 bytes, rows contiguous: no swizzle, 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (8ull << 32) | (1ull << 46);
}
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Whether the producer loads row `row` of the sorted table when blocks with at most 32 / 64 routed rows load only
// those (a block's routed rows come first).
__device__ __forceinline__ bool row_in_small_box(const int32_t* sorted_ids, int row) {
  const int r = row & 127, b0 = row & ~127;
  if (r < 32) return true;
  if (sorted_ids[b0 + 32] < 0) return false;
  return r < 64 || sorted_ids[b0 + 64] >= 0;
}

// ue8m0 exponent of the smallest power of two >= amax / 448 (frexp rule of the reference's _mxfp8):
// returns the unbiased exponent in [-126, 127]; amax == 0 gives 0 (scale 1).
__device__ __forceinline__ int mxfp8_exponent(float amax) {
  if (amax == 0.0f) return 0;
  const uint32_t bits = __float_as_uint(__fdiv_rn(amax, 448.0f));
  int e = static_cast<int>(bits >> 23) - 127 + ((bits & 0x7FFFFFu) != 0u ? 1 : 0);
  return e < -126 ? -126 : (e > 127 ? 127 : e);
}

// MXFP4 activations (aklr/ops/fused_moe/reference.py:21-37): the exponent that puts the group's largest value
// in (3, 6] -- frexp(max(amax, 1e-10)) = (m, e), exponent e - 3 + (m > 0.75) -- clamped to [-127, 127].
__device__ __forceinline__ int mxfp4_exponent(float amax) {
  const uint32_t bits = __float_as_uint(fmaxf(amax, 1e-10f));
  const int e = static_cast<int>(bits >> 23) - 127 - 2 + ((bits & 0x7FFFFFu) > 0x400000u ? 1 : 0);
  return e < -127 ? -127 : (e > 127 ? 127 : e);
}
// Two values already divided by their group's scale -> the e4m3 bytes of their nearest e2m1 grid values
// (0, .5, 1, 1.5, 2, 3, 4, 6; exact ties to the even code, which is round-to-nearest-even in e2m1).
__device__ __forceinline__ uint16_t e2m1_grid_as_e4m3x2(float s0, float s1) {
  const __nv_fp4x2_storage_t q = __nv_cvt_float2_to_fp4x2(make_float2(s0, s1), __NV_E2M1, cudaRoundNearest);
  const __half2_raw back = __nv_cvt_fp4x2_to_halfraw2(q, __NV_E2M1);
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&back));
  return cvt_e4m3x2(f.x, f.y);
}

// Two values already divided by their group's scale -> their e4m3 codes and the codes of what the
// first rounding left over, times lo_mul (2^4 unless the second scale was clamped): hi + lo / lo_mul
// is the input exactly when it has 8 significant bits, as a bf16 value has.
__device__ __forceinline__ void e4m3x2_two_terms(float s0, float s1, float lo_mul, uint16_t& hi, uint16_t& lo) {
  hi = cvt_e4m3x2(s0, s1);
  const __half2_raw back = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(hi), __NV_E4M3);
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&back));
  lo = cvt_e4m3x2((s0 - f.x) * lo_mul, (s1 - f.y) * lo_mul);
}

// act(gate) * up for the activations of the reference's experts-only op other than SiLU
// (aklr/ops/fused_moe/reference.py:113-121).  Deliberately NOT inlined: the epilogue calls it from a
// loop unrolled 64 times, and with erff and tanhf expanded in every copy the loop grew to hundreds of
// KB of straight-line code that missed the instruction cache once per element (gate_up epilogue
// 6 k -> 77 k cycles per tile, the whole kernel 1.7x slower, SiLU included).
__device__ __noinline__ float gated_product_other(int activation, float gate, float up, float beta, float linear_beta) {
  switch (activation) {
    case AKLR_ACT_GELU:  // exact (erf) GELU
      return 0.5f * gate * (1.0f + erff(gate * 0.70710678118654752f)) * up;
    case AKLR_ACT_SWIGLU_OAI:  // gpt-oss: alpha 1.702, up biased by 1
      return __fdividef(gate, 1.0f + __expf(-1.702f * gate)) * (up + 1.0f);
    default:  // AKLR_ACT_SITUV2
      return beta * tanhf(__fdividef(gate, beta)) * __fdividef(1.0f, 1.0f + __expf(-gate)) *
             (linear_beta * tanhf(__fdividef(up, linear_beta)));
  }
}

// SPLIT: the activations are bf16 values carried as two e4m3 terms (MxQuantParams): per K step the
// MMA warp issues the product of each term with the SAME weight tile and weight scales into the same
// accumulator -- twice the tensor work of the MXFP8 path, no rounding of the activations.
template <bool GATE_UP, bool SPLIT>
__global__ void __launch_bounds__(kThreads, 1) grouped_gemm_mx_kernel(const __grid_constant__ MxGemmParams p) {
  constexpr int kStageBytes = stage_bytes(SPLIT);
  constexpr int kOffB = stage_b_offset(SPLIT);
  constexpr int kOffSf = kOffB + kBBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int KB = p.k >> 7;
  const int S = p.stages;
  const MxLayout L = mx_layout(S, GATE_UP, SPLIT);
  int* rid_s = reinterpret_cast<int*>(smem + L.off_rid);
  float* wgt_s = reinterpret_cast<float*>(smem + L.off_wgt);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.off_bars);
  uint64_t* empty = full + S;
  uint64_t* sf_full = empty + S;
  uint64_t* acc_full = sf_full + S;
  uint64_t* acc_empty = acc_full + 1;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(acc_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
      mbar_init(&sf_full[s], 1);  // the staging warp that owns the K-block
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, kEpi / 32);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&p.map_w);
    tma_prefetch_desc(&p.map_x);
    if (SPLIT) tma_prefetch_desc(&p.map_x_lo);
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, 512);
    tmem_relinquish();
  }
  // A block with few routed rows loads a 32- or 64-row box; the MMA still multiplies all 128 rows of the stage.
  // Start them as zeros: in a decode batch, where every block is such a block, they stay zero, and what the tensor
  // core draws -- and with it the clock the part holds -- depends on the operands.
  for (int s = 0; s < S; ++s)
    for (int i = threadIdx.x; i < kOffB / 16; i += kThreads)
      reinterpret_cast<uint4*>(smem + s * kStageBytes)[i] = make_uint4(0u, 0u, 0u, 0u);
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr;
  griddep_wait();  // everything below reads what earlier kernels of the call wrote
  griddep_launch();  // after the wait: a dependent that starts knows every kernel before this one is complete
  int nb = *p.num_blocks;
  if (nb > p.max_blocks) nb = p.max_blocks;
  const int tiles_per_block = GATE_UP ? (p.out_dim >> 7) : (p.out_dim >> 8);
  const int total_tiles = nb * tiles_per_block;

  if (warp == 0) {
    // ------------------------------- TMA producer ------------------------------------------
    if (lane == 0) {
      int s = 0;  // ring position and the parity of its current use
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int b = t / tiles_per_block, j = t - b * tiles_per_block;
        const int e = p.block_expert[b];
        const int w_row = e * p.rows_per_expert + (GATE_UP ? j * 128 : j * 256);
        // A decode batch leaves most of a 128-row block as padding (the sort puts the routed rows
        // first, -1 after them).  Loading all 128 activation rows per K-block made shared-memory
        // fill traffic from L2, not HBM, the bound (32 KB per K-block against 16 KB of weights): a
        // block with at most 32 or 64 routed rows loads only those.  The rows left stale feed TMEM
        // lanes whose results are never stored.
        const CUtensorMap* map_x = &p.map_x;
        uint32_t x_bytes = kABytes;
        if (!SPLIT && p.small_boxes) {
          const int id32 = p.sorted_ids[b * kBM + 32], id64 = p.sorted_ids[b * kBM + 64];
          if (id32 < 0) { map_x = &p.map_x_rows32; x_bytes = 32 * 128; }
          else if (id64 < 0) { map_x = &p.map_x_rows64; x_bytes = 64 * 128; }
        }
        for (int kb = 0; kb < KB; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 21)) { ok = false; break; }
          uint8_t* st = smem + s * kStageBytes;
          // the transaction count of the unpacking fp4 load is its packed size (what crosses from
          // global memory), not the padded bytes it writes: expecting the padded size never completes
          mbar_expect_tx(&full[s], (SPLIT ? 2 : 1) * x_bytes + kBBytes / 2);
          tma_load_2d(st, map_x, &full[s], kb * 128, b * kBM);
          if (SPLIT) tma_load_2d(st + kABytes, &p.map_x_lo, &full[s], kb * 128, b * kBM);
          if (GATE_UP) {
            tma_load_2d(st + kOffB, &p.map_w, &full[s], kb * 128, w_row);
            tma_load_2d(st + kOffB + kBBytes / 2, &p.map_w, &full[s], kb * 128, w_row + p.out_dim);
          } else {
            tma_load_2d(st + kOffB, &p.map_w, &full[s], kb * 128, w_row);
          }
          if (++s == S) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer --------------------------------------------
    if (lane == 0) {
      // A lone thread pays the full latency of every instruction: ring position, phase and the
      // five descriptors are carried forward, not recomputed.
      uint32_t it = 0, tile_no = 0;
      int s = 0;
      uint32_t ph = 0;
      const uint32_t base = smem_u32(smem);
      const uint64_t da0 = umma_desc_sw128(base), db0 = umma_desc_sw128(base + kOffB);
      const uint64_t sfa0 = sf_desc(base + kOffSf);
      uint32_t step = 0;  // (stage * kStageBytes) >> 4, added to the address field of each descriptor
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_no) {
        // the single accumulator must have been read out by the previous tile's epilogue
        bool got;
        got = mbar_wait(acc_empty, (tile_no & 1) ^ 1, abort_flag, p.status, 22);
        if (!got) break;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          got = mbar_wait(&full[s], ph, abort_flag, p.status, 23);
          if (!got) { ok = false; break; }
          got = mbar_wait(&sf_full[s], ph, abort_flag, p.status, 24);
          if (!got) { ok = false; break; }
          tc_fence_after_sync();
          const uint64_t sfa = sfa0 + step;
          tmem_cp_32x128b_warpx4(tmem_base + kSfaCol, sfa);
          tmem_cp_32x128b_warpx4(tmem_base + kSfbCol, sfa + (kSfaBytes >> 4));
          tmem_cp_32x128b_warpx4(tmem_base + kSfbCol + 4, sfa + ((kSfaBytes + 512) >> 4));
          if (SPLIT) tmem_cp_32x128b_warpx4(tmem_base + kSfaLoCol, sfa + (kSfLoOffset >> 4));
          const uint64_t da = da0 + step, db = db0 + step;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            umma_mx(tmem_base, da + 2 * k, db + 2 * k, mx_idesc(kBN, k), tmem_base + kSfaCol, tmem_base + kSfbCol,
                    (kb > 0 || k > 0) ? 1u : 0u);
            if (SPLIT)  // the second term: the next 16 KB of the stage, its own activation scales
              umma_mx(tmem_base, da + (kABytes >> 4) + 2 * k, db + 2 * k, mx_idesc(kBN, k), tmem_base + kSfaLoCol,
                      tmem_base + kSfbCol, 1u);
          }
          tc_commit(&empty[s]);
          step += kStageBytes >> 4;
          if (++s == S) { s = 0; ph ^= 1; step = 0; }
        }
        if (ok) tc_commit(acc_full);
      }
    }
  } else if (warp >= 10) {
    // ------------------- scale-factor staging, running ahead of the MMA warp -------------------
    // The two staging warps take alternate K-blocks, so each has two MMA periods per stage; a
    // lane moves 8 weight-row words (rows lane, lane+32, ...) and 16 bytes of activation scales.
    const int sw = warp - 10;
    const int KS = p.k >> 5;  // scale bytes per weight row
    uint32_t it0 = 0;         // K-blocks before this tile
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, it0 += KB) {
      const int b = t / tiles_per_block, j = t - b * tiles_per_block;
      const int e = p.block_expert[b];
      const uint8_t* wsf[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const int i = lane + q * 32;
        const int wrow = GATE_UP ? (i < 128 ? j * 128 + i : p.out_dim + j * 128 + (i - 128)) : j * 256 + i;
        wsf[q] = p.w_scale + (static_cast<size_t>(e) * p.rows_per_expert + wrow) * KS;
      }
      const uint8_t* xsf = p.x_scale + static_cast<size_t>(b) * KB * kSfaBytes;
      const uint8_t* xsf_lo = SPLIT ? p.x_scale_lo + static_cast<size_t>(b) * KB * kSfaBytes : nullptr;
      const int first = ((it0 & 1u) == static_cast<uint32_t>(sw)) ? 0 : 1;
      // ring of kDepth own K-blocks of scale words in registers: loaded long before their stage
      // frees up (down-projection rows are 64 bytes apart and miss to HBM on first touch)
      constexpr int kDepth = 3;
      uint32_t wq[kDepth][8];
      uint4 aq[kDepth], aq_lo[SPLIT ? kDepth : 1];
#pragma unroll
      for (int d = 0; d < kDepth; ++d) {
        const int kb = first + 2 * d;
#pragma unroll
        for (int q = 0; q < 8; ++q) wq[d][q] = kb < KB ? __ldg(reinterpret_cast<const uint32_t*>(wsf[q] + kb * 4)) : 0u;
        aq[d] = kb < KB ? __ldg(reinterpret_cast<const uint4*>(xsf + kb * kSfaBytes) + lane) : make_uint4(0, 0, 0, 0);
        if (SPLIT) aq_lo[d] = kb < KB ? __ldg(reinterpret_cast<const uint4*>(xsf_lo + kb * kSfaBytes) + lane) : make_uint4(0, 0, 0, 0);
      }
      for (int kb0 = first; kb0 < KB && ok; kb0 += 2 * kDepth) {
#pragma unroll
        for (int d = 0; d < kDepth; ++d) {
          const int kb = kb0 + 2 * d;
          if (kb < KB && ok) {
            const uint32_t it = it0 + kb;
            const int s = it % S;
            const uint32_t ph = (it / S) & 1;
            bool got;
            got = mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 25);
            if (!got) ok = false;
            uint8_t* sf = smem + s * kStageBytes + kOffSf;
            *reinterpret_cast<uint4*>(sf + lane * 16) = aq[d];
            if (SPLIT) *reinterpret_cast<uint4*>(sf + kSfLoOffset + lane * 16) = aq_lo[d];
#pragma unroll
            for (int q = 0; q < 8; ++q)  // row lane + 32 q -> 16-byte line `lane`, word q % 4, chunk q / 4
              *reinterpret_cast<uint32_t*>(sf + kSfaBytes + (q >> 2) * 512 + lane * 16 + (q & 3) * 4) = wq[d][q];
            fence_proxy_async_smem();  // tcgen05.cp reads these bytes through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(&sf_full[s]);
            const int nk = kb + 2 * kDepth;
            if (nk < KB) {
#pragma unroll
              for (int q = 0; q < 8; ++q) wq[d][q] = __ldg(reinterpret_cast<const uint32_t*>(wsf[q] + nk * 4));
              aq[d] = __ldg(reinterpret_cast<const uint4*>(xsf + nk * kSfaBytes) + lane);
              if (SPLIT) aq_lo[d] = __ldg(reinterpret_cast<const uint4*>(xsf_lo + nk * kSfaBytes) + lane);
            }
          }
        }
      }
    }
  } else {
    // ------------------------------------ epilogue warps ---------------------------------------
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int et = threadIdx.x - 64;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    uint32_t tile_no = 0;
    bool bad = false;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++tile_no) {
      if (epi_any(*abort_flag)) break;
      const int b = t / tiles_per_block, j = t - b * tiles_per_block;
      if (et < kBM) {
        const int rid = p.sorted_ids[b * kBM + et];
        rid_s[et] = rid;
        // down: the route weight, or 1 when the gate_up projection already carried it; gate_up: the
        // route weight when it is applied there (doweight_stage1), else 1
        const float* weights = GATE_UP ? p.stage1_weights : p.topk_weights;
        wgt_s[et] = rid < 0 ? 0.0f : (weights ? weights[rid] : 1.0f);
      }
      // gate_up: rows the down projection's producer will load (padding rows among them get zero codes)
      int box_rows = kBM;
      if (GATE_UP && !SPLIT && p.small_boxes) {
        if (p.sorted_ids[b * kBM + 32] < 0) box_rows = 32;
        else if (p.sorted_ids[b * kBM + 64] < 0) box_rows = 64;
      }
      epi_sync();  // the epilogue reads other threads' entries
      // ---- epilogue: the whole K reduction is in TMEM ----
      {
        bool got;
        got = mbar_wait(acc_full, tile_no & 1, abort_flag, p.status, 26);
        if (!got) bad = true;
      }
      tc_fence_after_sync();
      float acc[128];
      {
        // tcgen05.ld is latency-bound: all eight loads in flight, one wait, so that the accumulator
        // goes back to the MMA warp after one round trip
        uint32_t r[128];
        const uint32_t t0 = tmem_base + lane_addr + (GATE_UP ? half * 64 : half * 128);
#pragma unroll
        for (int c = 0; c < 128; c += 16) {
          const uint32_t at = GATE_UP ? (c < 64 ? t0 + c : t0 + 128 + (c - 64)) : t0 + c;
          AKLR_TMEM_LD_16(at, (r + c));
        }
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 128; ++i) acc[i] = __uint_as_float(r[i]);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);

      const int rid = rid_s[row];
      if (GATE_UP) {
        const int IB = p.out_dim >> 7;
        const float w1row = p.stage1_weights ? wgt_s[row] : 1.0f;  // exact when the weight is not applied here
        const bool silu = p.activation == AKLR_ACT_SILU;  // uniform over the grid
        // two 1 x 32 groups of this thread's 64 h channels
        uint32_t packed[16], packed_lo[SPLIT ? 16 : 1];
        uint32_t scale_bytes = 0, scale_bytes_lo = 0;
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          float m = 0.0f;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float gate = acc[g * 32 + i] * w1row, up = acc[64 + g * 32 + i] * w1row;
            if (p.swiglu_limit > 0.0f) {
              gate = fminf(gate, p.swiglu_limit);
              up = fminf(fmaxf(up, -p.swiglu_limit), p.swiglu_limit);
            }
            const float h = silu ? __fdividef(gate, 1.0f + __expf(-gate)) * up
                                 : gated_product_other(p.activation, gate, up, p.beta, p.linear_beta);
            acc[g * 32 + i] = __bfloat162float(__float2bfloat16_rn(h));
            m = fmaxf(m, fabsf(acc[g * 32 + i]));
          }
          const int ex = p.act_fp4 ? mxfp4_exponent(m) : mxfp8_exponent(m);
          const float inv = __uint_as_float(static_cast<uint32_t>(127 - ex) << 23);  // 2^-ex, exact
          scale_bytes |= static_cast<uint32_t>(ex + 127) << (8 * g);
          if (!SPLIT && p.act_fp4) {
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              packed[g * 8 + i / 4] = e2m1_grid_as_e4m3x2(acc[g * 32 + i] * inv, acc[g * 32 + i + 1] * inv) |
                                      (static_cast<uint32_t>(e2m1_grid_as_e4m3x2(acc[g * 32 + i + 2] * inv, acc[g * 32 + i + 3] * inv)) << 16);
          } else if (SPLIT) {
            // h stays the bf16 value it is: two e4m3 terms, the second at 2^(ex-4) (see MxQuantParams)
            const int ex_lo = ex - 4 < -127 ? -127 : ex - 4;
            const float lo_mul = __uint_as_float(static_cast<uint32_t>(127 + ex - ex_lo) << 23);
            scale_bytes_lo |= static_cast<uint32_t>(ex_lo + 127) << (8 * g);
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              uint16_t h0, l0, h1, l1;
              e4m3x2_two_terms(acc[g * 32 + i] * inv, acc[g * 32 + i + 1] * inv, lo_mul, h0, l0);
              e4m3x2_two_terms(acc[g * 32 + i + 2] * inv, acc[g * 32 + i + 3] * inv, lo_mul, h1, l1);
              packed[g * 8 + i / 4] = h0 | (static_cast<uint32_t>(h1) << 16);
              packed_lo[g * 8 + i / 4] = l0 | (static_cast<uint32_t>(l1) << 16);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              packed[g * 8 + i / 4] = cvt_e4m3x2(acc[g * 32 + i] * inv, acc[g * 32 + i + 1] * inv) |
                                      (static_cast<uint32_t>(cvt_e4m3x2(acc[g * 32 + i + 2] * inv, acc[g * 32 + i + 3] * inv)) << 16);
          }
        }
        if (rid < 0 && row < box_rows && !bad) {
          uint8_t* dst = p.out_q + static_cast<size_t>(b * kBM + row) * p.out_dim + j * 128 + half * 64;
#pragma unroll
          for (int v = 0; v < 4; ++v) *reinterpret_cast<uint4*>(dst + v * 16) = make_uint4(0u, 0u, 0u, 0u);
          if (SPLIT) {
            uint8_t* dst_lo = p.out_q_lo + static_cast<size_t>(b * kBM + row) * p.out_dim + j * 128 + half * 64;
#pragma unroll
            for (int v = 0; v < 4; ++v) *reinterpret_cast<uint4*>(dst_lo + v * 16) = make_uint4(0u, 0u, 0u, 0u);
          }
        }
        if (rid >= 0 && !bad) {
          uint8_t* dst = p.out_q + static_cast<size_t>(b * kBM + row) * p.out_dim + j * 128 + half * 64;
#pragma unroll
          for (int v = 0; v < 4; ++v)
            *reinterpret_cast<uint4*>(dst + v * 16) = make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
          // scale bytes in the order the down projection's tcgen05.cp wants them
          const size_t scale_at = (static_cast<size_t>(b) * IB + j) * kSfaBytes + (row & 31) * 16 + (row >> 5) * 4 + half * 2;
          *reinterpret_cast<uint16_t*>(p.out_scale + scale_at) = static_cast<uint16_t>(scale_bytes);
          if (SPLIT) {
            uint8_t* dst_lo = p.out_q_lo + static_cast<size_t>(b * kBM + row) * p.out_dim + j * 128 + half * 64;
#pragma unroll
            for (int v = 0; v < 4; ++v)
              *reinterpret_cast<uint4*>(dst_lo + v * 16) =
                  make_uint4(packed_lo[4 * v], packed_lo[4 * v + 1], packed_lo[4 * v + 2], packed_lo[4 * v + 3]);
            *reinterpret_cast<uint16_t*>(p.out_scale_lo + scale_at) = static_cast<uint16_t>(scale_bytes_lo);
          }
        }
      } else {
        // A thread owns 128 channels of one token: direct stores would be 16 bytes per lane at 32
        // different rows (half-filled sectors, one L1 wavefront per lane), and that store traffic
        // also delays the scale-staging warps, which share the load/store path.  Each warp stages
        // 32 rows x 32 channels in shared memory (16-byte chunks XOR-swizzled by row) and writes 64
        // contiguous bytes of 8 rows per instruction.
        const float w = wgt_s[row];
        uint8_t* stage = smem + L.off_out + (warp - 2) * (32 * kOutPassCols * 2);
#pragma unroll
        for (int pass = 0; pass < 128 / kOutPassCols; ++pass) {
#pragma unroll
          for (int v = 0; v < kOutPassCols / 8; ++v) {
            uint32_t o[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int i = pass * kOutPassCols + v * 8 + 2 * q;
              const __nv_bfloat162 two = __floats2bfloat162_rn(acc[i] * w, acc[i + 1] * w);
              o[q] = *reinterpret_cast<const uint32_t*>(&two);
            }
            *reinterpret_cast<uint4*>(stage + lane * (kOutPassCols * 2) + ((v ^ ((lane >> 1) & 3)) << 4)) =
                make_uint4(o[0], o[1], o[2], o[3]);
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int r = 8 * i + (lane >> 2), c = lane & 3;  // row of this warp's 32, 16-byte chunk
            const int rr = rid_s[quarter * 32 + r];
            const uint4 val = *reinterpret_cast<const uint4*>(stage + r * (kOutPassCols * 2) + ((c ^ ((r >> 1) & 3)) << 4));
            if (rr >= 0 && !bad)
              *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.out_rows) +
                                        (static_cast<size_t>(rr) * p.out_dim + j * 256 + half * 128 +
                                         pass * kOutPassCols + c * 8) * 2) = val;
          }
          __syncwarp();
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) publish_wait_failure(p.status, p.host_status);
    const uint64_t start = global_timer_ns();
    while (global_timer_ns() - start < 200000ull) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// Four lanes x 8 values per 1 x 32 group: rows
// gathered through the sorted route table, e4m3 codes row-major, scale bytes in tcgen05.cp order.
__global__ void __launch_bounds__(256) gather_quant_mxfp8_kernel(MxQuantParams p) {
  griddep_wait();
  griddep_launch();
  const int groups_per_row = p.hidden >> 5;
  const int n_rows = p.num_rows ? min(*p.num_rows, p.n_rows) : p.n_rows;
  const int64_t total = static_cast<int64_t>(n_rows) * groups_per_row;
  const int sub = threadIdx.x & 3;
  const uint32_t group_mask = 0xFu << (threadIdx.x & 28);
  const int64_t quads = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 2;
  const int KB = p.hidden >> 7;
  for (int64_t g = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 2; g < total; g += quads) {
    const int row = static_cast<int>(static_cast<uint32_t>(g) / static_cast<uint32_t>(groups_per_row));  // total < 2^31: checked at launch
    const int grp = static_cast<int>(static_cast<uint32_t>(g) - static_cast<uint32_t>(row) * static_cast<uint32_t>(groups_per_row));
    const int rid = p.sorted_ids ? p.sorted_ids[row] : row;  // no table: quantise the rows in place order
    if (rid < 0) {
      if (p.zero_padding == 1 || (p.zero_padding == 2 && row_in_small_box(p.sorted_ids, row))) {
        *reinterpret_cast<uint2*>(p.q + static_cast<size_t>(row) * p.hidden + grp * 32 + sub * 8) = make_uint2(0u, 0u);
        if (p.q_lo) *reinterpret_cast<uint2*>(p.q_lo + static_cast<size_t>(row) * p.hidden + grp * 32 + sub * 8) = make_uint2(0u, 0u);
      }
      continue;
    }
    const int token = rid / p.routes_per_token;
    if (p.q_in) {  // rows quantised by their sender: move codes and scale byte
      *reinterpret_cast<uint2*>(p.q + static_cast<size_t>(row) * p.hidden + grp * 32 + sub * 8) =
          *reinterpret_cast<const uint2*>(p.q_in + static_cast<size_t>(token) * p.hidden + grp * 32 + sub * 8);
      if (sub == 0) {
        const int b = row >> 7, r = row & 127, kb = grp >> 2, ks = grp & 3;
        p.scales[(static_cast<size_t>(b) * KB + kb) * kSfaBytes + (r & 31) * 16 + (r >> 5) * 4 + ks] =
            p.scales_in[static_cast<size_t>(token) * groups_per_row + grp];
      }
      continue;
    }
    const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.x) +
                                                      static_cast<size_t>(token) * p.hidden + grp * 32 + sub * 8);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    float v[8];
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
      m = fmaxf(m, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
    }
    m = fmaxf(m, __shfl_xor_sync(group_mask, m, 2, 4));
    m = fmaxf(m, __shfl_xor_sync(group_mask, m, 1, 4));
    const int ex = p.act_fp4 ? mxfp4_exponent(m) : mxfp8_exponent(m);
    const float inv = __uint_as_float(static_cast<uint32_t>(127 - ex) << 23);
    uint2 out;
    if (p.act_fp4) {
      out.x = e2m1_grid_as_e4m3x2(v[0] * inv, v[1] * inv) | (static_cast<uint32_t>(e2m1_grid_as_e4m3x2(v[2] * inv, v[3] * inv)) << 16);
      out.y = e2m1_grid_as_e4m3x2(v[4] * inv, v[5] * inv) | (static_cast<uint32_t>(e2m1_grid_as_e4m3x2(v[6] * inv, v[7] * inv)) << 16);
    } else if (p.q_lo) {  // the value itself, as two e4m3 terms
      const int ex_lo = ex - 4 < -127 ? -127 : ex - 4;
      const float lo_mul = __uint_as_float(static_cast<uint32_t>(127 + ex - ex_lo) << 23);
      uint16_t hi[4], lo[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) e4m3x2_two_terms(v[2 * i] * inv, v[2 * i + 1] * inv, lo_mul, hi[i], lo[i]);
      out.x = hi[0] | (static_cast<uint32_t>(hi[1]) << 16);
      out.y = hi[2] | (static_cast<uint32_t>(hi[3]) << 16);
      uint2 out_lo;
      out_lo.x = lo[0] | (static_cast<uint32_t>(lo[1]) << 16);
      out_lo.y = lo[2] | (static_cast<uint32_t>(lo[3]) << 16);
      *reinterpret_cast<uint2*>(p.q_lo + static_cast<size_t>(row) * p.hidden + grp * 32 + sub * 8) = out_lo;
      if (sub == 0) {
        const int b = row >> 7, r = row & 127, kb = grp >> 2, ks = grp & 3;
        p.scales_lo[(static_cast<size_t>(b) * KB + kb) * kSfaBytes + (r & 31) * 16 + (r >> 5) * 4 + ks] =
            static_cast<uint8_t>(ex_lo + 127);
      }
    } else {
      out.x = cvt_e4m3x2(v[0] * inv, v[1] * inv) | (static_cast<uint32_t>(cvt_e4m3x2(v[2] * inv, v[3] * inv)) << 16);
      out.y = cvt_e4m3x2(v[4] * inv, v[5] * inv) | (static_cast<uint32_t>(cvt_e4m3x2(v[6] * inv, v[7] * inv)) << 16);
    }
    *reinterpret_cast<uint2*>(p.q + static_cast<size_t>(row) * p.hidden + grp * 32 + sub * 8) = out;
    if (sub == 0) {
      if (p.row_major_scales) {  // for transport to another rank: [row, hidden/32]
        p.scales[static_cast<size_t>(row) * groups_per_row + grp] = static_cast<uint8_t>(ex + 127);
      } else {
        const int b = row >> 7, r = row & 127, kb = grp >> 2, ks = grp & 3;
        p.scales[(static_cast<size_t>(b) * KB + kb) * kSfaBytes + (r & 31) * 16 + (r >> 5) * 4 + ks] =
            static_cast<uint8_t>(ex + 127);
      }
    }
  }
}

// Rows quantised before (each token once, or by the sender of an expert-parallel dispatch): copy
// row rid's codes into the expert-sorted table and its scale bytes into tcgen05.cp order.  A CTA
// moves four rows at a time, every thread with four independent 16-byte loads in flight; a
// K-block's four scale bytes of a row move as one word.
constexpr int kGatherRows = 4;
__global__ void __launch_bounds__(256) gather_rows_mxfp8_kernel(MxQuantParams p) {
  __shared__ int src_s[kGatherRows];
  griddep_wait();
  griddep_launch();
  const int vec_per_row = p.hidden >> 4;
  const int KB = p.hidden >> 7;
  const size_t q_pitch = p.q_in_stride ? p.q_in_stride : p.hidden;
  const size_t s_pitch = p.scales_in_stride ? p.scales_in_stride : KB * 4;
  const int n_rows = p.num_rows ? min(*p.num_rows, p.n_rows) : p.n_rows;
  for (int row0 = blockIdx.x * kGatherRows; row0 < n_rows; row0 += gridDim.x * kGatherRows) {
    if (threadIdx.x < kGatherRows) {
      const int row = row0 + threadIdx.x;
      const int rid = row < n_rows ? p.sorted_ids[row] : -1;
      src_s[threadIdx.x] = rid < 0 ? -1 : rid / p.routes_per_token;
    }
    __syncthreads();
    int src[kGatherRows];
#pragma unroll
    for (int r = 0; r < kGatherRows; ++r) src[r] = src_s[r];
    bool zero[kGatherRows];  // a padding row that the GEMM's producer loads
#pragma unroll
    for (int r = 0; r < kGatherRows; ++r)
      zero[r] = src[r] < 0 && row0 + r < n_rows &&
                (p.zero_padding == 1 || (p.zero_padding == 2 && row_in_small_box(p.sorted_ids, row0 + r)));
    for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
      uint4 val[kGatherRows];
#pragma unroll
      for (int r = 0; r < kGatherRows; ++r) {
        val[r] = make_uint4(0u, 0u, 0u, 0u);
        if (src[r] >= 0)
          val[r] = __ldg(reinterpret_cast<const uint4*>(p.q_in + static_cast<size_t>(src[r]) * q_pitch) + v);
      }
#pragma unroll
      for (int r = 0; r < kGatherRows; ++r)
        if (src[r] >= 0 || zero[r]) reinterpret_cast<uint4*>(p.q + static_cast<size_t>(row0 + r) * p.hidden)[v] = val[r];
    }
    for (int i = threadIdx.x; i < kGatherRows * KB; i += blockDim.x) {
      const int r = i / KB, kb = i - r * KB;
      const int row = row0 + r;
      if (src_s[r] >= 0) {
        const uint32_t word = __ldg(reinterpret_cast<const uint32_t*>(p.scales_in + static_cast<size_t>(src_s[r]) * s_pitch) + kb);
        if (p.row_major_scales) {  // for transport to another rank: [row, hidden/32]
          *reinterpret_cast<uint32_t*>(p.scales + static_cast<size_t>(row) * (KB * 4) + kb * 4) = word;
        } else {
          const int b = row >> 7, rr = row & 127;
          *reinterpret_cast<uint32_t*>(p.scales + (static_cast<size_t>(b) * KB + kb) * kSfaBytes + (rr & 31) * 16 + (rr >> 5) * 4) = word;
        }
      }
    }
    __syncthreads();
  }
}

}  // namespace


int launch_gather_quant_mxfp8(const MxQuantParams& p, cudaStream_t stream) {
  if (p.hidden % 128 != 0) return AKLR_ERR_UNSUPPORTED_SHAPE;
  if ((p.q_lo != nullptr) != (p.scales_lo != nullptr) || (p.q_lo && (p.q_in || p.row_major_scales || p.act_fp4))) return AKLR_ERR_BAD_ARGUMENT;
  if (p.n_rows == 0) return AKLR_OK;
  if (p.q_in) {
    if (!p.sorted_ids || !p.scales_in) return AKLR_ERR_BAD_ARGUMENT;
    const int64_t blocks = (static_cast<int64_t>(p.n_rows) + kGatherRows - 1) / kGatherRows;
    const int grid = static_cast<int>(blocks < 148 * 32 ? blocks : 148 * 32);
    return launch_kernel(gather_rows_mxfp8_kernel, dim3(grid), dim3(256), 0, stream, 1, p) == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
  }
  const int64_t groups = static_cast<int64_t>(p.n_rows) * (p.hidden / 32);
  if (groups >= (int64_t{1} << 31)) return AKLR_ERR_TOO_LARGE;
  const int64_t blocks = (groups * 4 + 255) / 256;
  const int grid = static_cast<int>(blocks < 148 * 16 ? blocks : 148 * 16);
  return launch_kernel(gather_quant_mxfp8_kernel, dim3(grid), dim3(256), 0, stream, 1, p) == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

int grouped_gemm_mx_pick_stages(bool gate_up, bool split) {
  for (int s = 4; s >= 2; --s)
    if (mx_layout(s, gate_up, split).total + 1024 <= 227 * 1024) return s;
  return 0;
}

int launch_grouped_gemm_mx(const MxGemmParams& p, bool gate_up, int sm_count, cudaStream_t stream) {
  if (p.k % 128 != 0 || p.max_blocks < 1 || p.stages < 2) return AKLR_ERR_UNSUPPORTED_SHAPE;
  if (gate_up ? (p.out_dim % 128 != 0) : (p.out_dim % 256 != 0)) return AKLR_ERR_UNSUPPORTED_SHAPE;
  const bool split = p.split != 0;
  if (split && (!p.x_scale_lo || (gate_up && (!p.out_q_lo || !p.out_scale_lo)))) return AKLR_ERR_BAD_ARGUMENT;
  const size_t smem = static_cast<size_t>(mx_layout(p.stages, gate_up, split).total) + 1024;
  if (smem > 227 * 1024) return AKLR_ERR_UNSUPPORTED_SHAPE;
  const long long tiles = static_cast<long long>(p.max_blocks) * (gate_up ? p.out_dim / 128 : p.out_dim / 256);
  const int grid = static_cast<int>(tiles < sm_count ? tiles : sm_count);
  auto run = [&](auto kernel) {
    if (ensure_max_dynamic_smem(reinterpret_cast<const void*>(kernel)) != AKLR_OK) return AKLR_ERR_CUDA;
    return launch_kernel(kernel, dim3(grid), dim3(kThreads), smem, stream, 1, p) == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
  };
  if (split) return gate_up ? run(grouped_gemm_mx_kernel<true, true>) : run(grouped_gemm_mx_kernel<false, true>);
  return gate_up ? run(grouped_gemm_mx_kernel<true, false>) : run(grouped_gemm_mx_kernel<false, false>);
}

}  // namespace aklr
