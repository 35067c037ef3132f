// Top-k routing and the moe_align token sort, sm_100a.
//
// Routing: each expert's ranking value becomes a 64-bit key (order-preserving image of the float in
// the high word, ~expert in the low word), so "greater key" means the larger value and, among
// equals, the lower expert id -- the order the reference's stable descending sort defines
// (aklr/plugins/sglang/models/deepseek_v2/reference.py:114-143,
//  aklr/plugins/sglang/models/qwen3_moe/reference.py:34-41, aklr/ops/topk/reference.py:17-35).
// Two kernels pick by those keys and give bit-identical tables: large batches take one warp per
// token (every pick a warp arg-max), batches up to 2048 tokens one CTA per token with one thread per
// expert that COUNTS the keys greater than its own (no chain of dependent reductions: ~3 us
// instead of ~15 us for a handful of tokens).  One to eight tokens run routing and sort as one CTA.
//
// Sort: a stable counting sort of routes (token*K + slot) by expert, each expert's run padded
// with -1 to a multiple of block_m, plus a block -> expert table.  The reference defines no order
// here (its kernels use atomics); this one is deterministic.
#include "common.cuh"
#include "kernels.h"

namespace aklr {

__device__ __forceinline__ uint32_t ordered_bits(float v) {
  v += 0.0f;  // -0 -> +0, so equal values have equal images
  const uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct Key {
  uint32_t hi, lo;
};
__device__ __forceinline__ bool key_greater(Key a, Key b) { return a.hi > b.hi || (a.hi == b.hi && a.lo > b.lo); }

// warp-wide max of 64-bit keys given as two words (all lanes take part)
__device__ __forceinline__ Key warp_max_key(Key k) {
  const uint32_t hi = __reduce_max_sync(0xFFFFFFFFu, k.hi);
  const uint32_t lo = __reduce_max_sync(0xFFFFFFFFu, k.hi == hi ? k.lo : 0u);
  return Key{hi, lo};
}

__device__ __forceinline__ float sigmoid_exact(float x) { return __fdiv_rn(1.0f, 1.0f + expf(-x)); }

// VPT: values per lane; expert e = i*32 + lane sits in register i.
template <int VPT>
__global__ void __launch_bounds__(256) route_kernel(RouteParams p) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  griddep_wait();
  griddep_launch();
  if (token >= p.n_tokens) return;
  const int E = p.n_routed;
  const int ktot = p.topk + p.n_shared;

  float score[VPT];   // what weighs the expert (softmax: the logit; sigmoid: the score)
  uint32_t rank[VPT]; // ordered image of what ranks it; 0 = not a candidate
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int e = i * 32 + lane;
    score[i] = 0.0f;
    rank[i] = 0u;
    if (e < E) {
      float logit;
      uint32_t bits16 = 0;
      if (p.logits_are_bf16) {
        bits16 = reinterpret_cast<const uint16_t*>(p.logits)[static_cast<size_t>(token) * E + e];
        logit = bf16_bits_to_float(bits16);
      } else {
        logit = reinterpret_cast<const float*>(p.logits)[static_cast<size_t>(token) * E + e];
      }
      if (p.scoring == AKLR_SCORING_SIGMOID) {
        const float s = (p.logits_are_bf16 && p.sigmoid_table) ? p.sigmoid_table[bits16] : sigmoid_exact(logit);
        float b = 0.0f;
        if (p.bias) b = p.bias_is_bf16 ? bf16_bits_to_float(reinterpret_cast<const uint16_t*>(p.bias)[e])
                                       : reinterpret_cast<const float*>(p.bias)[e];
        score[i] = s;
        rank[i] = ordered_bits(s + b);
      } else {
        score[i] = logit;
        rank[i] = ordered_bits(logit);
      }
    }
  }

  // ---- grouped routing: keep the topk_group groups whose two best biased scores sum highest ----
  if (p.num_expert_group > 1 && p.topk_group < p.num_expert_group) {
    const int G = p.num_expert_group;
    const int gs = E / G;
    int gid[VPT];  // group of each register's expert (one division each, not one per group and pass)
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int e = i * 32 + lane;
      gid[i] = e < E ? e / gs : -1;
    }
    float my_group_score = 0.0f;  // lane g holds group g's score
    for (int g = 0; g < G; ++g) {
      Key best{0u, 0u};
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int e = i * 32 + lane;
        const Key k{gid[i] == g ? rank[i] : 0u, ~static_cast<uint32_t>(e)};
        if (key_greater(k, best)) best = k;
      }
      const Key first = warp_max_key(best);
      Key second_local{0u, 0u};
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int e = i * 32 + lane;
        const Key k{gid[i] == g ? rank[i] : 0u, ~static_cast<uint32_t>(e)};
        const bool is_first = (k.hi == first.hi && k.lo == first.lo);
        if (!is_first && key_greater(k, second_local)) second_local = k;
      }
      const Key second = warp_max_key(second_local);
      // recover the floats from their ordered images
      auto value_of = [](uint32_t o) {
        const uint32_t u = (o & 0x80000000u) ? (o & 0x7FFFFFFFu) : ~o;
        return __uint_as_float(u);
      };
      const float sum = value_of(first.hi) + value_of(second.hi);
      if (lane == g) my_group_score = sum;
    }
    uint32_t kept_mask = 0u;
    Key gk{lane < G ? ordered_bits(my_group_score) : 0u, ~static_cast<uint32_t>(lane)};
    for (int j = 0; j < p.topk_group; ++j) {
      const Key top = warp_max_key(gk);
      const int g = static_cast<int>(~top.lo);
      kept_mask |= 1u << g;
      if (lane == g) gk.hi = 0u;
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i)
      if (gid[i] >= 0 && !((kept_mask >> gid[i]) & 1u)) rank[i] = 0u;
  }

  // ---- top-k by key; lane j keeps the j-th pick ----
  int my_id = -1;
  float my_score = 0.0f;
  for (int j = 0; j < p.topk; ++j) {
    Key best{0u, 0u};
    float best_score = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const Key k{rank[i], ~static_cast<uint32_t>(i * 32 + lane)};
      if (key_greater(k, best)) {
        best = k;
        best_score = score[i];
      }
    }
    const Key top = warp_max_key(best);
    const int e = static_cast<int>(~top.lo);
    const bool mine = (best.hi == top.hi && best.lo == top.lo);
    const float s = __shfl_sync(0xFFFFFFFFu, best_score, __ffs(__ballot_sync(0xFFFFFFFFu, mine)) - 1);
#pragma unroll
    for (int i = 0; i < VPT; ++i)
      if (mine && i * 32 + lane == e) rank[i] = 0u;
    if (lane == j) {
      my_id = e;
      my_score = s;
    }
  }

  // ---- weights ----
  float w = 0.0f;
  if (p.scoring == AKLR_SCORING_SIGMOID) {
    float total = 0.0f;
    for (int j = 0; j < p.topk; ++j) total += __shfl_sync(0xFFFFFFFFu, my_score, j);
    w = p.renormalize ? __fdiv_rn(my_score, total) : my_score;
    w *= p.routed_scaling_factor;
  } else {
    // softmax over the chosen logits (lane 0 holds the largest)
    const float top_logit = __shfl_sync(0xFFFFFFFFu, my_score, 0);
    const float ex = lane < p.topk ? expf(my_score - top_logit) : 0.0f;
    float total = 0.0f;
    for (int j = 0; j < p.topk; ++j) total += __shfl_sync(0xFFFFFFFFu, ex, j);
    w = __fdiv_rn(ex, total);
  }
  if (lane < p.topk) {
    p.topk_ids[static_cast<size_t>(token) * ktot + lane] = my_id;
    p.topk_weights[static_cast<size_t>(token) * ktot + lane] = w;
  } else if (lane < ktot) {  // shared experts: the slots after the routed ones, at weight 1
    p.topk_ids[static_cast<size_t>(token) * ktot + lane] = E + (lane - p.topk);
    p.topk_weights[static_cast<size_t>(token) * ktot + lane] = 1.0f;
  }
}

// ---------------------------------------------------------------------------------------------
// Routing by counting: one thread per expert, for small batches.  The warp-per-token kernel above
// walks ~2500 dependent instructions (every pick is a warp reduction); at a handful of tokens that
// chain IS the latency.  Here an expert's position in the order is the number of keys greater than
// its own, counted from shared memory with no cross-thread dependency, and keys are the same
// (value image, ~expert) pairs, so the picks, their order and the weights are bit-identical.
// Grouped routing counts inside the group first (the two best give the group score, the topk best
// are the only candidates that can be picked), ranks the groups the same way, then counts among the
// kept groups' candidates.
// ---------------------------------------------------------------------------------------------
template <int kExperts, int kCandidates>
struct RouteSharedT {
  unsigned long long key[kExperts];      // per expert
  unsigned long long cand[kCandidates];  // [group][topk]: candidates of the kept groups, 0 elsewhere
  unsigned long long gkey[32];    // per group
  float gtop[64];                 // [group][2]: its two best biased scores
  int kept[32];
  int sel_id[32];
  float sel_score[32];
};
using RouteShared = RouteSharedT<1024, 1024>;  // any shape launch_route accepts

__device__ __forceinline__ unsigned long long route_key(uint32_t image, int index) {
  return (static_cast<unsigned long long>(image) << 32) | static_cast<uint32_t>(~index);
}

__device__ __forceinline__ float value_of_image(uint32_t o) {
  const uint32_t u = (o & 0x80000000u) ? (o & 0x7FFFFFFFu) : ~o;
  return __uint_as_float(u);
}

// Thread e's expert of ``token``: what weighs it (``s``) and the image of what ranks it.  Split from
// the counting so that a CTA routing several tokens has all their loads in flight at once.
__device__ __forceinline__ void route_load(const RouteParams& p, int token, int e, float& s, uint32_t& image) {
  const int E = p.n_routed;
  s = 0.0f;
  image = 0u;
  if (e < E) {
    float logit;
    uint32_t bits16 = 0;
    if (p.logits_are_bf16) {
      bits16 = reinterpret_cast<const uint16_t*>(p.logits)[static_cast<size_t>(token) * E + e];
      logit = bf16_bits_to_float(bits16);
    } else {
      logit = reinterpret_cast<const float*>(p.logits)[static_cast<size_t>(token) * E + e];
    }
    if (p.scoring == AKLR_SCORING_SIGMOID) {
      s = (p.logits_are_bf16 && p.sigmoid_table) ? p.sigmoid_table[bits16] : sigmoid_exact(logit);
      float b = 0.0f;
      if (p.bias) b = p.bias_is_bf16 ? bf16_bits_to_float(reinterpret_cast<const uint16_t*>(p.bias)[e])
                                     : reinterpret_cast<const float*>(p.bias)[e];
      image = ordered_bits(s + b);
    } else {
      s = logit;
      image = ordered_bits(logit);
    }
  }
}

// A team of ``team`` threads (a multiple of 32, at least max(n_routed, 32)) routes one token: thread
// ``e`` of the team owns expert e, threads past n_routed only keep the barriers.  ``barrier`` 0 is
// the CTA's (the team is the CTA); teams sharing a CTA each pass their own named barrier 1..15.
__device__ __forceinline__ void team_sync(int barrier, int team) {
  if (barrier == 0) __syncthreads();
  else asm volatile("bar.sync %0, %1;" ::"r"(barrier), "r"(team) : "memory");
}

template <class Shared>
__device__ void route_by_counting(const RouteParams& p, int token, int e, int team, int barrier, float s, uint32_t image,
                                  Shared& sh) {
  const int E = p.n_routed;
  const bool has = e < E;
  const unsigned long long key = has ? route_key(image, e) : 0ull;
  const bool grouped = p.num_expert_group > 1 && p.topk_group < p.num_expert_group;
  const int G = grouped ? p.num_expert_group : 1;
  const int gs = E / G;
  sh.key[e] = key;
  for (int i = e; i < G * p.topk; i += team) sh.cand[i] = 0ull;
  team_sync(barrier, team);
  int g = 0, rank = 0;  // the expert's group and its position inside it
  if (has) {
    g = e / gs;
    const unsigned long long* mine = sh.key + g * gs;
    for (int i = 0; i < gs; ++i) rank += mine[i] > key;
  }
  int final_rank = rank;
  if (grouped) {
    if (has && rank < 2) sh.gtop[g * 2 + rank] = value_of_image(image);
    team_sync(barrier, team);
    if (e < G) sh.gkey[e] = route_key(ordered_bits(sh.gtop[2 * e] + sh.gtop[2 * e + 1]), e);
    team_sync(barrier, team);
    if (e < G) {
      int ahead = 0;
      for (int i = 0; i < G; ++i) ahead += sh.gkey[i] > sh.gkey[e];
      sh.kept[e] = ahead < p.topk_group;
    }
    team_sync(barrier, team);
    const bool candidate = has && rank < p.topk && sh.kept[g];
    if (candidate) sh.cand[g * p.topk + rank] = key;
    team_sync(barrier, team);
    final_rank = p.topk;  // not picked
    if (candidate) {
      final_rank = 0;
      for (int i = 0; i < G * p.topk; ++i) final_rank += sh.cand[i] > key;
    }
  }
  if (has && final_rank < p.topk) {
    sh.sel_id[final_rank] = e;
    sh.sel_score[final_rank] = s;
  }
  team_sync(barrier, team);
  const int ktot = p.topk + p.n_shared;
  if (e < p.topk) {
    const float my_score = sh.sel_score[e];
    float w;
    if (p.scoring == AKLR_SCORING_SIGMOID) {
      float total = 0.0f;
      for (int j = 0; j < p.topk; ++j) total += sh.sel_score[j];
      w = p.renormalize ? __fdiv_rn(my_score, total) : my_score;
      w *= p.routed_scaling_factor;
    } else {  // softmax over the chosen logits (slot 0 holds the largest)
      const float top_logit = sh.sel_score[0];
      float total = 0.0f;
      for (int j = 0; j < p.topk; ++j) total += expf(sh.sel_score[j] - top_logit);
      w = __fdiv_rn(expf(my_score - top_logit), total);
    }
    p.topk_ids[static_cast<size_t>(token) * ktot + e] = sh.sel_id[e];
    p.topk_weights[static_cast<size_t>(token) * ktot + e] = w;
  } else if (e < ktot) {  // shared experts: the slots after the routed ones, at weight 1
    p.topk_ids[static_cast<size_t>(token) * ktot + e] = E + (e - p.topk);
    p.topk_weights[static_cast<size_t>(token) * ktot + e] = 1.0f;
  }
  team_sync(barrier, team);  // the next token reuses the shared arrays
}

__global__ void __launch_bounds__(1024) route_count_kernel(RouteParams p) {
  __shared__ RouteShared sh;
  griddep_wait();
  griddep_launch();
  float s;
  uint32_t image;
  route_load(p, blockIdx.x, threadIdx.x, s, image);
  route_by_counting(p, blockIdx.x, threadIdx.x, blockDim.x, 0, s, image, sh);
}

// Batches up to this many tokens are routed by counting (one CTA per token).
constexpr int kCountingRouteTokens = 2048;

static int check_route_shape(const RouteParams& p) {
  if (p.n_routed < 1 || p.n_routed > 1024 || p.topk < 1 || p.topk + p.n_shared > 32 || p.topk > p.n_routed)
    return AKLR_ERR_UNSUPPORTED_SHAPE;
  if (p.num_expert_group > 1) {
    if (p.num_expert_group > 32 || p.n_routed % p.num_expert_group != 0 || p.topk_group > p.num_expert_group ||
        p.topk_group < 1 || p.topk > p.topk_group * (p.n_routed / p.num_expert_group))
      return AKLR_ERR_UNSUPPORTED_SHAPE;
    // a group's score is the sum of its two best experts; when every group is kept the kernels
    // never form it, so single-expert groups are fine there
    if (p.topk_group < p.num_expert_group && p.n_routed / p.num_expert_group < 2) return AKLR_ERR_UNSUPPORTED_SHAPE;
  }
  return AKLR_OK;
}

int launch_route(const RouteParams& p, cudaStream_t stream) {
  if (p.n_tokens == 0) return AKLR_OK;
  if (int rc = check_route_shape(p)) return rc;
  if (p.n_tokens <= kCountingRouteTokens) {
    const int per_token = p.n_routed < 32 ? 32 : (p.n_routed + 31) & ~31;
    return launch_kernel(route_count_kernel, dim3(p.n_tokens), dim3(per_token), 0, stream, 1, p) == cudaSuccess
               ? AKLR_OK : AKLR_ERR_CUDA;
  }
  const int threads = 256, warps = threads / 32;
  const int blocks = (p.n_tokens + warps - 1) / warps;
  const int vpt = (p.n_routed + 31) / 32;
  cudaError_t err = cudaSuccess;
  if (vpt <= 1) err = launch_kernel(route_kernel<1>, dim3(blocks), dim3(threads), 0, stream, 1, p);
  else if (vpt <= 2) err = launch_kernel(route_kernel<2>, dim3(blocks), dim3(threads), 0, stream, 1, p);
  else if (vpt <= 4) err = launch_kernel(route_kernel<4>, dim3(blocks), dim3(threads), 0, stream, 1, p);
  else if (vpt <= 8) err = launch_kernel(route_kernel<8>, dim3(blocks), dim3(threads), 0, stream, 1, p);
  else if (vpt <= 16) err = launch_kernel(route_kernel<16>, dim3(blocks), dim3(threads), 0, stream, 1, p);
  else err = launch_kernel(route_kernel<32>, dim3(blocks), dim3(threads), 0, stream, 1, p);
  return err == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

// =============================================================================================
// moe_align: stable counting sort of routes by expert with per-expert padding
// =============================================================================================
constexpr int kSortChunk = 1024;  // routes per CTA, one per thread

__device__ __forceinline__ int local_expert(const AlignParams& p, int route) {
  int e = p.topk_ids[route];
  if (e < 0 || e >= p.n_experts_global) return -1;
  // rows a rank did not receive (aklr/ops/fused_moe/reference.py:85-86)
  if (p.num_local_tokens && route / p.routes_per_token >= __ldg(p.num_local_tokens)) return -1;
  if (p.expert_map) e = p.expert_map[e];
  return (e >= 0 && e < p.n_experts) ? e : -1;
}

// Pass 1: histogram of each 1024-route chunk -> chunk_hist[chunk][expert]
__global__ void __launch_bounds__(kSortChunk) align_count_kernel(AlignParams p) {
  extern __shared__ int hist[];
  griddep_wait();
  griddep_launch();
  for (int e = threadIdx.x; e < p.n_experts; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int route = blockIdx.x * kSortChunk + threadIdx.x;
  if (route < p.n_routes) {
    const int e = local_expert(p, route);
    if (e >= 0) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < p.n_experts; e += blockDim.x)
    p.chunk_hist[static_cast<size_t>(blockIdx.x) * p.n_experts + e] = hist[e];
}

// Exclusive prefix sum of one value per thread over the CTA (blockDim.x a multiple of 32, <= 1024):
// warp shuffles, then the warp totals by warp 0.  ``scratch`` holds >= 33 ints.  Two barriers.
__device__ int block_exclusive_scan(int v, int* scratch, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  int inc = v;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int u = __shfl_up_sync(0xFFFFFFFFu, inc, off);
    if (lane >= off) inc += u;
  }
  __syncthreads();  // earlier readers of scratch are done
  if (lane == 31) scratch[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = lane < n_warps ? scratch[lane] : 0;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int u = __shfl_up_sync(0xFFFFFFFFu, w, off);
      if (lane >= off) w += u;
    }
    scratch[lane] = w;  // inclusive totals of warps 0..lane
    if (lane == 31) scratch[32] = w;
  }
  __syncthreads();
  *total = scratch[32];
  return inc - v + (warp > 0 ? scratch[warp - 1] : 0);
}

// Shared by the scan kernel and the one-CTA path: from per-expert totals in smem ``total`` compute
// padded bases, the block table, counts, the pad fill.  ``base`` receives each expert's first row.
__device__ void plan_blocks(const AlignParams& p, const int* total, int* base, int* scratch) {
  // serial-in-chunks exclusive scan over experts of padded block counts (n_experts <= 1025)
  const int tid = threadIdx.x, nt = blockDim.x;
  const int per = (p.n_experts + nt - 1) / nt;
  int local_sum = 0;
  for (int i = 0; i < per; ++i) {
    const int e = tid * per + i;
    if (e < p.n_experts) local_sum += (total[e] + p.block_m - 1) / p.block_m;
  }
  int all_blocks;
  int running = block_exclusive_scan(local_sum, scratch, &all_blocks);  // blocks before this thread's experts
  if (tid == nt - 1) {
    p.num_blocks[0] = all_blocks;
    p.num_blocks[1] = all_blocks * p.block_m;
  }
  int pair_running = 0;  // runs of <= 2 blocks before this thread's experts
  if (p.pair_table) {
    __syncthreads();
    int local_pairs = 0;
    for (int i = 0; i < per; ++i) {
      const int e = tid * per + i;
      if (e < p.n_experts) local_pairs += ((total[e] + p.block_m - 1) / p.block_m + 1) / 2;
    }
    int all_pairs;
    pair_running = block_exclusive_scan(local_pairs, scratch, &all_pairs);
    if (tid == nt - 1) p.num_blocks[2] = all_pairs;
  }
  for (int i = 0; i < per; ++i) {
    const int e = tid * per + i;
    if (e < p.n_experts) {
      const int c = total[e];
      const int nb = (c + p.block_m - 1) / p.block_m;
      base[e] = running * p.block_m;
      p.counts[e] = c;
      for (int b = 0; b < nb; ++b) p.block_expert[running + b] = e;
      if (p.pair_table) {
        for (int b = 0; b < nb; b += 2)
          p.pair_table[pair_running++] = (running + b) | (b + 1 < nb ? static_cast<int>(0x80000000u) : 0);
      }
      for (int r = c; r < nb * p.block_m; ++r) p.sorted_ids[running * p.block_m + r] = -1;
      running += nb;
    }
  }
  __syncthreads();
}

// Stable placement of one chunk: thread t holds route chunk_start + t.  ``cursor[e]`` is the next
// free row of expert e for this chunk (smem, updated in warp order so the order stays stable).
__device__ void place_chunk(const AlignParams& p, int route, int* cursor) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int e = route < p.n_routes ? local_expert(p, route) : -1;
  const uint32_t active = __ballot_sync(0xFFFFFFFFu, e >= 0);
  uint32_t same = 0;
  if (e >= 0) same = __match_any_sync(active, e);
  const int rank_in_warp = __popc(same & ((1u << lane) - 1u));
  const bool leader = e >= 0 && rank_in_warp == 0;
  int start = 0;
  const int chunk_first = route - static_cast<int>(threadIdx.x);  // first route of this chunk
  const int in_chunk = p.n_routes - chunk_first < static_cast<int>(blockDim.x) ? p.n_routes - chunk_first
                                                                                : static_cast<int>(blockDim.x);
  const int busy_warps = in_chunk > 0 ? (in_chunk + 31) >> 5 : 0;  // warps past these hold no route
  for (int w = 0; w < busy_warps; ++w) {
    if (warp == w && leader) {
      start = cursor[e];
      cursor[e] = start + __popc(same);
    }
    __syncthreads();
  }
  if (e >= 0) {
    start = __shfl_sync(same, start, __ffs(same) - 1);
    p.sorted_ids[start + rank_in_warp] = route;
  }
}

// Pass 2 (one CTA): per-expert totals, per-chunk offsets, block table.
__global__ void __launch_bounds__(1024) align_scan_kernel(AlignParams p, int n_chunks) {
  extern __shared__ int sm[];
  griddep_wait();
  griddep_launch();
  int* total = sm;                  // [n_experts]
  int* base = sm + p.n_experts;     // [n_experts]
  int* scratch = base + p.n_experts;  // [blockDim]
  // One thread per expert walks the chunks; the loads of eight chunks are issued together (a load that
  // waits for the store before it costs an L2 round trip per chunk: 36 of them at 4096 tokens).
  constexpr int kScanBatch = 8;
  for (int e = threadIdx.x; e < p.n_experts; e += blockDim.x) {
    int run = 0;
    for (int c0 = 0; c0 < n_chunks; c0 += kScanBatch) {
      int h[kScanBatch];
#pragma unroll
      for (int u = 0; u < kScanBatch; ++u)
        h[u] = c0 + u < n_chunks ? p.chunk_hist[static_cast<size_t>(c0 + u) * p.n_experts + e] : 0;
#pragma unroll
      for (int u = 0; u < kScanBatch; ++u) {
        if (c0 + u < n_chunks) p.chunk_hist[static_cast<size_t>(c0 + u) * p.n_experts + e] = run;  // exclusive offset of the chunk inside expert e
        run += h[u];
      }
    }
    total[e] = run;
  }
  __syncthreads();
  plan_blocks(p, total, base, scratch);
  for (int e = threadIdx.x; e < p.n_experts; e += blockDim.x) {
    const int add = base[e];
    for (int c0 = 0; c0 < n_chunks; c0 += kScanBatch) {
      int h[kScanBatch];
#pragma unroll
      for (int u = 0; u < kScanBatch; ++u)
        h[u] = c0 + u < n_chunks ? p.chunk_hist[static_cast<size_t>(c0 + u) * p.n_experts + e] : 0;
#pragma unroll
      for (int u = 0; u < kScanBatch; ++u)
        if (c0 + u < n_chunks) p.chunk_hist[static_cast<size_t>(c0 + u) * p.n_experts + e] = h[u] + add;
    }
  }
}

// Pass 3: scatter each chunk
__global__ void __launch_bounds__(kSortChunk) align_scatter_kernel(AlignParams p) {
  extern __shared__ int cursor[];
  griddep_wait();
  griddep_launch();
  for (int e = threadIdx.x; e < p.n_experts; e += blockDim.x)
    cursor[e] = p.chunk_hist[static_cast<size_t>(blockIdx.x) * p.n_experts + e];
  __syncthreads();
  place_chunk(p, blockIdx.x * kSortChunk + threadIdx.x, cursor);
}

// All three passes in one CTA, for up to kSmallRoutes routes (decode batches).
constexpr int kSmallRoutes = 4096;
__device__ void align_small_body(const AlignParams& p, int* sm) {
  int* total = sm;
  int* base = sm + p.n_experts;
  int* scratch = base + p.n_experts;
  for (int e = threadIdx.x; e < p.n_experts; e += blockDim.x) total[e] = 0;
  __syncthreads();
  for (int r = threadIdx.x; r < p.n_routes; r += blockDim.x) {
    const int e = local_expert(p, r);
    if (e >= 0) atomicAdd(&total[e], 1);
  }
  __syncthreads();
  plan_blocks(p, total, base, scratch);
  for (int start = 0; start < p.n_routes; start += blockDim.x) {  // a chunk is one route per thread
    place_chunk(p, start + threadIdx.x, base);
    __syncthreads();
  }
}

__global__ void __launch_bounds__(kSortChunk) align_small_kernel(AlignParams p) {
  extern __shared__ int sm[];
  griddep_wait();
  griddep_launch();
  align_small_body(p, sm);
}

// Routing and sort of a decode call in one CTA: route each token by counting, then sort the routes
// (the sort reads the ids the same CTA just wrote, after a barrier).  At one to eight tokens the two
// kernels this replaces spend their time on launch and drain, not on work.  The activation
// quantisation stays a kernel of its own: it is memory latency over many rows and needs many SMs
// (inside this CTA it took 50 us for one token, 300 us for eight).
constexpr int kPrologueTeams = kSortChunk / kDecodePrologueExperts;  // tokens routed side by side
__global__ void __launch_bounds__(kSortChunk) decode_prologue_kernel(RouteParams rp, AlignParams ap) {
  extern __shared__ int sm[];
  using TeamShared = RouteSharedT<kDecodePrologueExperts, kDecodePrologueExperts>;
  __shared__ TeamShared sh[kPrologueTeams];
  griddep_wait();
  griddep_launch();
  // Teams of 256 threads route tokens team, team + 4, ... side by side, each on its own named
  // barrier.  A team's loads for both of its tokens are issued before it counts (one memory round
  // trip), and the counting is a rolled loop: a decode call streams hundreds of MB through L2 between
  // two runs of this kernel, so its instructions come from DRAM every time and unrolled copies cost
  // more in instruction fetch than they save.
  const int team = threadIdx.x / kDecodePrologueExperts, e = threadIdx.x % kDecodePrologueExperts;
  constexpr int kRounds = kDecodePrologueTokens / kPrologueTeams;
  float s[kRounds];
  uint32_t image[kRounds];
#pragma unroll
  for (int r = 0; r < kRounds; ++r) {
    const int token = team + r * kPrologueTeams;
    if (token < rp.n_tokens) route_load(rp, token, e, s[r], image[r]);
  }
#pragma unroll
  for (int r = 0; r < kRounds; ++r) {
    const int token = team + r * kPrologueTeams;  // uniform over the team
    if (token < rp.n_tokens)
      route_by_counting(rp, token, e, kDecodePrologueExperts, 1 + team, s[r], image[r], sh[team]);
  }
  __syncthreads();  // every token's ids are written
  align_small_body(ap, sm);
}

int launch_decode_prologue(const RouteParams& rp, const AlignParams& ap, cudaStream_t stream) {
  if (rp.n_tokens < 1 || rp.n_tokens > kDecodePrologueTokens || rp.n_routed > kDecodePrologueExperts || ap.n_routes > kSmallRoutes)
    return AKLR_ERR_UNSUPPORTED_SHAPE;
  if (ap.n_experts < 1 || ap.n_experts > 2048 || ap.block_m < 1) return AKLR_ERR_UNSUPPORTED_SHAPE;
  if (int rc = check_route_shape(rp)) return rc;
  const int groups = rp.num_expert_group > 1 && rp.topk_group < rp.num_expert_group ? rp.num_expert_group : 1;
  if (groups * rp.topk > kDecodePrologueExperts) return AKLR_ERR_UNSUPPORTED_SHAPE;  // the teams' candidate tables
  const size_t smem = (2 * static_cast<size_t>(ap.n_experts) + 1024) * sizeof(int);
  return launch_kernel(decode_prologue_kernel, dim3(1), dim3(kSortChunk), smem, stream, 1, rp, ap) == cudaSuccess
             ? AKLR_OK : AKLR_ERR_CUDA;
}

int launch_align(const AlignParams& p, cudaStream_t stream) {
  if (p.n_experts < 1 || p.n_experts > 2048 || p.block_m < 1) return AKLR_ERR_UNSUPPORTED_SHAPE;
  const size_t smem = (2 * static_cast<size_t>(p.n_experts) + 1024) * sizeof(int);
  cudaError_t err = cudaSuccess;
  if (p.n_routes <= kSmallRoutes) {
    err = launch_kernel(align_small_kernel, dim3(1), dim3(kSortChunk), smem, stream, 1, p);
  } else {
    const int chunks = (p.n_routes + kSortChunk - 1) / kSortChunk;
    err = launch_kernel(align_count_kernel, dim3(chunks), dim3(kSortChunk), p.n_experts * sizeof(int), stream, 1, p);
    if (err == cudaSuccess) err = launch_kernel(align_scan_kernel, dim3(1), dim3(1024), smem, stream, 1, p, chunks);
    if (err == cudaSuccess)
      err = launch_kernel(align_scatter_kernel, dim3(chunks), dim3(kSortChunk), p.n_experts * sizeof(int), stream, 1, p);
  }
  return err == cudaSuccess ? AKLR_OK : AKLR_ERR_CUDA;
}

}  // namespace aklr
