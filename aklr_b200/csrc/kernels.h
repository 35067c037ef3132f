// Internal launch interface between the kernel files and the C ABI (abi.cu).
#pragma once

#include <cuda.h>
#include <utility>
#include <cuda_runtime.h>
#include <stdint.h>

#define AKLR_SCORING_SOFTMAX 0
#define AKLR_SCORING_SIGMOID 1
#ifndef AKLR_ACT_SILU  // the public header defines the same values
#define AKLR_ACT_SILU 0
#define AKLR_ACT_GELU 1
#define AKLR_ACT_SWIGLU_OAI 2
#define AKLR_ACT_SITUV2 3
#endif

namespace aklr {

struct RouteParams {
  const void* logits;          // [n_tokens, n_routed] bf16 or f32
  const void* bias;            // [n_routed] bf16 or f32, or null
  const float* sigmoid_table;  // 65536 floats indexed by bf16 bits, or null
  int32_t* topk_ids;           // [n_tokens, topk + n_shared]
  float* topk_weights;         // [n_tokens, topk + n_shared]
  int n_tokens, n_routed, n_shared, topk;
  int scoring, num_expert_group, topk_group, renormalize;
  int logits_are_bf16, bias_is_bf16;
  float routed_scaling_factor;
};
int launch_route(const RouteParams& p, cudaStream_t stream);

struct AlignParams {
  const int32_t* topk_ids;    // [n_routes] global expert ids (negative: dropped)
  const int32_t* expert_map;  // [n_experts_global] -> local id or -1, or null (identity)
  int32_t* sorted_ids;        // [capacity] route ids, -1 in padding
  int32_t* block_expert;      // [max_blocks]
  int32_t* counts;            // [n_experts]
  int32_t* num_blocks;        // [2]: blocks used, rows used (= blocks * block_m); [3] with pair_table: + pairs
  int32_t* pair_table;        // optional [max_blocks]: first block of every run of <= 2 blocks of one
                              // expert; bit 31 set when the second block exists
  int32_t* chunk_hist;        // [ceil(n_routes/1024) * n_experts] scratch
  const int32_t* num_local_tokens;  // optional device scalar: routes of tokens at or past it are dropped
  int n_routes, n_experts, n_experts_global, block_m;
  int routes_per_token;       // read with num_local_tokens only
};
int launch_align(const AlignParams& p, cudaStream_t stream);

// rows of the sorted table an align call can use at most
inline int64_t align_max_blocks(int64_t n_routes, int64_t n_experts, int64_t block_m) {
  const int64_t nonempty = n_routes < n_experts ? n_routes : n_experts;
  return n_routes / block_m + nonempty;
}

struct GatherQuantParams {
  const void* x;              // [n_tokens, hidden] bf16
  const uint8_t* q_in;        // gather_rows only: [n_tokens, hidden] e4m3 quantised by the sender
  const float* scales_in;     // gather_rows only: [n_tokens, hidden/128]
  const int32_t* sorted_ids;  // [capacity] or null: row r reads token r
  const int32_t* num_rows;    // device count of rows in use (null: n_rows)
  uint8_t* q;                 // [rows, hidden] e4m3
  float* scales;              // block_m == 0: [rows, hidden/128]; else [rows/block_m, hidden/128, block_m]
  int n_rows, hidden, routes_per_token, block_m;
  int q_in_stride, scales_in_stride;  // gather_rows only: bytes between source rows (0: dense)
  int zero_padding;  // non-zero: padding rows of the table get zero codes (see gather_rows_fp8_kernel)
};
int launch_gather_quant_fp8(const GatherQuantParams& p, cudaStream_t stream);

// Routing and sort of a decode batch (1..kDecodePrologueTokens tokens, up to kDecodePrologueExperts routed
// experts) in one CTA.
constexpr int kDecodePrologueTokens = 8;
constexpr int kDecodePrologueExperts = 256;
int launch_decode_prologue(const RouteParams& rp, const AlignParams& ap, cudaStream_t stream);
int launch_gather_rows_fp8(const GatherQuantParams& p, cudaStream_t stream);

// standalone quant ops
int launch_per_group_quant_fp8(const void* x_bf16, uint8_t* q, float* scales_group_major, int rows, int hidden,
                               cudaStream_t stream);
int launch_per_group_quant_mxfp8(const void* x_bf16, uint8_t* q, uint8_t* scales_e8m0, int rows, int hidden,
                                 cudaStream_t stream);

struct GroupedGemmParams {
  CUtensorMap map_w;   // weights flattened to [experts*rows_per_expert, k], box 128 x 128
  CUtensorMap map_x;   // activations [capacity, k] e4m3, box block_m x 128
  const float* w_scale;        // [experts, rows_per_expert/128, k/128]
  const float* x_scale;        // [max_blocks, k/128, block_m]
  const int32_t* sorted_ids;   // [capacity]
  const int32_t* block_expert; // [max_blocks]
  const int32_t* num_blocks;   // device count ([2] = number of block pairs)
  const int32_t* pair_table;   // CTA-pair kernel only
  const float* topk_weights;   // [n_routes] (down projection only)
  uint8_t* out_q;              // gate_up: [capacity, inter] e4m3
  float* out_scale;            // gate_up: [max_blocks, inter/128, block_m]
  void* out_rows;              // down: [n_routes, hidden] bf16 per-route contributions
  int32_t* status;             // [2] error word + location
  int32_t* host_status;        // the device's host-visible copy of a failure (or null)
  int k;                       // reduction length (hidden for gate_up, inter for down)
  int out_dim;                 // inter (gate_up) or hidden (down)
  int rows_per_expert;         // 2*inter (gate_up) or hidden (down)
  int block_m;                 // tokens per block: 16, 32, 64 or 128
  int max_blocks;              // upper bound used to size the tile loop
  int stages;
  int w_tiled;                 // weights in the tile-contiguous layout: [expert][row/128][k/128][128 rows][128 bytes]
  int wide;                    // weight-major down projection on 256-channel tiles (grouped_gemm_down_is_wide)
};
int launch_grouped_gemm_gate_up(const GroupedGemmParams& p, int sm_count, cudaStream_t stream);
int launch_grouped_gemm_down(const GroupedGemmParams& p, int sm_count, cudaStream_t stream);
// token-major variant for full 128-token blocks (grouped_gemm_prefill.cu); its down projection
// needs map_w built with a 256-row box
bool grouped_gemm_is_token_major(bool gate_up, int block_m, int out_dim);
// pair: two CTAs of a cluster share one M=256 MMA over two token blocks of an expert (needs
// pair_table; map_w with a 128-row box for both projections)
int grouped_gemm_prefill_pick_stages(bool gate_up, bool pair);
int launch_grouped_gemm_prefill(const GroupedGemmParams& p, bool gate_up, bool pair, int sm_count, cudaStream_t stream);
// the same on 128 x 128 tiles with four TMEM partials in flight (grouped_gemm_deep.cu); map_w with a
// 64-row box for gate_up and a 128-row box for down; out_dim a multiple of 128 for both
int grouped_gemm_deep_pick_stages(bool gate_up);
int launch_grouped_gemm_deep(const GroupedGemmParams& p, bool gate_up, int sm_count, cudaStream_t stream);
// Tile-contiguous FP8 weights (a layout a checkpoint loader can convert to once): every 128-row x 128-byte tile
// the TMA fetches is one contiguous 16 KB run of HBM instead of 128 row segments k bytes apart.  The map is then
// over [tiles * 128 rows, 128 bytes] and a tile's box starts at row tile_index * 128.
int launch_exact_divide_selftest(const float* x, const float* scale, int64_t n, int32_t* mismatches, cudaStream_t stream);
int launch_tile_weights_fp8(const void* src, void* dst, int64_t matrices, int rows, int cols, cudaStream_t stream);
size_t grouped_gemm_smem_bytes(bool gate_up, int block_m, int k, int stages, bool wide = false);
int grouped_gemm_pick_stages(bool gate_up, int block_m, int k, bool wide = false);
bool grouped_gemm_down_is_wide(int block_m, int out_dim, int max_blocks, int sm_count);

// ---- MXFP4 weights / MXFP8 activations (grouped_gemm_mx.cu), always 128-token blocks ----------
struct MxQuantParams {
  const void* x;              // [n_tokens, hidden] bf16
  const int32_t* sorted_ids;  // [capacity]
  const int32_t* num_rows;    // device count of rows in use
  uint8_t* q;                 // [capacity, hidden] e4m3
  uint8_t* scales;            // [capacity/128, hidden/128, 512] e8m0 bytes in tcgen05.cp order
  const uint8_t* q_in;        // rows already quantised by a sender ([n, hidden] e4m3), or null
  const uint8_t* scales_in;   // their scale bytes [n, hidden/32]
  int n_rows, hidden, routes_per_token;
  int row_major_scales;       // write scales as [row, hidden/32] (for transport) instead
  int q_in_stride, scales_in_stride;  // rows quantised before: bytes between source rows (0: dense)
  // Activations kept in bf16 (no MXFP8 rounding): every value travels as TWO e4m3 codes whose block
  // scales are 2^ex and 2^(ex-4), hi + lo = the bf16 value exactly (8 significant bits = 4 + 4) except
  // for elements below 2^-22 of their group's largest.  q_lo / scales_lo: the second term, same shapes.
  uint8_t* q_lo;
  uint8_t* scales_lo;
  // Activations quantised to MXFP4 instead of MXFP8 (the reference's act_quant 4): the scale puts the
  // group's largest value in (3, 6], values round to the e2m1 grid (ties to the even code).  Every e2m1
  // value is also an e4m3 value, so the codes are stored as e4m3 bytes and the same MMAs consume them.
  int act_fp4;
  // Padding rows of the table that the GEMM's producer loads get zero codes (they are multiplied although never
  // read back, and zero operands cost the tensor core least): 0 off, 1 every padding row, 2 only those inside the
  // 32- or 64-row box of a block with that few routed rows (MxGemmParams::small_boxes).
  int zero_padding;
};
int launch_gather_quant_mxfp8(const MxQuantParams& p, cudaStream_t stream);

struct MxGemmParams {
  CUtensorMap map_w;           // packed e2m1 weights [experts*rows_per_expert, k], 16U4_ALIGN16B, box 128 x 128|256
  CUtensorMap map_x;           // e4m3 activations [capacity, k], box 128 x 128
  CUtensorMap map_x_rows32;    // the same matrix with boxes of 32 and 64 rows: a block with that few routed
  CUtensorMap map_x_rows64;    // rows loads only those (the tile's other rows are never read back)
  int small_boxes;             // non-zero: the two maps above are set
  const uint8_t* w_scale;      // e8m0 [experts, rows_per_expert, k/32]
  const uint8_t* x_scale;      // e8m0 [max_blocks, k/128, 512]
  const int32_t* sorted_ids;
  const int32_t* block_expert;
  const int32_t* num_blocks;
  const float* topk_weights;   // down only
  uint8_t* out_q;              // gate_up: [capacity, inter] e4m3
  uint8_t* out_scale;          // gate_up: [max_blocks, inter/128, 512]
  void* out_rows;              // down: [n_routes, hidden] bf16
  int32_t* status;
  int32_t* host_status;        // the device's host-visible copy of a failure (or null)
  float swiglu_limit;          // > 0: clamp gate above and up on both sides before the activation
  int activation;              // gate_up: AKLR_ACT_* of the public header
  float beta, linear_beta;     // gate_up, AKLR_ACT_SITUV2: saturation of gate and up
  const float* stage1_weights; // gate_up: route weights applied to the projection before the activation, or null
  int k, out_dim, rows_per_expert, max_blocks, stages;
  // bf16 activations as two e4m3 terms (see MxQuantParams): the second term's operand map, scales and,
  // for gate_up, outputs; split != 0 issues two MMAs per K step on the same weight tile
  int split;
  int act_fp4;  // gate_up: requantise the gated product to the MXFP4 grid (see MxQuantParams)
  CUtensorMap map_x_lo;
  const uint8_t* x_scale_lo;
  uint8_t* out_q_lo;
  uint8_t* out_scale_lo;
};
int grouped_gemm_mx_pick_stages(bool gate_up, bool split = false);
int launch_grouped_gemm_mx(const MxGemmParams& p, bool gate_up, int sm_count, cudaStream_t stream);

struct CombineParams {
  const void* rows;          // [n_tokens * routes_per_token, hidden] bf16
  const int32_t* topk_ids;   // [n_tokens, routes_per_token] global ids
  const int32_t* expert_map; // null or global -> local (-1: not here, the route adds nothing)
  void* out;                 // [n_tokens, hidden] bf16
  const int32_t* num_local_tokens;  // optional device scalar: tokens at or past it get zeros
  int n_tokens, hidden, routes_per_token, n_experts_global;
};
int launch_combine(const CombineParams& p, cudaStream_t stream);

// ---- expert parallelism: sender-side packing and home-side combine --------------------------
struct EpMetaParams {
  const int32_t* sorted_ids;    // [n_send] routes ordered by destination rank (moe_align, block_m 1)
  const int32_t* topk_ids;      // [n_routes] global expert ids
  const float* topk_weights;    // [n_routes]
  int32_t* send_expert;         // [n_send] expert id local to the destination rank
  float* send_weight;           // [n_send]
  int32_t* position_of_route;   // [n_routes] where the route sits in the send order (-1: not sent)
  int n_send, n_routes, experts_per_rank;
};
int launch_ep_meta(const EpMetaParams& p, cudaStream_t stream);

struct EpPlanParams {
  const int32_t* topk_ids;     // [n_tokens, topk] global expert ids (negative: no route)
  int32_t* first_rank;         // [n_tokens, topk] destination rank of the first slot per (token, rank), else -1
  int32_t* position_of_route;  // [n_tokens, topk] set to -1
  int n_tokens, topk, experts_per_rank;
};
int launch_ep_first_slots(const EpPlanParams& p, cudaStream_t stream);

struct EpPackParams {
  const uint8_t* tokens_q;      // [n_tokens, hidden] e4m3, each token quantised once
  const uint8_t* tokens_scale;  // [n_tokens, scale_bytes]
  const int32_t* sorted_ids;    // [n_send] first slots (token * topk + slot) ordered by destination rank
  const int32_t* n_send_device; // optional device count of rows to send (the host only knows the bound n_send)
  const int32_t* topk_ids;      // [n_tokens, topk]
  const float* topk_weights;    // [n_tokens, topk]
  uint8_t* packed;              // [n_send, row_bytes]
  int32_t* position_of_route;   // [n_tokens, topk]: send position of the first slots
  int n_send, n_tokens, topk, hidden, scale_bytes, row_bytes, experts_per_rank;
};
int launch_ep_pack(const EpPackParams& p, cudaStream_t stream);
int launch_ep_unpack_meta(const uint8_t* packed, int n_rows, int row_bytes, int meta_offset, int topk, int32_t* ids,
                          float* weights, cudaStream_t stream);

int launch_ep_counts_to_host(const int32_t* send_counts, const int32_t* recv_counts, int world, int32_t* host_mapped,
                             cudaStream_t stream);

struct EpCombineParams {
  const void* rows;                  // [n_send, hidden] bf16, weighted, in send order
  const int32_t* position_of_route;  // [n_tokens * topk]
  const void* shared_rows;           // [n_tokens, hidden] bf16 or null
  void* out;                         // [n_tokens, hidden] bf16
  int n_tokens, topk, hidden;
};
int launch_ep_combine(const EpCombineParams& p, cudaStream_t stream);

// tensor-core router GEMM (router_gemm.cu): maps are bf16 [T,H] box 64 x 128 and [E,H] box 64 x n_tile
int launch_router_gemm_tc(const CUtensorMap& map_x, const CUtensorMap& map_w, void* logits, int n_tokens, int hidden,
                          int n_routed, int n_tile, int32_t* host_status, cudaStream_t stream);

// Shared by the files that hold extern "C" entry points: the device check (sm_100 only) and the
// process-wide count of kernels this library has launched (aklr_kernel_launch_count).
int require_sm100_device(char* message, size_t message_bytes);
void count_kernel_launches(int n);
// Two int32 of mapped pinned host memory per device (error code, location) that a kernel whose wait
// gave up writes and every entry point reads before it launches anything; the device-side address
// for the current device, or null when it could not be set up (then only the workspace's status
// words report a failure).  ``stream`` is looked at only to avoid setting up inside a capture.
int32_t* host_visible_status(cudaStream_t stream);

// Opt a kernel in to the full 227 KB of dynamic shared memory, once per (kernel, device).
int ensure_max_dynamic_smem(const void* kernel);

// Launch, with programmatic stream serialisation (see griddep_wait in common.cuh) unless AKLR_PDL=0 is in
// the environment.  ``cluster`` > 1 adds a cluster dimension.
bool pdl_enabled();
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 int cluster, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int n = 0;
  if (pdl_enabled()) {
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster > 1) {
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = static_cast<unsigned>(cluster);
    attrs[n].val.clusterDim.y = 1;
    attrs[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

int launch_shared_gate(const void* x_bf16, const void* gate_bf16, const int32_t* ids_in, const float* weights_in,
                       int32_t* ids, float* weights, int n_tokens, int hidden, int topk, int shared_slot, cudaStream_t stream);
int launch_silu_mul_bf16(const void* gate_up_bf16, void* out_bf16, int n_tokens, int inter, cudaStream_t stream);
int launch_add_gated_rows(const void* x_bf16, const void* gate_bf16, const void* rows_bf16, void* out_bf16, int n_tokens,
                          int hidden, cudaStream_t stream);
int launch_router_gemm_f32(const void* x_bf16, const float* w, float* logits, int n_tokens, int hidden, int n_routed,
                           cudaStream_t stream);
int launch_router_gemm(const void* x_bf16, const void* w_bf16, void* logits_bf16, int n_tokens, int hidden,
                       int n_routed, cudaStream_t stream);

}  // namespace aklr
