/* C ABI of the B200 (sm_100a) fused-MoE library, libaklr_b200.so.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as void*: a
 * cudaStream_t) and launches on that stream.  The compute entry points never synchronise, never
 * allocate device memory and keep no state between calls: scratch comes from the caller as one
 * workspace buffer whose size aklr_moe_fp8_workspace gives.  The exceptions say so where they are
 * declared: aklr_moe_align_noalloc keeps its scratch in an array inside the library that all its
 * calls on a device share; aklr_moe_read_status and aklr_profile_read wait for the stream because
 * their job is to read a result back; aklr_profile_begin switches a process-wide event recorder.
 * Return value: 0, or a negative AKLR_ERR_* code (aklr_status_string names it).  Nothing here falls
 * back to a CPU path.
 *
 * Each function cites the reference interface it stands in for (paths inside the reference
 * project).  The reference's kernels are Python `run(*, <tensors>, out)` callables served by its
 * dispatch registry (aklr/ops/README.md:183-251); its native-extension precedent registers
 * `run(Tensor..., Tensor(a!) out) -> ()` (aklr/ops/README.md:269-279).  A binding passes
 * tensor.data_ptr() values to the functions below.
 */
#ifndef AKLR_B200_H
#define AKLR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AKLR_B200_ABI_VERSION 2

#define AKLR_OK 0
#define AKLR_ERR_BAD_ARGUMENT -1
#define AKLR_ERR_WORKSPACE_TOO_SMALL -2
#define AKLR_ERR_CUDA -3
#define AKLR_ERR_UNSUPPORTED_SHAPE -4
#define AKLR_ERR_NO_DEVICE -5
#define AKLR_ERR_KERNEL_WAIT_TIMEOUT -6
#define AKLR_ERR_TOO_LARGE -7

#define AKLR_SCORING_SOFTMAX 0
#define AKLR_SCORING_SIGMOID 1
#define AKLR_DTYPE_BF16 0
#define AKLR_DTYPE_F32 1
/* act(gate) in act(gate) * up (aklr/ops/fused_moe/reference.py:113-121) */
#define AKLR_ACT_SILU 0       /* gate * sigmoid(gate) */
#define AKLR_ACT_GELU 1       /* exact (erf) GELU */
#define AKLR_ACT_SWIGLU_OAI 2 /* gpt-oss: gate * sigmoid(1.702 gate) * (up + 1) */
#define AKLR_ACT_SITUV2 3     /* beta tanh(gate/beta) sigmoid(gate) * linear_beta tanh(up/linear_beta) */

/* One fused-MoE layer call.  Expert slots in w1/w2: the n_routed routed experts, then n_shared
 * shared experts every token visits at weight 1 (aklr/plugins/sglang/models/deepseek_v2/
 * reference.py:80-88).  Routes per token = topk + n_shared. */
typedef struct aklr_moe_config {
  int32_t n_tokens;
  int32_t hidden;            /* model dim, multiple of 128 */
  int32_t inter;             /* expert intermediate dim, multiple of 128 */
  int32_t n_routed;          /* router columns, <= 1024 */
  int32_t n_shared;          /* shared experts appended after the routed ones */
  int32_t topk;
  int32_t scoring;           /* AKLR_SCORING_* */
  int32_t num_expert_group;  /* 1 = ungrouped */
  int32_t topk_group;
  int32_t renormalize;       /* sigmoid scoring only; softmax always renormalises over the chosen */
  float routed_scaling_factor;
  int32_t logits_dtype;      /* AKLR_DTYPE_* of router logits */
  int32_t bias_dtype;        /* AKLR_DTYPE_* of correction_bias */
  int32_t block_m;           /* tokens per expert block: 16/32/64/128, 0 = library picks */
  int32_t n_experts_global;  /* experts-only entry with an expert map: ids range over this; else 0 */
  int32_t variant;           /* 0, or AKLR_VARIANT_* bits: kernel choices of THIS call (nothing global) */
} aklr_moe_config;

/* aklr_moe_config::variant.  Each bit overrides one kernel choice the library otherwise makes by
 * itself, for this call only, so that two variants can be compared on the same inputs (the results
 * agree; the tests check it).  No counterpart in the reference. */
#define AKLR_VARIANT_WEIGHT_MAJOR 1           /* 128-token blocks: down projection through the weight-major (decode) GEMM */
#define AKLR_VARIANT_CTA_PAIRS 2              /* token-major GEMMs as CTA pairs (cta_group::2, no multicast) */
#define AKLR_VARIANT_SEPARATE_PROLOGUE 4      /* 1..8 tokens: routing and sort as two kernels, not one */
#define AKLR_VARIANT_FULL_ACTIVATION_BOXES 8  /* MXFP4 GEMMs load all 128 activation rows of every block */
#define AKLR_VARIANT_DEEP_PIPELINE 64         /* FP8 token-major GEMMs on 128 x 128 tiles with four partials in flight */
/* w1 / w2 of the FP8 entry points are in the tile-contiguous layout aklr_tile_weights_fp8 writes (block scales are
 * unchanged).  A layout variant of the weights, as the reference's `is_shuffled` is one of its own
 * (aklr/plugins/sglang/models/deepseek_v2/contract.py:181-185, 310-318): results are bit-identical to row-major. */
#define AKLR_VARIANT_TILED_WEIGHTS 128
/* A numerics mode rather than a kernel choice (it also sizes the workspace, so set it before asking for the layout):
 * the MXFP4 expert entry points keep the activations in bf16 instead of rounding them to MXFP8 -- what the reference's
 * fused_moe does under gate_mode "interleave" and for gpt-oss swiglu below 256 rows (aklr/ops/fused_moe/
 * reference.py:90-93) and its deepseek_v2_mxfp4_moe always (aklr/plugins/sglang/models/deepseek_v2/reference.py:91-111).
 * Every activation enters the block-scaled MMAs as TWO e4m3 terms at scales 2^ex and 2^(ex-4) whose sum is the bf16 value
 * exactly (8 significant bits = 4 + 4; elements below 2^-22 of their 32-group's largest lose low bits). */
#define AKLR_VARIANT_BF16_ACTIVATIONS 16
/* Another numerics mode of the MXFP4 expert entry points: activations (the input and the gated product) quantised to
 * MXFP4 per 1 x 32 as the reference's fused_moe does at its default act_quant 4 (aklr/ops/fused_moe/reference.py:21-37):
 * scale 2^e with the group's largest value in (3, 6], values rounded to the e2m1 grid, ties to the even code.  The codes
 * travel as e4m3 bytes (every e2m1 value is an e4m3 value), so the products are exact and the MMAs are the MXFP8 path's. */
#define AKLR_VARIANT_MXFP4_ACTIVATIONS 32

/* Byte offsets of the intermediates inside the workspace (for tests and debuggers). */
typedef struct aklr_moe_workspace_layout {
  int64_t total_bytes;
  int64_t status;        /* int32[2]: first failed device wait (0 = none), its location */
  int64_t topk_ids;      /* int32 [n_tokens, routes] */
  int64_t topk_weights;  /* float [n_tokens, routes] */
  int64_t sorted_ids;    /* int32 [capacity] route ids grouped by expert, -1 = padding */
  int64_t block_expert;  /* int32 [max_blocks] */
  int64_t counts;        /* int32 [experts] routes per expert */
  int64_t num_blocks;    /* int32 [2] blocks in use, rows in use */
  int64_t chunk_hist;    /* int32 sort scratch */
  int64_t xq;            /* e4m3 [capacity, hidden] */
  int64_t xs;            /* float [max_blocks, hidden/128, block_m] */
  int64_t hq;            /* e4m3 [capacity, inter] */
  int64_t hs;            /* float [max_blocks, inter/128, block_m] */
  int64_t rows;          /* bf16 [n_tokens*routes, hidden] weighted per-route outputs */
  int32_t block_m;
  int32_t max_blocks;
  int32_t capacity;      /* max_blocks * block_m */
  int32_t n_experts;     /* expert slots sorted over */
} aklr_moe_workspace_layout;

int aklr_abi_version(void);
const char* aklr_status_string(int code);
/* Message of the last failing call on this thread ("" if none). */
const char* aklr_last_error(void);

/* Workspace of aklr_moe_fp8_forward / aklr_moe_fp8_experts for this config. */
int aklr_moe_fp8_workspace(const aklr_moe_config* cfg, aklr_moe_workspace_layout* layout);

/* Whole layer from router logits: routing, sort, quant, gate_up, down, combine.
 * Stands in for the kernels behind `deepseek_v2_fp8_moe` / `qwen3_moe_fp8_moe`
 * (aklr/plugins/sglang/models/deepseek_v2/api.py:35-50, .../qwen3_moe/api.py:14-23; arithmetic:
 * .../deepseek_v2/reference.py:163-183, .../qwen3_moe/reference.py:64-88) after the router GEMM.
 *   hidden_states bf16 [T,H]; logits [T,n_routed]; bias [n_routed] or NULL;
 *   sigmoid_table float[65536] on the device indexed by bf16 bits, or NULL (computed in-kernel);
 *   w1 e4m3 [E,2I,H] gate rows then up rows; w1_scale float [E,2I/128,H/128];
 *   w2 e4m3 [E,H,I]; w2_scale float [E,H/128,I/128]; out bf16 [T,H]. */
int aklr_moe_fp8_forward(const aklr_moe_config* cfg, const void* hidden_states, const void* logits,
                         const void* bias, const float* sigmoid_table, const void* w1, const float* w1_scale,
                         const void* w2, const float* w2_scale, void* out, void* workspace,
                         size_t workspace_bytes, void* stream);

/* Experts only, routing given: stands in for the kernels behind `fused_moe` with FP8 128x128
 * weights (aklr/ops/fused_moe/api.py:17-44; expert_mask semantics
 * aklr/ops/fused_moe/reference.py:78-84).  topk_ids int32 [T, topk + n_shared] hold ids in
 * [0, n_experts_global); expert_map int32 [n_experts_global] maps them to this rank's slot or -1
 * (NULL: identity).  topk_weights float [T, topk + n_shared]. */
int aklr_moe_fp8_experts(const aklr_moe_config* cfg, const void* hidden_states, const int32_t* topk_ids,
                         const float* topk_weights, const int32_t* expert_map, const void* w1,
                         const float* w1_scale, const void* w2, const float* w2_scale, void* out,
                         void* workspace, size_t workspace_bytes, void* stream);

/* MXFP4 experts with MXFP8 activations: the kernels behind `fused_moe` at quant_type per_1x32 with
 * act_quant 8 (aklr/ops/fused_moe/api.py:17-44, reference.py:40-127) and the local compute of
 * `mega_moe` (aklr/ops/mega_moe/reference.py:18-48).  w1 packed e2m1 [E, 2I, H/2] (low nibble
 * first), w1_scale e8m0 bytes [E, 2I, H/32]; w2 [E, H, I/2], w2_scale [E, H, I/32]; activations
 * are quantised per 1 x 32 to e4m3 at the smallest power-of-two scale >= amax/448, the gated
 * product is rounded to bf16 and quantised the same way.  swiglu_limit > 0 clamps gate (above) and
 * up (both sides) before the activation; <= 0: no clamp.  cfg->block_m must be 128, hidden % 256 == 0.
 * aklr_moe_mxfp4_forward routes from logits first (the DeepSeek routing of aklr_moe_fp8_forward). */
int aklr_moe_mxfp4_experts(const aklr_moe_config* cfg, const void* hidden_states, const int32_t* topk_ids,
                           const float* topk_weights, const int32_t* expert_map, const void* w1,
                           const uint8_t* w1_scale, const void* w2, const uint8_t* w2_scale, float swiglu_limit,
                           void* out, void* workspace, size_t workspace_bytes, void* stream);
int aklr_moe_mxfp4_forward(const aklr_moe_config* cfg, const void* hidden_states, const void* logits,
                           const void* bias, const float* sigmoid_table, const void* w1, const uint8_t* w1_scale,
                           const void* w2, const uint8_t* w2_scale, float swiglu_limit, void* out, void* workspace,
                           size_t workspace_bytes, void* stream);

/* The remaining attributes of `fused_moe` (aklr/ops/fused_moe/contract.py:90-140, reference.py:85-127).
 * A zeroed struct is aklr_moe_mxfp4_experts with no clamp. */
typedef struct aklr_mx_options {
  int32_t activation;              /* AKLR_ACT_* */
  int32_t weight_in_stage1;        /* doweight_stage1: the route weight multiplies the gate_up projection
                                      (before clamp and activation) instead of the expert's output */
  float swiglu_limit;              /* > 0: clamp gate (above) and up (both sides) before the activation */
  float beta, linear_beta;         /* AKLR_ACT_SITUV2 only; both > 0 */
  const int32_t* num_local_tokens; /* device scalar or NULL: routes of tokens at or past it add nothing and
                                      their output rows are zero (rows this rank did not receive) */
} aklr_mx_options;
int aklr_moe_mxfp4_experts_ex(const aklr_moe_config* cfg, const void* hidden_states, const int32_t* topk_ids,
                              const float* topk_weights, const int32_t* expert_map, const void* w1,
                              const uint8_t* w1_scale, const void* w2, const uint8_t* w2_scale,
                              const aklr_mx_options* options, void* out, void* workspace, size_t workspace_bytes,
                              void* stream);

/* Expert parallelism (the reference's `mega_moe` contract: every rank holds n_local experts, global
 * expert e is local e % n_local of rank e / n_local; aklr/ops/mega_moe/contract.py:42-51,
 * reference.py:25,38).  The host code orders routes by destination rank with aklr_moe_align
 * (block_m 1, an expert map global expert -> rank), then:
 *   aklr_ep_gather_quant    FP8 rows + row-major scales [n_send, H/128] of the routes in send order;
 *   aklr_ep_dispatch_meta   per sent route its expert id on the destination and its weight, and
 *                           the inverse map route -> send position (-1 must be pre-filled);
 *   (NCCL all-to-all of rows, scales, expert ids, weights -- issued by the caller)
 *   aklr_moe_fp8_experts_prequant  on the receiver: experts over rows that arrive quantised, one
 *                           route per row (cfg: n_tokens = rows, topk 1, n_shared 0, n_routed =
 *                           local expert slots); writes weighted bf16 rows [rows, H], no combine;
 *   (NCCL all-to-all of the bf16 rows back)
 *   aklr_ep_combine         out[t] = bf16(sum_k rows[position(t,k)] + shared_rows[t]). */
int aklr_ep_gather_quant(const void* hidden_states, const int32_t* sorted_ids, int32_t n_send, int32_t hidden,
                         int32_t routes_per_token, void* rows_q, float* rows_scale, void* stream);
int aklr_ep_dispatch_meta(const int32_t* sorted_ids, const int32_t* topk_ids, const float* topk_weights,
                          int32_t n_send, int32_t n_routes, int32_t experts_per_rank, int32_t* send_expert,
                          float* send_weight, int32_t* position_of_route, void* stream);
int aklr_moe_fp8_experts_prequant(const aklr_moe_config* cfg, const void* rows_q, const float* rows_scale,
                                  const int32_t* expert_ids, const float* weights, const void* w1,
                                  const float* w1_scale, const void* w2, const float* w2_scale, void* out_rows,
                                  void* workspace, size_t workspace_bytes, void* stream);
/* The MXFP4 counterparts for `mega_moe` (MXFP8 rows travel with one e8m0 byte per 32 values,
 * rows_scale uint8 [n, H/32] row-major). */
/* The same packing from rows quantised once per token (aklr_ep_gather_quant[_mxfp8] with the
 * identity table and routes_per_token 1): copies token rid / routes_per_token's codes and row-major
 * scales to send position.  mx = 0: float scales [*, H/128]; mx = 1: e8m0 bytes [*, H/32]. */
int aklr_ep_gather_rows(const void* tokens_q, const void* tokens_scale, const int32_t* sorted_ids, int32_t n_send,
                        int32_t hidden, int32_t routes_per_token, int32_t mx, void* rows_q, void* rows_scale,
                        void* stream);
int aklr_ep_gather_quant_mxfp8(const void* hidden_states, const int32_t* sorted_ids, int32_t n_send, int32_t hidden,
                               int32_t routes_per_token, void* rows_q, uint8_t* rows_scale, void* stream);
int aklr_moe_mxfp4_experts_prequant(const aklr_moe_config* cfg, const void* rows_q, const uint8_t* rows_scale,
                                    const int32_t* expert_ids, const float* weights, const void* w1,
                                    const uint8_t* w1_scale, const void* w2, const uint8_t* w2_scale,
                                    float swiglu_limit, void* out_rows, void* workspace, size_t workspace_bytes,
                                    void* stream);
int aklr_ep_combine(const void* rows, const int32_t* position_of_route, const void* shared_rows, void* out,
                    int32_t n_tokens, int32_t topk, int32_t hidden, void* stream);

/* One row per (token, destination rank) instead of one per route: a token whose routes name several
 * experts of one rank sends that rank its row once, the rank runs all of them and returns their weighted
 * sum as one row -- the "pre-sum per (token, rank)" the reference's expert-parallel notes describe for
 * mega_moe (aklr/ops/mega_moe/contract.py:44-51 fixes who owns what; message shape: the reference's
 * mega_moe_buffers, kernel e9d234d2dd4d06d9, mega_moe_buffers.py:154-167).
 *   aklr_ep_plan      first_rank[t, s] = rank of slot s if no earlier slot of token t goes to that rank, else -1
 *                     (sort it by rank with aklr_moe_align, block_m 1); position_of_route[t, s] = -1;
 *   aklr_ep_pack      send row i = [hidden e4m3 codes][scales][topk int32 ids local to the destination, -1 where the
 *                     slot goes elsewhere][topk float weights], aklr_ep_row_bytes(hidden, topk, mx) bytes a row, from
 *                     tokens quantised once (aklr_moe_act_quant_fp8: float scales [T, H/128]; mx: aklr_ep_gather_quant_mxfp8
 *                     with the identity table: e8m0 bytes [T, H/32]); records position_of_route for the sent slots;
 *                     n_send is the host's bound on the rows, n_send_device (or NULL) the device's count of them;
 *   (ONE NCCL all-to-all of the packed rows -- issued by the caller)
 *   aklr_ep_unpack_meta  the ids / weights tables [rows, topk] of the rows received;
 *   aklr_moe_fp8_experts_rows / aklr_moe_mxfp4_experts_rows  experts over rows that arrive quantised, topk routes
 *                     per row (negative id: none), codes and scales read in place from the packed rows (pitches in
 *                     bytes, 0 = dense); out [rows, H] bf16 = each row's weighted sum;
 *   (ONE NCCL all-to-all of the bf16 rows back), then aklr_ep_combine as above. */
/* The split sizes of the uneven all-to-all for the host: [send_counts | recv_counts] (2 x world int32) stored
 * by a kernel into pinned host memory the device can address (cudaHostAlloc memory under unified addressing),
 * not by a device-to-host copy, which would wait on the copy engine behind any large copy in flight there.
 * The caller records an event after it and waits for that event before reading. */
int aklr_ep_counts_to_host(const int32_t* send_counts, const int32_t* recv_counts, int32_t world, int32_t* host_mapped,
                           void* stream);
int32_t aklr_ep_row_bytes(int32_t hidden, int32_t topk, int32_t mx);
int aklr_ep_plan(const int32_t* topk_ids, int32_t n_tokens, int32_t topk, int32_t experts_per_rank, int32_t* first_rank,
                 int32_t* position_of_route, void* stream);
int aklr_ep_pack(const void* tokens_q, const void* tokens_scale, const int32_t* sorted_ids, const int32_t* topk_ids,
                 const float* topk_weights, int32_t n_send, int32_t n_tokens, int32_t topk, int32_t hidden,
                 int32_t experts_per_rank, int32_t mx, const int32_t* n_send_device, void* packed,
                 int32_t* position_of_route, void* stream);
int aklr_ep_unpack_meta(const void* packed, int32_t n_rows, int32_t hidden, int32_t topk, int32_t mx, int32_t* topk_ids,
                        float* topk_weights, void* stream);
int aklr_moe_fp8_experts_rows(const aklr_moe_config* cfg, const void* rows_q, int32_t rows_q_pitch, const float* rows_scale,
                              int32_t rows_scale_pitch, const int32_t* topk_ids, const float* topk_weights, const void* w1,
                              const float* w1_scale, const void* w2, const float* w2_scale, void* out, void* workspace,
                              size_t workspace_bytes, void* stream);
int aklr_moe_mxfp4_experts_rows(const aklr_moe_config* cfg, const void* rows_q, int32_t rows_q_pitch, const uint8_t* rows_scale,
                                int32_t rows_scale_pitch, const int32_t* topk_ids, const float* topk_weights, const void* w1,
                                const uint8_t* w1_scale, const void* w2, const uint8_t* w2_scale, float swiglu_limit, void* out,
                                void* workspace, size_t workspace_bytes, void* stream);

/* Routing alone: `biased_grouped_topk` (aklr/ops/topk/api.py:12-22, reference.py:17-35) and the
 * routing halves of the two layer ops.  Writes topk_ids int32 / topk_weights float
 * [T, topk + n_shared]. */
int aklr_moe_route(const aklr_moe_config* cfg, const void* logits, const void* bias, const float* sigmoid_table,
                   int32_t* topk_ids, float* topk_weights, void* stream);

/* moe_align: stable sort of routes by expert, padded per expert to block_m.  The reference has no
 * function for it (its kernels sort inside, e.g. deepseek_v2 kernel e5adae63cb11d836,
 * kernel.py:276-361).  chunk_scratch: int32 [ceil(n_routes/1024) * n_experts]. */
int aklr_moe_align(const int32_t* topk_ids, const int32_t* expert_map, int32_t n_routes, int32_t n_experts,
                   int32_t n_experts_global, int32_t block_m, int32_t* sorted_ids, int32_t* block_expert,
                   int32_t* counts, int32_t* num_blocks, int32_t* chunk_scratch, void* stream);
int64_t aklr_moe_align_max_blocks(int64_t n_routes, int64_t n_experts, int64_t block_m);

/* moe_align without a scratch argument.  It has no counterpart in the reference.  For callers
 * that cannot allocate device memory where they sort (a frozen memory pool, a hook handed only the
 * engine's tensors, a binding with no allocator): the histogram scratch is a 1 MiB array inside
 * the library, held by every GPU that loads it.  Limit: ceil(n_routes/1024) * n_experts <=
 * aklr_moe_align_noalloc_max_scratch_ints() (262144), else AKLR_ERR_TOO_LARGE.  The first call on
 * a device resolves the array's address (make it before any stream capture); calls on one device
 * share the array, so calls whose kernels overlap on the GPU race.  Outputs as aklr_moe_align. */
int aklr_moe_align_noalloc(const int32_t* topk_ids, const int32_t* expert_map, int32_t n_routes,
                           int32_t n_experts, int32_t n_experts_global, int32_t block_m, int32_t* sorted_ids,
                           int32_t* block_expert, int32_t* counts, int32_t* num_blocks, void* stream);
int32_t aklr_moe_align_noalloc_max_scratch_ints(void);
const char* aklr_moe_align_noalloc_last_error(void);

/* Qwen2-MoE's gated shared expert (`_experts`, aklr/plugins/sglang/models/qwen2_moe/reference.py:84-90):
 * slot `topk` of the [T, topk+1] routing tables becomes expert `shared_slot` at weight
 * sigmoid(x . shared_gate_weight) (both bf16).  topk_ids_in / topk_weights_in [T, topk] are copied into the
 * first slots when given; NULL when those slots are already written (aklr_moe_route with n_shared 1). */
int aklr_moe_shared_gate(const void* x, const void* shared_gate_weight, const int32_t* topk_ids_in,
                         const float* topk_weights_in, int32_t* topk_ids, float* topk_weights, int32_t n_tokens,
                         int32_t hidden, int32_t topk, int32_t shared_slot, void* stream);

/* A shared expert held apart from the routed ones in bf16 (`qwen2_moe_mxfp4_moe_reference`,
 * aklr/plugins/sglang/models/qwen2_moe/reference.py:160-185): its two projections are plain dense bf16 GEMMs
 * (the caller's GEMM library); these are the steps around them.
 * aklr_silu_mul_bf16: out bf16 [T, inter] = silu(gate_up[:, :inter]) * gate_up[:, inter:], gate_up bf16 [T, 2*inter].
 * aklr_moe_add_gated_rows: out[t] = bf16(out[t] + sigmoid(x[t] . shared_gate_weight) * rows[t]), all bf16 [T, hidden]
 * (shared_gate_weight bf16 [hidden]); out is the routed experts' sum the layer call wrote. */
int aklr_silu_mul_bf16(const void* gate_up, void* out, int32_t n_tokens, int32_t inter, void* stream);
int aklr_moe_add_gated_rows(const void* x, const void* shared_gate_weight, const void* rows, void* out, int32_t n_tokens,
                            int32_t hidden, void* stream);

/* Self-test: the activation quantiser divides by a group's scale through a reciprocal and one exact residual
 * step instead of an IEEE division per value (the reference divides: `_fp8_input`,
 * aklr/plugins/sglang/models/qwen3_moe/reference.py:44-54).  Adds to *mismatches (int32, device, zeroed by the
 * caller) the number of pairs (x[i], scale[i]), float32 on the device, where the two differ in any bit. */
int aklr_selftest_exact_divide(const float* x, const float* scale, int64_t n, int32_t* mismatches, void* stream);

/* Load-time converter, outside any layer call: `matrices` row-major FP8 matrices [rows, cols] (an expert tensor
 * [E, rows, cols] is E of them) -> [matrix][rows/128][cols/128][128][128 bytes], every 128 x 128-byte tile one
 * contiguous 16 KB run.  rows and cols multiples of 128; src and dst 16-byte aligned, not overlapping.  The
 * reference's layout variants are converted the same way, by the engine at load time
 * (`Preshuffle`, aklr/core/contract/semantics/_layouts.py:103-121). */
int aklr_tile_weights_fp8(const void* src, void* dst, int64_t matrices, int32_t rows, int32_t cols, void* stream);

/* logits float32 [T,E] = x (bf16 [T,H]) @ w (float32 [E,H])^T, nothing rounded: the gate of
 * `minimax_m2_fp8_moe` (aklr/plugins/sglang/models/minimax_m2/reference.py:43-50). */
int aklr_router_gemm_f32(const void* x, const float* w, float* logits, int32_t n_tokens, int32_t hidden,
                         int32_t n_routed, void* stream);

/* logits bf16 [T,E] = bf16(x [T,H] @ w [E,H]^T): `_router_logits`
 * (aklr/plugins/sglang/models/qwen3_moe/reference.py:24-31). */
int aklr_router_gemm_bf16(const void* x, const void* w, void* logits, int32_t n_tokens, int32_t hidden,
                          int32_t n_routed, void* stream);

/* `per_group_quant_fp8` (aklr/ops/quant/api.py:8-9, reference.py:9-28): x bf16 [T,H] ->
 * q e4m3 [T,H], scales float [H/128, T] (group-major). */
int aklr_per_group_quant_fp8(const void* x, void* q, float* scales, int32_t rows, int32_t hidden, void* stream);
/* `per_group_quant_mxfp8` (aklr/ops/quant/api.py:12-13, reference.py:31-48): q e4m3 [T,H],
 * scales e8m0 bytes [T, H/32]. */
int aklr_per_group_quant_mxfp8(const void* x, void* q, uint8_t* scales, int32_t rows, int32_t hidden,
                               void* stream);
/* The layer's own activation quantiser (division form, row-major scales [T,H/128]):
 * `_fp8_input` (aklr/plugins/sglang/models/qwen3_moe/reference.py:44-54). */
int aklr_moe_act_quant_fp8(const void* x, void* q, float* scales, int32_t rows, int32_t hidden, void* stream);

/* Copies the workspace's status words to host_status[2] and waits for the stream: 0 = every
 * device-side wait completed. */
int aklr_moe_read_status(const void* workspace, int32_t* host_status, void* stream);

/* A failed device-side wait, heard by callers that never read a workspace.  Every wait inside the
 * kernels is bounded; one that gives up makes its kernel drain and return, and records
 * (AKLR_ERR_KERNEL_WAIT_TIMEOUT, location) in the workspace AND in two int32 of pinned host memory
 * per device.  Every entry point reads that pair first (a host read; no copy, no synchronisation):
 * the first call on the device after such a failure launches nothing, returns the code (the message
 * names the location) and clears the pair.  What the failed call and the calls enqueued after it
 * wrote is not valid.  aklr_device_status reads (and optionally clears) the current device's pair
 * without launching anything.  The pinned words are allocated once per process at the first eager
 * call.  No counterpart in the reference, whose kernels have no bounded waits. */
int aklr_device_status(int32_t* code_and_location, int32_t clear);
/* Self-test of that path: one thread waits, for at most limit_cycles SM cycles, on a barrier that
 * nothing arrives on, then reports as a stuck pipeline would (status: int32[2] on the device, and
 * the device's host-visible pair).  The kernel always returns; the context stays usable.  Lets an
 * integrator see what their error handling does with the code without needing a real failure. */
int aklr_selftest_wait_expiry(int64_t limit_cycles, int32_t* status, void* stream);

/* Measurement aids (no counterpart in the reference, which times with rocprofiler:
 * aklr/core/utils/testing.py:171-252).  aklr_kernel_launch_count: kernels this library has
 * launched in this process.  aklr_profile_begin(n): record CUDA events around the six stages
 * (route, sort, quant, gate_up, down, combine) of the next n layer calls of this process;
 * n = 0 switches it off.  aklr_profile_read(call, ms[6]) waits for that call and gives its
 * stage durations in milliseconds. */
int64_t aklr_kernel_launch_count(void);
int aklr_profile_begin(int32_t max_calls);
int aklr_profile_read(int32_t call, float* stage_ms);

#ifdef __cplusplus
}
#endif
#endif /* AKLR_B200_H */
