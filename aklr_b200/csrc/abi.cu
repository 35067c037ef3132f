// extern "C" surface of libaklr_b200.so: argument checks, workspace layout, TMA descriptors and
// the launch sequence of one fused-MoE layer.  No allocation, no synchronisation (except
// aklr_moe_read_status, whose purpose is to read a result back), no state between calls.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <atomic>
#include <mutex>
#include <vector>

#include "../../include/aklr_b200.h"
#include "common.cuh"
#include "kernels.h"

namespace {

thread_local char g_error[512] = "";

// ---- optional stage timing: a ring of CUDA events the caller switches on for a measurement ----
constexpr int kStages = 6;  // route, sort, quant, gate_up, down, combine
constexpr int kQuantOncePerTokenFrom = 512;  // tokens from which activations are quantised once per token, then gathered
struct StageProfile {
  std::vector<cudaEvent_t> events;  // (kStages + 1) per recorded call
  int capacity = 0, used = 0;
  bool on = false;
};
StageProfile g_profile;
std::atomic<long long> g_launches{0};

// Kernel choices a caller can override per call (aklr_moe_config::variant, AKLR_VARIANT_*).
// CTA pairs are off unless asked for: they cut a CTA's operand traffic by a third, but measured
// within 2% of the single-CTA kernel at 8+ blocks per expert and slower where experts have one or
// two blocks (an odd last block wastes half a pair).
bool force_weight_major(const aklr_moe_config& c) { return (c.variant & AKLR_VARIANT_WEIGHT_MAJOR) != 0; }
bool use_cta_pairs(const aklr_moe_config& c) { return (c.variant & AKLR_VARIANT_CTA_PAIRS) != 0; }
bool deep_pipeline(const aklr_moe_config& c) { return (c.variant & AKLR_VARIANT_DEEP_PIPELINE) != 0; }
bool tiled_weights(const aklr_moe_config& c) { return (c.variant & AKLR_VARIANT_TILED_WEIGHTS) != 0; }
bool small_activation_boxes(const aklr_moe_config& c) { return (c.variant & AKLR_VARIANT_FULL_ACTIVATION_BOXES) == 0; }
bool bf16_activations(const aklr_moe_config& c) { return (c.variant & AKLR_VARIANT_BF16_ACTIVATIONS) != 0; }
bool mxfp4_activations(const aklr_moe_config& c) { return (c.variant & AKLR_VARIANT_MXFP4_ACTIVATIONS) != 0; }

void profile_mark(cudaStream_t stream, int slot, int stage) {
  if (g_profile.on && slot >= 0) cudaEventRecord(g_profile.events[slot * (kStages + 1) + stage], stream);
}
int profile_slot() {
  if (!g_profile.on || g_profile.used >= g_profile.capacity) return -1;
  return g_profile.used++;
}

int fail(int code, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
  return code;
}

int cuda_fail(cudaError_t err, const char* what) {
  return fail(AKLR_ERR_CUDA, "%s: %s", what, cudaGetErrorString(err));
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess)
      sym = nullptr;
    return reinterpret_cast<EncodeTiledFn>(sym);
  }();
  return fn;
}

// 2-D map over a row-major byte matrix [rows, cols]; box = box_rows x 128 bytes, SWIZZLE_128B.
int make_map_u8(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (!encode) return fail(AKLR_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0 || cols % 16 != 0)
    return fail(AKLR_ERR_BAD_ARGUMENT, "TMA operand must be 16-byte aligned with a 16-byte multiple row pitch");
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols};
  const cuuint32_t box[2] = {128, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(AKLR_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return AKLR_OK;
}

// Packed e2m1 matrix [rows, cols elements]: the TMA unpacks 16 nibbles (8 bytes) to 16 bytes in shared
// memory, the layout the mixed f8f6f4 MMA reads.  Box = box_rows x 128 elements, SWIZZLE_128B.
int make_map_fp4(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (!encode) return fail(AKLR_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if (reinterpret_cast<uintptr_t>(base) % 32 != 0 || (cols / 2) % 32 != 0)
    return fail(AKLR_ERR_BAD_ARGUMENT, "packed fp4 TMA operand must be 32-byte aligned with a 32-byte multiple row pitch");
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols / 2};
  const cuuint32_t box[2] = {128, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, const_cast<void*>(base), dims, strides, box,
                            elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(AKLR_ERR_CUDA, "cuTensorMapEncodeTiled (packed fp4) failed with CUresult %d", (int)r);
  return AKLR_OK;
}

// bf16 matrix [rows, cols]: box = box_rows x 64 elements (128 bytes), SWIZZLE_128B, zero fill outside.
int make_map_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (!encode) return fail(AKLR_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0 || (cols * 2) % 16 != 0)
    return fail(AKLR_ERR_BAD_ARGUMENT, "TMA operand must be 16-byte aligned with a 16-byte multiple row pitch");
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(AKLR_ERR_CUDA, "cuTensorMapEncodeTiled (bf16) failed with CUresult %d", (int)r);
  return AKLR_OK;
}

int sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  return n;
}

// ---- a failure every later call hears of ---------------------------------------------------------
// A kernel whose bounded wait gave up records it in the call's workspace, which only a caller that
// asks (aklr_moe_read_status) ever reads.  So the kernel also writes the pair (code, location) into
// two int32 of mapped pinned host memory that belong to its device, and every entry point looks at
// them -- a plain host read, no copy, no synchronisation -- before it launches anything: the first
// call after a failure returns AKLR_ERR_KERNEL_WAIT_TIMEOUT and clears the pair.
constexpr int kMaxDevices = 64;
std::mutex g_host_status_lock;
int32_t* g_host_status = nullptr;            // [kMaxDevices][2], one allocation for the process
int32_t* g_host_status_dev[kMaxDevices] = {};  // the same words as each device addresses them

int32_t* host_status_words(int dev, cudaStream_t stream) {
  if (dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> guard(g_host_status_lock);
  if (g_host_status_dev[dev]) return g_host_status_dev[dev];
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &capturing) != cudaSuccess || capturing != cudaStreamCaptureStatusNone) {
    cudaGetLastError();
    return nullptr;  // never set up inside a capture; the next eager call does it
  }
  if (!g_host_status) {
    void* host = nullptr;
    if (cudaHostAlloc(&host, sizeof(int32_t) * 2 * kMaxDevices, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    memset(host, 0, sizeof(int32_t) * 2 * kMaxDevices);
    g_host_status = static_cast<int32_t*>(host);
  }
  void* device_view = nullptr;
  if (cudaHostGetDevicePointer(&device_view, g_host_status + 2 * dev, 0) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  g_host_status_dev[dev] = static_cast<int32_t*>(device_view);
  return g_host_status_dev[dev];
}

// Entry-point check: an sm_100 device is current and no earlier kernel on it reported a failed wait.
int check_device() {
  int rc = aklr::require_sm100_device(g_error, sizeof(g_error));
  if (rc) return rc;
  int dev = 0;
  cudaGetDevice(&dev);
  if (g_host_status && dev >= 0 && dev < kMaxDevices) {
    volatile int32_t* words = g_host_status + 2 * dev;
    const int32_t code = words[0];
    if (code != 0) {
      const int32_t where = words[1];
      words[0] = 0;
      words[1] = 0;
      return fail(code, "a kernel of an earlier call on device %d gave up a wait (location %d): what that call and the "
                        "calls after it wrote is not valid; this call launched nothing", dev, where);
    }
  }
  return AKLR_OK;
}

// Waits on a barrier nothing arrives on, with the caller's limit: what a stuck pipeline looks like
// to the error path, without one (aklr_selftest_wait_expiry).
__global__ void wait_expiry_kernel(long long limit_cycles, int32_t* status, int32_t* host_status) {
  __shared__ uint64_t never;
  __shared__ int abort_word;
  if (threadIdx.x == 0) {
    aklr::mbar_init(&never, 1);
    abort_word = 0;
    aklr::fence_mbar_init();
    volatile int* abort_flag = &abort_word;
    aklr::mbar_wait(&never, 0, abort_flag, status, 99, limit_cycles);
    if (abort_word) aklr::publish_wait_failure(status, host_status);
  }
}

int pick_block_m(const aklr_moe_config& c) {
  if (c.block_m) return c.block_m;
  const double avg = static_cast<double>(c.n_tokens) * c.topk / (c.n_routed > 0 ? c.n_routed : 1);
  // Measured on the DeepSeek-V3 layer: from ~28 rows per expert the token-major kernels on 128-token
  // blocks (mostly padding at that point) already beat the weight-major ones on smaller blocks --
  // T=1024 (32 rows per expert): 2.28-2.57 ms against 2.66 (block 32) and 2.60-2.67 (block 64); T=768 (24):
  // 2.38-2.44 ms against 2.19-2.23 (block 32) and 2.54 (block 64).  Blocks of 64 lose to blocks of 32 at every
  // count from 384 to 1536 tokens (their down projection has no 256-channel tiles), so they are never picked.
  if (avg >= 28.0) return 128;
  int bm = 16;
  while (bm < 32 && bm < avg * 1.5) bm *= 2;
  return bm;
}

int check_config(const aklr_moe_config& c) {
  if (c.n_tokens < 0 || c.hidden < 128 || c.inter < 128 || c.hidden % 128 || c.inter % 128)
    return fail(AKLR_ERR_UNSUPPORTED_SHAPE, "hidden (%d) and inter (%d) must be positive multiples of 128", c.hidden, c.inter);
  if (c.n_routed < 1 || c.n_routed > 1024 || c.n_shared < 0 || c.topk < 1 || c.topk + c.n_shared > 32 || c.topk > c.n_routed)
    return fail(AKLR_ERR_UNSUPPORTED_SHAPE, "n_routed=%d topk=%d n_shared=%d is outside 1..1024 experts, <=32 routes", c.n_routed, c.topk, c.n_shared);
  if (c.block_m != 0 && c.block_m != 16 && c.block_m != 32 && c.block_m != 64 && c.block_m != 128)
    return fail(AKLR_ERR_BAD_ARGUMENT, "block_m must be 0, 16, 32, 64 or 128");
  if (static_cast<int64_t>(c.n_tokens) * (c.topk + c.n_shared) > (1ll << 30))
    return fail(AKLR_ERR_TOO_LARGE, "too many routes");
  return AKLR_OK;
}

int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

void layout_of(const aklr_moe_config& c, aklr_moe_workspace_layout* l) {
  const int64_t routes_per_token = c.topk + c.n_shared;
  const int64_t routes = static_cast<int64_t>(c.n_tokens) * routes_per_token;
  const int64_t experts = c.n_routed + c.n_shared;
  const int bm = pick_block_m(c);
  int64_t max_blocks = aklr::align_max_blocks(routes, experts, bm);
  if (max_blocks < 1) max_blocks = 1;
  const int64_t cap = max_blocks * bm;
  const int64_t chunks = (routes + 1023) / 1024;
  int64_t at = 0;
  auto take = [&](int64_t bytes, int64_t align) {
    at = align_up(at, align);
    const int64_t here = at;
    at += bytes;
    return here;
  };
  l->status = take(16, 256);
  l->num_blocks = take(16, 16);
  l->topk_ids = take(routes * 4, 256);
  l->topk_weights = take(routes * 4, 256);
  l->sorted_ids = take(cap * 4, 256);
  l->block_expert = take(max_blocks * 8, 256);  // block -> expert, then the table of block pairs
  l->counts = take(experts * 4, 256);
  l->chunk_hist = take((chunks > 0 ? chunks : 1) * experts * 4, 256);
  // activations kept in bf16 travel as two e4m3 terms: every one of these four buffers twice, the
  // second term right after the first (offsets below name the first)
  const int64_t terms = bf16_activations(c) ? 2 : 1;
  l->xq = take(terms * align_up(cap * c.hidden, 1024), 1024);
  l->xs = take(terms * align_up(cap * (c.hidden / 128) * 4, 256), 256);
  l->hq = take(terms * align_up(cap * c.inter, 1024), 1024);
  l->hs = take(terms * align_up(cap * (c.inter / 128) * 4, 256), 256);
  l->rows = take(routes * c.hidden * 2, 1024);
  l->total_bytes = align_up(at, 256);
  l->block_m = bm;
  l->max_blocks = static_cast<int32_t>(max_blocks);
  l->capacity = static_cast<int32_t>(cap);
  l->n_experts = static_cast<int32_t>(experts);
}

// Everything after the routing table exists: sort, quantise, two grouped GEMMs, combine.
aklr::RouteParams route_params(const aklr_moe_config& c, const void* logits, const void* bias, const float* sigmoid_table,
                               int32_t* topk_ids, float* topk_weights) {
  aklr::RouteParams p{};
  p.logits = logits;
  p.bias = bias;
  p.sigmoid_table = sigmoid_table;
  p.topk_ids = topk_ids;
  p.topk_weights = topk_weights;
  p.n_tokens = c.n_tokens;
  p.n_routed = c.n_routed;
  p.n_shared = c.n_shared;
  p.topk = c.topk;
  p.scoring = c.scoring;
  p.num_expert_group = c.num_expert_group < 1 ? 1 : c.num_expert_group;
  p.topk_group = c.topk_group < 1 ? 1 : c.topk_group;
  p.renormalize = c.renormalize;
  p.logits_are_bf16 = c.logits_dtype == AKLR_DTYPE_BF16;
  p.bias_is_bf16 = c.bias_dtype == AKLR_DTYPE_BF16;
  p.routed_scaling_factor = c.routed_scaling_factor;
  return p;
}

// Whether a call's routing and sort run as the one-CTA decode prologue.
bool fused_prologue_serves(const aklr_moe_config& c) {
  return (c.variant & AKLR_VARIANT_SEPARATE_PROLOGUE) == 0 && c.n_tokens >= 1 && c.n_tokens <= aklr::kDecodePrologueTokens && c.n_routed <= aklr::kDecodePrologueExperts &&
         c.n_tokens * (c.topk + c.n_shared) <= 1024 &&
         (c.num_expert_group > 1 && c.topk_group < c.num_expert_group ? c.num_expert_group : 1) * c.topk <=
             aklr::kDecodePrologueExperts;
}

int run_experts(const aklr_moe_config& c, const aklr_moe_workspace_layout& l, const void* hidden_states,
                const int32_t* topk_ids, const float* topk_weights, const int32_t* expert_map,
                int n_experts_global, const void* w1, const float* w1_scale, const void* w2,
                const float* w2_scale, void* out, uint8_t* ws, cudaStream_t stream, int slot,
                const uint8_t* q_in = nullptr, const float* scales_in = nullptr, void* rows_out = nullptr,
                const aklr::RouteParams* route = nullptr, int q_in_stride = 0, int scales_in_stride = 0) {
  // q_in/scales_in: the rows arrive already quantised (expert-parallel receive side);
  // rows_out: write the weighted per-route rows there and skip the combine;
  // route: the routing has not run yet -- a decode batch does it and the sort in one kernel (the
  // caller checked fused_prologue_serves).
  using namespace aklr;
  const int routes_per_token = c.topk + c.n_shared;
  const int routes = c.n_tokens * routes_per_token;
  const int experts = c.n_routed + c.n_shared;
  int32_t* status = reinterpret_cast<int32_t*>(ws + l.status);
  int32_t* num_blocks = reinterpret_cast<int32_t*>(ws + l.num_blocks);
  int32_t* sorted_ids = reinterpret_cast<int32_t*>(ws + l.sorted_ids);
  int32_t* block_expert = reinterpret_cast<int32_t*>(ws + l.block_expert);

  AlignParams ap{};
  ap.topk_ids = topk_ids;
  ap.expert_map = expert_map;
  ap.sorted_ids = sorted_ids;
  ap.block_expert = block_expert;
  ap.counts = reinterpret_cast<int32_t*>(ws + l.counts);
  ap.num_blocks = num_blocks;
  ap.chunk_hist = reinterpret_cast<int32_t*>(ws + l.chunk_hist);
  ap.n_routes = routes;
  ap.n_experts = experts;
  ap.n_experts_global = n_experts_global;
  ap.block_m = l.block_m;
  const bool tiled = tiled_weights(c);  // [expert][row tile][K-block][128][128]: the maps below are over tiles
  const bool pairs = l.block_m == 128 && !force_weight_major(c) && use_cta_pairs(c) && !tiled &&
                     grouped_gemm_is_token_major(true, l.block_m, c.inter) &&
                     grouped_gemm_is_token_major(false, l.block_m, c.hidden);
  int32_t* pair_table = block_expert + l.max_blocks;  // second half of the block table's space
  if (pairs) ap.pair_table = pair_table;
  int rc = AKLR_OK;
  if (route) {
    rc = launch_decode_prologue(*route, ap, stream);
    if (rc) return fail(rc, "decode prologue launch failed");
    g_launches += 1;
  } else {
    rc = launch_align(ap, stream);
    if (rc) return fail(rc, "moe_align launch failed");
    g_launches += routes <= 4096 ? 1 : 3;
  }
  profile_mark(stream, slot, 2);

  GatherQuantParams qp{};
  qp.x = hidden_states;
  qp.sorted_ids = sorted_ids;
  qp.num_rows = num_blocks + 1;
  qp.q = ws + l.xq;
  qp.scales = reinterpret_cast<float*>(ws + l.xs);
  qp.n_rows = l.capacity;
  qp.hidden = c.hidden;
  qp.routes_per_token = routes_per_token;
  qp.block_m = l.block_m;
  qp.q_in = q_in;
  qp.scales_in = scales_in;
  qp.q_in_stride = q_in_stride;
  qp.scales_in_stride = scales_in_stride;
  qp.zero_padding = l.block_m == 128;  // the token-major GEMM is where the padding rows' operands cost clock
  if (!q_in && routes_per_token > 1 && c.n_tokens >= kQuantOncePerTokenFrom) {
    // A token's routes all carry the same quantised row: quantise every token once, then copy.
    // The per-route output rows are not written before the down projection, so their space
    // holds the per-token codes and scales until then.
    uint8_t* tq = ws + l.rows;
    float* ts = reinterpret_cast<float*>(tq + align_up(static_cast<int64_t>(c.n_tokens) * c.hidden, 256));
    GatherQuantParams tp{};
    tp.x = hidden_states;
    tp.q = tq;
    tp.scales = ts;
    tp.n_rows = c.n_tokens;
    tp.hidden = c.hidden;
    tp.routes_per_token = 1;
    rc = launch_gather_quant_fp8(tp, stream);
    if (rc) return fail(rc, "activation quant launch failed");
    g_launches += 1;
    qp.q_in = tq;
    qp.scales_in = ts;
    rc = launch_gather_rows_fp8(qp, stream);
  } else {
    rc = q_in ? launch_gather_rows_fp8(qp, stream) : launch_gather_quant_fp8(qp, stream);
  }
  if (rc) return fail(rc, "activation quant launch failed");
  g_launches += 1;
  profile_mark(stream, slot, 3);

  const int sms = sm_count();
  GroupedGemmParams g1{};
  // 128-token blocks on 128 x 128 tiles, four partials in flight (both projections or neither)
  const bool deep = l.block_m == 128 && deep_pipeline(c) && !pairs && !force_weight_major(c) && c.inter % 128 == 0 &&
                    c.hidden % 128 == 0;
  rc = tiled ? make_map_u8(&g1.map_w, w1, static_cast<uint64_t>(experts) * 2 * c.inter * (c.hidden / 128), 128, deep ? 64 : 128)
             : make_map_u8(&g1.map_w, w1, static_cast<uint64_t>(experts) * 2 * c.inter, c.hidden, deep ? 64 : 128);
  g1.w_tiled = tiled ? 1 : 0;
  if (rc) return rc;
  rc = make_map_u8(&g1.map_x, ws + l.xq, l.capacity, c.hidden, l.block_m);
  if (rc) return rc;
  g1.w_scale = w1_scale;
  g1.x_scale = reinterpret_cast<const float*>(ws + l.xs);
  g1.sorted_ids = sorted_ids;
  g1.block_expert = block_expert;
  g1.num_blocks = num_blocks;
  g1.out_q = ws + l.hq;
  g1.out_scale = reinterpret_cast<float*>(ws + l.hs);
  g1.status = status;
  g1.host_status = aklr::host_visible_status(stream);
  g1.k = c.hidden;
  g1.out_dim = c.inter;
  g1.rows_per_expert = 2 * c.inter;
  g1.block_m = l.block_m;
  g1.max_blocks = l.max_blocks;
  const bool tm1 = grouped_gemm_is_token_major(true, l.block_m, c.inter);  // at 128 tokens per block always
  g1.pair_table = pairs ? pair_table : nullptr;
  g1.stages = deep ? grouped_gemm_deep_pick_stages(true)
              : tm1 ? grouped_gemm_prefill_pick_stages(true, pairs) : grouped_gemm_pick_stages(true, l.block_m, c.hidden);
  if (g1.stages < 2) return fail(AKLR_ERR_UNSUPPORTED_SHAPE, "hidden=%d needs more shared memory than one SM has", c.hidden);
  rc = deep ? launch_grouped_gemm_deep(g1, true, sms, stream)
       : tm1 ? launch_grouped_gemm_prefill(g1, true, pairs, sms, stream) : launch_grouped_gemm_gate_up(g1, sms, stream);
  if (rc) return fail(rc, "gate_up grouped GEMM launch failed");
  g_launches += 1;
  profile_mark(stream, slot, 4);

  GroupedGemmParams g2{};
  const bool tm2 = grouped_gemm_is_token_major(false, l.block_m, c.hidden) && !force_weight_major(c);
  rc = tiled ? make_map_u8(&g2.map_w, w2, static_cast<uint64_t>(experts) * c.hidden * (c.inter / 128), 128, 128)
             : make_map_u8(&g2.map_w, w2, static_cast<uint64_t>(experts) * c.hidden, c.inter, tm2 && !pairs && !deep ? 256 : 128);
  g2.w_tiled = tiled ? 1 : 0;
  if (rc) return rc;
  rc = make_map_u8(&g2.map_x, ws + l.hq, l.capacity, c.inter, l.block_m);
  if (rc) return rc;
  g2.w_scale = w2_scale;
  g2.x_scale = reinterpret_cast<const float*>(ws + l.hs);
  g2.sorted_ids = sorted_ids;
  g2.block_expert = block_expert;
  g2.num_blocks = num_blocks;
  g2.topk_weights = topk_weights;
  g2.out_rows = rows_out ? rows_out : ws + l.rows;
  g2.status = status;
  g2.host_status = g1.host_status;
  g2.k = c.inter;
  g2.out_dim = c.hidden;
  g2.rows_per_expert = c.hidden;
  g2.block_m = l.block_m;
  g2.max_blocks = l.max_blocks;
  g2.pair_table = pairs ? pair_table : nullptr;
  const bool wide2 = !tm2 && !deep && grouped_gemm_down_is_wide(l.block_m, c.hidden, l.max_blocks, sms);
  g2.wide = wide2 ? 1 : 0;
  g2.stages = deep ? grouped_gemm_deep_pick_stages(false)
              : tm2 ? grouped_gemm_prefill_pick_stages(false, pairs) : grouped_gemm_pick_stages(false, l.block_m, c.inter, wide2);
  if (g2.stages < 2) return fail(AKLR_ERR_UNSUPPORTED_SHAPE, "inter=%d needs more shared memory than one SM has", c.inter);
  rc = deep ? launch_grouped_gemm_deep(g2, false, sms, stream)
       : tm2 ? launch_grouped_gemm_prefill(g2, false, pairs, sms, stream) : launch_grouped_gemm_down(g2, sms, stream);
  if (rc) return fail(rc, "down grouped GEMM launch failed");
  g_launches += 1;
  profile_mark(stream, slot, 5);

  if (rows_out) {
    profile_mark(stream, slot, 6);
    return AKLR_OK;
  }
  CombineParams cp{};
  cp.rows = ws + l.rows;
  cp.topk_ids = topk_ids;
  cp.expert_map = expert_map;
  cp.out = out;
  cp.n_tokens = c.n_tokens;
  cp.hidden = c.hidden;
  cp.routes_per_token = routes_per_token;
  cp.n_experts_global = n_experts_global;
  rc = launch_combine(cp, stream);
  if (rc) return fail(rc, "combine launch failed");
  g_launches += 1;
  profile_mark(stream, slot, 6);
  return AKLR_OK;
}

// MXFP4 experts after the routing table exists: sort, MXFP8 quant, two block-scaled GEMMs, combine.
int run_mx_experts(const aklr_moe_config& c, const aklr_moe_workspace_layout& l, const void* hidden_states,
                   const int32_t* topk_ids, const float* topk_weights, const int32_t* expert_map,
                   int n_experts_global, const void* w1, const uint8_t* w1_scale, const void* w2,
                   const uint8_t* w2_scale, const aklr_mx_options& opt, void* out, uint8_t* ws, cudaStream_t stream,
                   const uint8_t* q_in = nullptr, const uint8_t* scales_in = nullptr, void* rows_out = nullptr,
                   int slot = -1, int q_in_stride = 0, int scales_in_stride = 0) {
  using namespace aklr;
  if (tiled_weights(c)) return fail(AKLR_ERR_BAD_ARGUMENT, "the tile-contiguous weight layout is an FP8 layout: packed MXFP4 weights stay row-major");
  const int routes_per_token = c.topk + c.n_shared;
  const int routes = c.n_tokens * routes_per_token;
  const int experts = c.n_routed + c.n_shared;
  int32_t* status = reinterpret_cast<int32_t*>(ws + l.status);
  int32_t* num_blocks = reinterpret_cast<int32_t*>(ws + l.num_blocks);
  int32_t* sorted_ids = reinterpret_cast<int32_t*>(ws + l.sorted_ids);
  int32_t* block_expert = reinterpret_cast<int32_t*>(ws + l.block_expert);

  AlignParams ap{};
  ap.topk_ids = topk_ids;
  ap.expert_map = expert_map;
  ap.sorted_ids = sorted_ids;
  ap.block_expert = block_expert;
  ap.counts = reinterpret_cast<int32_t*>(ws + l.counts);
  ap.num_blocks = num_blocks;
  ap.chunk_hist = reinterpret_cast<int32_t*>(ws + l.chunk_hist);
  ap.n_routes = routes;
  ap.n_experts = experts;
  ap.n_experts_global = n_experts_global;
  ap.block_m = 128;
  ap.num_local_tokens = opt.num_local_tokens;
  ap.routes_per_token = routes_per_token;
  int rc = launch_align(ap, stream);
  if (rc) return fail(rc, "moe_align launch failed");
  g_launches += routes <= 4096 ? 1 : 3;
  profile_mark(stream, slot, 2);

  MxQuantParams qp{};
  qp.x = hidden_states;
  qp.sorted_ids = sorted_ids;
  qp.num_rows = num_blocks + 1;
  qp.q = ws + l.xq;
  qp.scales = ws + l.xs;
  qp.n_rows = l.capacity;
  qp.hidden = c.hidden;
  qp.routes_per_token = routes_per_token;
  qp.q_in = q_in;
  qp.scales_in = scales_in;
  qp.q_in_stride = q_in_stride;
  qp.scales_in_stride = scales_in_stride;
  const bool split = bf16_activations(c);
  const bool fp4 = mxfp4_activations(c);
  if (split && fp4) return fail(AKLR_ERR_BAD_ARGUMENT, "activations are kept in bf16 or quantised to MXFP4, not both");
  if (fp4 && q_in) return fail(AKLR_ERR_BAD_ARGUMENT, "rows that arrive quantised are MXFP8");
  qp.act_fp4 = fp4;
  qp.zero_padding = small_activation_boxes(c) && !split ? 2 : 1;
  const int64_t cap = l.capacity;
  uint8_t* xq_lo = ws + l.xq + align_up(cap * c.hidden, 1024);
  uint8_t* xs_lo = ws + l.xs + align_up(cap * (c.hidden / 128) * 4, 256);
  uint8_t* hq_lo = ws + l.hq + align_up(cap * c.inter, 1024);
  uint8_t* hs_lo = ws + l.hs + align_up(cap * (c.inter / 128) * 4, 256);
  if (split) {
    if (q_in) return fail(AKLR_ERR_BAD_ARGUMENT, "rows that arrive quantised cannot be bf16 activations");
    qp.q_lo = xq_lo;
    qp.scales_lo = xs_lo;
  }
  if (!split && !q_in && routes_per_token > 1 && c.n_tokens >= kQuantOncePerTokenFrom) {
    // quantise every token once (codes and row-major scale bytes parked in the space of the
    // per-route output rows, unused until the down projection), then copy per route
    uint8_t* tq = ws + l.rows;
    uint8_t* ts = tq + align_up(static_cast<int64_t>(c.n_tokens) * c.hidden, 256);
    MxQuantParams tp{};
    tp.x = hidden_states;
    tp.q = tq;
    tp.scales = ts;
    tp.n_rows = c.n_tokens;
    tp.hidden = c.hidden;
    tp.routes_per_token = 1;
    tp.row_major_scales = 1;
    tp.act_fp4 = fp4;
    rc = launch_gather_quant_mxfp8(tp, stream);
    if (rc) return fail(rc, "MXFP8 activation quant launch failed");
    g_launches += 1;
    qp.q_in = tq;
    qp.scales_in = ts;
  }
  rc = launch_gather_quant_mxfp8(qp, stream);
  if (rc) return fail(rc, "MXFP8 activation quant launch failed");
  g_launches += 1;
  profile_mark(stream, slot, 3);

  const int sms = sm_count();
  MxGemmParams g1{};
  rc = make_map_fp4(&g1.map_w, w1, static_cast<uint64_t>(experts) * 2 * c.inter, c.hidden, 128);
  if (rc) return rc;
  rc = make_map_u8(&g1.map_x, ws + l.xq, l.capacity, c.hidden, 128);
  if (rc) return rc;
  rc = make_map_u8(&g1.map_x_rows32, ws + l.xq, l.capacity, c.hidden, 32);
  if (rc) return rc;
  rc = make_map_u8(&g1.map_x_rows64, ws + l.xq, l.capacity, c.hidden, 64);
  if (rc) return rc;
  g1.small_boxes = small_activation_boxes(c) && !split;
  g1.split = split;
  g1.act_fp4 = fp4;
  if (split) {
    rc = make_map_u8(&g1.map_x_lo, xq_lo, l.capacity, c.hidden, 128);
    if (rc) return rc;
    g1.x_scale_lo = xs_lo;
    g1.out_q_lo = hq_lo;
    g1.out_scale_lo = hs_lo;
  }
  g1.w_scale = w1_scale;
  g1.x_scale = ws + l.xs;
  g1.sorted_ids = sorted_ids;
  g1.block_expert = block_expert;
  g1.num_blocks = num_blocks;
  g1.out_q = ws + l.hq;
  g1.out_scale = ws + l.hs;
  g1.status = status;
  g1.host_status = aklr::host_visible_status(stream);
  g1.swiglu_limit = opt.swiglu_limit;
  g1.activation = opt.activation;
  g1.beta = opt.beta;
  g1.linear_beta = opt.linear_beta;
  g1.stage1_weights = opt.weight_in_stage1 ? topk_weights : nullptr;
  g1.k = c.hidden;
  g1.out_dim = c.inter;
  g1.rows_per_expert = 2 * c.inter;
  g1.max_blocks = l.max_blocks;
  g1.stages = grouped_gemm_mx_pick_stages(true, split);
  rc = launch_grouped_gemm_mx(g1, true, sms, stream);
  if (rc) return fail(rc, "MX gate_up grouped GEMM launch failed");
  g_launches += 1;
  profile_mark(stream, slot, 4);

  MxGemmParams g2{};
  rc = make_map_fp4(&g2.map_w, w2, static_cast<uint64_t>(experts) * c.hidden, c.inter, 256);
  if (rc) return rc;
  rc = make_map_u8(&g2.map_x, ws + l.hq, l.capacity, c.inter, 128);
  if (rc) return rc;
  rc = make_map_u8(&g2.map_x_rows32, ws + l.hq, l.capacity, c.inter, 32);
  if (rc) return rc;
  rc = make_map_u8(&g2.map_x_rows64, ws + l.hq, l.capacity, c.inter, 64);
  if (rc) return rc;
  g2.small_boxes = small_activation_boxes(c) && !split;
  g2.split = split;
  if (split) {
    rc = make_map_u8(&g2.map_x_lo, hq_lo, l.capacity, c.inter, 128);
    if (rc) return rc;
    g2.x_scale_lo = hs_lo;
  }
  g2.w_scale = w2_scale;
  g2.x_scale = ws + l.hs;
  g2.sorted_ids = sorted_ids;
  g2.block_expert = block_expert;
  g2.num_blocks = num_blocks;
  g2.topk_weights = opt.weight_in_stage1 ? nullptr : topk_weights;
  g2.out_rows = rows_out ? rows_out : ws + l.rows;
  g2.status = status;
  g2.host_status = g1.host_status;
  g2.k = c.inter;
  g2.out_dim = c.hidden;
  g2.rows_per_expert = c.hidden;
  g2.max_blocks = l.max_blocks;
  g2.stages = grouped_gemm_mx_pick_stages(false, split);
  rc = launch_grouped_gemm_mx(g2, false, sms, stream);
  if (rc) return fail(rc, "MX down grouped GEMM launch failed");
  g_launches += 1;
  profile_mark(stream, slot, 5);
  if (rows_out) {
    profile_mark(stream, slot, 6);
    return AKLR_OK;
  }

  CombineParams cp{};
  cp.rows = ws + l.rows;
  cp.topk_ids = topk_ids;
  cp.expert_map = expert_map;
  cp.out = out;
  cp.n_tokens = c.n_tokens;
  cp.hidden = c.hidden;
  cp.routes_per_token = routes_per_token;
  cp.n_experts_global = n_experts_global;
  cp.num_local_tokens = opt.num_local_tokens;
  rc = launch_combine(cp, stream);
  if (rc) return fail(rc, "combine launch failed");
  g_launches += 1;
  profile_mark(stream, slot, 6);
  return AKLR_OK;
}

aklr_mx_options clamp_only(float swiglu_limit) {
  aklr_mx_options opt{};
  opt.swiglu_limit = swiglu_limit;
  return opt;
}

int prepare(const aklr_moe_config* cfg, aklr_moe_workspace_layout* l, void* workspace, size_t workspace_bytes,
            cudaStream_t stream) {
  if (!cfg) return fail(AKLR_ERR_BAD_ARGUMENT, "cfg is NULL");
  int rc = check_config(*cfg);
  if (rc) return rc;
  rc = check_device();
  if (rc) return rc;
  layout_of(*cfg, l);
  if (!workspace || workspace_bytes < static_cast<size_t>(l->total_bytes))
    return fail(AKLR_ERR_WORKSPACE_TOO_SMALL, "workspace holds %zu bytes, the call needs %lld", workspace_bytes,
                static_cast<long long>(l->total_bytes));
  if (reinterpret_cast<uintptr_t>(workspace) % 1024 != 0)
    return fail(AKLR_ERR_BAD_ARGUMENT, "workspace must be 1024-byte aligned");
  const cudaError_t err = cudaMemsetAsync(static_cast<uint8_t*>(workspace) + l->status, 0, 32, stream);
  if (err != cudaSuccess) return cuda_fail(err, "clearing the status words");
  return AKLR_OK;
}

}  // namespace

namespace aklr {
int require_sm100_device(char* message, size_t message_bytes) {
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    snprintf(message, message_bytes, "no CUDA device is current");
    return AKLR_ERR_NO_DEVICE;
  }
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (major != 10) {
    snprintf(message, message_bytes, "this library holds sm_100a code only; device has capability %d.x", major);
    return AKLR_ERR_NO_DEVICE;
  }
  return AKLR_OK;
}
void count_kernel_launches(int n) { g_launches += n; }
int32_t* host_visible_status(cudaStream_t stream) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  return host_status_words(dev, stream);
}
}  // namespace aklr

extern "C" {

int aklr_abi_version(void) { return AKLR_B200_ABI_VERSION; }

const char* aklr_status_string(int code) {
  switch (code) {
    case AKLR_OK: return "ok";
    case AKLR_ERR_BAD_ARGUMENT: return "bad argument";
    case AKLR_ERR_WORKSPACE_TOO_SMALL: return "workspace too small";
    case AKLR_ERR_CUDA: return "CUDA runtime or driver error";
    case AKLR_ERR_UNSUPPORTED_SHAPE: return "unsupported shape";
    case AKLR_ERR_NO_DEVICE: return "no sm_100 device";
    case AKLR_ERR_KERNEL_WAIT_TIMEOUT: return "a device-side wait gave up";
    case AKLR_ERR_TOO_LARGE: return "problem too large";
    default: return "unknown status";
  }
}

const char* aklr_last_error(void) { return g_error; }

int aklr_moe_fp8_workspace(const aklr_moe_config* cfg, aklr_moe_workspace_layout* layout) {
  if (!cfg || !layout) return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  const int rc = check_config(*cfg);
  if (rc) return rc;
  layout_of(*cfg, layout);
  return AKLR_OK;
}

int aklr_moe_fp8_forward(const aklr_moe_config* cfg, const void* hidden_states, const void* logits,
                         const void* bias, const float* sigmoid_table, const void* w1, const float* w1_scale,
                         const void* w2, const float* w2_scale, void* out, void* workspace,
                         size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  aklr_moe_workspace_layout l;
  int rc = prepare(cfg, &l, workspace, workspace_bytes, stream);
  if (rc) return rc;
  if (cfg->n_tokens == 0) return AKLR_OK;  // nothing to do; empty tensors may have NULL pointers
  if (!hidden_states || !logits || !w1 || !w1_scale || !w2 || !w2_scale || !out)
    return fail(AKLR_ERR_BAD_ARGUMENT, "NULL tensor argument");
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int32_t* ids = reinterpret_cast<int32_t*>(ws + l.topk_ids);
  float* weights = reinterpret_cast<float*>(ws + l.topk_weights);
  const int slot = profile_slot();
  profile_mark(stream, slot, 0);
  if (fused_prologue_serves(*cfg)) {
    const aklr::RouteParams route = route_params(*cfg, logits, bias, sigmoid_table, ids, weights);
    profile_mark(stream, slot, 1);
    return run_experts(*cfg, l, hidden_states, ids, weights, nullptr, cfg->n_routed + cfg->n_shared, w1, w1_scale, w2,
                       w2_scale, out, ws, stream, slot, nullptr, nullptr, nullptr, &route);
  }
  rc = aklr_moe_route(cfg, logits, bias, sigmoid_table, ids, weights, stream_);
  if (rc) return rc;
  profile_mark(stream, slot, 1);
  return run_experts(*cfg, l, hidden_states, ids, weights, nullptr, cfg->n_routed + cfg->n_shared, w1, w1_scale, w2,
                     w2_scale, out, ws, stream, slot);
}

int aklr_moe_fp8_experts(const aklr_moe_config* cfg, const void* hidden_states, const int32_t* topk_ids,
                         const float* topk_weights, const int32_t* expert_map, const void* w1,
                         const float* w1_scale, const void* w2, const float* w2_scale, void* out,
                         void* workspace, size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  aklr_moe_workspace_layout l;
  int rc = prepare(cfg, &l, workspace, workspace_bytes, stream);
  if (rc) return rc;
  if (cfg->n_tokens == 0) return AKLR_OK;
  if (!hidden_states || !topk_ids || !topk_weights || !w1 || !w1_scale || !w2 || !w2_scale || !out)
    return fail(AKLR_ERR_BAD_ARGUMENT, "NULL tensor argument");
  const int local = cfg->n_routed + cfg->n_shared;
  const int global = expert_map ? cfg->n_experts_global : local;
  if (expert_map && global < 1) return fail(AKLR_ERR_BAD_ARGUMENT, "n_experts_global must be set with an expert map");
  const int slot = profile_slot();
  profile_mark(stream, slot, 0);
  profile_mark(stream, slot, 1);
  return run_experts(*cfg, l, hidden_states, topk_ids, topk_weights, expert_map, global, w1, w1_scale, w2, w2_scale,
                     out, static_cast<uint8_t*>(workspace), stream, slot);
}

int aklr_moe_fp8_experts_prequant(const aklr_moe_config* cfg, const void* rows_q, const float* rows_scale,
                                  const int32_t* expert_ids, const float* weights, const void* w1,
                                  const float* w1_scale, const void* w2, const float* w2_scale, void* out_rows,
                                  void* workspace, size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  aklr_moe_workspace_layout l;
  if (cfg && (cfg->topk != 1 || cfg->n_shared != 0)) return fail(AKLR_ERR_BAD_ARGUMENT, "prequantised rows carry one route each: topk 1, n_shared 0");
  int rc = prepare(cfg, &l, workspace, workspace_bytes, stream);
  if (rc) return rc;
  if (cfg->n_tokens == 0) return AKLR_OK;
  if (!rows_q || !rows_scale || !expert_ids || !weights || !w1 || !w1_scale || !w2 || !w2_scale || !out_rows)
    return fail(AKLR_ERR_BAD_ARGUMENT, "NULL tensor argument");
  const int slot = profile_slot();
  profile_mark(stream, slot, 0);
  profile_mark(stream, slot, 1);
  return run_experts(*cfg, l, nullptr, expert_ids, weights, nullptr, cfg->n_routed, w1, w1_scale, w2, w2_scale, nullptr,
                     static_cast<uint8_t*>(workspace), stream, slot, static_cast<const uint8_t*>(rows_q), rows_scale,
                     out_rows);
}

int aklr_moe_mxfp4_experts_ex(const aklr_moe_config* cfg, const void* hidden_states, const int32_t* topk_ids,
                              const float* topk_weights, const int32_t* expert_map, const void* w1,
                              const uint8_t* w1_scale, const void* w2, const uint8_t* w2_scale,
                              const aklr_mx_options* options, void* out, void* workspace, size_t workspace_bytes,
                              void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!cfg || !options) return fail(AKLR_ERR_BAD_ARGUMENT, "cfg or options is NULL");
  if (cfg->block_m != 128) return fail(AKLR_ERR_BAD_ARGUMENT, "the MXFP4 path works on 128-token blocks: set block_m = 128");
  if (cfg->hidden % 256 != 0) return fail(AKLR_ERR_UNSUPPORTED_SHAPE, "the MXFP4 path needs hidden %% 256 == 0 (got %d)", cfg->hidden);
  if (options->activation < AKLR_ACT_SILU || options->activation > AKLR_ACT_SITUV2)
    return fail(AKLR_ERR_BAD_ARGUMENT, "activation %d is not one of AKLR_ACT_*", options->activation);
  if (options->activation == AKLR_ACT_SITUV2 && !(options->beta > 0.0f && options->linear_beta > 0.0f))
    return fail(AKLR_ERR_BAD_ARGUMENT, "AKLR_ACT_SITUV2 needs beta > 0 and linear_beta > 0");
  aklr_moe_workspace_layout l;
  int rc = prepare(cfg, &l, workspace, workspace_bytes, stream);
  if (rc) return rc;
  if (cfg->n_tokens == 0) return AKLR_OK;
  if (!hidden_states || !topk_ids || !topk_weights || !w1 || !w1_scale || !w2 || !w2_scale || !out)
    return fail(AKLR_ERR_BAD_ARGUMENT, "NULL tensor argument");
  const int local = cfg->n_routed + cfg->n_shared;
  const int global = expert_map ? cfg->n_experts_global : local;
  if (expert_map && global < 1) return fail(AKLR_ERR_BAD_ARGUMENT, "n_experts_global must be set with an expert map");
  return run_mx_experts(*cfg, l, hidden_states, topk_ids, topk_weights, expert_map, global, w1, w1_scale, w2, w2_scale,
                        *options, out, static_cast<uint8_t*>(workspace), stream);
}

int aklr_moe_mxfp4_experts(const aklr_moe_config* cfg, const void* hidden_states, const int32_t* topk_ids,
                           const float* topk_weights, const int32_t* expert_map, const void* w1,
                           const uint8_t* w1_scale, const void* w2, const uint8_t* w2_scale, float swiglu_limit,
                           void* out, void* workspace, size_t workspace_bytes, void* stream_) {
  const aklr_mx_options options = clamp_only(swiglu_limit);
  return aklr_moe_mxfp4_experts_ex(cfg, hidden_states, topk_ids, topk_weights, expert_map, w1, w1_scale, w2, w2_scale,
                                   &options, out, workspace, workspace_bytes, stream_);
}

int aklr_moe_mxfp4_forward(const aklr_moe_config* cfg, const void* hidden_states, const void* logits,
                           const void* bias, const float* sigmoid_table, const void* w1, const uint8_t* w1_scale,
                           const void* w2, const uint8_t* w2_scale, float swiglu_limit, void* out, void* workspace,
                           size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!cfg) return fail(AKLR_ERR_BAD_ARGUMENT, "cfg is NULL");
  if (cfg->block_m != 128) return fail(AKLR_ERR_BAD_ARGUMENT, "the MXFP4 path works on 128-token blocks: set block_m = 128");
  if (cfg->hidden % 256 != 0) return fail(AKLR_ERR_UNSUPPORTED_SHAPE, "the MXFP4 path needs hidden %% 256 == 0 (got %d)", cfg->hidden);
  aklr_moe_workspace_layout l;
  int rc = prepare(cfg, &l, workspace, workspace_bytes, stream);
  if (rc) return rc;
  if (cfg->n_tokens == 0) return AKLR_OK;
  if (!hidden_states || !logits || !w1 || !w1_scale || !w2 || !w2_scale || !out)
    return fail(AKLR_ERR_BAD_ARGUMENT, "NULL tensor argument");
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int32_t* ids = reinterpret_cast<int32_t*>(ws + l.topk_ids);
  float* weights = reinterpret_cast<float*>(ws + l.topk_weights);
  const int slot = profile_slot();
  profile_mark(stream, slot, 0);
  rc = aklr_moe_route(cfg, logits, bias, sigmoid_table, ids, weights, stream_);
  if (rc) return rc;
  profile_mark(stream, slot, 1);
  return run_mx_experts(*cfg, l, hidden_states, ids, weights, nullptr, cfg->n_routed + cfg->n_shared, w1, w1_scale, w2,
                        w2_scale, clamp_only(swiglu_limit), out, ws, stream, nullptr, nullptr, nullptr, slot);
}

int aklr_moe_mxfp4_experts_prequant(const aklr_moe_config* cfg, const void* rows_q, const uint8_t* rows_scale,
                                    const int32_t* expert_ids, const float* weights, const void* w1,
                                    const uint8_t* w1_scale, const void* w2, const uint8_t* w2_scale,
                                    float swiglu_limit, void* out_rows, void* workspace, size_t workspace_bytes,
                                    void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!cfg) return fail(AKLR_ERR_BAD_ARGUMENT, "cfg is NULL");
  if (cfg->topk != 1 || cfg->n_shared != 0 || cfg->block_m != 128)
    return fail(AKLR_ERR_BAD_ARGUMENT, "prequantised rows carry one route each: topk 1, n_shared 0, block_m 128");
  if (cfg->hidden % 256 != 0) return fail(AKLR_ERR_UNSUPPORTED_SHAPE, "the MXFP4 path needs hidden %% 256 == 0");
  aklr_moe_workspace_layout l;
  int rc = prepare(cfg, &l, workspace, workspace_bytes, stream);
  if (rc) return rc;
  if (cfg->n_tokens == 0) return AKLR_OK;
  if (!rows_q || !rows_scale || !expert_ids || !weights || !w1 || !w1_scale || !w2 || !w2_scale || !out_rows)
    return fail(AKLR_ERR_BAD_ARGUMENT, "NULL tensor argument");
  const int slot = profile_slot();
  profile_mark(stream, slot, 0);
  profile_mark(stream, slot, 1);
  return run_mx_experts(*cfg, l, nullptr, expert_ids, weights, nullptr, cfg->n_routed, w1, w1_scale, w2, w2_scale,
                        clamp_only(swiglu_limit), nullptr, static_cast<uint8_t*>(workspace), stream,
                        static_cast<const uint8_t*>(rows_q), rows_scale, out_rows, slot);
}

int aklr_moe_fp8_experts_rows(const aklr_moe_config* cfg, const void* rows_q, int32_t rows_q_pitch, const float* rows_scale,
                              int32_t rows_scale_pitch, const int32_t* topk_ids, const float* topk_weights, const void* w1,
                              const float* w1_scale, const void* w2, const float* w2_scale, void* out, void* workspace,
                              size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  aklr_moe_workspace_layout l;
  if (cfg && cfg->n_shared != 0) return fail(AKLR_ERR_BAD_ARGUMENT, "rows that arrive quantised have no shared slots: n_shared 0");
  if (rows_q_pitch < 0 || rows_scale_pitch < 0 || rows_q_pitch % 16 != 0 || rows_scale_pitch % 4 != 0)
    return fail(AKLR_ERR_BAD_ARGUMENT, "row pitches must be multiples of 16 (codes) and 4 (scales) bytes, or 0 for dense rows");
  int rc = prepare(cfg, &l, workspace, workspace_bytes, stream);
  if (rc) return rc;
  if (cfg->n_tokens == 0) return AKLR_OK;
  if (!rows_q || !rows_scale || !topk_ids || !topk_weights || !w1 || !w1_scale || !w2 || !w2_scale || !out)
    return fail(AKLR_ERR_BAD_ARGUMENT, "NULL tensor argument");
  if (reinterpret_cast<uintptr_t>(rows_q) % 16 != 0 || reinterpret_cast<uintptr_t>(rows_scale) % 4 != 0)
    return fail(AKLR_ERR_BAD_ARGUMENT, "rows_q must be 16-byte aligned and rows_scale 4-byte aligned");
  const int slot = profile_slot();
  profile_mark(stream, slot, 0);
  profile_mark(stream, slot, 1);
  return run_experts(*cfg, l, nullptr, topk_ids, topk_weights, nullptr, cfg->n_routed, w1, w1_scale, w2, w2_scale, out,
                     static_cast<uint8_t*>(workspace), stream, slot, static_cast<const uint8_t*>(rows_q), rows_scale, nullptr,
                     nullptr, rows_q_pitch, rows_scale_pitch);
}

int aklr_moe_mxfp4_experts_rows(const aklr_moe_config* cfg, const void* rows_q, int32_t rows_q_pitch, const uint8_t* rows_scale,
                                int32_t rows_scale_pitch, const int32_t* topk_ids, const float* topk_weights, const void* w1,
                                const uint8_t* w1_scale, const void* w2, const uint8_t* w2_scale, float swiglu_limit, void* out,
                                void* workspace, size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!cfg) return fail(AKLR_ERR_BAD_ARGUMENT, "cfg is NULL");
  if (cfg->n_shared != 0 || cfg->block_m != 128)
    return fail(AKLR_ERR_BAD_ARGUMENT, "rows that arrive quantised: n_shared 0, block_m 128");
  if (cfg->hidden % 256 != 0) return fail(AKLR_ERR_UNSUPPORTED_SHAPE, "the MXFP4 path needs hidden %% 256 == 0");
  if (rows_q_pitch < 0 || rows_scale_pitch < 0 || rows_q_pitch % 16 != 0 || rows_scale_pitch % 4 != 0)
    return fail(AKLR_ERR_BAD_ARGUMENT, "row pitches must be multiples of 16 (codes) and 4 (scales) bytes, or 0 for dense rows");
  aklr_moe_workspace_layout l;
  int rc = prepare(cfg, &l, workspace, workspace_bytes, stream);
  if (rc) return rc;
  if (cfg->n_tokens == 0) return AKLR_OK;
  if (!rows_q || !rows_scale || !topk_ids || !topk_weights || !w1 || !w1_scale || !w2 || !w2_scale || !out)
    return fail(AKLR_ERR_BAD_ARGUMENT, "NULL tensor argument");
  if (reinterpret_cast<uintptr_t>(rows_q) % 16 != 0 || reinterpret_cast<uintptr_t>(rows_scale) % 4 != 0)
    return fail(AKLR_ERR_BAD_ARGUMENT, "rows_q must be 16-byte aligned and rows_scale 4-byte aligned");
  const int slot = profile_slot();
  profile_mark(stream, slot, 0);
  profile_mark(stream, slot, 1);
  return run_mx_experts(*cfg, l, nullptr, topk_ids, topk_weights, nullptr, cfg->n_routed, w1, w1_scale, w2, w2_scale,
                        clamp_only(swiglu_limit), out, static_cast<uint8_t*>(workspace), stream,
                        static_cast<const uint8_t*>(rows_q), rows_scale, nullptr, slot, rows_q_pitch, rows_scale_pitch);
}

int32_t aklr_ep_row_bytes(int32_t hidden, int32_t topk, int32_t mx) {
  const int scale_bytes = mx ? hidden / 32 : hidden / 128 * 4;
  return (hidden + scale_bytes + 8 * topk + 15) / 16 * 16;
}

int aklr_ep_plan(const int32_t* topk_ids, int32_t n_tokens, int32_t topk, int32_t experts_per_rank, int32_t* first_rank,
                 int32_t* position_of_route, void* stream) {
  if (!topk_ids || !first_rank || !position_of_route) return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  int rc = check_device();
  if (rc) return rc;
  aklr::EpPlanParams p{topk_ids, first_rank, position_of_route, n_tokens, topk, experts_per_rank};
  rc = aklr::launch_ep_first_slots(p, static_cast<cudaStream_t>(stream));
  if (rc) return fail(rc, "ep plan: %s", aklr_status_string(rc));
  g_launches += n_tokens > 0;
  return AKLR_OK;
}

int aklr_ep_pack(const void* tokens_q, const void* tokens_scale, const int32_t* sorted_ids, const int32_t* topk_ids,
                 const float* topk_weights, int32_t n_send, int32_t n_tokens, int32_t topk, int32_t hidden,
                 int32_t experts_per_rank, int32_t mx, const int32_t* n_send_device, void* packed,
                 int32_t* position_of_route, void* stream) {
  if (!tokens_q || !tokens_scale || !sorted_ids || !topk_ids || !topk_weights || !packed || !position_of_route)
    return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  int rc = check_device();
  if (rc) return rc;
  aklr::EpPackParams p{};
  p.tokens_q = static_cast<const uint8_t*>(tokens_q);
  p.tokens_scale = static_cast<const uint8_t*>(tokens_scale);
  p.sorted_ids = sorted_ids;
  p.n_send_device = n_send_device;
  p.topk_ids = topk_ids;
  p.topk_weights = topk_weights;
  p.packed = static_cast<uint8_t*>(packed);
  p.position_of_route = position_of_route;
  p.n_send = n_send;
  p.n_tokens = n_tokens;
  p.topk = topk;
  p.hidden = hidden;
  p.scale_bytes = mx ? hidden / 32 : hidden / 128 * 4;
  p.row_bytes = aklr_ep_row_bytes(hidden, topk, mx);
  p.experts_per_rank = experts_per_rank;
  rc = aklr::launch_ep_pack(p, static_cast<cudaStream_t>(stream));
  if (rc) return fail(rc, "ep pack: %s", aklr_status_string(rc));
  g_launches += n_send > 0;
  return AKLR_OK;
}

int aklr_ep_unpack_meta(const void* packed, int32_t n_rows, int32_t hidden, int32_t topk, int32_t mx, int32_t* topk_ids,
                        float* topk_weights, void* stream) {
  if (!packed || !topk_ids || !topk_weights) return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  int rc = check_device();
  if (rc) return rc;
  const int scale_bytes = mx ? hidden / 32 : hidden / 128 * 4;
  rc = aklr::launch_ep_unpack_meta(static_cast<const uint8_t*>(packed), n_rows, aklr_ep_row_bytes(hidden, topk, mx),
                                   hidden + scale_bytes, topk, topk_ids, topk_weights, static_cast<cudaStream_t>(stream));
  if (rc) return fail(rc, "ep unpack: %s", aklr_status_string(rc));
  g_launches += n_rows > 0;
  return AKLR_OK;
}

int aklr_ep_counts_to_host(const int32_t* send_counts, const int32_t* recv_counts, int32_t world, int32_t* host_mapped,
                           void* stream) {
  if (!send_counts || !recv_counts || !host_mapped) return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  int rc = check_device();
  if (rc) return rc;
  rc = aklr::launch_ep_counts_to_host(send_counts, recv_counts, world, host_mapped, static_cast<cudaStream_t>(stream));
  if (rc) return fail(rc, "ep counts to host: %s", aklr_status_string(rc));
  g_launches += 1;
  return AKLR_OK;
}

int aklr_ep_gather_quant_mxfp8(const void* hidden_states, const int32_t* sorted_ids, int32_t n_send, int32_t hidden,
                               int32_t routes_per_token, void* rows_q, uint8_t* rows_scale, void* stream) {
  if (!hidden_states || !sorted_ids || !rows_q || !rows_scale) return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  int rc = check_device();
  if (rc) return rc;
  aklr::MxQuantParams p{};
  p.x = hidden_states;
  p.sorted_ids = sorted_ids;
  p.q = static_cast<uint8_t*>(rows_q);
  p.scales = rows_scale;
  p.n_rows = n_send;
  p.hidden = hidden;
  p.routes_per_token = routes_per_token;
  p.row_major_scales = 1;
  rc = aklr::launch_gather_quant_mxfp8(p, static_cast<cudaStream_t>(stream));
  if (rc) return fail(rc, "ep MXFP8 gather quant: %s", aklr_status_string(rc));
  g_launches += n_send > 0;
  return AKLR_OK;
}

int aklr_ep_dispatch_meta(const int32_t* sorted_ids, const int32_t* topk_ids, const float* topk_weights,
                          int32_t n_send, int32_t n_routes, int32_t experts_per_rank, int32_t* send_expert,
                          float* send_weight, int32_t* position_of_route, void* stream) {
  if (!sorted_ids || !topk_ids || !topk_weights || !send_expert || !send_weight || !position_of_route || experts_per_rank < 1)
    return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  int rc = check_device();
  if (rc) return rc;
  aklr::EpMetaParams p{sorted_ids, topk_ids, topk_weights, send_expert, send_weight, position_of_route,
                       n_send, n_routes, experts_per_rank};
  rc = aklr::launch_ep_meta(p, static_cast<cudaStream_t>(stream));
  if (rc) return fail(rc, "ep dispatch meta: %s", aklr_status_string(rc));
  g_launches += n_send > 0;
  return AKLR_OK;
}

int aklr_ep_gather_quant(const void* hidden_states, const int32_t* sorted_ids, int32_t n_send, int32_t hidden,
                         int32_t routes_per_token, void* rows_q, float* rows_scale, void* stream) {
  if (!hidden_states || !sorted_ids || !rows_q || !rows_scale) return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  int rc = check_device();
  if (rc) return rc;
  aklr::GatherQuantParams p{};
  p.x = hidden_states;
  p.sorted_ids = sorted_ids;
  p.q = static_cast<uint8_t*>(rows_q);
  p.scales = rows_scale;
  p.n_rows = n_send;
  p.hidden = hidden;
  p.routes_per_token = routes_per_token;
  rc = aklr::launch_gather_quant_fp8(p, static_cast<cudaStream_t>(stream));
  if (rc) return fail(rc, "ep gather quant: %s", aklr_status_string(rc));
  g_launches += n_send > 0;
  return AKLR_OK;
}

int aklr_ep_gather_rows(const void* tokens_q, const void* tokens_scale, const int32_t* sorted_ids, int32_t n_send,
                        int32_t hidden, int32_t routes_per_token, int32_t mx, void* rows_q, void* rows_scale,
                        void* stream) {
  if (!tokens_q || !tokens_scale || !sorted_ids || !rows_q || !rows_scale) return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  int rc = check_device();
  if (rc) return rc;
  if (mx) {
    aklr::MxQuantParams p{};
    p.sorted_ids = sorted_ids;
    p.q = static_cast<uint8_t*>(rows_q);
    p.scales = static_cast<uint8_t*>(rows_scale);
    p.q_in = static_cast<const uint8_t*>(tokens_q);
    p.scales_in = static_cast<const uint8_t*>(tokens_scale);
    p.n_rows = n_send;
    p.hidden = hidden;
    p.routes_per_token = routes_per_token;
    p.row_major_scales = 1;
    rc = aklr::launch_gather_quant_mxfp8(p, static_cast<cudaStream_t>(stream));
  } else {
    aklr::GatherQuantParams p{};
    p.sorted_ids = sorted_ids;
    p.q = static_cast<uint8_t*>(rows_q);
    p.scales = static_cast<float*>(rows_scale);
    p.q_in = static_cast<const uint8_t*>(tokens_q);
    p.scales_in = static_cast<const float*>(tokens_scale);
    p.n_rows = n_send;
    p.hidden = hidden;
    p.routes_per_token = routes_per_token;
    p.block_m = 1;  // [row, hidden/128] scales
    rc = aklr::launch_gather_rows_fp8(p, static_cast<cudaStream_t>(stream));
  }
  if (rc) return fail(rc, "ep gather rows: %s", aklr_status_string(rc));
  g_launches += n_send > 0;
  return AKLR_OK;
}

int aklr_ep_combine(const void* rows, const int32_t* position_of_route, const void* shared_rows, void* out,
                    int32_t n_tokens, int32_t topk, int32_t hidden, void* stream) {
  if (!position_of_route || !out) return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  int rc = check_device();
  if (rc) return rc;
  aklr::EpCombineParams p{rows, position_of_route, shared_rows, out, n_tokens, topk, hidden};
  rc = aklr::launch_ep_combine(p, static_cast<cudaStream_t>(stream));
  if (rc) return fail(rc, "ep combine: %s", aklr_status_string(rc));
  g_launches += n_tokens > 0;
  return AKLR_OK;
}

int aklr_moe_route(const aklr_moe_config* cfg, const void* logits, const void* bias, const float* sigmoid_table,
                   int32_t* topk_ids, float* topk_weights, void* stream) {
  if (!cfg || !logits || !topk_ids || !topk_weights) return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  int rc = check_device();
  if (rc) return rc;
  const aklr::RouteParams p = route_params(*cfg, logits, bias, sigmoid_table, topk_ids, topk_weights);
  rc = aklr::launch_route(p, static_cast<cudaStream_t>(stream));
  if (rc) return fail(rc, "routing: %s", aklr_status_string(rc));
  g_launches += p.n_tokens > 0;
  return AKLR_OK;
}

int aklr_moe_align(const int32_t* topk_ids, const int32_t* expert_map, int32_t n_routes, int32_t n_experts,
                   int32_t n_experts_global, int32_t block_m, int32_t* sorted_ids, int32_t* block_expert,
                   int32_t* counts, int32_t* num_blocks, int32_t* chunk_scratch, void* stream) {
  if (!topk_ids || !sorted_ids || !block_expert || !counts || !num_blocks || !chunk_scratch)
    return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  int rc = check_device();
  if (rc) return rc;
  aklr::AlignParams p{};
  p.topk_ids = topk_ids;
  p.expert_map = expert_map;
  p.sorted_ids = sorted_ids;
  p.block_expert = block_expert;
  p.counts = counts;
  p.num_blocks = num_blocks;
  p.chunk_hist = chunk_scratch;
  p.n_routes = n_routes;
  p.n_experts = n_experts;
  p.n_experts_global = expert_map ? n_experts_global : n_experts;
  p.block_m = block_m;
  rc = aklr::launch_align(p, static_cast<cudaStream_t>(stream));
  if (rc) return fail(rc, "moe_align: %s", aklr_status_string(rc));
  g_launches += n_routes <= 4096 ? 1 : 3;
  return AKLR_OK;
}

int64_t aklr_moe_align_max_blocks(int64_t n_routes, int64_t n_experts, int64_t block_m) {
  return aklr::align_max_blocks(n_routes, n_experts, block_m);
}

int aklr_router_gemm_bf16(const void* x, const void* w, void* logits, int32_t n_tokens, int32_t hidden,
                          int32_t n_routed, void* stream) {
  if (!x || !w || !logits) return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  int rc = check_device();
  if (rc) return rc;
  // 64 tokens and up: tensor cores (128-token tiles); fewer: the warp-per-dot-product kernel, which
  // spreads the router weight over many SMs
  if (n_tokens >= 64 && hidden % 64 == 0 && n_routed >= 1) {
    int n_tile = (n_routed + 15) / 16 * 16;
    if (n_tile > 256) n_tile = 256;
    CUtensorMap map_x, map_w;
    rc = make_map_bf16(&map_x, x, n_tokens, hidden, 128);
    if (rc) return rc;
    rc = make_map_bf16(&map_w, w, n_routed, hidden, n_tile);
    if (rc) return rc;
    rc = aklr::launch_router_gemm_tc(map_x, map_w, logits, n_tokens, hidden, n_routed, n_tile,
                                     aklr::host_visible_status(static_cast<cudaStream_t>(stream)), static_cast<cudaStream_t>(stream));
  } else {
    rc = aklr::launch_router_gemm(x, w, logits, n_tokens, hidden, n_routed, static_cast<cudaStream_t>(stream));
  }
  if (rc) return fail(rc, "router GEMM: %s", aklr_status_string(rc));
  g_launches += 1;
  return AKLR_OK;
}

int aklr_moe_shared_gate(const void* x, const void* shared_gate_weight, const int32_t* topk_ids_in,
                         const float* topk_weights_in, int32_t* topk_ids, float* topk_weights, int32_t n_tokens,
                         int32_t hidden, int32_t topk, int32_t shared_slot, void* stream) {
  if (!x || !shared_gate_weight || !topk_ids || !topk_weights || (!topk_ids_in) != (!topk_weights_in))
    return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  int rc = check_device();
  if (rc) return rc;
  rc = aklr::launch_shared_gate(x, shared_gate_weight, topk_ids_in, topk_weights_in, topk_ids, topk_weights, n_tokens, hidden,
                                topk, shared_slot, static_cast<cudaStream_t>(stream));
  if (rc) return fail(rc, "shared expert gate: %s", aklr_status_string(rc));
  g_launches += n_tokens > 0;
  return AKLR_OK;
}

int aklr_silu_mul_bf16(const void* gate_up, void* out, int32_t n_tokens, int32_t inter, void* stream) {
  if (!gate_up || !out) return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  if (n_tokens < 0) return fail(AKLR_ERR_BAD_ARGUMENT, "n_tokens %d", n_tokens);
  int rc = check_device();
  if (rc) return rc;
  rc = aklr::launch_silu_mul_bf16(gate_up, out, n_tokens, inter, static_cast<cudaStream_t>(stream));
  if (rc) return fail(rc, "silu(gate) * up: %s", aklr_status_string(rc));
  g_launches += n_tokens > 0;
  return AKLR_OK;
}

int aklr_moe_add_gated_rows(const void* x, const void* shared_gate_weight, const void* rows, void* out, int32_t n_tokens,
                            int32_t hidden, void* stream) {
  if (!x || !shared_gate_weight || !rows || !out) return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  if (n_tokens < 0) return fail(AKLR_ERR_BAD_ARGUMENT, "n_tokens %d", n_tokens);
  int rc = check_device();
  if (rc) return rc;
  rc = aklr::launch_add_gated_rows(x, shared_gate_weight, rows, out, n_tokens, hidden, static_cast<cudaStream_t>(stream));
  if (rc) return fail(rc, "gated shared rows: %s", aklr_status_string(rc));
  g_launches += n_tokens > 0;
  return AKLR_OK;
}

int aklr_selftest_exact_divide(const float* x, const float* scale, int64_t n, int32_t* mismatches, void* stream) {
  if (!x || !scale || !mismatches || n < 0) return fail(AKLR_ERR_BAD_ARGUMENT, "bad argument");
  int rc = check_device();
  if (rc) return rc;
  rc = aklr::launch_exact_divide_selftest(x, scale, n, mismatches, static_cast<cudaStream_t>(stream));
  if (rc) return fail(rc, "division self-test launch failed");
  g_launches += n > 0;
  return AKLR_OK;
}

int aklr_tile_weights_fp8(const void* src, void* dst, int64_t matrices, int32_t rows, int32_t cols, void* stream) {
  if (!src || !dst) return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  int rc = check_device();
  if (rc) return rc;
  rc = aklr::launch_tile_weights_fp8(src, dst, matrices, rows, cols, static_cast<cudaStream_t>(stream));
  if (rc) return fail(rc, "tile-contiguous weight layout: %s (rows %d, cols %d, %lld matrices)", aklr_status_string(rc), rows, cols,
                      static_cast<long long>(matrices));
  g_launches += 1;
  return AKLR_OK;
}

int aklr_router_gemm_f32(const void* x, const float* w, float* logits, int32_t n_tokens, int32_t hidden,
                         int32_t n_routed, void* stream) {
  if (!x || !w || !logits) return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  int rc = check_device();
  if (rc) return rc;
  rc = aklr::launch_router_gemm_f32(x, w, logits, n_tokens, hidden, n_routed, static_cast<cudaStream_t>(stream));
  if (rc) return fail(rc, "router GEMM (float32 weights): %s", aklr_status_string(rc));
  g_launches += n_tokens > 0;
  return AKLR_OK;
}

int aklr_per_group_quant_fp8(const void* x, void* q, float* scales, int32_t rows, int32_t hidden, void* stream) {
  if (!x || !q || !scales) return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  int rc = check_device();
  if (rc) return rc;
  rc = aklr::launch_per_group_quant_fp8(x, static_cast<uint8_t*>(q), scales, rows, hidden,
                                        static_cast<cudaStream_t>(stream));
  if (rc) return fail(rc, "per_group_quant_fp8: %s", aklr_status_string(rc));
  g_launches += 1;
  return AKLR_OK;
}

int aklr_per_group_quant_mxfp8(const void* x, void* q, uint8_t* scales, int32_t rows, int32_t hidden,
                               void* stream) {
  if (!x || !q || !scales) return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  int rc = check_device();
  if (rc) return rc;
  rc = aklr::launch_per_group_quant_mxfp8(x, static_cast<uint8_t*>(q), scales, rows, hidden,
                                          static_cast<cudaStream_t>(stream));
  if (rc) return fail(rc, "per_group_quant_mxfp8: %s", aklr_status_string(rc));
  g_launches += 1;
  return AKLR_OK;
}

int aklr_moe_act_quant_fp8(const void* x, void* q, float* scales, int32_t rows, int32_t hidden, void* stream) {
  if (!x || !q || !scales) return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  int rc = check_device();
  if (rc) return rc;
  aklr::GatherQuantParams p{};
  p.x = x;
  p.q = static_cast<uint8_t*>(q);
  p.scales = scales;
  p.n_rows = rows;
  p.hidden = hidden;
  p.routes_per_token = 1;
  rc = aklr::launch_gather_quant_fp8(p, static_cast<cudaStream_t>(stream));
  if (rc) return fail(rc, "activation quant: %s", aklr_status_string(rc));
  g_launches += 1;
  return AKLR_OK;
}

int aklr_moe_read_status(const void* workspace, int32_t* host_status, void* stream_) {
  if (!workspace || !host_status) return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  cudaError_t err = cudaMemcpyAsync(host_status, workspace, 8, cudaMemcpyDeviceToHost, stream);
  if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
  if (err != cudaSuccess) return cuda_fail(err, "reading the status words");
  return host_status[0] == 0 ? AKLR_OK : fail(host_status[0], "device wait gave up at location %d", host_status[1]);
}

int64_t aklr_kernel_launch_count(void) { return g_launches.load(); }

int aklr_device_status(int32_t* code_and_location, int32_t clear) {
  int dev = 0;
  if (!code_and_location) return fail(AKLR_ERR_BAD_ARGUMENT, "NULL argument");
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return fail(AKLR_ERR_NO_DEVICE, "no CUDA device is current");
  code_and_location[0] = code_and_location[1] = 0;
  if (!g_host_status) return AKLR_OK;
  volatile int32_t* words = g_host_status + 2 * dev;
  code_and_location[0] = words[0];
  code_and_location[1] = words[1];
  if (clear) words[0] = words[1] = 0;
  return AKLR_OK;
}

int aklr_selftest_wait_expiry(int64_t limit_cycles, int32_t* status, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!status || limit_cycles < 1 || limit_cycles > 4000000000ll)
    return fail(AKLR_ERR_BAD_ARGUMENT, "status must be a device pointer and the limit 1..4e9 cycles");
  int rc = check_device();
  if (rc) return rc;
  cudaError_t err = cudaMemsetAsync(status, 0, 8, stream);
  if (err != cudaSuccess) return cuda_fail(err, "clearing the status words");
  wait_expiry_kernel<<<1, 32, 0, stream>>>(limit_cycles, status, aklr::host_visible_status(stream));
  err = cudaGetLastError();
  if (err != cudaSuccess) return cuda_fail(err, "launching the wait self-test");
  g_launches += 1;
  return AKLR_OK;
}

int aklr_profile_begin(int32_t max_calls) {
  for (cudaEvent_t e : g_profile.events) cudaEventDestroy(e);
  g_profile.events.clear();
  g_profile.capacity = g_profile.used = 0;
  g_profile.on = false;
  if (max_calls <= 0) return AKLR_OK;
  g_profile.events.resize(static_cast<size_t>(max_calls) * (kStages + 1));
  for (cudaEvent_t& e : g_profile.events) {
    const cudaError_t err = cudaEventCreate(&e);
    if (err != cudaSuccess) return cuda_fail(err, "creating profile events");
  }
  g_profile.capacity = max_calls;
  g_profile.on = true;
  return AKLR_OK;
}

int aklr_profile_read(int32_t call, float* stage_ms) {
  if (!stage_ms || call < 0 || call >= g_profile.used) return fail(AKLR_ERR_BAD_ARGUMENT, "no such recorded call");
  cudaEvent_t* ev = &g_profile.events[static_cast<size_t>(call) * (kStages + 1)];
  cudaError_t err = cudaEventSynchronize(ev[kStages]);
  for (int i = 0; i < kStages && err == cudaSuccess; ++i) err = cudaEventElapsedTime(&stage_ms[i], ev[i], ev[i + 1]);
  if (err != cudaSuccess) return cuda_fail(err, "reading profile events");
  return AKLR_OK;
}

}  // extern "C"
