// aklr_moe_align_noalloc: the token sort for callers that cannot hand the library a scratch buffer.
//
// aklr_moe_align needs a scratch array of int32 (one histogram per 1024 routes) that its caller
// allocates.  Some callers cannot allocate device memory at the point where they sort: code running
// under a memory pool that is frozen for the duration of a step, a plugin hook that is handed only
// the engine's own input and output tensors, a host language binding without an allocator of its
// own.  For them this file keeps the scratch in a fixed device array that lives inside the loaded
// library: every GPU that loads libaklr_b200.so holds kNoAllocScratchInts * 4 bytes (1 MiB) of it
// from load until the process exits.
//
// Set-up: in host code the array's name is only a handle, not a device address, so the first call
// on each device asks the runtime for the address (cudaGetSymbolAddress, with that device current)
// and remembers it per device.  Make that first call before any stream capture begins.
//
// Sharing: every call on a device uses the same array, which keeps whatever the last call left in
// it.  Nothing in it has to start at zero -- the sort's first pass writes each histogram whole
// before the second pass reads it -- but two calls whose kernels overlap on the GPU (different
// streams, or graphs replayed concurrently) race on it; run them one after another.
#include <cstdio>
#include <mutex>

#include "../../include/aklr_b200.h"
#include "common.cuh"
#include "kernels.h"

namespace {

constexpr int kNoAllocScratchInts = 262144;  // 1 MiB: ceil(n_routes / 1024) * n_experts must fit
constexpr int kMaxDevices = 64;

static __device__ __align__(256) int32_t g_align_scratch[kNoAllocScratchInts];

std::mutex g_setup_lock;
int32_t* g_scratch_address[kMaxDevices] = {};

thread_local char g_noalloc_error[256] = "";

// The device address of the scratch array on the current device, resolved once per device.
int scratch_for_current_device(int32_t** out) {
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess || device < 0 || device >= kMaxDevices) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error), "no usable current device (%s)", cudaGetErrorString(err));
    return AKLR_ERR_NO_DEVICE;
  }
  std::lock_guard<std::mutex> guard(g_setup_lock);
  if (g_scratch_address[device] == nullptr) {
    int32_t* address = nullptr;
    err = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_align_scratch);
    if (err != cudaSuccess || address == nullptr) {
      snprintf(g_noalloc_error, sizeof(g_noalloc_error), "cudaGetSymbolAddress on device %d: %s", device,
               cudaGetErrorString(err));
      return AKLR_ERR_CUDA;
    }
    g_scratch_address[device] = address;
  }
  *out = g_scratch_address[device];
  return AKLR_OK;
}

}  // namespace

extern "C" {

int32_t aklr_moe_align_noalloc_max_scratch_ints(void) { return kNoAllocScratchInts; }

const char* aklr_moe_align_noalloc_last_error(void) { return g_noalloc_error; }

int aklr_moe_align_noalloc(const int32_t* topk_ids, const int32_t* expert_map, int32_t n_routes, int32_t n_experts,
                           int32_t n_experts_global, int32_t block_m, int32_t* sorted_ids, int32_t* block_expert,
                           int32_t* counts, int32_t* num_blocks, void* stream) {
  g_noalloc_error[0] = 0;
  if (!topk_ids || !sorted_ids || !block_expert || !counts || !num_blocks || n_routes < 0 || n_experts < 1) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error), "NULL or negative argument");
    return AKLR_ERR_BAD_ARGUMENT;
  }
  const long long chunks = (static_cast<long long>(n_routes) + 1023) / 1024;
  const long long needed = chunks * n_experts;
  if (needed > kNoAllocScratchInts) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error),
             "n_routes=%d with n_experts=%d needs %lld scratch ints; the built-in array holds %d "
             "(use aklr_moe_align with a caller-provided scratch buffer)",
             n_routes, n_experts, needed, kNoAllocScratchInts);
    return AKLR_ERR_TOO_LARGE;
  }
  int rc = aklr::require_sm100_device(g_noalloc_error, sizeof(g_noalloc_error));
  if (rc) return rc;
  int32_t* scratch = nullptr;
  rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  aklr::AlignParams p{};
  p.topk_ids = topk_ids;
  p.expert_map = expert_map;
  p.sorted_ids = sorted_ids;
  p.block_expert = block_expert;
  p.counts = counts;
  p.num_blocks = num_blocks;
  p.chunk_hist = scratch;  // a device address: the kernels never see the host-side handle
  p.n_routes = n_routes;
  p.n_experts = n_experts;
  p.n_experts_global = expert_map ? n_experts_global : n_experts;
  p.block_m = block_m;
  rc = aklr::launch_align(p, static_cast<cudaStream_t>(stream));
  if (rc) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error), "moe_align launch failed (status %d)", rc);
    return rc;
  }
  aklr::count_kernel_launches(n_routes <= 4096 ? 1 : 3);
  return AKLR_OK;
}

}  // extern "C"
