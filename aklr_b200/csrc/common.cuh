// Shared device helpers for the sm_100a fused-MoE kernels: error codes, bounded mbarrier
// waits, TMA / tcgen05 PTX wrappers.  Every wait in this library is bounded: after
// AKLR_WAIT_LIMIT_CYCLES it gives up, records where in a status word the host can read, and the
// kernel drains and returns instead of hanging the device.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

// ---- status codes returned by the C ABI (0 = ok, negative = error) -------------------------
#define AKLR_OK 0
#define AKLR_ERR_BAD_ARGUMENT -1
#define AKLR_ERR_WORKSPACE_TOO_SMALL -2
#define AKLR_ERR_CUDA -3
#define AKLR_ERR_UNSUPPORTED_SHAPE -4
#define AKLR_ERR_NO_DEVICE -5
#define AKLR_ERR_KERNEL_WAIT_TIMEOUT -6
#define AKLR_ERR_TOO_LARGE -7

#ifndef AKLR_WAIT_LIMIT_CYCLES
#define AKLR_WAIT_LIMIT_CYCLES 4000000000ll  // about 2 s of SM clock
#endif

namespace aklr {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---- programmatic dependent launch ------------------------------------------------------------
// Kernels of a call are launched with programmatic stream serialisation: a kernel's CTAs may be
// scheduled while the previous kernel is still finishing, do their local set-up (barriers, TMEM,
// descriptor prefetch) and then wait here until everything before them in the stream is complete
// and visible.  Nothing produced by the PREVIOUS kernel may be read before griddep_wait().  Every kernel
// calls griddep_launch() only after its own griddep_wait(), so a kernel that has started also knows that
// whatever ran before its predecessor is complete: the weight-major GEMM reads the sort's block table
// (two kernels back) and starts its weight loads before it waits.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- mbarrier -------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false when the limit ran out or another thread of the CTA already
// gave up (``*abort_flag`` != 0); the first to give up records ``where`` in status[0..1].
// The loop polls mbarrier.try_wait (which itself suspends the thread for a short hardware-defined
// time) and looks at the SM's cycle counter only every 1024 polls: reading %globaltimer or
// sleeping here costs microseconds of wake-up latency per pipeline hand-off.
// SPIN: poll with the non-blocking test_wait instead of try_wait (barriers whose arrivals come from
// the other CTA of a pair).
template <bool SPIN = false>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int where, long long limit = AKLR_WAIT_LIMIT_CYCLES) {
  long long start = 0;
  for (uint32_t spin = 1;; ++spin) {
    if (SPIN ? mbar_test_wait(bar, parity) : mbar_try_wait(bar, parity)) return true;
    if ((spin & 1023u) == 0u) {
      if (*abort_flag) return false;
      const long long now = clock64();
      if (start == 0) start = now;
      if (now - start > limit) {
        *abort_flag = 1;
        if (atomicCAS(status, 0, AKLR_ERR_KERNEL_WAIT_TIMEOUT) == 0) status[1] = where;
        return false;
      }
    }
  }
}

// After a wait gave up, one thread of the CTA copies the call's status words to the device's
// host-visible pair (mapped pinned host memory, or null): the host looks at it at the start of every
// later call, so a caller that never reads its workspace's status still hears of the failure.
__device__ __forceinline__ void publish_wait_failure(const int* status, int32_t* host_visible) {
  if (host_visible == nullptr || status[0] == 0) return;
  volatile int32_t* v = host_visible;
  v[1] = status[1];
  __threadfence_system();
  v[0] = status[0];
  __threadfence_system();
}

// ---- TMA --------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
// 2-D tiled load global -> this CTA's shared memory; x is the innermost (contiguous) coordinate
// and x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x,
                                            int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Where a weight box starts in the TMA map: rows `row`.. of the flattened [experts * rows_per_expert, k] matrix at
// K-block `kb`.  Row-major weights: (kb * 128, row).  Tile-contiguous weights: the map is [tiles * 128, 128] and the
// box starts inside tile (row / 128) * (k / 128) + kb (a 64-row box may start at the tile's row 64).
__device__ __forceinline__ void weight_box(bool tiled, int k_blocks, int row, int kb, int* x, int* y) {
  if (tiled) {
    *x = 0;
    *y = (((row >> 7) * k_blocks + kb) << 7) + (row & 127);
  } else {
    *x = kb * 128;
    *y = row;
  }
}

// ---- tcgen05 ----------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
// ---- CTA pairs (cta_group::2): two CTAs of a cluster run one M=256 MMA, each holding its 128
// rows of A, half of B's rows and its half of the accumulator.  Nothing here is a multicast load:
// every CTA fetches its own operands; only barrier arrivals cross between the two.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of this CTA's shared-memory address ``addr`` in CTA ``rank`` of the cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-D tiled load into this CTA's shared memory whose bytes are counted on a barrier that may live in
// the pair's other CTA (a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t cluster_bar,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrive on the barrier at this shared-memory offset in every CTA of ``cta_mask`` once the MMAs
// issued so far are complete
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(cta_mask)
      : "memory");
}
// D[tmem, both CTAs] (+)= A * B with M = 256 over the pair; issued by one thread of the even CTA.
__device__ __forceinline__ void umma_f8f6f4_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t accumulate) {
  const uint32_t zero = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(zero)
      : "memory");
}

__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc], e4m3 x e4m3 -> f32, issued by one thread.
__device__ __forceinline__ void umma_f8f6f4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, stored as TMA's
// SWIZZLE_128B writes it: 8-row atoms of 1024 bytes (stride byte offset 1024), version 1.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) |
         (2ull << 61);
}

// kind::f8f6f4 instruction descriptor: f32 accumulator, e4m3 A and B, both K-major, M=128.
__host__ __device__ constexpr uint32_t umma_idesc_e4m3(int n, int m = 128) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

#define AKLR_TMEM_LD_8(taddr, r)                                                                       \
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"                \
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),   \
                 "=r"(r[7])                                                                            \
               : "r"(taddr))

#define AKLR_TMEM_LD_16(taddr, r)                                                                      \
  asm volatile(                                                                                        \
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "                                                        \
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"                                \
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), \
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),       \
        "=r"(r[15])                                                                                    \
      : "r"(taddr))

// ---- small numeric helpers ------------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

// max over the warp of non-negative floats (their bit patterns order like unsigned ints)
__device__ __forceinline__ float warp_max_nonneg(float v) {
  return __uint_as_float(__reduce_max_sync(0xFFFFFFFFu, __float_as_uint(v)));
}

__device__ __forceinline__ uint16_t cvt_e4m3x2(float lo, float hi) {
  return static_cast<uint16_t>(__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3));
}

}  // namespace aklr
