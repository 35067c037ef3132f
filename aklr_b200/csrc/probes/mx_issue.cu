// Issue stream of the MXFP4 grouped GEMM alone: per K-block the thread copies scale factors into TMEM with
// tcgen05.cp (0..4 copies) and issues four kind::mxf8f6f4.block_scale MMAs (M 128, N 256, K 32) on one accumulator.
// Cycles per K-block as a function of the number of copies, and with the copies writing alternating column sets.
#include <cstdio>
#include "../common.cuh"
using namespace aklr;

__device__ __forceinline__ uint32_t mx_idesc(int n, int sf_id) {
  return (static_cast<uint32_t>(sf_id) << 4) | (0u << 7) | (5u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (1u << 23) | (static_cast<uint32_t>(128 >> 4) << 24) | (static_cast<uint32_t>(sf_id) << 29);
}
__device__ __forceinline__ void umma_mx(uint32_t d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d), "l"(da), "l"(db), "r"(idesc), "r"(acc), "r"(sfa), "r"(sfb) : "memory");
}
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (8ull << 32) | (1ull << 46);
}
__device__ __forceinline__ void cp_32x128b_warpx4(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}

__global__ void __launch_bounds__(128, 1) probe(long long* out, int copies, int alternate, int kblocks) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t done;
  __shared__ uint32_t tptr;
  __shared__ int abortf; __shared__ int st[2];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // operands: e4m3 1.0 (0x38) for A; B as unpacked e2m1 bytes (0x02 = 1.0 in the low nibble); scale bytes 127 (2^0)
  for (int i = threadIdx.x; i < 16384 / 4; i += blockDim.x) ((uint32_t*)smem)[i] = 0x38383838u;
  for (int i = threadIdx.x; i < 32768 / 4; i += blockDim.x) ((uint32_t*)(smem + 16384))[i] = 0x02020202u;
  for (int i = threadIdx.x; i < 2048 / 4; i += blockDim.x) ((uint32_t*)(smem + 49152))[i] = 0x7F7F7F7Fu;
  if (threadIdx.x == 0) { mbar_init(&done, 1); fence_mbar_init(); abortf = 0; st[0] = st[1] = 0; }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 1) { tmem_alloc(&tptr, 512); tmem_relinquish(); }
  tc_fence_before_sync(); __syncthreads(); tc_fence_after_sync();
  const uint32_t tbase = tptr;
  if (warp == 1 && lane == 0) {
    const uint64_t da = umma_desc_sw128(smem_u32(smem));
    const uint64_t db = umma_desc_sw128(smem_u32(smem + 16384));
    const uint64_t sf = sf_desc(smem_u32(smem + 49152));
    // the scale columns must hold something valid before the first MMA reads them
    cp_32x128b_warpx4(tbase + 256, sf);
    cp_32x128b_warpx4(tbase + 260, sf + 32);
    cp_32x128b_warpx4(tbase + 264, sf + 64);
    cp_32x128b_warpx4(tbase + 272, sf);
    cp_32x128b_warpx4(tbase + 276, sf + 32);
    cp_32x128b_warpx4(tbase + 280, sf + 64);
    const long long t0 = clock64();
    for (int kb = 0; kb < kblocks; ++kb) {
      const uint32_t set = tbase + 256 + (alternate ? (kb & 1) * 16 : 0);
      if (copies > 0) cp_32x128b_warpx4(set, sf);
      if (copies > 1) cp_32x128b_warpx4(set + 4, sf + 32);
      if (copies > 2) cp_32x128b_warpx4(set + 8, sf + 64);
      if (copies > 3) cp_32x128b_warpx4(set + 12, sf + 96);
#pragma unroll
      for (int k = 0; k < 4; ++k) umma_mx(tbase, da + 2 * k, db + 2 * k, mx_idesc(256, k), set, set + 4, (kb | k) ? 1u : 0u);
    }
    const long long t_issue = clock64();
    tc_commit(&done);
    mbar_wait(&done, 0, &abortf, st, 9);
    out[blockIdx.x * 2] = clock64() - t0;
    out[blockIdx.x * 2 + 1] = t_issue - t0;
  }
  tc_fence_before_sync(); __syncthreads();
  if (warp == 1) { tc_fence_after_sync(); tmem_dealloc(tbase, 512); }
}

int main() {
  long long* d; cudaMalloc(&d, 148 * 2 * 8);
  cudaFuncSetAttribute(probe, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  const int kblocks = 2048;
  const int cfgs[][2] = {{0, 0}, {1, 0}, {2, 0}, {3, 0}, {4, 0}, {3, 1}, {4, 1}};
  for (auto& c : cfgs) {
    cudaMemset(d, 0, 148 * 2 * 8);
    probe<<<148, 128, 64 * 1024>>>(d, c[0], c[1], kblocks);
    cudaError_t e = cudaDeviceSynchronize();
    long long h[296]; cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
    long long a = 0, b = 0; for (int i = 0; i < 148; ++i) { a += h[2 * i]; b += h[2 * i + 1]; }
    printf("tcgen05.cp per K-block: %d%s  %s  cycles per K-block (4 block-scaled MMAs N=256): %.0f (issue loop alone %.0f)\n", c[0],
           c[1] ? ", alternating column sets" : "", cudaGetErrorString(e), a / 148.0 / kblocks, b / 148.0 / kblocks);
    fflush(stdout);
  }
  return 0;
}
