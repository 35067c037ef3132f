// What an issuing thread pays per tcgen05.mma and how far the tensor pipe lets it run ahead: bursts of n MMAs (M128, N256, K32)
// from an idle pipe, cycles until the issue loop returns and until the commit of the burst is seen.
#include <cstdio>
#include "../common.cuh"
using namespace aklr;
__global__ void __launch_bounds__(128, 1) probe(long long* out, int n) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t done[2];
  __shared__ uint32_t tptr;
  __shared__ int abortf; __shared__ int st[2];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 49152 / 4; i += blockDim.x) ((uint32_t*)smem)[i] = 0x38383838u;
  if (threadIdx.x == 0) { mbar_init(&done[0], 1); mbar_init(&done[1], 1); fence_mbar_init(); abortf = 0; st[0] = st[1] = 0; }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 1) { tmem_alloc(&tptr, 512); tmem_relinquish(); }
  tc_fence_before_sync(); __syncthreads(); tc_fence_after_sync();
  const uint32_t tbase = tptr;
  if (warp == 1 && lane == 0) {
    const uint64_t da = umma_desc_sw128(smem_u32(smem));
    const uint64_t db = umma_desc_sw128(smem_u32(smem + 16384));
    const uint32_t idesc = umma_idesc_e4m3(256);
    // warm: one MMA and wait
    umma_f8f6f4(tbase, da, db, idesc, 0);
    tc_commit(&done[0]);
    mbar_wait(&done[0], 0, &abortf, st, 9);
    long long t_issue_sum = 0, t_total_sum = 0;
    for (int rep = 0; rep < 16; ++rep) {
      const long long t0 = clock64();
      for (int i = 0; i < n; ++i) {
        umma_f8f6f4(tbase + (i & 1) * 256, da + 2 * (i & 3), db + 2 * (i & 3), idesc, 1);
      }
      const long long t1 = clock64();
      tc_commit(&done[1]);
      mbar_wait(&done[1], rep & 1, &abortf, st, 9);
      const long long t2 = clock64();
      t_issue_sum += t1 - t0; t_total_sum += t2 - t0;
    }
    out[blockIdx.x * 2] = t_issue_sum / 16;
    out[blockIdx.x * 2 + 1] = t_total_sum / 16;
  }
  tc_fence_before_sync(); __syncthreads();
  if (warp == 1) { tc_fence_after_sync(); tmem_dealloc(tbase, 512); }
}
int main() {
  long long* d; cudaMalloc(&d, 148 * 2 * 8);
  cudaFuncSetAttribute(probe, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  for (int n = 1; n <= 12; ++n) {
    probe<<<148, 128, 64 * 1024>>>(d, n);
    cudaError_t e = cudaDeviceSynchronize();
    long long h[296]; cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
    double a = 0, b = 0; for (int i = 0; i < 148; ++i) { a += h[2 * i]; b += h[2 * i + 1]; }
    printf("burst of %2d MMAs (N=256): issue loop returns after %.0f cycles, all complete (commit seen) after %.0f   %s\n", n, a / 148, b / 148, cudaGetErrorString(e));
  }
  return 0;
}
