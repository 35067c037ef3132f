// Tensor-pipe timing of tcgen05.mma kind::f8f6f4 (M128, K32): cycles per MMA as a function of N and of how
// many INDEPENDENT accumulators the issuing thread rotates over (1 = every MMA depends on the one before).
#include <cstdio>
#include "../common.cuh"
using namespace aklr;

__global__ void __launch_bounds__(128, 1) probe(long long* out, int n_cols, int chains, int total) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t done;
  __shared__ uint32_t tptr;
  __shared__ int abortf; __shared__ int st[2];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 49152 / 4; i += blockDim.x) ((uint32_t*)smem)[i] = 0x38383838u;
  if (threadIdx.x == 0) { mbar_init(&done, 1); fence_mbar_init(); abortf = 0; st[0] = st[1] = 0; }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 1) { tmem_alloc(&tptr, 512); tmem_relinquish(); }
  tc_fence_before_sync(); __syncthreads(); tc_fence_after_sync();
  const uint32_t tbase = tptr;
  if (warp == 1 && lane == 0) {
    const uint64_t da = umma_desc_sw128(smem_u32(smem));
    const uint64_t db = umma_desc_sw128(smem_u32(smem + 16384));
    const uint32_t idesc = umma_idesc_e4m3(n_cols);
    const long long t0 = clock64();
    int c = 0;
    for (int i = 0; i < total; ++i) {
      umma_f8f6f4(tbase + c * n_cols, da + 2 * (i & 3), db + 2 * (i & 3), idesc, i >= chains);
      if (++c == chains) c = 0;
    }
    const long long t_issue = clock64();
    tc_commit(&done);
    mbar_wait(&done, 0, &abortf, st, 9);
    const long long t1 = clock64();
    out[blockIdx.x * 2] = (t1 - t0);
    out[blockIdx.x * 2 + 1] = (t_issue - t0);
  }
  tc_fence_before_sync(); __syncthreads();
  if (warp == 1) { tc_fence_after_sync(); tmem_dealloc(tbase, 512); }
}

int main() {
  long long* d; cudaMalloc(&d, 148 * 2 * 8);
  cudaFuncSetAttribute(probe, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  const int total = 4096;
  const int cfgs[][2] = {{256, 1}, {256, 2}, {128, 1}, {128, 2}, {128, 3}, {128, 4}, {64, 1}, {64, 2}, {64, 4}, {64, 8}, {192, 1}, {192, 2}, {32, 1}, {32, 8}, {16, 1}};
  for (auto& c : cfgs) {
    cudaMemset(d, 0, 148 * 2 * 8);
    probe<<<148, 128, 64 * 1024>>>(d, c[0], c[1], total);
    cudaError_t e = cudaDeviceSynchronize();
    long long h[296]; cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
    long long a = 0, b = 0; for (int i = 0; i < 148; ++i) { a += h[2 * i]; b += h[2 * i + 1]; }
    printf("N=%3d chains=%d  %s  cycles per MMA: %.1f (issue loop alone %.1f)   = %.0f%% of the nominal N/2 cycles\n", c[0], c[1], cudaGetErrorString(e),
           a / 148.0 / total, b / 148.0 / total, 100.0 * (c[0] / 2.0) / (a / 148.0 / total));
    fflush(stdout);
  }
  return 0;
}
