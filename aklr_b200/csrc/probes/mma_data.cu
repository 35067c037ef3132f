// Does the tensor pipe's rate depend on WHAT it multiplies?  The same stream of tcgen05.mma kind::f8f6f4
// (M128, N256, K32, one issuing thread per SM, all 148 SMs) on constant operands (every byte e4m3 1.0) and on
// random bytes, short (4096 MMAs, 0.3 ms) and long (65536 MMAs, several ms): cycles per MMA from clock64,
// nanoseconds per MMA from the global timer, and the SM clock the two imply.
#include <cstdio>
#include "../common.cuh"
using namespace aklr;

__global__ void __launch_bounds__(128, 1) probe(long long* out, int random_data, int total) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t done;
  __shared__ uint32_t tptr;
  __shared__ int abortf; __shared__ int st[2];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 49152 / 4; i += blockDim.x) {
    uint32_t v = 0x38383838u;
    if (random_data) {  // a hash of the position; exponent bits kept below the NaN pattern
      v = (i + 1) * 2654435761u + blockIdx.x * 40503u;
      v ^= v >> 15; v *= 2246822519u; v ^= v >> 13;
      v &= 0xBFBFBFBFu;
      // modes 2, 3: the activation tile's rows from 64 / 32 on are zero (row r = bytes r * 128 .. of the first 16 KB)
      if (random_data >= 2 && i * 4 < 16384 && i * 4 >= (random_data == 2 ? 64 : 32) * 128) v = 0u;
    }
    ((uint32_t*)smem)[i] = v;
  }
  if (threadIdx.x == 0) { mbar_init(&done, 1); fence_mbar_init(); abortf = 0; st[0] = st[1] = 0; }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 1) { tmem_alloc(&tptr, 512); tmem_relinquish(); }
  tc_fence_before_sync(); __syncthreads(); tc_fence_after_sync();
  const uint32_t tbase = tptr;
  if (warp == 1 && lane == 0) {
    const uint64_t da = umma_desc_sw128(smem_u32(smem));
    const uint64_t db = umma_desc_sw128(smem_u32(smem + 16384));
    const uint32_t idesc = umma_idesc_e4m3(256);
    const uint64_t n0 = global_timer_ns();
    const long long t0 = clock64();
    for (int i = 0; i < total; ++i)
      umma_f8f6f4(tbase + (i & 4 ? 256 : 0), da + 2 * (i & 3), db + 2 * (i & 3), idesc, (i & 3) != 0);
    tc_commit(&done);
    mbar_wait(&done, 0, &abortf, st, 9);
    const long long t1 = clock64();
    const uint64_t n1 = global_timer_ns();
    out[blockIdx.x * 2] = (t1 - t0);
    out[blockIdx.x * 2 + 1] = static_cast<long long>(n1 - n0);
  }
  tc_fence_before_sync(); __syncthreads();
  if (warp == 1) { tc_fence_after_sync(); tmem_dealloc(tbase, 512); }
}

int main() {
  long long* d; cudaMalloc(&d, 148 * 2 * 8);
  cudaFuncSetAttribute(probe, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  const int cfgs[][2] = {{0, 4096}, {1, 4096}, {0, 65536}, {1, 65536}, {0, 262144}, {1, 262144}, {0, 4096}, {2, 65536}, {3, 65536}, {1, 65536}};
  for (auto& c : cfgs) {
    cudaMemset(d, 0, 148 * 2 * 8);
    probe<<<148, 128, 64 * 1024>>>(d, c[0], c[1]);
    cudaError_t e = cudaDeviceSynchronize();
    long long h[296]; cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
    double cyc = 0, ns = 0; for (int i = 0; i < 148; ++i) { cyc += h[2 * i]; ns += h[2 * i + 1]; }
    cyc /= 148.0 * c[1]; ns /= 148.0 * c[1];
    printf("%-26s operands, %6d MMAs  %s  cycles per MMA %.1f   ns per MMA %.1f   -> SM clock %.0f MHz, %.2f PFLOP/s over the GPU\n",
           c[0] == 0 ? "constant" : c[0] == 1 ? "random" : c[0] == 2 ? "random, A rows 64.. zero" : "random, A rows 32.. zero", c[1], cudaGetErrorString(e), cyc, ns, cyc / ns * 1e3,
           148.0 * 2 * 128 * 256 * 32 / ns / 1e6);
    fflush(stdout);
  }
  return 0;
}
