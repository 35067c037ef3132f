// Does a TMA ring writing shared memory slow the tensor core's reads of it?  148 CTAs; each runs
// (a) an MMA stream on a fixed operand pair in shared memory (M128 N256 K128 e4m3 per "K-block", two deep),
// (b) a TMA ring of 48 KB stages into OTHER shared memory, recycled at once,  alone and together.
#include <cstdio>
#include <cstdlib>
#include <cuda.h>
#include "../common.cuh"
using namespace aklr;

struct P { CUtensorMap map; long long* out; int kblocks; int with_mma, with_tma, n_mma_per_kb, n_cols; };

__global__ void __launch_bounds__(128, 1) probe(const __grid_constant__ P p) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  constexpr int kStage = 49152, kStages = 3;  // source rows stay inside a 58 MB window: L2 hits
  uint8_t* fixed = smem + kStages * kStage;  // 48 KB operand pair for the MMAs
  __shared__ uint64_t full[kStages], empty[kStages], done[2];
  __shared__ uint32_t tptr;
  __shared__ int abortf; __shared__ int st[2];
  __shared__ volatile int stop;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < kStage / 4; i += blockDim.x) ((uint32_t*)fixed)[i] = 0x38383838u;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(&done[0], 1); mbar_init(&done[1], 1);
    fence_mbar_init(); abortf = 0; st[0] = st[1] = 0; stop = 0;
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 1) { tmem_alloc(&tptr, 512); tmem_relinquish(); }
  tc_fence_before_sync(); __syncthreads(); tc_fence_after_sync();
  const uint32_t tbase = tptr;
  if (warp == 1 && lane == 0) {
    if (p.with_mma) {
      const uint64_t da = umma_desc_sw128(smem_u32(fixed));
      const uint64_t db = umma_desc_sw128(smem_u32(fixed + 16384));
      const uint32_t idesc = umma_idesc_e4m3(p.n_cols);
      const long long t0 = clock64();
      int b = 0;
      for (; b < p.kblocks; ++b) {
        for (int i = 0; i < 4; ++i) umma_f8f6f4(tbase + (b & 1) * 256, da + 2 * i, db + 2 * i, idesc, i);
        tc_commit(&done[b & 1]);
        if (b >= 1 && !mbar_wait(&done[(b - 1) & 1], ((b - 1) >> 1) & 1, &abortf, st, 9)) break;
      }
      if (b >= 1 && !abortf) mbar_wait(&done[(b - 1) & 1], ((b - 1) >> 1) & 1, &abortf, st, 9);
      p.out[blockIdx.x * 4 + 0] = (clock64() - t0) / (b ? b : 1);
    }
    stop = 1;
  } else if (warp == 2 && lane == 0) {
    if (p.with_tma) {
      int s = 0; uint32_t ph = 0; long long n = 0;
      const long long t0 = clock64();
      // until the MMA stream is done (or, alone, for kblocks stages)
      for (; p.with_mma ? !stop : n < p.kblocks; ++n) {
        if (!mbar_wait(&empty[s], ph ^ 1, &abortf, st, 10)) break;
        mbar_expect_tx(&full[s], kStage);
        const int row = (int)(((long long)blockIdx.x * 7919 + n * 3) % 60) * 128;
        const int col = (int)(n % 56) * 128;
        tma_load_2d(smem + s * kStage, &p.map, &full[s], col, row);
        tma_load_2d(smem + s * kStage + 16384, &p.map, &full[s], col, row + 128);
        tma_load_2d(smem + s * kStage + 32768, &p.map, &full[s], col, row + 256);
        if (++s == kStages) { s = 0; ph ^= 1; }
        if (n > 40000000) break;
      }
      p.out[blockIdx.x * 4 + 1] = n ? (clock64() - t0) / n : 0;
      p.out[blockIdx.x * 4 + 2] = n;
    }
  } else if (warp == 3 && lane == 0) {
    if (p.with_tma) {
      int s = 0; uint32_t ph = 0;
      for (long long n = 0;; ++n) {
        // stop once the producer has stopped issuing: bounded polling
        bool got = false;
        for (int spin = 0; spin < 200000; ++spin) { if (mbar_try_wait(&full[s], ph)) { got = true; break; } }
        if (!got) break;
        mbar_arrive(&empty[s]);
        if (++s == kStages) { s = 0; ph ^= 1; }
      }
    }
  }
  tc_fence_before_sync(); __syncthreads();
  if (warp == 1) { tc_fence_after_sync(); tmem_dealloc(tbase, 512); }
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
int main() {
  void* sym = nullptr; cudaDriverEntryPointQueryResult qr;
  cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qr);
  EncodeFn enc = (EncodeFn)sym;
  const uint64_t rows = 8000ull * 128 + 512, cols = 7168;
  uint8_t* w; cudaMalloc(&w, rows * cols); cudaMemset(w, 0x38, rows * cols);
  long long* d; cudaMalloc(&d, 148 * 4 * 8);
  P p{};
  const cuuint64_t dims[2] = {cols, rows}; const cuuint64_t strides[1] = {cols};
  const cuuint32_t box[2] = {128, 128}; const cuuint32_t elem[2] = {1, 1};
  if (enc(&p.map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) { printf("encode failed\n"); return 1; }
  p.out = d; p.kblocks = 20000;
  cudaFuncSetAttribute(probe, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  const int modes[][3] = {{1, 0, 256}, {0, 1, 256}, {1, 1, 256}, {1, 0, 128}, {1, 1, 128}};
  for (auto& m : modes) {
    p.with_mma = m[0]; p.with_tma = m[1]; p.n_cols = m[2];
    cudaMemset(d, 0, 148 * 4 * 8);
    cudaEventRecord(e0);
    probe<<<148, 128, 200 * 1024>>>(p);
    cudaEventRecord(e1);
    cudaError_t e = cudaDeviceSynchronize();
    float ms; cudaEventElapsedTime(&ms, e0, e1);
    long long h[148 * 4]; cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
    long long mma = 0, tma = 0, n = 0;
    for (int i = 0; i < 148; ++i) { mma += h[i * 4]; tma += h[i * 4 + 1]; n += h[i * 4 + 2]; }
    (void)ms;
    (void)n;
    printf("mma=%d (N=%d) tma=%d  %s   MMA cycles per K-block (avg over CTAs) %lld   TMA cycles per 48 KB stage %lld (%.0f bytes per cycle and SM)\n",
           m[0], m[2], m[1], cudaGetErrorString(e), mma / 148, tma / 148, tma ? 49152.0 / (tma / 148.0) : 0.0);
    fflush(stdout);
  }
  return 0;
}
