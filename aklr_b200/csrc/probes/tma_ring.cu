// L2 -> shared memory delivery ceiling for the grouped GEMM's load pattern: persistent CTAs that only
// run the TMA ring (no MMA, no fold).  Modes: tile shape (48 KB x 4 stages | 32 KB x 6 stages), weights
// L2-resident or streamed from HBM; and the MXFP4 kernel's weight loads, packed e2m1 in global memory that the TMA
// unpacks to one byte per element in shared memory (16U4_ALIGN16B).
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
#include <cstdlib>

#define CHECK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); exit(1);} } while (0)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory"); }
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err) {
  const long long start = clock64();
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try(bar, parity)) return true;
    if ((spin & 1023u) == 0u && clock64() - start > 2000000000ll) { *err = 1; return false; }
  }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

struct Params {
  CUtensorMap map_w, map_x;
  int K, rows_per_expert, n_experts, blocks_per_expert, n_tile, stages, tiles_per_block, total_tiles, load_a, fp4;
  int w_box;         // rows per weight box: 128 (two loads per 256-row tile) or 256 (one)
  int two_producers; // 1: a thread of another warp issues the weight loads
  int* err;
};

// tile t -> (block b, channel tile j): block's expert = b / blocks_per_expert
__global__ void __launch_bounds__(96, 1) probe(const __grid_constant__ Params p) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  const int a_bytes = p.load_a ? 16384 : 0;
  const int stage_bytes = 16384 + p.n_tile * 128;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.stages * stage_bytes);
  uint64_t* empty = full + p.stages;
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int KB = p.K / 128;
  if (threadIdx.x == 0 || (p.two_producers && threadIdx.x == 64)) {
    // one producer: barrier, activation box, weight boxes.  Two: thread 0 the barrier and the activation box,
    // thread 64 the weight boxes (its bytes may land before the expectation is posted: the count goes negative).
    const bool does_a = threadIdx.x == 0, does_w = !p.two_producers || threadIdx.x == 64;
    int s = 0; uint32_t ph = 0;
    for (int t = blockIdx.x; t < p.total_tiles; t += gridDim.x) {
      const int b = t / p.tiles_per_block, j = t - b * p.tiles_per_block;
      const int e = (b / p.blocks_per_expert) % p.n_experts;
      const int w_row = e * p.rows_per_expert + j * p.n_tile;
      for (int kb = 0; kb < KB; ++kb) {
        if (!mbar_wait(&empty[s], ph ^ 1, p.err)) return;
        uint8_t* st = smem + s * stage_bytes;
        if (does_a) {
          // an unpacking load counts the packed bytes that cross from global memory
          mbar_expect_tx(&full[s], a_bytes + (p.fp4 ? p.n_tile * 64 : p.n_tile * 128));
          if (p.load_a) tma_load_2d(st, &p.map_x, &full[s], kb * 128, b * 128);
        }
        if (does_w)
          for (int r = 0; r < p.n_tile; r += p.w_box) tma_load_2d(st + 16384 + r * 128, &p.map_w, &full[s], kb * 128, w_row + r);
        if (++s == p.stages) { s = 0; ph ^= 1; }
      }
    }
  } else if (threadIdx.x == 32) {
    int s = 0; uint32_t ph = 0;
    for (int t = blockIdx.x; t < p.total_tiles; t += gridDim.x) {
      for (int kb = 0; kb < KB; ++kb) {
        if (!mbar_wait(&full[s], ph, p.err)) return;
        mbar_arrive(&empty[s]);
        if (++s == p.stages) { s = 0; ph ^= 1; }
      }
    }
  }
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static void make_map(EncodeFn enc, CUtensorMap* m, void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, bool fp4 = false) {
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {fp4 ? cols / 2 : cols};
  const cuuint32_t box[2] = {128, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = enc(m, fp4 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { printf("encode failed %d\n", (int)r); exit(1); }
}

int main() {
  void* sym = nullptr; cudaDriverEntryPointQueryResult qr;
  CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qr));
  EncodeFn enc = reinterpret_cast<EncodeFn>(sym);
  const int K = 7168, rows_per_expert = 4096;
  const int blocks = 1184;  // 8 rounds of 148
  uint8_t *w, *x; int* err;
  const size_t w_bytes_big = (size_t)128 * rows_per_expert * K;  // 3.76 GB: streams from HBM
  CHECK(cudaMalloc(&w, w_bytes_big)); CHECK(cudaMemset(w, 1, w_bytes_big));
  CHECK(cudaMalloc(&x, (size_t)blocks * 128 * K)); CHECK(cudaMemset(x, 1, (size_t)blocks * 128 * K));
  CHECK(cudaMalloc(&err, 4)); CHECK(cudaMemset(err, 0, 4));
  cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  CHECK(cudaFuncSetAttribute(probe, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
  struct Mode { const char* name; int n_tile, stages, n_experts, blocks_per_expert, load_a, fp4, w_box, two_producers; };
  const Mode modes[] = {
      {"48KB x4, weights from HBM (128 experts x 5 blocks)", 256, 4, 128, 5, 1},
      {"48KB x4, weights L2-resident (2 experts)", 256, 4, 2, 5, 1},
      {"32KB x6, weights from HBM", 128, 6, 128, 5, 1},
      {"32KB x6, weights L2-resident (2 experts)", 128, 6, 2, 5, 1},
      {"B only 32KB x6 (stage 48KB), weights L2-resident", 256, 4, 2, 5, 0},
      {"B only, weights from HBM", 256, 4, 128, 5, 0},
      {"fp4 unpacked by the TMA: A 16KB + B 16KB packed -> 32KB, x4, from HBM", 256, 4, 128, 5, 1, 1},
      {"fp4 unpacked by the TMA: A + B, x4, L2-resident (2 experts)", 256, 4, 2, 5, 1, 1},
      {"fp4 unpacked by the TMA: B only, x4, from HBM", 256, 4, 128, 5, 0, 1},
      {"fp4 unpacked by the TMA: B only, x4, L2-resident", 256, 4, 2, 5, 0, 1},
      {"48KB x4 L2-resident, weights as ONE 256-row box (2 loads per stage)", 256, 4, 2, 5, 1, 0, 256},
      {"48KB x4 L2-resident, two producer threads (A | 2 weight boxes)", 256, 4, 2, 5, 1, 0, 128, 1},
      {"48KB x4 L2-resident, two producer threads, one 256-row weight box", 256, 4, 2, 5, 1, 0, 256, 1},
      {"48KB x4 from HBM, two producer threads, one 256-row weight box", 256, 4, 128, 5, 1, 0, 256, 1},
  };
  for (const Mode& m : modes) {
    Params p{};
    make_map(enc, &p.map_w, w, (uint64_t)128 * rows_per_expert, K, m.w_box ? m.w_box : 128, m.fp4 != 0);
    p.w_box = m.w_box ? m.w_box : 128; p.two_producers = m.two_producers;
    make_map(enc, &p.map_x, x, (uint64_t)blocks * 128, K, 128);
    p.K = K; p.rows_per_expert = rows_per_expert; p.n_experts = m.n_experts; p.blocks_per_expert = m.blocks_per_expert;
    p.n_tile = m.n_tile; p.stages = m.stages; p.tiles_per_block = rows_per_expert / m.n_tile; p.load_a = m.load_a; p.fp4 = m.fp4;
    p.total_tiles = blocks * p.tiles_per_block / 4;  // a quarter of the channel tiles: keeps a run ~10 ms
    p.tiles_per_block /= 4;
    p.err = err;
    const size_t smem = (size_t)m.stages * (16384 + m.n_tile * 128) + 2 * m.stages * 8 + 1024;
    for (int rep = 0; rep < 3; ++rep) {
      cudaEventRecord(e0);
      probe<<<148, 96, smem>>>(p);
      cudaEventRecord(e1);
      CHECK(cudaDeviceSynchronize());
      float ms; cudaEventElapsedTime(&ms, e0, e1);
      // bytes written to shared memory (an unpacked fp4 tile is twice its size in global memory)
      const double bytes = (double)p.total_tiles * (K / 128) * ((m.load_a ? 16384 : 0) + m.n_tile * 128);
      const double stages = (double)p.total_tiles * (K / 128) / 148;
      if (rep == 2) printf("%-72s %8.3f ms  %7.2f TB/s into shared memory (%.1f GB/s per SM, %.0f ns per stage)\n", m.name, ms, bytes / ms / 1e9, bytes / ms / 1e6 / 148, ms * 1e6 / stages);
    }
    int h = 0; CHECK(cudaMemcpy(&h, err, 4, cudaMemcpyDeviceToHost));
    if (h) { printf("a wait gave up\n"); return 1; }
    fflush(stdout);
  }
  return 0;
}
