// Microbenchmark: does alternating between tcgen05.mma shapes / accumulators cost extra cycles, and what
// does one commit -> mbarrier -> wake-up round trip add? (the per-block pattern of flash attention:
// 8 x 128x64x16 for P V, 4 x 128x128x16 for Q K^T). One CTA per SM, SM clock cycles per iteration.
// Build and run:
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o mma_switch benchmarks/micro/mma_switch.cu
//   ./mma_switch
#include <cstdio>
#include <cuda_runtime.h>
#include "../../csrc/common/ptx.cuh"
using namespace pico;

template <int MODE>
__global__ void __launch_bounds__(128, 1) k(long long* out, int iters, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bar = (uint64_t*)(smem + 96 * 1024);
  uint32_t* tptr = (uint32_t*)(bar + 1);
  volatile int* abort_word = (volatile int*)(tptr + 1);
  if (threadIdx.x == 0) { mbar_init(bar, 1); *abort_word = 0; mbar_fence_init(); }
  for (int i = threadIdx.x; i < 96 * 1024 / 4; i += blockDim.x) ((uint32_t*)smem)[i] = 0;
  fence_proxy_async_smem();
  if (threadIdx.x < 32) { tmem_alloc(tptr, 512); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  uint32_t tb = *tptr;
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
    constexpr uint32_t idesc_o = umma_idesc_bf16(128, 64, 0, 1);
    uint32_t a = smem_u32(smem), b = smem_u32(smem + 32 * 1024);
    long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
      // "PV": 8 MMAs N=64 (TS, B MN-major) into D1; "S": 4 MMAs N=128 (SS K-major) into D0
      if (MODE == 0 || MODE == 2) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          tc_mma_f16_ts(tb + 256, tb + 384 + kk * 8, umma_smem_desc(b + kk * 2048, 16384, 1024), idesc_o, 1u);
      }
      if (MODE == 1 || MODE == 2) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          tc_mma_f16_ss(tb, umma_smem_desc(a + off, 16, 1024), umma_smem_desc(b + off, 16, 1024), idesc_s, kk ? 1u : 0u);
        }
      }
      if (MODE == 3) {   // S with fresh accumulator each time + commit each iteration
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          tc_mma_f16_ts(tb + 256, tb + 384 + kk * 8, umma_smem_desc(b + kk * 2048, 16384, 1024), idesc_o, 1u);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          tc_mma_f16_ss(tb, umma_smem_desc(a + off, 16, 1024), umma_smem_desc(b + off, 16, 1024), idesc_s, kk ? 1u : 0u);
        }
        tc_commit(bar);
        if (!mbar_wait(bar, it & 1, abort_word, status, 1)) break;
        tc_fence_after();
      }
    }
    long long t1 = clock64();
    if (MODE != 3) { tc_commit(bar); mbar_wait(bar, 0, abort_word, status, 1); }
    long long t2 = clock64();
    if (blockIdx.x == 0) { out[0] = t1 - t0; out[1] = t2 - t0; }
  }
  tc_fence_before(); __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tb, 512); }
}
template <int MODE> void run(const char* name, long long* dout, int* status) {
  auto kern = k<MODE>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  const int iters = 64;
  for (int r = 0; r < 2; ++r) { kern<<<148, 128, 100 * 1024>>>(dout, iters, status); cudaDeviceSynchronize(); }
  long long h[2]; cudaMemcpy(h, dout, sizeof(h), cudaMemcpyDeviceToHost);
  printf("%-40s: %.0f clk per iteration (issue %.0f) err=%s\n", name, (double)h[1] / iters, (double)h[0] / iters, cudaGetErrorString(cudaGetLastError()));
}
int main() {
  long long* dout; int* status; cudaMalloc(&dout, 64); cudaMalloc(&status, 64); cudaMemset(status, 0, 64);
  run<0>("8 x (128x64x16 TS, MN-major B)", dout, status);
  run<1>("4 x (128x128x16 SS)", dout, status);
  run<2>("8 PV + 4 S alternating", dout, status);
  run<3>("8 PV + 4 S + commit + wait per iteration", dout, status);
  return 0;
}
