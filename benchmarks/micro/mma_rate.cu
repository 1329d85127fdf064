// Microbenchmark: SM cycles per tcgen05.mma (M=128, K=16, bf16) for N = 64 / 128, with the A operand
// in shared memory (SS) or tensor memory (TS) and B K-major or MN-major, while eight other warps of
// the CTA keep a chosen unit busy (mode 0 idle, 2 exp2 chain, 4 tcgen05.st). One CTA per SM.
// Build and run:
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 --use_fast_math -o mma_rate benchmarks/micro/mma_rate.cu
//   ./mma_rate
#include <cstdio>
#include <cuda_runtime.h>
#include "../../csrc/common/ptx.cuh"
using namespace pico;

template <int N, bool TS, int BMN = 0>
__global__ void __launch_bounds__(320, 1) rate_kernel(long long* out, int iters, int* status, int mode, float* sink) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bar = (uint64_t*)(smem + 96 * 1024);
  uint32_t* tptr = (uint32_t*)(bar + 1);
  volatile int* abort_word = (volatile int*)(tptr + 1);
  if (threadIdx.x == 0) { mbar_init(bar, 1); *abort_word = 0; mbar_fence_init(); }
  // zero the operand area
  for (int i = threadIdx.x; i < 96 * 1024 / 4; i += blockDim.x) ((uint32_t*)smem)[i] = 0;
  fence_proxy_async_smem();
  if (threadIdx.x < 32) { tmem_alloc(tptr, 512); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  uint32_t tb = *tptr;
  volatile int* done = abort_word + 1;
  if (threadIdx.x == 0) *done = 0;
  __syncthreads();
  if (threadIdx.x >= 64) {
    // background load from 8 other warps until the MMA thread is done
    const int w = threadIdx.x >> 5;
    const uint32_t lane_base = (uint32_t)((w & 3) * 32) << 16;
    float acc = threadIdx.x * 1e-3f;
    uint32_t v[32];
    for (int i = 0; i < 32; ++i) v[i] = threadIdx.x + i;
    int guard = 0;
    while (!*done && ++guard < 200000) {
      if (mode == 1) {
        tmem_ld_32x32b_x32(tb + 384 + lane_base, v);
        tmem_ld_wait();
        acc += __uint_as_float(v[3]);
      } else if (mode == 2) {
#pragma unroll
        for (int i = 0; i < 32; ++i) acc = exp2f(acc * 0.5f - 1.f) + __uint_as_float(v[i]);
      } else if (mode == 3) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          *reinterpret_cast<uint4*>(smem + 64 * 1024 + (threadIdx.x - 64) * 128 + ((i ^ (threadIdx.x & 7)) << 4)) = make_uint4(v[0], v[1], v[2], v[3]);
      } else if (mode == 4) {
        tmem_st_32x32b_x32(tb + 384 + lane_base, v);
        tmem_st_wait();
      } else if (mode == 5) {
#pragma unroll
        for (int i = 0; i < 32; ++i) acc = fmaf(acc, 0.5f, __uint_as_float(v[i]));
      } else {
        __nanosleep(200);
      }
    }
    if (acc == 123.456f) sink[0] = acc;
  }
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc = umma_idesc_bf16(128, N, 0, BMN);
    uint32_t a = smem_u32(smem), b = smem_u32(smem + 32 * 1024);
    long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
        if (TS && BMN) tc_mma_f16_ts(tb, tb + 256 + kk * 8, umma_smem_desc(b + kk * 2048, 16384, 1024), idesc, 1u);
        else if (TS) tc_mma_f16_ts(tb, tb + 256 + kk * 8, umma_smem_desc(b + off, 16, 1024), idesc, 1u);
        else tc_mma_f16_ss(tb, umma_smem_desc(a + off, 16, 1024), umma_smem_desc(b + off, 16, 1024), idesc, 1u);
      }
    }
    long long t1 = clock64();
    tc_commit(bar);
    bool ok = mbar_wait(bar, 0, abort_word, status, 1);
    long long t2 = clock64();
    if (blockIdx.x == 0) { out[0] = t1 - t0; out[1] = t2 - t0; out[2] = ok; }
    *done = 1;
  }
  tc_fence_before(); __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tb, 512); }
}

template <int N, bool TS, int BMN = 0>
void run(const char* name, long long* dout, int* status, int grid, int mode) {
  auto k = rate_kernel<N, TS, BMN>;
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  const int iters = 64;
  for (int r = 0; r < 2; ++r) {
    k<<<grid, 320, 100 * 1024>>>(dout, iters, status, mode, (float*)(dout + 4));
    cudaDeviceSynchronize();
  }
  long long h[3];
  cudaMemcpy(h, dout, sizeof(h), cudaMemcpyDeviceToHost);
  printf("mode %d %s N=%3d grid=%3d: issue %.1f clk/mma, complete %.1f clk/mma (ok=%lld) err=%s\n", mode, name, N, grid,
         (double)h[0] / (iters * 8), (double)h[1] / (iters * 8), h[2], cudaGetErrorString(cudaGetLastError()));
}

int main() {
  long long* dout; int* status;
  cudaMalloc(&dout, 64); cudaMalloc(&status, 64); cudaMemset(status, 0, 64);
  for (int mode : {0, 2, 4}) {
    run<64, true, 0>("TS Kmaj", dout, status, 148, mode);
    run<64, true, 1>("TS MNmaj", dout, status, 148, mode);
    run<128, true, 1>("TS MNmaj", dout, status, 148, mode);
  }
  return 0;
}
