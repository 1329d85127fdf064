// Microbenchmark: issue cycles per warp instruction of ex2.approx, cvt.rn.bf16x2.f32 and fma.rn.f32 per SM
// sub-partition (1, 2 or 4 warps per sub-partition) - the inputs of the softmax cost model of the
// attention kernels.
// Build and run:
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o alu_rate benchmarks/micro/alu_rate.cu
//   ./alu_rate
#include <cstdio>
#include <cuda_runtime.h>
#include <cstdint>
template <int MODE>
__global__ void k(float* out, long long* clk, int iters) {
  float a[8];
  for (int i = 0; i < 8; ++i) a[i] = threadIdx.x * 1e-3f + i * 0.01f;
  uint32_t acc = 0;
  __syncthreads();
  long long t0 = clock64();
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (MODE == 0) { asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(a[i])); }
      else if (MODE == 1) { uint32_t r; asm volatile("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(a[i]), "f"(a[(i + 1) & 7])); acc ^= r; }
      else if (MODE == 2) { asm volatile("fma.rn.f32 %0, %0, %1, %1;" : "+f"(a[i]) : "f"(0.5f)); }
      else if (MODE == 3) { asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(a[i])); asm volatile("fma.rn.f32 %0, %0, %1, %1;" : "+f"(a[i]) : "f"(0.5f)); asm volatile("add.f32 %0, %0, %1;" : "+f"(a[i]) : "f"(0.25f)); }
    }
  }
  long long t1 = clock64();
  float s = 0; for (int i = 0; i < 8; ++i) s += a[i];
  out[blockIdx.x * blockDim.x + threadIdx.x] = s + acc;
  if (threadIdx.x == 0 && blockIdx.x == 0) clk[0] = t1 - t0;
}
template <int MODE> void run(const char* name, int threads, float* out, long long* clk) {
  const int iters = 2048;
  for (int r = 0; r < 2; ++r) { k<MODE><<<148, threads>>>(out, clk, iters); cudaDeviceSynchronize(); }
  long long h; cudaMemcpy(&h, clk, 8, cudaMemcpyDeviceToHost);
  double per_warp_instr = (double)h / (iters * 8);
  int warps_per_smsp = threads / 32 / 4; if (warps_per_smsp < 1) warps_per_smsp = 1;
  printf("%-14s threads=%3d: %.2f clk per warp-instruction-group per warp; => %.2f clk per warp-instr per SMSP\n", name, threads, per_warp_instr, per_warp_instr / warps_per_smsp);
}
int main() {
  float* out; long long* clk; cudaMalloc(&out, 148 * 1024 * 4); cudaMalloc(&clk, 8);
  for (int threads : {128, 256, 512}) {
    run<0>("ex2", threads, out, clk);
    run<1>("cvt.bf16x2", threads, out, clk);
    run<2>("ffma", threads, out, clk);
    run<3>("ex2+ffma+fadd", threads, out, clk);
  }
  return 0;
}
