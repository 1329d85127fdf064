#include "dp_zero.h"

#include <cuda_bf16.h>

#include "../common/host.h"
#include "../runtime/flags.cuh"

namespace pico {

__global__ void __launch_bounds__(256)
zero1_adamw_kernel(PicoPeerTable grads, PicoPeerTable params, float* __restrict__ m, float* __restrict__ v,
                   float* __restrict__ master, int64_t shard_start, int64_t shard_len, int world, int my_rank, float lr,
                   float beta1, float beta2, float eps, float wd, float bc1, float bc2, float grad_scale,
                   const uint32_t* local_flags, int ready_slot, uint32_t epoch, uint64_t timeout_ns,
                   int* status) {
  if (!wait_slot_all(local_flags, ready_slot, world, epoch, timeout_ns, status, 800)) return;
  const float step_size = lr / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  const float decay = 1.f - lr * wd;
  const int64_t nvec = shard_len / 8;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e = shard_start + i * 8;
    float g[8];
    {
      const float4* gp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.ptr[0]) + e);
      const float4 a = gp[0], b = gp[1];
      g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w; g[4] = b.x; g[5] = b.y; g[6] = b.z; g[7] = b.w;
    }
    for (int r = 1; r < world; ++r) {
      const float4* gp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.ptr[r]) + e);
      const float4 a = gp[0], b = gp[1];
      g[0] += a.x; g[1] += a.y; g[2] += a.z; g[3] += a.w; g[4] += b.x; g[5] += b.y; g[6] += b.z; g[7] += b.w;
    }
    float pv[8], mv[8], vv[8];
    *reinterpret_cast<float4*>(&mv[0]) = reinterpret_cast<const float4*>(m + i * 8)[0];
    *reinterpret_cast<float4*>(&mv[4]) = reinterpret_cast<const float4*>(m + i * 8)[1];
    *reinterpret_cast<float4*>(&vv[0]) = reinterpret_cast<const float4*>(v + i * 8)[0];
    *reinterpret_cast<float4*>(&vv[4]) = reinterpret_cast<const float4*>(v + i * 8)[1];
    if (master) {
      *reinterpret_cast<float4*>(&pv[0]) = reinterpret_cast<const float4*>(master + i * 8)[0];
      *reinterpret_cast<float4*>(&pv[4]) = reinterpret_cast<const float4*>(master + i * 8)[1];
    } else {
      // every rank holds the same parameter values; read the local copy
      const uint4 raw = *reinterpret_cast<const uint4*>(
          reinterpret_cast<const __nv_bfloat16*>(params.ptr[my_rank]) + e);
      const __nv_bfloat162* pp = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = __bfloat1622float2(pp[j]);
        pv[2 * j] = t.x;
        pv[2 * j + 1] = t.y;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = g[j] * grad_scale;
      pv[j] *= decay;
      mv[j] = beta1 * mv[j] + (1.f - beta1) * gj;
      vv[j] = beta2 * vv[j] + (1.f - beta2) * gj * gj;
      pv[j] -= step_size * mv[j] / (sqrtf(vv[j]) * inv_sqrt_bc2 + eps);
    }
    reinterpret_cast<float4*>(m + i * 8)[0] = *reinterpret_cast<float4*>(&mv[0]);
    reinterpret_cast<float4*>(m + i * 8)[1] = *reinterpret_cast<float4*>(&mv[4]);
    reinterpret_cast<float4*>(v + i * 8)[0] = *reinterpret_cast<float4*>(&vv[0]);
    reinterpret_cast<float4*>(v + i * 8)[1] = *reinterpret_cast<float4*>(&vv[4]);
    if (master) {
      reinterpret_cast<float4*>(master + i * 8)[0] = *reinterpret_cast<float4*>(&pv[0]);
      reinterpret_cast<float4*>(master + i * 8)[1] = *reinterpret_cast<float4*>(&pv[4]);
    }
    uint4 packed;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int j = 0; j < 4; ++j) op[j] = __floats2bfloat162_rn(pv[2 * j], pv[2 * j + 1]);
    for (int r = 0; r < world; ++r)
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.ptr[r]) + e) = packed;
  }
}

}  // namespace pico

extern "C" int pico_zero1_adamw(PicoPeerTable grads, PicoPeerTable params, float* m, float* v, float* master,
                                int64_t shard_start, int64_t shard_len, int world, int my_rank, float lr, float beta1,
                                float beta2, float eps, float weight_decay, float bias_corr1, float bias_corr2,
                                float grad_scale, const uint32_t* local_flags, int ready_slot, uint32_t epoch,
                                uint32_t timeout_ms, cudaStream_t stream) {
  if (shard_len <= 0) return 0;
  if (world < 1 || world > PICO_MAX_PEERS || my_rank < 0 || my_rank >= world || (shard_start % 8) != 0 || (shard_len % 8) != 0) {
    pico_host::set_error("zero1_adamw: world %d, shard [%lld, +%lld) must be multiples of 8", world,
                         (long long)shard_start, (long long)shard_len);
    return -2;
  }
  int64_t blocks = (shard_len / 8 + 255) / 256;
  const int cap = pico_host::num_sms() * 8;
  if (blocks > cap) blocks = cap;
  pico::zero1_adamw_kernel<<<(int)blocks, 256, 0, stream>>>(
      grads, params, m, v, master, shard_start, shard_len, world, my_rank, lr, beta1, beta2, eps, weight_decay,
      bias_corr1, bias_corr2, grad_scale, local_flags, ready_slot, epoch, (uint64_t)timeout_ms * 1000000ull,
      pico_status_buffer());
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("zero1_adamw: %s", cudaGetErrorString(e));
  return (int)e;
}
