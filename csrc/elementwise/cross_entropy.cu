// Cross entropy over a (possibly vocabulary-sharded) bf16 logits matrix, split into the two
// halves a vocabulary-parallel loss needs:
//
//   pico_ce_stats     : per row, one streaming pass with an online softmax -> {max, sumexp,
//                       target logit}. Under tensor parallelism these triples are combined
//                       across vocabulary shards by the caller (max / rescaled sum / sum).
//   pico_ce_loss_grad : per row, loss = log(sum) + max - target and, in the same pass that
//                       re-reads the logits, dlogits = (softmax - onehot) * scale written in
//                       place, so no [rows, V] softmax tensor is ever kept.
//
// One CTA of 512 threads per row; 16-byte loads; V must be a multiple of 8.
#include <cuda_bf16.h>
#include <math_constants.h>

#include "../common/host.h"
#include "elementwise.h"

namespace pico {

constexpr int kCeThreads = 512;

__device__ __forceinline__ void ce_unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__global__ void __launch_bounds__(kCeThreads)
ce_stats_kernel(const __nv_bfloat16* __restrict__ logits, int64_t ldl,
                const int64_t* __restrict__ targets, float* __restrict__ stats, int rows, int V,
                int vocab_start) {
  __shared__ float s_max[kCeThreads / 32];
  __shared__ float s_sum[kCeThreads / 32];
  const int nvec = V / 8;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* lr = reinterpret_cast<const uint4*>(logits + (int64_t)row * ldl);
    float mx = -CUDART_INF_F, sum = 0.f;
    for (int v = threadIdx.x; v < nvec; v += kCeThreads) {
      float f[8];
      ce_unpack8(lr[v], f);
      float lm = f[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
      if (lm > mx) {
        sum *= __expf(mx - lm);
        mx = lm;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) sum += __expf(f[j] - mx);
    }
    // combine (max, sum) pairs across the CTA
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, mx, o);
      const float os = __shfl_xor_sync(0xffffffffu, sum, o);
      const float nm = fmaxf(mx, om);
      sum = (mx == -CUDART_INF_F ? 0.f : sum * __expf(mx - nm)) +
            (om == -CUDART_INF_F ? 0.f : os * __expf(om - nm));
      mx = nm;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) {
      s_max[warp] = mx;
      s_sum[warp] = sum;
    }
    __syncthreads();
    if (warp == 0) {
      mx = lane < kCeThreads / 32 ? s_max[lane] : -CUDART_INF_F;
      sum = lane < kCeThreads / 32 ? s_sum[lane] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, mx, o);
        const float os = __shfl_xor_sync(0xffffffffu, sum, o);
        const float nm = fmaxf(mx, om);
        sum = (mx == -CUDART_INF_F ? 0.f : sum * __expf(mx - nm)) +
              (om == -CUDART_INF_F ? 0.f : os * __expf(om - nm));
        mx = nm;
      }
      if (lane == 0) {
        const int64_t t = targets[row] - vocab_start;
        float tl = 0.f;
        if (t >= 0 && t < V) tl = __bfloat162float(logits[(int64_t)row * ldl + t]);
        stats[row * 3 + 0] = mx;
        stats[row * 3 + 1] = sum;
        stats[row * 3 + 2] = tl;
      }
    }
  }
}

__global__ void __launch_bounds__(kCeThreads)
ce_loss_grad_kernel(const __nv_bfloat16* __restrict__ logits, int64_t ldl,
                    const int64_t* __restrict__ targets, const float* __restrict__ stats,
                    float* __restrict__ loss, __nv_bfloat16* __restrict__ dlogits, int64_t ldd,
                    float grad_scale, int rows, int V, int vocab_start) {
  const int nvec = V / 8;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float mx = stats[row * 3 + 0];
    const float sum = stats[row * 3 + 1];
    const float tl = stats[row * 3 + 2];
    if (threadIdx.x == 0 && loss) loss[row] = __logf(sum) + mx - tl;
    if (!dlogits) continue;
    const float inv = grad_scale / sum;
    const int64_t t = targets[row] - vocab_start;
    const uint4* lr = reinterpret_cast<const uint4*>(logits + (int64_t)row * ldl);
    uint4* dr = reinterpret_cast<uint4*>(dlogits + (int64_t)row * ldd);
    for (int v = threadIdx.x; v < nvec; v += kCeThreads) {
      float f[8];
      ce_unpack8(lr[v], f);
      uint4 o;
      __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        f[j] = __expf(f[j] - mx) * inv;
        if ((int64_t)v * 8 + j == t) f[j] -= grad_scale;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) op[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
      dr[v] = o;
    }
  }
}

}  // namespace pico

extern "C" int pico_ce_stats(const void* logits, int64_t ldl, const int64_t* targets, float* stats,
                             int rows, int V, int vocab_start, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (V % 8 != 0 || ldl % 8 != 0) {
    pico_host::set_error("cross entropy: vocab shard %d and stride %lld must be multiples of 8", V,
                         (long long)ldl);
    return -2;
  }
  const int cap = pico_host::num_sms() * 4;
  pico::ce_stats_kernel<<<rows < cap ? rows : cap, pico::kCeThreads, 0, stream>>>(
      (const __nv_bfloat16*)logits, ldl, targets, stats, rows, V, vocab_start);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("ce_stats: %s", cudaGetErrorString(e));
  return (int)e;
}

extern "C" int pico_ce_loss_grad(const void* logits, int64_t ldl, const int64_t* targets,
                                 const float* stats, float* loss, void* dlogits, int64_t ldd,
                                 float grad_scale, int rows, int V, int vocab_start,
                                 cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (V % 8 != 0 || ldl % 8 != 0 || ldd % 8 != 0) {
    pico_host::set_error("cross entropy: vocab shard and strides must be multiples of 8");
    return -2;
  }
  const int cap = pico_host::num_sms() * 4;
  pico::ce_loss_grad_kernel<<<rows < cap ? rows : cap, pico::kCeThreads, 0, stream>>>(
      (const __nv_bfloat16*)logits, ldl, targets, stats, loss, (__nv_bfloat16*)dlogits, ldd,
      grad_scale, rows, V, vocab_start);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("ce_loss_grad: %s", cudaGetErrorString(e));
  return (int)e;
}
