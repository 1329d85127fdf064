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

#include <cstring>

#include "../common/host.h"
#include "../runtime/flags.cuh"
#include "elementwise.h"

namespace pico {

// Where ce_stats_kernel sends its triples when the vocabulary is sharded (world == 0: nowhere).
struct PicoCePush {
  PicoPeerTable dst, flags;
  int world, my_rank, slot;
  uint32_t epoch;
  unsigned int* counter;
};
// The gathered [world][rows][3] table ce_loss_grad_kernel merges (world == 0: stats are final).
struct PicoCeGathered {
  const uint32_t* local_flags;
  int world, slot;
  uint32_t epoch;
  uint64_t timeout_ns;
};

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
                int vocab_start, PicoCePush push) {
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
        if (stats) {
          stats[row * 3 + 0] = mx;
          stats[row * 3 + 1] = sum;
          stats[row * 3 + 2] = tl;
        }
        if (push.world > 0) {
          // this shard's triple goes into block my_rank of every rank's [world][rows][3] table
          const int64_t o = ((int64_t)push.my_rank * rows + row) * 3;
          for (int r = 0; r < push.world; ++r) {
            float* d = reinterpret_cast<float*>(push.dst.ptr[r]) + o;
            d[0] = mx;
            d[1] = sum;
            d[2] = tl;
          }
        }
      }
    }
  }
  if (push.world > 0)
    raise_flags_when_grid_done(push.counter, push.flags, push.world, push.my_rank, push.slot, push.epoch);
}

__global__ void __launch_bounds__(kCeThreads)
ce_loss_grad_kernel(const __nv_bfloat16* __restrict__ logits, int64_t ldl,
                    const int64_t* __restrict__ targets, const float* __restrict__ stats,
                    float* __restrict__ loss, __nv_bfloat16* __restrict__ dlogits, int64_t ldd,
                    float grad_scale, int rows, int V, int vocab_start, PicoCeGathered gat, int* status) {
  const int nvec = V / 8;
  if (gat.world > 0 &&
      !wait_slot_all(gat.local_flags, gat.slot, gat.world, gat.epoch, gat.timeout_ns, status, 1000))
    return;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    float mx, sum, tl;
    if (gat.world > 0) {
      // merge the shards' triples in rank order (every rank computes the same bits)
      const float* g = stats + (int64_t)row * 3;
      const int64_t blk = (int64_t)rows * 3;
      mx = g[0];
      for (int r = 1; r < gat.world; ++r) mx = fmaxf(mx, g[r * blk]);
      sum = 0.f;
      tl = 0.f;
      for (int r = 0; r < gat.world; ++r) {
        sum += g[r * blk + 1] * __expf(g[r * blk] - mx);
        tl += g[r * blk + 2];
      }
    } else {
      mx = stats[row * 3 + 0];
      sum = stats[row * 3 + 1];
      tl = stats[row * 3 + 2];
    }
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
  pico::PicoCePush none;
  memset(&none, 0, sizeof(none));
  pico::ce_stats_kernel<<<rows < cap ? rows : cap, pico::kCeThreads, 0, stream>>>(
      (const __nv_bfloat16*)logits, ldl, targets, stats, rows, V, vocab_start, none);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("ce_stats: %s", cudaGetErrorString(e));
  return (int)e;
}

namespace {
unsigned int* g_ce_counters[64] = {nullptr};
unsigned int* ce_counter() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!g_ce_counters[dev]) {
    unsigned int* p = nullptr;
    if (cudaMalloc(&p, 64) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 64);
    g_ce_counters[dev] = p;
  }
  return g_ce_counters[dev];
}
}  // namespace

extern "C" int pico_ce_stats_push(const void* logits, int64_t ldl, const int64_t* targets, int rows, int V,
                                  int vocab_start, PicoPeerTable dst, PicoPeerTable flags, int world,
                                  int my_rank, int slot, uint32_t epoch, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (V % 8 != 0 || ldl % 8 != 0 || world < 1 || world > PICO_MAX_PEERS || slot < 0 || slot >= PICO_FLAG_SLOTS) {
    pico_host::set_error("ce_stats_push: vocab shard %d / stride %lld must be multiples of 8, world %d, slot %d",
                         V, (long long)ldl, world, slot);
    return -2;
  }
  pico::PicoCePush push;
  push.dst = dst;
  push.flags = flags;
  push.world = world;
  push.my_rank = my_rank;
  push.slot = slot;
  push.epoch = epoch;
  push.counter = ce_counter();
  if (!push.counter) return -1;
  const int cap = pico_host::num_sms() * 4;
  pico::ce_stats_kernel<<<rows < cap ? rows : cap, pico::kCeThreads, 0, stream>>>(
      (const __nv_bfloat16*)logits, ldl, targets, nullptr, rows, V, vocab_start, push);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("ce_stats_push: %s", cudaGetErrorString(e));
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
  pico::PicoCeGathered none;
  memset(&none, 0, sizeof(none));
  pico::ce_loss_grad_kernel<<<rows < cap ? rows : cap, pico::kCeThreads, 0, stream>>>(
      (const __nv_bfloat16*)logits, ldl, targets, stats, loss, (__nv_bfloat16*)dlogits, ldd,
      grad_scale, rows, V, vocab_start, none, nullptr);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("ce_loss_grad: %s", cudaGetErrorString(e));
  return (int)e;
}

extern "C" int pico_ce_loss_grad_gathered(const void* logits, int64_t ldl, const int64_t* targets,
                                          const float* gathered_stats, float* loss, void* dlogits, int64_t ldd,
                                          float grad_scale, int rows, int V, int vocab_start,
                                          const uint32_t* local_flags, int world, int slot, uint32_t epoch,
                                          uint32_t timeout_ms, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (V % 8 != 0 || ldl % 8 != 0 || ldd % 8 != 0 || world < 1 || world > PICO_MAX_PEERS || slot < 0 ||
      slot >= PICO_FLAG_SLOTS) {
    pico_host::set_error("ce_loss_grad_gathered: vocab shard and strides must be multiples of 8, world %d, slot %d",
                         world, slot);
    return -2;
  }
  pico::PicoCeGathered gat;
  gat.local_flags = local_flags;
  gat.world = world;
  gat.slot = slot;
  gat.epoch = epoch;
  gat.timeout_ns = (uint64_t)timeout_ms * 1000000ull;
  const int cap = pico_host::num_sms() * 4;
  pico::ce_loss_grad_kernel<<<rows < cap ? rows : cap, pico::kCeThreads, 0, stream>>>(
      (const __nv_bfloat16*)logits, ldl, targets, gathered_stats, loss, (__nv_bfloat16*)dlogits, ldd,
      grad_scale, rows, V, vocab_start, gat, pico_status_buffer());
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("ce_loss_grad_gathered: %s", cudaGetErrorString(e));
  return (int)e;
}
