#include "ep_comm.h"

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "../common/host.h"
#include "../runtime/flags.cuh"

namespace pico {

// one warp per slot row; each lane handles 8 consecutive elements per step (d % 256 == 0 for
// the quantised path so that a 128-element block is covered by 16 lanes)
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const __nv_bfloat16* __restrict__ tokens, const int32_t* __restrict__ row_of_slot, int top_k,
                   PicoPeerTable payload, PicoPeerTable scales, PicoPeerTable flags, int ep, int my_rank, int L,
                   int C, int d, int quant, int slot, uint32_t epoch, unsigned int* counter) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const int64_t total = (int64_t)ep * L * C;
  for (int64_t idx = (int64_t)blockIdx.x * warps_per_cta + (threadIdx.x >> 5); idx < total;
       idx += (int64_t)gridDim.x * warps_per_cta) {
    const int s = (int)(idx % C);
    const int e = (int)(idx / C);
    const int dest = e / L, l = e % L;
    const int64_t drow = ((int64_t)l * ep + my_rank) * C + s;
    const int r = row_of_slot[idx];
    const __nv_bfloat16* src = r >= 0 ? tokens + (int64_t)(r / top_k) * d : nullptr;
    if (!quant) {
      uint4* out = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(payload.ptr[dest]) + drow * d);
      for (int v = lane; v < d / 8; v += 32)
        out[v] = src ? reinterpret_cast<const uint4*>(src)[v] : make_uint4(0, 0, 0, 0);
    } else {
      uint8_t* out = reinterpret_cast<uint8_t*>(payload.ptr[dest]) + drow * d;
      float* sc = reinterpret_cast<float*>(scales.ptr[dest]) + drow * (d / 128);
      for (int v = lane; v < d / 8; v += 32) {
        float f[8];
        if (src) {
          const uint4 raw = reinterpret_cast<const uint4*>(src)[v];
          const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 t = __bfloat1622float2(p2[j]);
            f[2 * j] = t.x;
            f[2 * j + 1] = t.y;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = 0.f;
        }
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
        // 16 lanes x 8 elements = one 128-element block
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float scale = fmaxf(amax, 1e-12f) / 448.f;
        const float inv = 1.f / scale;
        uint2 q;
        uint8_t* qb = reinterpret_cast<uint8_t*>(&q);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          qb[j] = (uint8_t)__nv_cvt_float_to_fp8(fminf(fmaxf(f[j] * inv, -448.f), 448.f), __NV_SATFINITE, __NV_E4M3);
        reinterpret_cast<uint2*>(out)[v] = q;
        if ((lane & 15) == 0) sc[v / 16] = scale;
      }
    }
  }
  raise_flags_when_grid_done(counter, flags, ep, my_rank, slot, epoch);
}

__global__ void __launch_bounds__(256)
ep_dequant_kernel(const uint8_t* __restrict__ payload, const float* __restrict__ scales,
                  __nv_bfloat16* __restrict__ out, int64_t rows, int d, const uint32_t* local_flags, int ep,
                  int slot, uint32_t epoch, uint64_t timeout_ns, int* status) {
  if (!wait_slot_all(local_flags, slot, ep, epoch, timeout_ns, status, 600)) return;
  const int64_t nvec = rows * d / 8;
  const int vec_per_row = d / 8;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / vec_per_row;
    const int v = (int)(i % vec_per_row);
    const float scale = scales[row * (d / 128) + v / 16];
    const uint2 q = reinterpret_cast<const uint2*>(payload)[i];
    const uint8_t* qb = reinterpret_cast<const uint8_t*>(&q);
    uint4 o;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __half_raw h0 = __nv_cvt_fp8_to_halfraw(qb[2 * j], __NV_E4M3);
      const __half_raw h1 = __nv_cvt_fp8_to_halfraw(qb[2 * j + 1], __NV_E4M3);
      op[j] = __floats2bfloat162_rn(__half2float(__half(h0)) * scale, __half2float(__half(h1)) * scale);
    }
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

__global__ void __launch_bounds__(256)
ep_block_exchange_kernel(const uint4* __restrict__ src, PicoPeerTable dst, PicoPeerTable flags, int ep, int my_rank,
                         int L, int C, int vec_per_row, int to_expert_major, int slot, uint32_t epoch,
                         unsigned int* counter) {
  const int64_t block_vecs = (int64_t)C * vec_per_row;
  const int64_t total = (int64_t)ep * L * block_vecs;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t blk = i / block_vecs;
    const int64_t within = i - blk * block_vecs;
    int dest;
    int64_t dblk;
    if (!to_expert_major) {      // src [L][ep][C]: block (l, r) -> rank r, block (my_rank * L + l)
      const int l = (int)(blk / ep), r = (int)(blk % ep);
      dest = r;
      dblk = (int64_t)my_rank * L + l;
    } else {                     // src [E][C]: block e = r*L + l -> rank r, block (l * ep + my_rank)
      const int r = (int)(blk / L), l = (int)(blk % L);
      dest = r;
      dblk = (int64_t)l * ep + my_rank;
    }
    reinterpret_cast<uint4*>(dst.ptr[dest])[dblk * block_vecs + within] = src[i];
  }
  raise_flags_when_grid_done(counter, flags, ep, my_rank, slot, epoch);
}

constexpr int kEpMaxDev = 64;
unsigned int* g_ep_counters[kEpMaxDev] = {nullptr};
static unsigned int* ep_counter() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kEpMaxDev) return nullptr;
  if (!g_ep_counters[dev]) {
    unsigned int* p = nullptr;
    if (cudaMalloc(&p, 64 * sizeof(unsigned int)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 64 * sizeof(unsigned int));
    g_ep_counters[dev] = p;
  }
  return g_ep_counters[dev];
}

}  // namespace pico

using namespace pico;

static int ep_check(const char* what, int ep, int slot, int d) {
  if (ep < 1 || ep > PICO_MAX_PEERS || slot < 0 || slot >= PICO_FLAG_SLOTS || d % 8 != 0) {
    pico_host::set_error("%s: ep %d / flag slot %d / row width %d out of range", what, ep, slot, d);
    return -2;
  }
  return 0;
}

extern "C" int pico_ep_dispatch(const void* tokens, const int32_t* row_of_slot, int top_k, PicoPeerTable payload,
                                PicoPeerTable scales, PicoPeerTable flags, int ep, int my_rank, int L, int C, int d,
                                int quant, int slot, uint32_t epoch, cudaStream_t stream) {
  if (int rc = ep_check("ep_dispatch", ep, slot, d)) return rc;
  if (quant && d % 256 != 0) {
    pico_host::set_error("ep_dispatch: quantised dispatch needs a row width that is a multiple of 256 (got %d)", d);
    return -2;
  }
  unsigned int* counter = ep_counter();
  if (!counter) return -1;
  const int64_t total = (int64_t)ep * L * C;
  int64_t blocks = (total + 7) / 8;
  const int cap = pico_host::num_sms() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  ep_dispatch_kernel<<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)tokens, row_of_slot, top_k, payload, scales,
                                                     flags, ep, my_rank, L, C, d, quant, slot, epoch, counter);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("ep_dispatch: %s", cudaGetErrorString(e));
  return (int)e;
}

extern "C" int pico_ep_dequant(const void* payload, const float* scales, void* out, int64_t rows, int d,
                               const uint32_t* local_flags, int ep, int slot, uint32_t epoch, uint32_t timeout_ms,
                               cudaStream_t stream) {
  if (int rc = ep_check("ep_dequant", ep, slot, d)) return rc;
  if (d % 128 != 0) {
    pico_host::set_error("ep_dequant: row width %d must be a multiple of 128", d);
    return -2;
  }
  int64_t blocks = (rows * d / 8 + 255) / 256;
  const int cap = pico_host::num_sms() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  ep_dequant_kernel<<<(int)blocks, 256, 0, stream>>>((const uint8_t*)payload, scales, (__nv_bfloat16*)out, rows, d,
                                                    local_flags, ep, slot, epoch, (uint64_t)timeout_ms * 1000000ull,
                                                    pico_status_buffer());
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("ep_dequant: %s", cudaGetErrorString(e));
  return (int)e;
}

extern "C" int pico_ep_block_exchange(const void* src, PicoPeerTable dst, PicoPeerTable flags, int ep, int my_rank,
                                      int L, int C, int d, int to_expert_major, int slot, uint32_t epoch,
                                      cudaStream_t stream) {
  if (int rc = ep_check("ep_block_exchange", ep, slot, d)) return rc;
  unsigned int* counter = ep_counter();
  if (!counter) return -1;
  const int64_t total = (int64_t)ep * L * C * (d / 8);
  int64_t blocks = (total + 255) / 256;
  const int cap = pico_host::num_sms() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  ep_block_exchange_kernel<<<(int)blocks, 256, 0, stream>>>((const uint4*)src, dst, flags, ep, my_rank, L, C, d / 8,
                                                           to_expert_major, slot, epoch, counter + 8);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("ep_block_exchange: %s", cudaGetErrorString(e));
  return (int)e;
}
