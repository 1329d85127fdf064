#include "ep_var.h"

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "../common/host.h"
#include "../common/ptx.cuh"
#include "../runtime/flags.cuh"

namespace pico {

__device__ __forceinline__ int pad128(int n) { return (n + 127) & ~127; }

// One CTA; the table has at most 8 x 512 entries, so plain loops in a few threads are enough.
__global__ void ep_var_layout_kernel(const int32_t* __restrict__ counts, int ep, int L, int my_rank, int max_rows,
                                     int32_t* __restrict__ send_blocks, int32_t* __restrict__ return_blocks,
                                     int32_t* __restrict__ seg_start, int32_t* __restrict__ seg_len,
                                     int32_t* __restrict__ tile_group, int* status) {
  const int E = ep * L;
  __shared__ int s_total;
  // ---- my outgoing blocks: one thread per destination rank walks that rank's experts
  if (threadIdx.x < ep) {
    const int r = threadIdx.x;
    // where my rows of expert e start in my expert-sorted rows
    int my_start = 0;
    for (int e = 0; e < r * L; ++e) my_start += counts[my_rank * E + e];
    int seg = 0;   // start of the destination's segment of the current expert
    for (int l = 0; l < L; ++l) {
      const int e = r * L + l;
      int total = 0, before_me = 0;
      for (int s = 0; s < ep; ++s) {
        const int c = counts[s * E + e];
        if (s < my_rank) before_me += c;
        total += c;
      }
      int cnt = counts[my_rank * E + e];
      const int dst_row = seg + before_me;
      // an expert whose segment does not fit into the destination's buffer takes no rows and no
      // space there (the receiver applies the same rule); the loss is reported
      const bool fits = seg + pad128(total) <= max_rows;
      if (!fits) {
        if (cnt > 0) report_error(status, PICO_ERR_BOUNDS, 3100, e);
        cnt = 0;
      }
      send_blocks[e * 4 + 0] = cnt;
      send_blocks[e * 4 + 1] = my_start;
      send_blocks[e * 4 + 2] = r;
      send_blocks[e * 4 + 3] = fits ? dst_row : 0;
      my_start += counts[my_rank * E + e];
      if (fits) seg += pad128(total);
    }
  }
  // ---- my receive buffer: segments of my local experts and the blocks on their way back
  if (threadIdx.x == 32) {
    int seg = 0;
    for (int l = 0; l < L; ++l) {
      const int e = my_rank * L + l;
      int total = 0;
      for (int s = 0; s < ep; ++s) total += counts[s * E + e];
      const bool fits = seg + pad128(total) <= max_rows;
      seg_start[l] = seg;
      seg_len[l] = fits ? total : 0;
      int within = 0;
      for (int s = 0; s < ep; ++s) {
        const int c = counts[s * E + e];
        // first row of expert e in source s's expert-sorted rows
        int s_start = 0;
        for (int e2 = 0; e2 < e; ++e2) s_start += counts[s * E + e2];
        int32_t* rb = return_blocks + (s * L + l) * 4;
        rb[0] = fits ? c : 0;
        rb[1] = seg + within;
        rb[2] = s;
        rb[3] = s_start;
        within += c;
      }
      if (fits) seg += pad128(total);
    }
    seg_start[L] = seg;
    s_total = seg;
  }
  __syncthreads();
  // ---- expert of every 128-row tile of my buffer
  const int num_tiles = max_rows / 128;
  for (int t = threadIdx.x; t < num_tiles; t += blockDim.x) {
    const int row = t * 128;
    int g = -1;
    if (row < s_total) {
      for (int l = 0; l < L; ++l)
        if (row >= seg_start[l] && row < seg_start[l + 1]) g = l;
    }
    tile_group[t] = g;
  }
}

// one warp per row; the rows of every block are spread over all warps of the grid.
// QUANT: rows are quantised to FP8 E4M3 with one fp32 scale per 1 x 128 block while they are being
// sent (d bytes per row into `dst`, d / 128 floats per row into `scales`).
template <bool QUANT>
__global__ void __launch_bounds__(256)
ep_var_exchange_kernel(const __nv_bfloat16* __restrict__ src, const int32_t* __restrict__ row_index, int index_div,
                       const int32_t* __restrict__ blocks, int num_blocks, PicoPeerTable dst, PicoPeerTable scales,
                       PicoPeerTable flags, int ep, int my_rank, int d, int slot, uint32_t epoch,
                       unsigned int* counter) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const int gwarp = blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
  const int nwarps = gridDim.x * warps_per_cta;
  const int vec = d / 8;
  for (int b = 0; b < num_blocks; ++b) {
    const int cnt = __ldg(blocks + b * 4 + 0);
    const int src_row = __ldg(blocks + b * 4 + 1);
    const int dst_rank = __ldg(blocks + b * 4 + 2);
    const int dst_row = __ldg(blocks + b * 4 + 3);
    for (int j = gwarp; j < cnt; j += nwarps) {
      const int64_t srow = row_index ? (int64_t)(__ldg(row_index + src_row + j) / index_div) : (int64_t)(src_row + j);
      const uint4* in = reinterpret_cast<const uint4*>(src + srow * d);
      const int64_t drow = (int64_t)dst_row + j;
      if (!QUANT) {
        uint4* o = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst.ptr[dst_rank]) + drow * d);
        for (int v = lane; v < vec; v += 32) o[v] = in[v];
      } else {
        uint8_t* out = reinterpret_cast<uint8_t*>(dst.ptr[dst_rank]) + drow * d;
        float* sc = reinterpret_cast<float*>(scales.ptr[dst_rank]) + drow * (d / 128);
        for (int v = lane; v < vec; v += 32) {   // d % 256 == 0: all 32 lanes take part in the shuffles
          const uint4 raw = in[v];
          const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
          float f[8];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 t = __bfloat1622float2(p2[q]);
            f[2 * q] = t.x;
            f[2 * q + 1] = t.y;
          }
          float amax = 0.f;
#pragma unroll
          for (int q = 0; q < 8; ++q) amax = fmaxf(amax, fabsf(f[q]));
          // 16 lanes x 8 elements = one 128-element block
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
          const float scale = fmaxf(amax, 1e-12f) / 448.f;
          const float inv = 1.f / scale;
          uint2 qv;
          uint8_t* qb = reinterpret_cast<uint8_t*>(&qv);
#pragma unroll
          for (int q = 0; q < 8; ++q)
            qb[q] = (uint8_t)__nv_cvt_float_to_fp8(fminf(fmaxf(f[q] * inv, -448.f), 448.f), __NV_SATFINITE, __NV_E4M3);
          reinterpret_cast<uint2*>(out)[v] = qv;
          if ((lane & 15) == 0) sc[v / 16] = scale;
        }
      }
    }
  }
  raise_flags_when_grid_done(counter, flags, ep, my_rank, slot, epoch);
}

// payload / scales -> bf16 for the rows in use (their number is read from device memory)
__global__ void __launch_bounds__(256)
ep_var_dequant_kernel(const uint8_t* __restrict__ payload, const float* __restrict__ scales,
                      __nv_bfloat16* __restrict__ out, const int32_t* __restrict__ rows_in_use, int d) {
  const int64_t rows = *rows_in_use;
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

__global__ void ep_var_zero_padding_kernel(__nv_bfloat16* __restrict__ buf, const int32_t* __restrict__ seg_start,
                                           const int32_t* __restrict__ seg_len, int L, int d) {
  const int vec = d / 8;
  for (int l = blockIdx.x; l < L; l += gridDim.x) {
    const int first = seg_start[l] + seg_len[l];
    const int last = seg_start[l + 1];
    const int64_t n = (int64_t)(last - first) * vec;
    uint4* p = reinterpret_cast<uint4*>(buf + (int64_t)first * d);
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) p[i] = make_uint4(0, 0, 0, 0);
  }
}

// rows [0, *rows_in_use) of src -> dst (16-byte vectors)
__global__ void ep_var_copy_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                        const int32_t* __restrict__ rows_in_use, int vec_per_row) {
  const int64_t n = (int64_t)(*rows_in_use) * vec_per_row;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    dst[i] = src[i];
}

constexpr int kVarMaxDev = 64;
static unsigned int* g_var_counters[kVarMaxDev] = {nullptr};
static unsigned int* var_counter() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kVarMaxDev) return nullptr;
  if (!g_var_counters[dev]) {
    unsigned int* p = nullptr;
    if (cudaMalloc(&p, 64 * sizeof(unsigned int)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 64 * sizeof(unsigned int));
    g_var_counters[dev] = p;
  }
  return g_var_counters[dev];
}

}  // namespace pico

using namespace pico;

extern "C" int pico_ep_var_layout(const int32_t* counts_table, int ep, int L, int my_rank, int max_rows,
                                  int32_t* send_blocks, int32_t* return_blocks, int32_t* seg_start,
                                  int32_t* seg_len, int32_t* tile_group, cudaStream_t stream) {
  if (ep < 1 || ep > PICO_MAX_PEERS || L < 1 || max_rows < 128 || max_rows % 128 != 0) {
    pico_host::set_error("ep_var_layout: ep %d / L %d / max_rows %d (multiple of 128) out of range", ep, L, max_rows);
    return -2;
  }
  ep_var_layout_kernel<<<1, 256, 0, stream>>>(counts_table, ep, L, my_rank, max_rows, send_blocks, return_blocks,
                                              seg_start, seg_len, tile_group, pico_status_buffer());
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("ep_var_layout: %s", cudaGetErrorString(e));
  return (int)e;
}

extern "C" int pico_ep_var_exchange(const void* src, const int32_t* row_index, int index_div,
                                    const int32_t* blocks, int num_blocks, PicoPeerTable dst, PicoPeerTable scales,
                                    PicoPeerTable flags, int ep, int my_rank, int d, int quant, int slot,
                                    uint32_t epoch, cudaStream_t stream) {
  if (ep < 1 || ep > PICO_MAX_PEERS || d % 8 != 0 || slot < 0 || slot >= PICO_FLAG_SLOTS || index_div < 1 ||
      (quant && d % 256 != 0)) {
    pico_host::set_error("ep_var_exchange: ep %d / d %d (multiple of 8; of 256 when quantising) / slot %d out of range",
                         ep, d, slot);
    return -2;
  }
  unsigned int* counter = var_counter();
  if (!counter) return -1;
  const int grid = pico_host::num_sms() * 2;
  if (quant)
    ep_var_exchange_kernel<true><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)src, row_index, index_div, blocks,
                                                           num_blocks, dst, scales, flags, ep, my_rank, d, slot, epoch,
                                                           counter);
  else
    ep_var_exchange_kernel<false><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)src, row_index, index_div, blocks,
                                                            num_blocks, dst, scales, flags, ep, my_rank, d, slot, epoch,
                                                            counter);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("ep_var_exchange: %s", cudaGetErrorString(e));
  return (int)e;
}

extern "C" int pico_ep_var_dequant(const void* payload, const float* scales, void* out, const int32_t* rows_in_use,
                                   int max_rows, int d, cudaStream_t stream) {
  if (d % 128 != 0 || max_rows < 1) {
    pico_host::set_error("ep_var_dequant: row width %d must be a multiple of 128", d);
    return -2;
  }
  int64_t blocks = ((int64_t)max_rows * d / 8 + 255) / 256;
  const int cap = pico_host::num_sms() * 8;
  if (blocks > cap) blocks = cap;
  ep_var_dequant_kernel<<<(int)blocks, 256, 0, stream>>>((const uint8_t*)payload, scales, (__nv_bfloat16*)out,
                                                        rows_in_use, d);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("ep_var_dequant: %s", cudaGetErrorString(e));
  return (int)e;
}

extern "C" int pico_ep_var_copy_rows(const void* src, void* dst, const int32_t* rows_in_use, int max_rows, int d,
                                     cudaStream_t stream) {
  if (d % 8 != 0 || max_rows < 1) {
    pico_host::set_error("ep_var_copy_rows: row width %d must be a multiple of 8", d);
    return -2;
  }
  int64_t blocks = ((int64_t)max_rows * (d / 8) + 255) / 256;
  const int cap = pico_host::num_sms() * 8;
  if (blocks > cap) blocks = cap;
  ep_var_copy_rows_kernel<<<(int)blocks, 256, 0, stream>>>((const uint4*)src, (uint4*)dst, rows_in_use, d / 8);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("ep_var_copy_rows: %s", cudaGetErrorString(e));
  return (int)e;
}

extern "C" int pico_ep_var_zero_padding(void* buf, const int32_t* seg_start, const int32_t* seg_len, int L, int d,
                                        cudaStream_t stream) {
  if (L < 1 || d % 8 != 0) {
    pico_host::set_error("ep_var_zero_padding: L %d / d %d out of range", L, d);
    return -2;
  }
  ep_var_zero_padding_kernel<<<L, 256, 0, stream>>>((__nv_bfloat16*)buf, seg_start, seg_len, L, d);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("ep_var_zero_padding: %s", cudaGetErrorString(e));
  return (int)e;
}
