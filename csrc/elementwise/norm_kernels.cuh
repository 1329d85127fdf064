// Device code of the RMSNorm kernels, shared by the launchers in norm.cu and by the
// allocation-free entry point in norm_noalloc.cu.
#pragma once
#include <cuda_bf16.h>

namespace pico {

constexpr int kNormThreads = 256;
constexpr int kMaxVec = 8;  // vectors of 8 bf16 per thread kept in registers: H <= 16384

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < kNormThreads / 32) ? red[lane] : 0.f;
  return warp_sum(t);
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

template <int NV>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out, int rows, int H,
                   float eps) {
  __shared__ float red[kNormThreads / 32];
  const int nvec = H / 8;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * H);
    const uint4* rr = residual ? reinterpret_cast<const uint4*>(residual + (size_t)row * H) : nullptr;
    float vals[NV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        unpack8(xr[v], vals[i]);
        if (rr) {
          float r[8];
          unpack8(rr[v], r);
#pragma unroll
          for (int j = 0; j < 8; ++j) vals[i][j] += r[j];
          // the summed stream is rounded to bf16 before it is normalised, as an unfused
          // add followed by a norm would do
          uint4 hv = pack8(vals[i]);
          unpack8(hv, vals[i]);
          if (h_out) reinterpret_cast<uint4*>(h_out + (size_t)row * H)[v] = hv;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
      }
    }
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / (float)H + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float wv[8], o[8];
        unpack8(reinterpret_cast<const uint4*>(w)[v], wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * rstd * wv[j];
        reinterpret_cast<uint4*>(y + (size_t)row * H)[v] = pack8(o);
      }
    }
  }
}

// dw partials: dw_partial[blockIdx.x][H] fp32
template <int NV>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dh,
                   float* __restrict__ dw_partial, int rows, int H) {
  __shared__ float red[kNormThreads / 32];
  const int nvec = H / 8;
  float dw_acc[NV][8];
  float wv[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
#pragma unroll
    for (int j = 0; j < 8; ++j) dw_acc[i][j] = 0.f;
    if (v < nvec) unpack8(reinterpret_cast<const uint4*>(w)[v], wv[i]);
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rstd = rstd_in[row];
    float g[NV][8], hv[NV][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float d[8];
        unpack8(reinterpret_cast<const uint4*>(dy + (size_t)row * H)[v], d);
        unpack8(reinterpret_cast<const uint4*>(h + (size_t)row * H)[v], hv[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          g[i][j] = d[j] * wv[i][j];
          dot += g[i][j] * hv[i][j];
          dw_acc[i][j] += d[j] * hv[i][j] * rstd;
        }
      }
    }
    dot = block_sum(dot, red);
    const float c = dot / (float)H * rstd * rstd * rstd;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * g[i][j] - hv[i][j] * c;
        if (dres) {
          float r[8];
          unpack8(reinterpret_cast<const uint4*>(dres + (size_t)row * H)[v], r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        reinterpret_cast<uint4*>(dh + (size_t)row * H)[v] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      float4* out = reinterpret_cast<float4*>(dw_partial + (size_t)blockIdx.x * H + (size_t)v * 8);
      out[0] = make_float4(dw_acc[i][0], dw_acc[i][1], dw_acc[i][2], dw_acc[i][3]);
      out[1] = make_float4(dw_acc[i][4], dw_acc[i][5], dw_acc[i][6], dw_acc[i][7]);
    }
  }
}

// Warp-per-row variant for H = 256 * NVW (NVW <= 8, i.e. H <= 2048): no block-level barrier per
// row, each lane owns NVW vectors of 8 columns and keeps its weight-gradient partials in
// registers; the warps of a CTA combine theirs through shared memory at the end.
template <int NVW>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_warp_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                        const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                        const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dh,
                        float* __restrict__ dw_partial, int rows, int H) {
  constexpr int kWarps = kNormThreads / 32;
  __shared__ float red[kWarps][32 * 8 + 8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float dw_acc[NVW][8];
  float wv[NVW][8];
#pragma unroll
  for (int i = 0; i < NVW; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) dw_acc[i][j] = 0.f;
    unpack8(reinterpret_cast<const uint4*>(w)[lane + i * 32], wv[i]);
  }
  const float inv_h = 1.f / (float)H;
  for (int row = blockIdx.x * kWarps + warp; row < rows; row += gridDim.x * kWarps) {
    const float rstd = rstd_in[row];
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + (size_t)row * H);
    const uint4* hr = reinterpret_cast<const uint4*>(h + (size_t)row * H);
    uint4 draw[NVW], hraw[NVW];
#pragma unroll
    for (int i = 0; i < NVW; ++i) {
      draw[i] = dyr[lane + i * 32];
      hraw[i] = hr[lane + i * 32];
    }
    float g[NVW][8], hv[NVW][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NVW; ++i) {
      float d[8];
      unpack8(draw[i], d);
      unpack8(hraw[i], hv[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        g[i][j] = d[j] * wv[i][j];
        dot += g[i][j] * hv[i][j];
        dw_acc[i][j] += d[j] * hv[i][j] * rstd;
      }
    }
    dot = warp_sum(dot);
    const float c = dot * inv_h * rstd * rstd * rstd;
#pragma unroll
    for (int i = 0; i < NVW; ++i) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rstd * g[i][j] - hv[i][j] * c;
      if (dres) {
        float r[8];
        unpack8(reinterpret_cast<const uint4*>(dres + (size_t)row * H)[lane + i * 32], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += r[j];
      }
      reinterpret_cast<uint4*>(dh + (size_t)row * H)[lane + i * 32] = pack8(o);
    }
  }
  // combine the warps' partials (fixed order) and write this CTA's row of dw_partial
#pragma unroll 1
  for (int i = 0; i < NVW; ++i) {
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 8; ++j) red[warp][lane * 8 + j] = dw_acc[i][j];
    __syncthreads();
    // 256 columns of this slice, one per thread
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < kWarps; ++k) s += red[k][threadIdx.x];
    dw_partial[(size_t)blockIdx.x * H + i * 256 + threadIdx.x] = s;
  }
}

// Row-group variant for H = 2048 * NV: one CTA works on R rows at a time, every thread owning NV
// vectors of 8 columns of each row. The R row dot products share one pair of barriers, the
// weight-gradient partials are 8 * NV registers per thread, so many CTAs fit an SM and enough
// loads are in flight to keep the memory system busy (the warp-per-row kernel holds 64 partials per
// lane and runs at a quarter of the copy bandwidth).
template <int NV, int R>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_rows_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                        const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                        const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dh,
                        float* __restrict__ dw_partial, int rows, int H) {
  constexpr int kWarps = kNormThreads / 32;
  __shared__ float red[R][kWarps];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = H / 8;                       // == NV * kNormThreads
  float dw_acc[NV][8];
  float wv[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) dw_acc[i][j] = 0.f;
    unpack8(reinterpret_cast<const uint4*>(w)[threadIdx.x + i * kNormThreads], wv[i]);
  }
  const float inv_h = 1.f / (float)H;
  for (int row0 = blockIdx.x * R; row0 < rows; row0 += gridDim.x * R) {
    uint4 draw[R][NV], hraw[R][NV];
    float rstd[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = row0 + r;
      rstd[r] = row < rows ? rstd_in[row] : 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const size_t off = (size_t)min(row, rows - 1) * nvec + threadIdx.x + i * kNormThreads;
        draw[r][i] = reinterpret_cast<const uint4*>(dy)[off];
        hraw[r][i] = reinterpret_cast<const uint4*>(h)[off];
      }
    }
    float dot[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      dot[r] = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        float d[8], hv[8];
        unpack8(draw[r][i], d);
        unpack8(hraw[r][i], hv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dot[r] += d[j] * wv[i][j] * hv[j];
          dw_acc[i][j] += d[j] * hv[j] * rstd[r];      // rstd = 0 for rows past the end
        }
      }
      dot[r] = warp_sum(dot[r]);
    }
    __syncthreads();                            // the previous iteration's readers are done with red
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r) red[r][warp] = dot[r];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = row0 + r;
      if (row >= rows) break;
      float tot = 0.f;
#pragma unroll
      for (int k = 0; k < kWarps; ++k) tot += red[r][k];
      const float c = tot * inv_h * rstd[r] * rstd[r] * rstd[r];
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        float d[8], hv[8], o[8];
        unpack8(draw[r][i], d);
        unpack8(hraw[r][i], hv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd[r] * d[j] * wv[i][j] - hv[j] * c;
        const size_t off = (size_t)row * nvec + threadIdx.x + i * kNormThreads;
        if (dres) {
          float rr[8];
          unpack8(reinterpret_cast<const uint4*>(dres)[off], rr);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += rr[j];
        }
        reinterpret_cast<uint4*>(dh)[off] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    float4* out = reinterpret_cast<float4*>(dw_partial + (size_t)blockIdx.x * H +
                                            (size_t)(threadIdx.x + i * kNormThreads) * 8);
    out[0] = make_float4(dw_acc[i][0], dw_acc[i][1], dw_acc[i][2], dw_acc[i][3]);
    out[1] = make_float4(dw_acc[i][4], dw_acc[i][5], dw_acc[i][6], dw_acc[i][7]);
  }
}

// The same row-group scheme with the next group's rows already in flight while the current group
// is reduced and written: the loads of group g+1 are issued before the barriers of group g, so the
// memory system never idles between the load and the store phase of a CTA.
template <int NV, int R>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_rows_pf_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                           const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                           const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dh,
                           float* __restrict__ dw_partial, int rows, int H) {
  constexpr int kWarps = kNormThreads / 32;
  __shared__ float red[R][kWarps];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = H / 8;                       // == NV * kNormThreads
  float dw_acc[NV][8];
  float wv[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) dw_acc[i][j] = 0.f;
    unpack8(reinterpret_cast<const uint4*>(w)[threadIdx.x + i * kNormThreads], wv[i]);
  }
  const float inv_h = 1.f / (float)H;
  uint4 dnext[R][NV], hnext[R][NV];
  float rnext[R];
  const int stride = gridDim.x * R;
  int row0 = blockIdx.x * R;
  if (row0 < rows) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = row0 + r;
      rnext[r] = row < rows ? rstd_in[row] : 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const size_t off = (size_t)min(row, rows - 1) * nvec + threadIdx.x + i * kNormThreads;
        dnext[r][i] = reinterpret_cast<const uint4*>(dy)[off];
        hnext[r][i] = reinterpret_cast<const uint4*>(h)[off];
      }
    }
  }
  for (; row0 < rows; row0 += stride) {
    uint4 draw[R][NV], hraw[R][NV];
    float rstd[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      rstd[r] = rnext[r];
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        draw[r][i] = dnext[r][i];
        hraw[r][i] = hnext[r][i];
      }
    }
    const int next0 = row0 + stride;
    if (next0 < rows) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int row = next0 + r;
        rnext[r] = row < rows ? rstd_in[row] : 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const size_t off = (size_t)min(row, rows - 1) * nvec + threadIdx.x + i * kNormThreads;
          dnext[r][i] = reinterpret_cast<const uint4*>(dy)[off];
          hnext[r][i] = reinterpret_cast<const uint4*>(h)[off];
        }
      }
    }
    float dot[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      dot[r] = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        float d[8], hv[8];
        unpack8(draw[r][i], d);
        unpack8(hraw[r][i], hv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dot[r] += d[j] * wv[i][j] * hv[j];
          dw_acc[i][j] += d[j] * hv[j] * rstd[r];      // rstd = 0 for rows past the end
        }
      }
      dot[r] = warp_sum(dot[r]);
    }
    __syncthreads();                            // the previous iteration's readers are done with red
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r) red[r][warp] = dot[r];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = row0 + r;
      if (row >= rows) break;
      float tot = 0.f;
#pragma unroll
      for (int k = 0; k < kWarps; ++k) tot += red[r][k];
      const float c = tot * inv_h * rstd[r] * rstd[r] * rstd[r];
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        float d[8], hv[8], o[8];
        unpack8(draw[r][i], d);
        unpack8(hraw[r][i], hv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd[r] * d[j] * wv[i][j] - hv[j] * c;
        const size_t off = (size_t)row * nvec + threadIdx.x + i * kNormThreads;
        if (dres) {
          float rr[8];
          unpack8(reinterpret_cast<const uint4*>(dres)[off], rr);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += rr[j];
        }
        reinterpret_cast<uint4*>(dh)[off] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    float4* out = reinterpret_cast<float4*>(dw_partial + (size_t)blockIdx.x * H +
                                            (size_t)(threadIdx.x + i * kNormThreads) * 8);
    out[0] = make_float4(dw_acc[i][0], dw_acc[i][1], dw_acc[i][2], dw_acc[i][3]);
    out[1] = make_float4(dw_acc[i][4], dw_acc[i][5], dw_acc[i][6], dw_acc[i][7]);
  }
}

// dw[H] (=|+=) sum_p partial[p][H]; fixed summation order (deterministic)
static __global__ void colsum_kernel(const float* __restrict__ partial, int nparts, int H,
                                     float* __restrict__ out_f32, __nv_bfloat16* __restrict__ out_bf16,
                                     int accumulate) {
  // block = 32 columns x 8 row groups; each thread sums every 8th partial row of its column, the
  // eight sub-sums are then added in a fixed order
  __shared__ float red[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s = 0.f;
  if (c < H)
    for (int p = ry; p < nparts; p += 8) s += partial[(size_t)p * H + c];
  red[ry][cx] = s;
  __syncthreads();
  if (ry == 0 && c < H) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][cx];
    if (out_f32) out_f32[c] = accumulate ? out_f32[c] + t : t;
    if (out_bf16) out_bf16[c] = __float2bfloat16(accumulate ? __bfloat162float(out_bf16[c]) + t : t);
  }
}

}  // namespace pico
