// Memory-bound pointwise kernels: rotary embedding, SwiGLU, AdamW, embedding gather /
// scatter, gradient accumulation. Every kernel moves 16-byte vectors and is sized as a
// grid-stride loop over a multiple of the SM count.
#include <cuda_bf16.h>

#include "../common/host.h"
#include "elementwise.h"

namespace pico {

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

static inline int grid_for(int64_t work_items, int threads) {
  int64_t blocks = (work_items + threads - 1) / threads;
  int64_t cap = (int64_t)pico_host::num_sms() * 16;
  return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

static inline int finish(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("%s: %s", what, cudaGetErrorString(e));
  return (int)e;
}

// ------------------------------------------------------------------------------ RoPE
// one work item = 8 elements of the first half of a head + the matching 8 of the second half
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, int64_t row_stride, int rows, int seq,
                            int pos_offset, int nheads, int d, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, float sign) {
  const int half = d / 2;
  const int vec_per_head = half / 8;
  const int64_t total = (int64_t)rows * nheads * vec_per_head;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec_per_head);
    const int64_t t = i / vec_per_head;
    const int head = (int)(t % nheads);
    const int64_t row = t / nheads;
    const int pos = pos_offset + (int)(row % seq);
    __nv_bfloat16* base = x + row * row_stride + (int64_t)head * d + v * 8;
    float a[8], b[8], c[8], s[8];
    unpack8(*reinterpret_cast<const uint4*>(base), a);
    unpack8(*reinterpret_cast<const uint4*>(base + half), b);
    const float4* cp = reinterpret_cast<const float4*>(cos_t + (int64_t)pos * half + v * 8);
    const float4* sp = reinterpret_cast<const float4*>(sin_t + (int64_t)pos * half + v * 8);
    *reinterpret_cast<float4*>(&c[0]) = cp[0];
    *reinterpret_cast<float4*>(&c[4]) = cp[1];
    *reinterpret_cast<float4*>(&s[0]) = sp[0];
    *reinterpret_cast<float4*>(&s[4]) = sp[1];
    float oa[8], ob[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sj = s[j] * sign;
      oa[j] = a[j] * c[j] - b[j] * sj;
      ob[j] = b[j] * c[j] + a[j] * sj;
    }
    *reinterpret_cast<uint4*>(base) = pack8(oa);
    *reinterpret_cast<uint4*>(base + half) = pack8(ob);
  }
}

// ------------------------------------------------------------------------------ SwiGLU
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, int64_t ld_gu,
                                  __nv_bfloat16* __restrict__ y, int rows, int I, const int* __restrict__ rows_dev) {
  if (rows_dev) rows = min(rows, *rows_dev);   // row count known only on the device (dropless MoE buffers)
  const int vec_per_row = I / 8;
  const int64_t total = (int64_t)rows * vec_per_row;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec_per_row);
    const int64_t row = i / vec_per_row;
    float g[8], u[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(gu + row * ld_gu + v * 8), g);
    unpack8(*reinterpret_cast<const uint4*>(gu + row * ld_gu + I + v * 8), u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    *reinterpret_cast<uint4*>(y + row * (int64_t)I + v * 8) = pack8(o);
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                  const __nv_bfloat16* __restrict__ gu, int64_t ld_gu,
                                  __nv_bfloat16* __restrict__ dgu, int64_t ld_dgu, int rows, int I,
                                  const int* __restrict__ rows_dev) {
  if (rows_dev) rows = min(rows, *rows_dev);
  const int vec_per_row = I / 8;
  const int64_t total = (int64_t)rows * vec_per_row;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec_per_row);
    const int64_t row = i / vec_per_row;
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(*reinterpret_cast<const uint4*>(gu + row * ld_gu + v * 8), g);
    unpack8(*reinterpret_cast<const uint4*>(gu + row * ld_gu + I + v * 8), u);
    unpack8(*reinterpret_cast<const uint4*>(dy + row * (int64_t)I + v * 8), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * sg;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * sg * (1.f + g[j] * (1.f - sg));
    }
    *reinterpret_cast<uint4*>(dgu + row * ld_dgu + v * 8) = pack8(dg);
    *reinterpret_cast<uint4*>(dgu + row * ld_dgu + I + v * 8) = pack8(du);
  }
}

// ------------------------------------------------------------------------------ AdamW
__global__ void adamw_kernel(__nv_bfloat16* __restrict__ p, float* __restrict__ master,
                             float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                             int64_t n, float lr, float beta1, float beta2, float eps, float wd,
                             float bc1, float bc2, float grad_scale, int zero_grad) {
  const int64_t nvec = n / 4;
  const float step_size = lr / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec;
       i += (int64_t)gridDim.x * blockDim.x) {
    float4 gv = reinterpret_cast<float4*>(g)[i];
    float4 mv = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float pv[4];
    if (master) {
      float4 t = reinterpret_cast<float4*>(master)[i];
      pv[0] = t.x; pv[1] = t.y; pv[2] = t.z; pv[3] = t.w;
    } else {
      const __nv_bfloat162* pp = reinterpret_cast<const __nv_bfloat162*>(p + i * 4);
      float2 a = __bfloat1622float2(pp[0]), b = __bfloat1622float2(pp[1]);
      pv[0] = a.x; pv[1] = a.y; pv[2] = b.x; pv[3] = b.y;
    }
    float ga[4] = {gv.x * grad_scale, gv.y * grad_scale, gv.z * grad_scale, gv.w * grad_scale};
    float ma[4] = {mv.x, mv.y, mv.z, mv.w};
    float va[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      pv[j] *= (1.f - lr * wd);
      ma[j] = beta1 * ma[j] + (1.f - beta1) * ga[j];
      va[j] = beta2 * va[j] + (1.f - beta2) * ga[j] * ga[j];
      const float denom = sqrtf(va[j]) * inv_sqrt_bc2 + eps;
      pv[j] -= step_size * ma[j] / denom;
    }
    reinterpret_cast<float4*>(m)[i] = make_float4(ma[0], ma[1], ma[2], ma[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(va[0], va[1], va[2], va[3]);
    if (master) reinterpret_cast<float4*>(master)[i] = make_float4(pv[0], pv[1], pv[2], pv[3]);
    if (p) {
      __nv_bfloat162* pp = reinterpret_cast<__nv_bfloat162*>(p + i * 4);
      pp[0] = __floats2bfloat162_rn(pv[0], pv[1]);
      pp[1] = __floats2bfloat162_rn(pv[2], pv[3]);
    }
    if (zero_grad) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  // scalar tail (n not a multiple of 4)
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const int64_t i = nvec * 4 + threadIdx.x;
    float pvs = master ? master[i] : __bfloat162float(p[i]);
    const float gs = g[i] * grad_scale;
    pvs *= (1.f - lr * wd);
    const float ms = beta1 * m[i] + (1.f - beta1) * gs;
    const float vs = beta2 * v[i] + (1.f - beta2) * gs * gs;
    pvs -= step_size * ms / (sqrtf(vs) * inv_sqrt_bc2 + eps);
    m[i] = ms;
    v[i] = vs;
    if (master) master[i] = pvs;
    if (p) p[i] = __float2bfloat16(pvs);
    if (zero_grad) g[i] = 0.f;
  }
}

// ------------------------------------------------------------------------------ embedding
__global__ void embedding_fwd_kernel(const __nv_bfloat16* __restrict__ W,
                                     const int64_t* __restrict__ ids, __nv_bfloat16* __restrict__ out,
                                     int rows, int H, int Vlocal, int vocab_start) {
  const int vec_per_row = H / 8;
  const int64_t total = (int64_t)rows * vec_per_row;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec_per_row);
    const int64_t row = i / vec_per_row;
    const int64_t id = ids[row] - vocab_start;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (id >= 0 && id < Vlocal) val = reinterpret_cast<const uint4*>(W + id * (int64_t)H)[v];
    reinterpret_cast<uint4*>(out + row * (int64_t)H)[v] = val;
  }
}

__global__ void embedding_bwd_kernel(const __nv_bfloat16* __restrict__ dout,
                                     const int64_t* __restrict__ ids, float* __restrict__ dW,
                                     int rows, int H, int Vlocal, int vocab_start) {
  const int vec_per_row = H / 8;
  const int64_t total = (int64_t)rows * vec_per_row;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec_per_row);
    const int64_t row = i / vec_per_row;
    const int64_t id = ids[row] - vocab_start;
    if (id < 0 || id >= Vlocal) continue;
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(dout + row * (int64_t)H)[v], f);
    float* dst = dW + id * (int64_t)H + v * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dst + j, f[j]);
  }
}

// ------------------------------------------------------------------------------ misc
__global__ void accumulate_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst,
                                  int64_t n) {
  const int64_t nvec = n / 8;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec;
       i += (int64_t)gridDim.x * blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(src)[i], f);
    float4* d = reinterpret_cast<float4*>(dst) + i * 2;
    float4 a = d[0], b = d[1];
    a.x += f[0]; a.y += f[1]; a.z += f[2]; a.w += f[3];
    b.x += f[4]; b.y += f[5]; b.z += f[6]; b.w += f[7];
    d[0] = a;
    d[1] = b;
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {
    const int64_t i = nvec * 8 + threadIdx.x;
    dst[i] += __bfloat162float(src[i]);
  }
}

__global__ void fill_kernel(uint32_t* __restrict__ dst, uint32_t value, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    dst[i] = value;
}

}  // namespace pico

using namespace pico;

// Exact merge of two partial attention results over disjoint key sets (online softmax):
// lse' = log(exp(lse_a) + exp(lse_b)); out' = out_a * exp(lse_a - lse') + out_b * exp(lse_b - lse').
// out_a: fp32 or bf16 [b, s, H, d]; out_b: bf16; result fp32 (may alias out_a when that is fp32).
// lse: fp32 [b, H, s]. One warp per (b, s, h) row. A row that has seen no key on either side
// (both lse = -inf) stays zero with lse = -inf.
template <typename TA>
__global__ void attn_merge_kernel(const TA* __restrict__ out_a, const float* __restrict__ lse_a,
                                  const __nv_bfloat16* __restrict__ out_b, const float* __restrict__ lse_b,
                                  float* __restrict__ out, float* __restrict__ lse, int B, int S, int H, int D) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t rows = (int64_t)B * S * H;
  for (int64_t r = warp; r < rows; r += nwarps) {
    const int h = (int)(r % H);
    const int64_t bs = r / H;
    const int s = (int)(bs % S);
    const int b = (int)(bs / S);
    const int64_t li = ((int64_t)b * H + h) * S + s;
    const float la = lse_a[li], lb = lse_b[li];
    const float mx = fmaxf(la, lb);
    float wa = 0.f, wb = 0.f, ln = -INFINITY;
    if (mx > -INFINITY) {
      const float ea = __expf(la - mx), eb = __expf(lb - mx);
      ln = mx + __logf(ea + eb);
      wa = ea / (ea + eb);
      wb = eb / (ea + eb);
    }
    for (int c = lane; c < D; c += 32) {
      const float a = (float)out_a[r * D + c];
      const float bb = __bfloat162float(out_b[r * D + c]);
      out[r * D + c] = a * wa + bb * wb;
    }
    if (lane == 0) lse[li] = ln;
  }
}

extern "C" int pico_attn_merge(const void* out_a, int a_is_f32, const float* lse_a, const void* out_b,
                               const float* lse_b, float* out, float* lse, int B, int S, int H, int D,
                               cudaStream_t stream) {
  const int64_t rows = (int64_t)B * S * H;
  if (rows <= 0) return 0;
  const int grid = grid_for(rows * 32, 256);
  if (a_is_f32)
    attn_merge_kernel<float><<<grid, 256, 0, stream>>>((const float*)out_a, lse_a, (const __nv_bfloat16*)out_b,
                                                       lse_b, out, lse, B, S, H, D);
  else
    attn_merge_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)out_a, lse_a,
                                                               (const __nv_bfloat16*)out_b, lse_b, out, lse, B, S, H, D);
  return finish("attn_merge");
}

// x *= *scale unless *scale == 1 (the usual case costs one scalar load per thread and no traffic)
__global__ void scale_unless_one_kernel(uint4* __restrict__ x, int64_t nvec, const float* __restrict__ scale) {
  const float sc = *scale;
  if (sc == 1.0f) return;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec;
       i += (int64_t)gridDim.x * blockDim.x) {
    uint4 v = x[i];
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(p[j]);
      p[j] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
    }
    x[i] = v;
  }
}

extern "C" int pico_scale_unless_one(void* x_bf16, int64_t n, const float* scale_dev, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n % 8 != 0) {
    pico_host::set_error("scale_unless_one: %lld elements, need a multiple of 8", (long long)n);
    return -2;
  }
  scale_unless_one_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>((uint4*)x_bf16, n / 8, scale_dev);
  return finish("scale_unless_one");
}

extern "C" int pico_rope_inplace(void* x, int64_t row_stride, int rows, int seq, int pos_offset,
                                 int nheads, int d, const float* cos, const float* sin, int sign,
                                 cudaStream_t stream) {
  if (rows <= 0 || nheads <= 0) return 0;
  if (d % 16 != 0 || row_stride % 8 != 0) {
    pico_host::set_error("rope: head_dim %d must be a multiple of 16 and row stride %lld of 8", d,
                         (long long)row_stride);
    return -2;
  }
  const int64_t total = (int64_t)rows * nheads * (d / 16);
  rope_kernel<<<grid_for(total, 256), 256, 0, stream>>>((__nv_bfloat16*)x, row_stride, rows, seq,
                                                        pos_offset, nheads, d, cos, sin,
                                                        sign >= 0 ? 1.f : -1.f);
  return finish("rope");
}

extern "C" int pico_swiglu_fwd(const void* gu, int64_t ld_gu, void* y, int rows, int I, const int* rows_dev,
                               cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (I % 8 != 0 || ld_gu % 8 != 0) {
    pico_host::set_error("swiglu: width %d and stride %lld must be multiples of 8", I, (long long)ld_gu);
    return -2;
  }
  swiglu_fwd_kernel<<<grid_for((int64_t)rows * (I / 8), 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)gu, ld_gu, (__nv_bfloat16*)y, rows, I, rows_dev);
  return finish("swiglu_fwd");
}

extern "C" int pico_swiglu_bwd(const void* dy, const void* gu, int64_t ld_gu, void* dgu,
                               int64_t ld_dgu, int rows, int I, const int* rows_dev, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (I % 8 != 0 || ld_gu % 8 != 0 || ld_dgu % 8 != 0) {
    pico_host::set_error("swiglu: width and strides must be multiples of 8");
    return -2;
  }
  swiglu_bwd_kernel<<<grid_for((int64_t)rows * (I / 8), 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)gu, ld_gu, (__nv_bfloat16*)dgu, ld_dgu, rows, I, rows_dev);
  return finish("swiglu_bwd");
}

extern "C" int pico_adamw(void* p_bf16, float* master, float* g, float* m, float* v, int64_t n,
                          float lr, float beta1, float beta2, float eps, float weight_decay,
                          float bias_corr1, float bias_corr2, float grad_scale, int zero_grad,
                          cudaStream_t stream) {
  if (n <= 0) return 0;
  if (!p_bf16 && !master) {
    pico_host::set_error("adamw: need bf16 params or fp32 master params");
    return -2;
  }
  adamw_kernel<<<grid_for(n / 4 + 1, 256), 256, 0, stream>>>(
      (__nv_bfloat16*)p_bf16, master, g, m, v, n, lr, beta1, beta2, eps, weight_decay, bias_corr1,
      bias_corr2, grad_scale, zero_grad);
  return finish("adamw");
}

extern "C" int pico_embedding_fwd(const void* W, const int64_t* ids, void* out, int rows, int H,
                                  int Vlocal, int vocab_start, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H % 8 != 0) {
    pico_host::set_error("embedding: hidden size %d must be a multiple of 8", H);
    return -2;
  }
  embedding_fwd_kernel<<<grid_for((int64_t)rows * (H / 8), 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)W, ids, (__nv_bfloat16*)out, rows, H, Vlocal, vocab_start);
  return finish("embedding_fwd");
}

extern "C" int pico_embedding_bwd(const void* dout, const int64_t* ids, float* dW, int rows, int H,
                                  int Vlocal, int vocab_start, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H % 8 != 0) {
    pico_host::set_error("embedding: hidden size %d must be a multiple of 8", H);
    return -2;
  }
  embedding_bwd_kernel<<<grid_for((int64_t)rows * (H / 8), 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)dout, ids, dW, rows, H, Vlocal, vocab_start);
  return finish("embedding_bwd");
}

extern "C" int pico_accumulate_bf16_into_f32(const void* src, float* dst, int64_t n,
                                             cudaStream_t stream) {
  if (n <= 0) return 0;
  accumulate_kernel<<<grid_for(n / 8 + 1, 256), 256, 0, stream>>>((const __nv_bfloat16*)src, dst, n);
  return finish("accumulate");
}

extern "C" int pico_fill_u32(void* dst, uint32_t value, int64_t n_words, cudaStream_t stream) {
  if (n_words <= 0) return 0;
  fill_kernel<<<grid_for(n_words, 256), 256, 0, stream>>>((uint32_t*)dst, value, n_words);
  return finish("fill");
}
