// Mixture-of-experts routing on the device, in three kernels that replace ~15 eager tensor ops per
// layer and direction (softmax, bias add, top-k, gather, renormalise, counts; stable sort, cumsum
// and scatter for the slot assignment; gather * weight + sum over k for the combine):
//
//   pico_moe_route       one warp per token: fp32 softmax over the E router logits, selection of
//                        the top-k experts on probs (+ bias when loss-free balancing is on), weights
//                        = the un-biased probabilities, renormalised over the k selected; also the
//                        per-expert row counts. Backward: pico_moe_route_bwd (weights -> logits,
//                        plus an optional dense gradient w.r.t. the probabilities, which is how the
//                        auxiliary balancing loss enters).
//   pico_moe_slots       one CTA per expert: position of every routed row inside its expert's queue
//                        in row order (deterministic), and the table row_of_slot[e * C + pos] = row
//                        for the rows that fit the capacity C (-1 elsewhere).
//   pico_moe_combine     y[t] = sum_k w[t,k] * expert_out[e(t,k) * C + pos(t,k)] over the rows that
//                        fit the capacity, k in fixed order; backward: pico_moe_combine_bwd gives the
//                        gradient of expert_out (each slot has exactly one reader, so no atomics)
//                        and of the weights (one dot product per routed row).
//
// Reference: picotron/expert_parallel/expert_parallel.py:168-224 (router, balancing, weighting),
// capacity_moe.py:44-57 (slot assignment).
#include <cuda_bf16.h>
#include <math_constants.h>

#include "../common/host.h"
#include "elementwise.h"

namespace pico {

constexpr int kMaxExpertsPerLane = 8;   // E <= 256
constexpr int kMaxTopK = 8;

__device__ __forceinline__ float route_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float route_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// logits: bf16 [T, E] (row stride ldl). probs: fp32 [T, E]. idx: int32 [T, k]. w: fp32 [T, k].
// counts: int32 [E], must be zero on entry.
__global__ void __launch_bounds__(256)
moe_route_kernel(const __nv_bfloat16* __restrict__ logits, int64_t ldl, const float* __restrict__ bias,
                 float* __restrict__ probs, int32_t* __restrict__ idx, float* __restrict__ w,
                 int32_t* __restrict__ counts, int T, int E, int k, int renorm) {
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int t = warp; t < T; t += nwarps) {
    float p[kMaxExpertsPerLane], s[kMaxExpertsPerLane];
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
      const int e = lane + 32 * i;
      p[i] = e < E ? __bfloat162float(logits[(int64_t)t * ldl + e]) : -CUDART_INF_F;
      mx = fmaxf(mx, p[i]);
    }
    mx = route_warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
      p[i] = (lane + 32 * i) < E ? __expf(p[i] - mx) : 0.f;
      sum += p[i];
    }
    sum = route_warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
      const int e = lane + 32 * i;
      p[i] *= inv;
      if (e < E) {
        probs[(int64_t)t * E + e] = p[i];
        s[i] = p[i] + (bias ? bias[e] : 0.f);
      } else {
        s[i] = -CUDART_INF_F;
      }
    }
    // k rounds of arg-max over the warp; ties go to the lower expert index
    float sel_w[kMaxTopK];
    int sel_e[kMaxTopK];
    float wsum = 0.f;
    for (int j = 0; j < k; ++j) {
      float best = -CUDART_INF_F;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < kMaxExpertsPerLane; ++i) {
        const int e = lane + 32 * i;
        if (s[i] > best || (s[i] == best && e < best_e)) {
          best = s[i];
          best_e = e;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) {
          best = ob;
          best_e = oe;
        }
      }
      // the lane that owns the winner hands out its un-biased probability and retires the entry
      float pw = 0.f;
#pragma unroll
      for (int i = 0; i < kMaxExpertsPerLane; ++i)
        if (lane + 32 * i == best_e) {
          pw = p[i];
          s[i] = -CUDART_INF_F;
        }
      pw = __shfl_sync(0xffffffffu, pw, best_e & 31);
      sel_w[j] = pw;
      sel_e[j] = best_e;
      wsum += pw;
    }
    if (lane == 0) {
      const float scale = (renorm && k > 1) ? 1.f / wsum : 1.f;
      for (int j = 0; j < k; ++j) {
        idx[(int64_t)t * k + j] = sel_e[j];
        w[(int64_t)t * k + j] = sel_w[j] * scale;
        atomicAdd(counts + sel_e[j], 1);
      }
    }
  }
}

// dlogits[t, :] (fp32) from dw[t, :k] and (optional) dprobs[t, :E].
__global__ void __launch_bounds__(256)
moe_route_bwd_kernel(const float* __restrict__ probs, const int32_t* __restrict__ idx, const float* __restrict__ w,
                     const float* __restrict__ dw, const float* __restrict__ dprobs, float* __restrict__ dlogits,
                     int T, int E, int k, int renorm) {
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int t = warp; t < T; t += nwarps) {
    float p[kMaxExpertsPerLane], g[kMaxExpertsPerLane];
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
      const int e = lane + 32 * i;
      p[i] = e < E ? probs[(int64_t)t * E + e] : 0.f;
      g[i] = (e < E && dprobs) ? dprobs[(int64_t)t * E + e] : 0.f;
    }
    // w_j = p_j / S over the selected set (S = 1 without renormalisation):
    // dL/dp_j = (dw_j - sum_i dw_i w_i) / S, with S = p_j / w_j for any selected j
    float dot = 0.f, S = 1.f;
    if (renorm && k > 1) {
      float psel = 0.f;
      for (int j = 0; j < k; ++j) {
        dot += dw[(int64_t)t * k + j] * w[(int64_t)t * k + j];
        const int e = idx[(int64_t)t * k + j];
        float pj = 0.f;
#pragma unroll
        for (int i = 0; i < kMaxExpertsPerLane; ++i)
          if (lane + 32 * i == e) pj = p[i];
        psel += __shfl_sync(0xffffffffu, pj, e & 31);
      }
      S = psel;
    }
    for (int j = 0; j < k; ++j) {
      const int e = idx[(int64_t)t * k + j];
      const float gj = (renorm && k > 1) ? (dw[(int64_t)t * k + j] - dot) / S : dw[(int64_t)t * k + j];
#pragma unroll
      for (int i = 0; i < kMaxExpertsPerLane; ++i)
        if (lane + 32 * i == e) g[i] += gj;
    }
    // softmax backward: dlogit_e = p_e (g_e - sum_e' g_e' p_e')
    float gp = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) gp += g[i] * p[i];
    gp = route_warp_sum(gp);
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
      const int e = lane + 32 * i;
      if (e < E) dlogits[(int64_t)t * E + e] = p[i] * (g[i] - gp);
    }
  }
}

// One CTA per expert e: pos[r] = number of rows r' < r with idx[r'] == e, for the rows of expert e;
// row_of_slot[e * C + pos] = r when pos < C (the table must hold -1 on entry).
__global__ void __launch_bounds__(1024)
moe_slots_kernel(const int32_t* __restrict__ idx, int R, int C, int32_t* __restrict__ pos,
                 int32_t* __restrict__ row_of_slot) {
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __shared__ int warp_tot[32];
  __shared__ int running;
  if (threadIdx.x == 0) running = 0;
  __syncthreads();
  for (int base = 0; base < R; base += blockDim.x) {
    const int r = base + threadIdx.x;
    const bool mine = r < R && idx[r] == e;
    const unsigned ballot = __ballot_sync(0xffffffffu, mine);
    const int before = __popc(ballot & ((1u << lane) - 1u));
    if (lane == 0) warp_tot[warp] = __popc(ballot);
    __syncthreads();
    int off = running;
    for (int wi = 0; wi < warp; ++wi) off += warp_tot[wi];
    if (mine) {
      const int ps = off + before;
      pos[r] = ps;
      if (row_of_slot != nullptr && ps < C) row_of_slot[(int64_t)e * C + ps] = r;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int wi = 0; wi < (int)(blockDim.x >> 5); ++wi) tot += warp_tot[wi];
      running += tot;
    }
    __syncthreads();
  }
}

// y[t, :] = sum_j [pos < C] w[t,j] * out[(idx[t,j] * C + pos[t,j]), :]; one warp per token, d % 8 == 0.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ out, const int32_t* __restrict__ idx,
                   const int32_t* __restrict__ pos, const float* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   int T, int k, int C, int d) {
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int nvec = d / 8;
  for (int t = warp; t < T; t += nwarps) {
    for (int v = lane; v < nvec; v += 32) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int j = 0; j < k; ++j) {
        const int ps = pos[(int64_t)t * k + j];
        if (ps >= C) continue;
        const float wj = w[(int64_t)t * k + j];
        const uint4 raw = reinterpret_cast<const uint4*>(out + ((int64_t)idx[(int64_t)t * k + j] * C + ps) * d)[v];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h[i]);
          acc[2 * i] += wj * f.x;
          acc[2 * i + 1] += wj * f.y;
        }
      }
      uint4 o;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) oh[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
      reinterpret_cast<uint4*>(y + (int64_t)t * d)[v] = o;
    }
  }
}

// One warp per slot s of the [E*C, d] expert-output table: row = row_of_slot[s];
// dout[s, :] = w[row] * dy[row / k, :] (zeros for an empty slot) and dw[row] = <dy[row / k], out[s]>.
// dw must be zero on entry for the rows that did not fit the capacity (they get no slot).
__global__ void __launch_bounds__(256)
moe_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ out,
                       const int32_t* __restrict__ row_of_slot, const float* __restrict__ w,
                       __nv_bfloat16* __restrict__ dout, float* __restrict__ dw, int64_t slots, int k, int d) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int nvec = d / 8;
  for (int64_t s = warp; s < slots; s += nwarps) {
    const int row = row_of_slot[s];
    if (row < 0) {
      for (int v = lane; v < nvec; v += 32) reinterpret_cast<uint4*>(dout + s * d)[v] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const float wr = w[row];
    const int t = row / k;
    float dot = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      const uint4 g = reinterpret_cast<const uint4*>(dy + (int64_t)t * d)[v];
      const uint4 o = reinterpret_cast<const uint4*>(out + s * d)[v];
      const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
      const __nv_bfloat162* oh = reinterpret_cast<const __nv_bfloat162*>(&o);
      uint4 r;
      __nv_bfloat162* rh = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 gf = __bfloat1622float2(gh[i]);
        const float2 of = __bfloat1622float2(oh[i]);
        dot += gf.x * of.x + gf.y * of.y;
        rh[i] = __floats2bfloat162_rn(wr * gf.x, wr * gf.y);
      }
      reinterpret_cast<uint4*>(dout + s * d)[v] = r;
    }
    dot = route_warp_sum(dot);
    if (lane == 0) dw[row] = dot;
  }
}

static int route_check(const char* what, int T, int E, int k) {
  if (T < 0 || E < 1 || E > 32 * kMaxExpertsPerLane || k < 1 || k > kMaxTopK || k > E) {
    pico_host::set_error("%s: %d tokens, %d experts (max %d), top-%d (max %d)", what, T, E, 32 * kMaxExpertsPerLane, k,
                         kMaxTopK);
    return -2;
  }
  return 0;
}

static int warp_grid(int64_t items) {
  int64_t blocks = (items + 7) / 8;       // 8 warps per CTA
  const int cap = pico_host::num_sms() * 8;
  if (blocks > cap) blocks = cap;
  return blocks < 1 ? 1 : (int)blocks;
}

}  // namespace pico

using namespace pico;

extern "C" int pico_moe_route(const void* logits, int64_t ldl, const float* bias, float* probs, int32_t* idx,
                              float* w, int32_t* counts, int T, int E, int k, int renorm, cudaStream_t stream) {
  if (int rc = route_check("moe_route", T, E, k)) return rc;
  if (T == 0) return 0;
  moe_route_kernel<<<warp_grid(T), 256, 0, stream>>>((const __nv_bfloat16*)logits, ldl, bias, probs, idx, w, counts,
                                                    T, E, k, renorm);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("moe_route: %s", cudaGetErrorString(e));
  return (int)e;
}

extern "C" int pico_moe_route_bwd(const float* probs, const int32_t* idx, const float* w, const float* dw,
                                  const float* dprobs, float* dlogits, int T, int E, int k, int renorm,
                                  cudaStream_t stream) {
  if (int rc = route_check("moe_route_bwd", T, E, k)) return rc;
  if (T == 0) return 0;
  moe_route_bwd_kernel<<<warp_grid(T), 256, 0, stream>>>(probs, idx, w, dw, dprobs, dlogits, T, E, k, renorm);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("moe_route_bwd: %s", cudaGetErrorString(e));
  return (int)e;
}

extern "C" int pico_moe_slots(const int32_t* idx, int R, int E, int C, int32_t* pos, int32_t* row_of_slot,
                              cudaStream_t stream) {
  if (R < 0 || E < 1 || C < 0) {
    pico_host::set_error("moe_slots: %d rows, %d experts, capacity %d", R, E, C);
    return -2;
  }
  if (R == 0) return 0;
  moe_slots_kernel<<<E, 1024, 0, stream>>>(idx, R, C, pos, row_of_slot);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("moe_slots: %s", cudaGetErrorString(e));
  return (int)e;
}

extern "C" int pico_moe_combine(const void* out, const int32_t* idx, const int32_t* pos, const float* w, void* y,
                                int T, int k, int C, int d, cudaStream_t stream) {
  if (d % 8 != 0 || k < 1 || k > kMaxTopK) {
    pico_host::set_error("moe_combine: row width %d must be a multiple of 8, top-%d at most %d", d, k, kMaxTopK);
    return -2;
  }
  if (T <= 0) return 0;
  moe_combine_kernel<<<warp_grid(T), 256, 0, stream>>>((const __nv_bfloat16*)out, idx, pos, w, (__nv_bfloat16*)y, T,
                                                      k, C, d);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("moe_combine: %s", cudaGetErrorString(e));
  return (int)e;
}

extern "C" int pico_moe_combine_bwd(const void* dy, const void* out, const int32_t* row_of_slot, const float* w,
                                    void* dout, float* dw, int64_t slots, int k, int d, cudaStream_t stream) {
  if (d % 8 != 0 || k < 1) {
    pico_host::set_error("moe_combine_bwd: row width %d must be a multiple of 8", d);
    return -2;
  }
  if (slots <= 0) return 0;
  moe_combine_bwd_kernel<<<warp_grid(slots), 256, 0, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)out,
                                                              row_of_slot, w, (__nv_bfloat16*)dout, dw, slots, k, d);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("moe_combine_bwd: %s", cudaGetErrorString(e));
  return (int)e;
}
