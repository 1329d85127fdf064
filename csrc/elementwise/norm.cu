// RMSNorm forward / backward for bf16 activations with fp32 statistics, with the
// residual-stream add folded in:
//
//   forward :  h = x (+ residual);  rstd = rsqrt(mean(h^2) + eps);  y = h * rstd * w
//   backward:  g = dy * w;  dh = rstd * g - h * rstd^3 * mean(g * h) (+ dres);
//              dw = sum_rows(dy * h * rstd)
//
// One CTA of 256 threads owns a row at a time (persistent over rows in the backward so
// the weight-gradient partials stay in registers); all global traffic is 16-byte vectors.
// The hidden size must be a multiple of 8.
#include <cuda_bf16.h>

#include <type_traits>

#include "../common/host.h"
#include "elementwise.h"
#include "norm_kernels.cuh"

namespace pico {

template <typename F>
static int pick_nv(int H, F&& f) {
  const int nvec = H / 8;
  const int need = (nvec + kNormThreads - 1) / kNormThreads;
  if (need <= 1) return f(std::integral_constant<int, 1>());
  if (need <= 2) return f(std::integral_constant<int, 2>());
  if (need <= 4) return f(std::integral_constant<int, 4>());
  if (need <= kMaxVec) return f(std::integral_constant<int, kMaxVec>());
  pico_host::set_error("rmsnorm: hidden size %d too large (max %d)", H, kNormThreads * 8 * kMaxVec);
  return -2;
}

}  // namespace pico

extern "C" int pico_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y,
                                void* h_out, float* rstd, int rows, int H, float eps,
                                cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H % 8 != 0) {
    pico_host::set_error("rmsnorm: hidden size %d must be a multiple of 8", H);
    return -2;
  }
  int grid = rows < pico_host::num_sms() * 8 ? rows : pico_host::num_sms() * 8;
  int rc = pico::pick_nv(H, [&](auto nv) {
    pico::rmsnorm_fwd_kernel<decltype(nv)::value><<<grid, pico::kNormThreads, 0, stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)residual, (const __nv_bfloat16*)w,
        (__nv_bfloat16*)y, (__nv_bfloat16*)h_out, rstd, rows, H, eps);
    return 0;
  });
  if (rc) return rc;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("rmsnorm_fwd: %s", cudaGetErrorString(e));
  return (int)e;
}

extern "C" int pico_rmsnorm_bwd_num_partials(void) { return pico_host::num_sms() * 4; }

extern "C" int pico_rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd,
                                const void* dres, void* dh, float* dw_partial, float* dw_f32,
                                void* dw_bf16, int accumulate, int rows, int H,
                                cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H % 8 != 0) {
    pico_host::set_error("rmsnorm: hidden size %d must be a multiple of 8", H);
    return -2;
  }
  const int grid = pico_rmsnorm_bwd_num_partials();
  if (H == 2048 || H == 4096) {
    const __nv_bfloat16* a = (const __nv_bfloat16*)dy;
    const __nv_bfloat16* b = (const __nv_bfloat16*)h;
    const __nv_bfloat16* c = (const __nv_bfloat16*)w;
    const __nv_bfloat16* d = (const __nv_bfloat16*)dres;
    __nv_bfloat16* o = (__nv_bfloat16*)dh;
    int parts = grid;
    if (H == 2048) {
      // two rows per step with the next two in flight: 78 registers, three CTAs resident per SM and
      // exactly that many launched (48 us against 58 us for four rows per step without prefetch)
      parts = pico_host::num_sms() * 3;
      pico::rmsnorm_bwd_rows_pf_kernel<1, 2><<<parts, pico::kNormThreads, 0, stream>>>(a, b, c, rstd, d, o, dw_partial, rows, H);
    } else {
      pico::rmsnorm_bwd_rows_kernel<2, 2><<<grid, pico::kNormThreads, 0, stream>>>(a, b, c, rstd, d, o, dw_partial, rows, H);
    }
    pico::colsum_kernel<<<(H + 31) / 32, 256, 0, stream>>>(dw_partial, parts, H, dw_f32,
                                                             (__nv_bfloat16*)dw_bf16, accumulate);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) pico_host::set_error("rmsnorm_bwd: %s", cudaGetErrorString(e));
    return (int)e;
  }
  if (H % 256 == 0 && H <= 2048) {
    const __nv_bfloat16* a = (const __nv_bfloat16*)dy;
    const __nv_bfloat16* b = (const __nv_bfloat16*)h;
    const __nv_bfloat16* c = (const __nv_bfloat16*)w;
    const __nv_bfloat16* d = (const __nv_bfloat16*)dres;
    __nv_bfloat16* o = (__nv_bfloat16*)dh;
    switch (H / 256) {
#define PICO_W(N) case N: pico::rmsnorm_bwd_warp_kernel<N><<<grid, pico::kNormThreads, 0, stream>>>(a, b, c, rstd, d, o, dw_partial, rows, H); break;
      PICO_W(1) PICO_W(2) PICO_W(3) PICO_W(4) PICO_W(5) PICO_W(6) PICO_W(7) PICO_W(8)
#undef PICO_W
    }
    pico::colsum_kernel<<<(H + 31) / 32, 256, 0, stream>>>(dw_partial, grid, H, dw_f32,
                                                             (__nv_bfloat16*)dw_bf16, accumulate);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) pico_host::set_error("rmsnorm_bwd: %s", cudaGetErrorString(e));
    return (int)e;
  }
  int rc = pico::pick_nv(H, [&](auto nv) {
    pico::rmsnorm_bwd_kernel<decltype(nv)::value><<<grid, pico::kNormThreads, 0, stream>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w, rstd,
        (const __nv_bfloat16*)dres, (__nv_bfloat16*)dh, dw_partial, rows, H);
    return 0;
  });
  if (rc) return rc;
  pico::colsum_kernel<<<(H + 31) / 32, 256, 0, stream>>>(dw_partial, grid, H, dw_f32,
                                                           (__nv_bfloat16*)dw_bf16, accumulate);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("rmsnorm_bwd: %s", cudaGetErrorString(e));
  return (int)e;
}
