// RMSNorm backward that allocates nothing: the per-CTA weight-gradient partials live in a
// file-scope device array instead of caller-provided scratch. See no_alloc.h for who needs
// this and for the rules of use.
#include "no_alloc.h"

#include <atomic>
#include <mutex>

#include "../common/host.h"
#include "norm_kernels.cuh"

namespace {

// [partials][hidden] fp32. In host code this name is only a handle for the runtime's symbol
// lookup, never a device pointer: kernels get the address that cudaGetSymbolAddress returns.
static __device__ __align__(256) float g_dw_scratch[PICO_NOALLOC_MAX_PARTIALS * PICO_NOALLOC_MAX_HIDDEN];

constexpr int kMaxDevices = 64;
// written once per device under the mutex, read without it: hence atomic
std::atomic<float*> g_scratch_ptr[kMaxDevices];
std::mutex g_setup_mu;

// Device address of the scratch on the current device, resolved once per device.
float* scratch_for_current_device() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    pico_host::set_error("rmsnorm_bwd_noalloc: cannot identify the current device (%s)",
                         cudaGetErrorString(e));
    return nullptr;
  }
  if (float* known = g_scratch_ptr[dev].load(std::memory_order_acquire)) return known;
  std::lock_guard<std::mutex> lk(g_setup_mu);
  if (float* known = g_scratch_ptr[dev].load(std::memory_order_acquire)) return known;
  float* ptr = nullptr;
  e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_dw_scratch);
  if (e != cudaSuccess || ptr == nullptr) {
    pico_host::set_error("rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed on device %d (%s)", dev,
                         cudaGetErrorString(e));
    return nullptr;
  }
  g_scratch_ptr[dev].store(ptr, std::memory_order_release);
  return ptr;
}

}  // namespace

extern "C" int pico_rmsnorm_bwd_noalloc(const void* dy, const void* h, const void* w,
                                        const float* rstd, const void* dres, void* dh,
                                        float* dw_f32, void* dw_bf16, int accumulate, int rows,
                                        int H, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H % 8 != 0 || H <= 0) {
    pico_host::set_error("rmsnorm_bwd_noalloc: hidden size %d must be a positive multiple of 8", H);
    return -2;
  }
  if (H > PICO_NOALLOC_MAX_HIDDEN) {
    pico_host::set_error(
        "rmsnorm_bwd_noalloc: hidden size %d exceeds the built-in scratch (max %d); use "
        "pico_rmsnorm_bwd with caller-provided scratch instead",
        H, PICO_NOALLOC_MAX_HIDDEN);
    return -2;
  }
  float* scratch = scratch_for_current_device();
  if (!scratch) return -1;
  int grid = pico_host::num_sms();
  if (grid > PICO_NOALLOC_MAX_PARTIALS) grid = PICO_NOALLOC_MAX_PARTIALS;
  const __nv_bfloat16* dyp = static_cast<const __nv_bfloat16*>(dy);
  const __nv_bfloat16* hp = static_cast<const __nv_bfloat16*>(h);
  const __nv_bfloat16* wp = static_cast<const __nv_bfloat16*>(w);
  const __nv_bfloat16* rp = static_cast<const __nv_bfloat16*>(dres);
  __nv_bfloat16* dhp = static_cast<__nv_bfloat16*>(dh);
  // every CTA writes its full H-wide row of partials (zeros if it owned no rows), so the
  // column sum below never reads stale contents of the shared array
  const int need = (H / 8 + pico::kNormThreads - 1) / pico::kNormThreads;
  if (need <= 1)
    pico::rmsnorm_bwd_kernel<1><<<grid, pico::kNormThreads, 0, stream>>>(dyp, hp, wp, rstd, rp, dhp, scratch, rows, H);
  else if (need <= 2)
    pico::rmsnorm_bwd_kernel<2><<<grid, pico::kNormThreads, 0, stream>>>(dyp, hp, wp, rstd, rp, dhp, scratch, rows, H);
  else
    pico::rmsnorm_bwd_kernel<4><<<grid, pico::kNormThreads, 0, stream>>>(dyp, hp, wp, rstd, rp, dhp, scratch, rows, H);
  pico::colsum_kernel<<<(H + 31) / 32, 256, 0, stream>>>(scratch, grid, H, dw_f32,
                                                           static_cast<__nv_bfloat16*>(dw_bf16), accumulate);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    pico_host::set_error("rmsnorm_bwd_noalloc: %s", cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}
