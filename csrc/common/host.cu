#include "host.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "ptx.cuh"

namespace {
thread_local char g_err[512] = "";
constexpr int kMaxDevices = 64;
int* g_status[kMaxDevices] = {nullptr};
int g_num_sms[kMaxDevices] = {0};
std::mutex g_mu;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

EncodeTiledFn get_encode() {
  if (g_encode) return g_encode;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_encode) return g_encode;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e =
      cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || fn == nullptr) {
    pico_host::set_error("cuTensorMapEncodeTiled entry point unavailable (%s)",
                         cudaGetErrorString(e));
    return nullptr;
  }
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return g_encode;
}
}  // namespace

namespace pico_host {

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int make_tmap_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int elem_bytes,
                 uint64_t inner, uint64_t outer, uint64_t ld_bytes, uint32_t box_inner,
                 uint32_t box_outer, Swizzle sw) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  // The driver call needs this thread to have the device's primary context current. Threads
  // that have only been handed tensors (autograd worker threads) may not have bound it yet.
  {
    thread_local int bound_dev = -1;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev != bound_dev) {
      cudaSetDevice(dev);
      bound_dev = dev;
    }
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld_bytes & 15) != 0) {
    set_error("TMA operand must be 16-byte aligned with a 16-byte multiple pitch (ptr=%p pitch=%llu)",
              base, (unsigned long long)ld_bytes);
    return -2;
  }
  if (sw == Swizzle::B128 && box_inner * (uint32_t)elem_bytes != 128) {
    set_error("128B-swizzled box must be exactly 128 bytes wide");
    return -2;
  }
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   sw == Swizzle::B128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (inner=%llu outer=%llu pitch=%llu box=%ux%u)",
              (int)r, (unsigned long long)inner, (unsigned long long)outer,
              (unsigned long long)ld_bytes, box_inner, box_outer);
    return -3;
  }
  return 0;
}

int make_tmap_bshd(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int elem_bytes,
                   uint64_t d, uint64_t heads, uint64_t seq, uint64_t batch, uint64_t row_stride_bytes,
                   uint64_t batch_stride_bytes, uint32_t box_d, uint32_t box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  {
    thread_local int bound_dev = -1;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev != bound_dev) {
      cudaSetDevice(dev);
      bound_dev = dev;
    }
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (row_stride_bytes & 15) != 0 ||
      (batch_stride_bytes & 15) != 0 || ((d * elem_bytes) & 15) != 0 || box_d * (uint32_t)elem_bytes != 128) {
    set_error("attention operand: base/strides must be 16-byte aligned and the box 128 bytes wide "
              "(ptr=%p row=%llu batch=%llu d=%llu)", base, (unsigned long long)row_stride_bytes,
              (unsigned long long)batch_stride_bytes, (unsigned long long)d);
    return -2;
  }
  cuuint64_t dims[4] = {d, heads, seq, batch};
  cuuint64_t strides[3] = {d * (uint64_t)elem_bytes, row_stride_bytes, batch_stride_bytes};
  cuuint32_t box[4] = {box_d, 1, box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, dtype, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled(4d) failed with CUresult %d (d=%llu heads=%llu seq=%llu batch=%llu "
              "row=%llu batchstride=%llu)", (int)r, (unsigned long long)d, (unsigned long long)heads,
              (unsigned long long)seq, (unsigned long long)batch, (unsigned long long)row_stride_bytes,
              (unsigned long long)batch_stride_bytes);
    return -3;
  }
  return 0;
}

int num_sms() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  if (g_num_sms[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    g_num_sms[dev] = n > 0 ? n : 148;
  }
  return g_num_sms[dev];
}

}  // namespace pico_host

extern "C" const char* pico_last_error(void) { return g_err; }

extern "C" int* pico_status_buffer(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (g_status[dev]) return g_status[dev];
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_status[dev]) return g_status[dev];
  int* p = nullptr;
  if (cudaMalloc(&p, sizeof(int) * pico::PICO_STATUS_WORDS) != cudaSuccess) return nullptr;
  cudaMemset(p, 0, sizeof(int) * pico::PICO_STATUS_WORDS);
  g_status[dev] = p;
  return p;
}

extern "C" int pico_status_fetch(int* out) {
  int* p = pico_status_buffer();
  if (!p) return -1;
  int host[pico::PICO_STATUS_WORDS];
  if (cudaMemcpy(host, p, sizeof(host), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (host[0] != 0) cudaMemset(p, 0, sizeof(host));
  if (out) memcpy(out, host, sizeof(host));
  return host[0];
}
