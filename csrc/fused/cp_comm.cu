#include "cp_comm.h"

#include <cuda_bf16.h>

#include "../common/host.h"
#include "../runtime/flags.cuh"

namespace pico {

// TO_SEQ: src[b][s][r][c] -> dst_r[b][my_rank * s_local + s][c]
// else  : src[b][r][s][c] -> dst_r[b][s][my_rank][c]
// c counts 16-byte vectors (vec = cols / 8).
template <bool TO_SEQ>
__global__ void a2a_kernel(const uint4* __restrict__ src, PicoPeerTable dst, PicoPeerTable flags, int world,
                           int my_rank, int batch, int s_local, int vec, int slot, uint32_t epoch,
                           unsigned int* counter) {
  const int64_t total = (int64_t)batch * s_local * world * vec;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % vec);
    int64_t t = i / vec;
    int r, s, b;
    if (TO_SEQ) {
      r = (int)(t % world);
      t /= world;
      s = (int)(t % s_local);
      b = (int)(t / s_local);
      const int64_t o = (((int64_t)b * world + my_rank) * s_local + s) * vec + c;
      reinterpret_cast<uint4*>(dst.ptr[r])[o] = src[i];
    } else {
      s = (int)(t % s_local);
      t /= s_local;
      r = (int)(t % world);
      b = (int)(t / world);
      const int64_t o = ((((int64_t)b * s_local + s) * world) + my_rank) * vec + c;
      reinterpret_cast<uint4*>(dst.ptr[r])[o] = src[i];
    }
  }
  raise_flags_when_grid_done(counter, flags, world, my_rank, slot, epoch);
}

constexpr int kMaxDevA2A = 64;
static unsigned int* g_a2a_counters[kMaxDevA2A] = {nullptr};

// One zero-initialised word per device for the "last CTA" detection; created on first use.
static unsigned int* a2a_counter() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevA2A) return nullptr;
  if (!g_a2a_counters[dev]) {
    unsigned int* p = nullptr;
    if (cudaMalloc(&p, 64 * sizeof(unsigned int)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 64 * sizeof(unsigned int));
    g_a2a_counters[dev] = p;
  }
  return g_a2a_counters[dev];
}

template <bool TO_SEQ>
static int launch_a2a(const char* what, const void* src, PicoPeerTable dst, PicoPeerTable flags, int world,
                      int my_rank, int batch, int s_local, int cols, int slot, uint32_t epoch,
                      cudaStream_t stream) {
  if (world < 1 || world > PICO_MAX_PEERS || slot < 0 || slot >= PICO_FLAG_SLOTS || cols % 8 != 0 || batch < 1 ||
      s_local < 1) {
    pico_host::set_error("%s: world %d / slot %d / cols %d (multiple of 8) out of range", what, world, slot, cols);
    return -2;
  }
  unsigned int* counter = a2a_counter();
  if (!counter) return -1;
  const int vec = cols / 8;
  const int64_t total = (int64_t)batch * s_local * world * vec;
  int grid = (int)((total + 255) / 256);
  const int cap = pico_host::num_sms() * 4;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  a2a_kernel<TO_SEQ><<<grid, 256, 0, stream>>>((const uint4*)src, dst, flags, world, my_rank, batch, s_local, vec,
                                               slot, epoch, counter + (TO_SEQ ? 0 : 1));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("%s: %s", what, cudaGetErrorString(e));
  return (int)e;
}

}  // namespace pico

extern "C" int pico_a2a_heads_to_seq(const void* src, PicoPeerTable dst, PicoPeerTable flags, int world,
                                     int my_rank, int batch, int s_local, int cols, int slot, uint32_t epoch,
                                     cudaStream_t stream) {
  return pico::launch_a2a<true>("a2a_heads_to_seq", src, dst, flags, world, my_rank, batch, s_local, cols, slot,
                                epoch, stream);
}

extern "C" int pico_a2a_seq_to_heads(const void* src, PicoPeerTable dst, PicoPeerTable flags, int world,
                                     int my_rank, int batch, int s_local, int cols, int slot, uint32_t epoch,
                                     cudaStream_t stream) {
  return pico::launch_a2a<false>("a2a_seq_to_heads", src, dst, flags, world, my_rank, batch, s_local, cols, slot,
                                 epoch, stream);
}
