#include "symm.h"

#include <cstring>

#include "../common/host.h"
#include "flags.cuh"

namespace pico {

__global__ void signal_peers_kernel(PicoPeerTable flags, int world, int my_rank, int slot,
                                    uint32_t epoch) {
  // make every earlier write of this stream (also those to peer memory) visible first
  __threadfence_system();
  const int t = threadIdx.x;
  if (t < world)
    st_release_sys(flag_word(flags.ptr[t], slot, my_rank), flag_value(flags.ptr[my_rank], slot, epoch, kFlagDone));
}

__global__ void wait_flags_kernel(const uint32_t* local_flags, int world, int slot, uint32_t epoch,
                                  uint64_t timeout_ns, int* status) {
  const int t = threadIdx.x;
  if (t < world)
    wait_flag_ge(local_flags + slot * PICO_MAX_PEERS + t, flag_value(local_flags, slot, epoch, kFlagDone),
                 timeout_ns, status, 900 + t);
}

__global__ void epoch_base_add_kernel(uint32_t* local_flags, PicoEpochDeltas d) {
  const int t = threadIdx.x;
  if (t < d.n) local_flags[PICO_FLAG_SLOTS * PICO_MAX_PEERS + d.slot[t]] += d.delta[t];
}

}  // namespace pico

extern "C" int pico_epoch_base_add(uint32_t* local_flags, const PicoEpochDeltas* deltas, cudaStream_t stream) {
  if (deltas->n < 0 || deltas->n > PICO_MAX_EPOCH_DELTAS) {
    pico_host::set_error("epoch_base_add: %d entries (at most %d)", deltas->n, PICO_MAX_EPOCH_DELTAS);
    return -2;
  }
  for (int i = 0; i < deltas->n; ++i)
    if (deltas->slot[i] < 0 || deltas->slot[i] >= PICO_FLAG_SLOTS) {
      pico_host::set_error("epoch_base_add: slot %d out of range", deltas->slot[i]);
      return -2;
    }
  pico::epoch_base_add_kernel<<<1, PICO_MAX_EPOCH_DELTAS, 0, stream>>>(local_flags, *deltas);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("epoch_base_add: %s", cudaGetErrorString(e));
  return (int)e;
}

extern "C" int pico_symm_alloc(size_t bytes, void** ptr, unsigned char* handle64) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) {
    pico_host::set_error("symm_alloc: cudaMalloc(%zu): %s", bytes, cudaGetErrorString(e));
    return (int)e;
  }
  cudaMemset(*ptr, 0, bytes);
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, *ptr);
  if (e != cudaSuccess) {
    pico_host::set_error("symm_alloc: cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
    cudaFree(*ptr);
    return (int)e;
  }
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  cudaDeviceSynchronize();
  return 0;
}

extern "C" int pico_symm_open(const unsigned char* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    pico_host::set_error("symm_open: cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

extern "C" int pico_symm_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }
extern "C" int pico_symm_free(void* ptr) { return (int)cudaFree(ptr); }

extern "C" int pico_signal_peers(PicoPeerTable flags, int world, int my_rank, int slot,
                                 uint32_t epoch, cudaStream_t stream) {
  if (world > PICO_MAX_PEERS || slot < 0 || slot >= PICO_FLAG_SLOTS) {
    pico_host::set_error("signal_peers: world %d / slot %d out of range", world, slot);
    return -2;
  }
  pico::signal_peers_kernel<<<1, 32, 0, stream>>>(flags, world, my_rank, slot, epoch);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("signal_peers: %s", cudaGetErrorString(e));
  return (int)e;
}

extern "C" int pico_wait_flags(const uint32_t* local_flags, int world, int slot, uint32_t epoch,
                               uint32_t timeout_ms, cudaStream_t stream) {
  if (world > PICO_MAX_PEERS || slot < 0 || slot >= PICO_FLAG_SLOTS) {
    pico_host::set_error("wait_flags: world %d / slot %d out of range", world, slot);
    return -2;
  }
  pico::wait_flags_kernel<<<1, 32, 0, stream>>>(local_flags, world, slot, epoch,
                                                (uint64_t)timeout_ms * 1000000ull, pico_status_buffer());
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("wait_flags: %s", cudaGetErrorString(e));
  return (int)e;
}
