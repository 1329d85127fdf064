// Device-side flag primitives (system-scope release/acquire, bounded waits).
#pragma once
#include <stdint.h>

#include "../common/ptx.cuh"
#include "symm.h"

namespace pico {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint32_t* flag_word(void* flags_base, int slot, int src) {
  return reinterpret_cast<uint32_t*>(flags_base) + slot * PICO_MAX_PEERS + src;
}

// Epochs reach the kernels as an offset from a per-slot base word kept behind the flag words of
// this rank's own flag buffer. Eager launches run with the host's mirror of that word, so the sum
// is the absolute epoch; a captured CUDA graph keeps its offsets and a node at its end advances
// the base by the number of epochs the graph used, which makes every replay continue the count.
__device__ __forceinline__ uint32_t epoch_base(const void* local_flags, int slot) {
  return __ldcg(reinterpret_cast<const uint32_t*>(local_flags) + PICO_FLAG_SLOTS * PICO_MAX_PEERS + slot);
}

// A flag word holds (absolute epoch << 8) | progress. Progress kFlagDone means the operation of that
// epoch is complete; 1 .. 254 mean that many parts of it are (the all-gather pushes report piece by
// piece so that their consumer can start on the first pieces). Waits compare with a wrap-safe ">=",
// so a waiter for part k is also released by any later part, by kFlagDone and by later epochs.
constexpr uint32_t kFlagDone = 0xFFu;
__device__ __forceinline__ uint32_t flag_value(const void* local_flags, int slot, uint32_t rel_epoch,
                                               uint32_t progress) {
  return ((epoch_base(local_flags, slot) + rel_epoch) << 8) | progress;
}

// Spin until *p >= epoch or `timeout_ns` passes. On timeout records error 2 and returns false.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* p, uint32_t epoch, uint64_t timeout_ns,
                                             int* status, int site) {
  if ((int32_t)(ld_acquire_sys(p) - epoch) >= 0) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if ((int32_t)(ld_acquire_sys(p) - epoch) >= 0) return true;
    if ((++spins & 0xff) == 0) {
      if (global_timer_ns() - t0 > timeout_ns) {
        report_error(status, PICO_ERR_FLAG_TIMEOUT, site, (int)epoch);
        return false;
      }
      __nanosleep(200);
    }
  }
}

// Waits for words [slot][src] >= base + rel_epoch for src = threadIdx.x < world (call with all
// threads of the CTA; returns false in every thread if any wait gave up).
__device__ __forceinline__ bool wait_slot_all(const uint32_t* local_flags, int slot, int world,
                                              uint32_t rel_epoch, uint64_t timeout_ns, int* status,
                                              int site) {
  __shared__ int pico_wait_ok;
  if (threadIdx.x == 0) pico_wait_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < world) {
    const uint32_t want = flag_value(local_flags, slot, rel_epoch, kFlagDone);
    if (!wait_flag_ge(local_flags + slot * PICO_MAX_PEERS + threadIdx.x, want, timeout_ns, status,
                      site + threadIdx.x))
      pico_wait_ok = 0;
  }
  __syncthreads();
  return pico_wait_ok != 0;
}

// Grid-wide completion: the last CTA to arrive raises flag [slot][my_rank] to (epoch, progress) on
// every rank of `flags`. `counter` is a device word that returns to zero after each use.
__device__ __forceinline__ void raise_flags_when_grid_done(unsigned int* counter, PicoPeerTable flags,
                                                           int world, int my_rank, int slot,
                                                           uint32_t rel_epoch, uint32_t progress = kFlagDone) {
  __threadfence_system();
  __syncthreads();
  __shared__ bool pico_last_cta;
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(counter, 1u) + 1u;
    pico_last_cta = (done == gridDim.x);
    if (pico_last_cta) *counter = 0;
  }
  __syncthreads();
  if (pico_last_cta && (int)threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(flag_word(flags.ptr[threadIdx.x], slot, my_rank),
                   flag_value(flags.ptr[my_rank], slot, rel_epoch, progress));
  }
}

}  // namespace pico
