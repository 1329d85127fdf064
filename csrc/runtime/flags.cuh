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

}  // namespace pico
