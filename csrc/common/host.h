// Host-side helpers shared by the launchers: error strings, the per-device status
// buffer that kernels report bounded-wait failures into, and TMA tensor-map encoding
// through the driver entry point (no link-time dependency on libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

#ifdef __cplusplus
extern "C" {
#endif

// 0 on success; otherwise a negative pico error or a positive cudaError_t.
// pico_last_error() returns a human-readable description of the last failure on this thread.
const char* pico_last_error(void);

// Per-device status words (device memory, zero when healthy). Allocated on first use.
int* pico_status_buffer(void);
// Copies the status words to the host (synchronises the device) and clears them.
// Returns the error code in word 0 (0 = ok); `out` may be NULL or hold 8 ints.
int pico_status_fetch(int* out);

#ifdef __cplusplus
}

namespace pico_host {

void set_error(const char* fmt, ...);

enum class Swizzle { None, B128 };

// 2-D row-major tensor map: `inner` elements contiguous, `outer` rows of `ld_bytes` pitch.
// Returns 0 on success.
int make_tmap_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int elem_bytes,
                 uint64_t inner, uint64_t outer, uint64_t ld_bytes, uint32_t box_inner,
                 uint32_t box_outer, Swizzle sw);

// 4-D map for [batch, seq, heads, head_dim] tensors: dims (d, heads, seq, batch), box
// (box_d, 1, box_rows, 1), 128-byte swizzle. Strides in bytes.
int make_tmap_bshd(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int elem_bytes,
                   uint64_t d, uint64_t heads, uint64_t seq, uint64_t batch, uint64_t row_stride_bytes,
                   uint64_t batch_stride_bytes, uint32_t box_d, uint32_t box_rows);

int num_sms();

}  // namespace pico_host
#endif
