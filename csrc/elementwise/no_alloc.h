// Allocation-free entry point. It has no counterpart in the reference framework.
//
// Some callers of this library must not allocate device memory at the moment they launch
// work: a host program that embeds these kernels behind a fixed memory budget and has handed
// every byte of the device to its own arena, a callback that runs while another component
// holds the allocator lock, or code on a path where cudaMalloc's implicit device
// synchronisation would stall other streams. The regular RMSNorm backward needs a scratch
// matrix for its per-CTA weight-gradient partial sums, which somebody has to allocate. This
// variant keeps that scratch in a fixed array inside the library image instead, so the caller
// passes only inputs and outputs.
//
// What to know before using it:
//  * The scratch is PICO_NOALLOC_MAX_PARTIALS x PICO_NOALLOC_MAX_HIDDEN floats (5 MiB). Every
//    GPU on which this library is loaded holds that much until the process exits, whether or
//    not the entry point is ever called.
//  * Hidden sizes above PICO_NOALLOC_MAX_HIDDEN (or not a multiple of 8) are rejected with an
//    error; nothing is launched.
//  * The first call on each device looks up the device address of the array (with that device
//    current). Make that first call outside any stream capture.
//  * All calls on a device share the one array and it keeps whatever the last call left in it.
//    Each call overwrites every element it later reads, so nothing has to be cleared, but two
//    calls whose kernels can overlap on the GPU (different streams without an ordering
//    between them) race on the scratch and produce garbage: order them.
//  * It calls no cudaMalloc, cudaFree or any allocating library routine.
#pragma once
#include <cuda_runtime.h>

#define PICO_NOALLOC_MAX_PARTIALS 160
#define PICO_NOALLOC_MAX_HIDDEN 8192

#ifdef __cplusplus
extern "C" {
#endif

// Same contract as pico_rmsnorm_bwd (elementwise.h) minus the dw_partial argument:
//   dh = d(norm)/dh (+ dres);  dw (fp32 and/or bf16, = or += when accumulate) = sum_rows dy*h*rstd
// Returns 0 on success, non-zero otherwise with a message in pico_last_error().
int pico_rmsnorm_bwd_noalloc(const void* dy, const void* h, const void* w, const float* rstd,
                             const void* dres, void* dh, float* dw_f32, void* dw_bf16,
                             int accumulate, int rows, int H, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
