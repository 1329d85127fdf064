// Kernels that move tensor-parallel activations between GPUs through peer memory, fused with the
// memory-bound op that produces or consumes them. Together with the flag-gated / scattering GEMM
// (gemm.h) they replace the all-gather and reduce-scatter collectives of sequence parallelism.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../runtime/symm.h"

#ifdef __cplusplus
extern "C" {
#endif

// Copy this rank's shard src[rows, cols] (bf16, contiguous) into row block `my_rank` of the
// gather buffer of every rank in `dst` (buffers of [world*rows, cols]), then raise flag
// [slot][my_rank] = epoch on every rank (flags table). One launch: all-gather by pushing.
int pico_push_rows(const void* src, PicoPeerTable dst, PicoPeerTable flags, int world, int my_rank,
                   int rows, int cols, int slot, uint32_t epoch, cudaStream_t stream);

// RMSNorm forward whose output goes straight into every rank's gather buffer (and, when y_local is
// given, into a local tensor as well): h = x (+ residual); y = norm(h) * w pushed as row block
// my_rank; then the flag is raised like pico_push_rows.
int pico_rmsnorm_fwd_push(const void* x, const void* residual, const void* w, void* y_local,
                          void* h_out, float* rstd, PicoPeerTable dst, PicoPeerTable flags, int world,
                          int my_rank, int rows, int H, float eps, int slot, uint32_t epoch,
                          cudaStream_t stream);

// Raise flag [slot][my_rank] = epoch on every rank once all earlier work of the stream is done
// (used after a scattering GEMM).  (= pico_signal_peers, re-exported for symmetry.)

// out[rows, cols] = sum_{s < world} staging[s][rows, cols] (+ addend), summed in rank order so the
// result is bit-identical on every run. Waits (bounded) for flags [slot][s] >= epoch of all ranks
// first: every writer raises its flag after its scattering GEMM.
int pico_slot_sum(const void* staging, int world, int rows, int cols, const void* addend, void* out,
                  const uint32_t* local_flags, int slot, uint32_t epoch, uint32_t timeout_ms,
                  cudaStream_t stream);

// Same, summing only slots first_slot .. world-1 (all flags are still awaited). With
// first_slot == world the result is the addend (or zero).
int pico_slot_sum_from(const void* staging, int world, int first_slot, int rows, int cols,
                       const void* addend, void* out, const uint32_t* local_flags, int slot, uint32_t epoch,
                       uint32_t timeout_ms, cudaStream_t stream);

// Row block o of src[num_dst*rows, cols] (bf16, contiguous) goes into slot `my_rank` of rank o's
// staging buffer ([world slots][rows][cols]) for o < num_dst; then flag [slot][my_rank] = epoch is
// raised on every rank. The scatter half of a reduce-scatter whose contributions differ per
// destination (context parallelism: a rank only holds gradients for the key blocks before its own).
int pico_scatter_rows(const void* src, PicoPeerTable dst, PicoPeerTable flags, int world, int my_rank,
                      int num_dst, int rows, int cols, int slot, uint32_t epoch, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
