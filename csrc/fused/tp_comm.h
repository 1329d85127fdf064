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

// Copy this rank's shard src[rows, cols] (bf16, contiguous) into the gather buffer of every rank in
// `dst` (buffers of [world*rows, cols]), then raise flag [slot][my_rank] = epoch on every rank (flags
// table). One launch: all-gather by pushing. The shard is a sequence of pieces of piece_rows rows
// (0 = one piece); source piece p becomes piece p * world + my_rank of the gathered tensor, i.e. a
// [batch, sequence/world] shard lands in its place inside [batch, sequence] (piece_rows =
// sequence/world), and one piece gives the plain "block my_rank" layout.
// skip_self: 0 = store to every rank; 1 = to the peers only (the caller fills this rank's own buffer
// itself, e.g. on another stream, so that local consumers need not wait for the remote stores);
// 2 = to this rank's own buffer only, without raising a flag (that local fill).
int pico_push_rows(const void* src, PicoPeerTable dst, PicoPeerTable flags, int world, int my_rank,
                   int rows, int cols, int piece_rows, int slot, uint32_t epoch, int skip_self,
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
// The source may also be a sequence of pieces of piece_rows rows (0 = `rows`: one piece per
// destination, as above); piece p then goes to destination p % num_dst as its (p / num_dst)-th piece.
int pico_scatter_rows(const void* src, PicoPeerTable dst, PicoPeerTable flags, int world, int my_rank,
                      int num_dst, int rows, int cols, int piece_rows, int slot, uint32_t epoch,
                      cudaStream_t stream);

#ifdef __cplusplus
}
#endif
