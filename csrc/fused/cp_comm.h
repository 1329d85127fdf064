// All-to-all layout exchanges of Ulysses context parallelism through peer memory: a rank trades its
// slice of the sequence (all heads) for the whole sequence of its slice of the heads, and back.
// One store kernel per tensor writes straight into the peers' buffers in the layout the attention
// kernel reads, so there are no chunk / concatenate copies around a library all-to-all.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../runtime/symm.h"

#ifdef __cplusplus
extern "C" {
#endif

// heads -> sequence: src[batch, s_local, world * cols] (bf16, contiguous; cols = heads_per_rank *
// head_dim). Column block r goes to rank r, which receives dst[batch, world * s_local, cols] with the
// rows of source rank q at sequence positions [q * s_local, (q + 1) * s_local). Afterwards flag
// [slot][my_rank] = epoch is raised on every rank.
int pico_a2a_heads_to_seq(const void* src, PicoPeerTable dst, PicoPeerTable flags, int world, int my_rank,
                          int batch, int s_local, int cols, int slot, uint32_t epoch, cudaStream_t stream);

// sequence -> heads (the inverse): src[batch, world * s_local, cols]; sequence block r goes to rank r,
// which receives dst[batch, s_local, world * cols] with source rank q's columns at [q * cols, (q+1) * cols).
int pico_a2a_seq_to_heads(const void* src, PicoPeerTable dst, PicoPeerTable flags, int world, int my_rank,
                          int batch, int s_local, int cols, int slot, uint32_t epoch, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
