// Expert-parallel dispatch and combine through NVLink peer memory for the fixed-capacity MoE
// layout: every (expert, source rank) pair owns C row slots, so all offsets are static and no
// counts have to be exchanged.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../runtime/symm.h"

#ifdef __cplusplus
extern "C" {
#endif

// Dispatch. This rank's routed rows are described by row_of_slot[E*C] (index of the routed row
// that occupies slot s of expert e, or -1) and `top_k` (routed row r belongs to token r / top_k).
// Slot (e, s) is sent to rank e / L, local expert l = e % L, and lands in that rank's receive slab
// at row (l * ep + my_rank) * C + s. Empty slots are written as zeros, so the receiver never has
// to clear its slab.
//   quant = 0: rows travel as bf16 into `payload` (d * 2 bytes per row)
//   quant = 1: rows are quantised to FP8 E4M3 with one fp32 scale per 1 x 128 block while they are
//              being sent: `payload` receives d bytes per row, `scales` d / 128 floats per row
// When the last CTA finishes, flag [slot][my_rank] = epoch is raised on every rank.
int pico_ep_dispatch(const void* tokens, const int32_t* row_of_slot, int top_k, PicoPeerTable payload,
                     PicoPeerTable scales, PicoPeerTable flags, int ep, int my_rank, int L, int C, int d,
                     int quant, int slot, uint32_t epoch, cudaStream_t stream);

// Receiver side of a quantised dispatch: payload/scales -> bf16 rows (waits for every source's
// flag first, bounded).
int pico_ep_dequant(const void* payload, const float* scales, void* out, int64_t rows, int d,
                    const uint32_t* local_flags, int ep, int slot, uint32_t epoch, uint32_t timeout_ms,
                    cudaStream_t stream);

// Block exchange used by combine (and by the backward passes): `src` is this rank's
// [L][ep][C][d] bf16 tensor; block (l, r) goes to rank r's buffer at row ((my_rank * L + l) * C),
// i.e. the receiver sees an [E][C][d] tensor indexed by global expert. With to_expert_major = 1
// the mapping is the reverse one: `src` is [E][C][d] and block (e = r*L + l) goes to rank r at row
// (l * ep + my_rank) * C (the dispatch layout, without quantisation). Raises the flag when done.
int pico_ep_block_exchange(const void* src, PicoPeerTable dst, PicoPeerTable flags, int ep, int my_rank,
                           int L, int C, int d, int to_expert_major, int slot, uint32_t epoch,
                           cudaStream_t stream);

#ifdef __cplusplus
}
#endif
