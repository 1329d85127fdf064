// Dropless expert-parallel dispatch and combine through NVLink peer memory with variable block
// sizes: no capacity, no dropped rows, no host synchronisation. Every rank publishes how many of
// its routed rows go to each expert; from the resulting [ep][E] table every rank derives the whole
// layout on the device (where each of its blocks lands in the receiver's expert-major buffer, the
// receiver's expert segments padded to 128-row tiles for the grouped GEMM, and the way back), and
// the rows are then stored straight into the peers' buffers at those offsets.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../runtime/symm.h"

#ifdef __cplusplus
extern "C" {
#endif

// Sizes of the int32 arrays that pico_ep_var_layout fills (E = ep * L experts):
//   send_blocks [E][4]      : for my block of expert e: {count, first row in my expert-sorted rows,
//                             destination rank, first row in the destination's receive buffer}
//   return_blocks [ep*L][4] : for the block of source s and local expert l in my receive buffer:
//                             {count, first row in my buffer, rank s, first row in s's sorted rows}
//   seg_start [L+1]         : my expert segments (multiples of 128); seg_start[L] = rows in use
//   seg_len [L]             : unpadded rows of each of my experts
//   tile_group [max_rows/128] : expert of every 128-row tile of my buffer, -1 past the end
// counts_table is the gathered [ep][E] table (device). If a buffer of max_rows rows (mine, or a
// destination's, all ranks use the same size) cannot hold its rows, the blocks that do not fit get
// count 0 and an error is recorded in the status words (the host raises on the next check).
int pico_ep_var_layout(const int32_t* counts_table, int ep, int L, int my_rank, int max_rows,
                       int32_t* send_blocks, int32_t* return_blocks, int32_t* seg_start, int32_t* seg_len,
                       int32_t* tile_group, cudaStream_t stream);

// Copy variable-size row blocks into peers' buffers: block b = blocks[b] = {count, src_row, dst_rank,
// dst_row}; row j of the block is read from src at row (row_index ? row_index[src_row + j] / index_div
// : src_row + j) and stored to dst.ptr[dst_rank] at row dst_row + j (rows of d bf16). With quant = 1
// the rows are quantised to FP8 E4M3 with one fp32 scale per 1 x 128 block while they are being sent:
// dst receives d bytes per row and `scales` d / 128 floats per row (d a multiple of 256). When the
// last CTA finishes, flag [slot][my_rank] = epoch is raised on every rank.
int pico_ep_var_exchange(const void* src, const int32_t* row_index, int index_div, const int32_t* blocks,
                         int num_blocks, PicoPeerTable dst, PicoPeerTable scales, PicoPeerTable flags, int ep,
                         int my_rank, int d, int quant, int slot, uint32_t epoch, cudaStream_t stream);

// Receiver side of a quantised exchange: payload / scales -> bf16 for rows [0, *rows_in_use) (a device
// integer, e.g. seg_start[L]); call after the senders' flags have been awaited.
int pico_ep_var_dequant(const void* payload, const float* scales, void* out, const int32_t* rows_in_use,
                        int max_rows, int d, cudaStream_t stream);

// dst[0 .. *rows_in_use) = src[0 .. *rows_in_use) for [max_rows, d] bf16 buffers (the fill level is a device
// integer): copies the used part of a receive buffer out of symmetric memory.
int pico_ep_var_copy_rows(const void* src, void* dst, const int32_t* rows_in_use, int max_rows, int d,
                          cudaStream_t stream);

// Zero the padding rows [seg_start[l] + seg_len[l], seg_start[l+1]) of a [rows, d] bf16 buffer, so
// that padded tiles contribute exact zeros to the grouped GEMMs.
int pico_ep_var_zero_padding(void* buf, const int32_t* seg_start, const int32_t* seg_len, int L, int d,
                             cudaStream_t stream);

#ifdef __cplusplus
}
#endif
