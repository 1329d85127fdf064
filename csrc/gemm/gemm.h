// C entry points of the tensor-core GEMM family. All pointers are device pointers; every
// function returns 0 on success and leaves a message in pico_last_error() otherwise.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// D[M,N] (=|+=) op(A) * op(B), bf16 inputs, fp32 accumulate.
//   a_mn_major: 0 -> A is [M,K] row-major (lda >= K); 1 -> A is [K,M] row-major (lda >= M)
//   b_mn_major: 0 -> B is [N,K] row-major (ldb >= K); 1 -> B is [K,N] row-major (ldb >= N)
//   out_mode  : 0 -> D bf16, 1 -> D fp32, 2 -> D fp32 accumulated in place (D += ...)
//   max_ctas  : cap on the persistent grid (0 = one CTA per SM); lets a caller leave SMs
//               free for a kernel running beside the GEMM on another stream
int pico_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, int lda, int ldb,
                   int ldd, int a_mn_major, int b_mn_major, int out_mode, int max_ctas,
                   cudaStream_t stream);

// Collective fusion (see csrc/runtime/symm.h for the symmetric-memory model).
//   Row geometry: the M rows are pieces of blk_rows rows (a multiple of 128); piece p belongs to
//   block p % num_blocks and is that block's (p / num_blocks)-th piece. One piece per block is the
//   plain split "rank r owns rows [r*M/n, (r+1)*M/n)"; several pieces per block describe a
//   [batch, sequence] tensor whose sequence dimension is split over the ranks (blk_rows = sequence
//   length per rank), which is how the sequence-parallel layers use it.
//   all-gather -> GEMM : A (K-major) is this GPU's gather buffer; block b was written by rank b and
//     is announced by flag [a_slot][b] >= a_epoch in a_flags (local flag buffer). The kernel visits
//     block first_block first (this rank's own rows, a_skip_block: never waited for) and loads the
//     other blocks as their flags arrive, so the transfer overlaps the math tile by tile.
//   GEMM -> reduce-scatter : the rows of block b are stored through d_ptrs[b] — the slot reserved
//     for this rank in rank b's staging buffer ([M / num_blocks, N], pieces in order) — instead of
//     D; the owner sums the slots afterwards (pico_slot_sum).
typedef struct {
  const unsigned int* a_flags;
  int a_slot;
  unsigned int a_epoch;
  int a_skip_block;
  int d_num_dest;
  void* d_ptrs[8];
  int blk_rows;
  int num_blocks;
  int first_block;
  unsigned int timeout_ms;
  // Grouped GEMM for the experts of a mixture-of-experts layer: one launch covers every local
  // expert. Rows of the activation matrices are expert-contiguous and every expert's segment
  // starts on a multiple of 128 rows (padding rows are zero), so a 128-row tile never mixes experts.
  //   row-grouped (forward / input gradient): tile_group[t] is the expert of row tile t (a device
  //     array of ceil(M/128) ints, -1 = tile not computed); B holds num_groups matrices of
  //     b_group_rows rows stacked along its rows ([G*N, K] for b_mn_major 0, [G*K, N] for 1).
  //   reduction-grouped (weight gradient): D holds num_groups [M, N] blocks stacked along its rows;
  //     block g = A[:, rows_g]^T-style product reduced over rows seg_start[g] .. seg_start[g+1]
  //     (device array of num_groups + 1 ints, multiples of 64) of the MN-major operands. K is the
  //     total number of rows. Blocks of empty groups are left untouched.
  const int* tile_group;
  int b_group_rows;
  const int* seg_start;
  int num_groups;
} PicoGemmComm;

int pico_gemm_bf16_ex(const void* A, const void* B, void* D, int M, int N, int K, int lda, int ldb,
                      int ldd, int a_mn_major, int b_mn_major, int out_mode, int max_ctas,
                      const PicoGemmComm* comm, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
