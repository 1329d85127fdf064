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
//   all-gather -> GEMM : A (K-major) is this GPU's gather buffer; row block b (a_rows_per_block
//     rows) is written by rank b and announced by flag [a_slot][b] >= a_epoch in a_flags (local
//     flag buffer). The kernel starts on block a_skip_block (this rank's own rows) and loads the
//     other blocks as their flags arrive, so the transfer overlaps the math tile by tile.
//   GEMM -> reduce-scatter : output row block b (d_rows_per_block rows) is stored through
//     d_ptrs[b] — the slot reserved for this rank in rank b's staging buffer — instead of D;
//     the owner sums the slots afterwards (pico_slot_sum / pico_slot_sum_add_rmsnorm).
//   m_rotate_rows shifts the order in which row blocks are visited.
typedef struct {
  const unsigned int* a_flags;
  int a_slot;
  unsigned int a_epoch;
  int a_rows_per_block;
  int a_skip_block;
  int d_num_dest;
  int d_rows_per_block;
  void* d_ptrs[8];
  int m_rotate_rows;
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
