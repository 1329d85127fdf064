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

#ifdef __cplusplus
}
#endif
