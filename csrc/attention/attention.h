// Flash attention (forward and backward) on tcgen05 tensor cores for sm_100a.
//
// Tensors use the [batch, seq, heads, head_dim] layout with arbitrary batch / sequence strides
// (so q, k and v can be column slices of one fused projection output); head_dim is contiguous and
// heads are head_dim apart. Grouped-query attention is native: query head h reads KV head
// h / (heads / kv_heads). bf16 in, fp32 softmax statistics and accumulation.
//
// Causal masking is expressed with global positions: a query at position q_pos0 + i attends keys
// at positions <= its own, keys starting at k_pos0. Whole-sequence attention uses 0 / 0; a
// ring-attention step passes the offsets of the blocks it holds.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
  int batch, seq_q, seq_k, heads, kv_heads, head_dim;
  // strides in elements
  int64_t q_batch_stride, q_row_stride;
  int64_t k_batch_stride, k_row_stride;
  int64_t v_batch_stride, v_row_stride;
  int64_t o_batch_stride, o_row_stride;
  float sm_scale;
  int causal;
  int q_pos0, k_pos0;
  // optional: device buffer of 1024 uint64; CTA (0,0,0) of the forward kernel records globaltimer
  // stamps of its pipeline phases there (performance debugging). NULL = off.
  unsigned long long* trace;
} PicoAttnParams;

// out[b, sq, H, d] (bf16) and lse[b, H, sq] (fp32, natural log; -inf for rows without keys).
int pico_attention_fwd(const void* q, const void* k, const void* v, void* out, float* lse,
                       const PicoAttnParams* p, cudaStream_t stream);

// Gradients. `delta` is scratch [b, H, sq] fp32, `dq_accum` scratch [b, sq, H, d] fp32 (zeroed by
// the call). dq/dk/dv use the strides of q/k/v in `p` when dq_row_stride etc. are 0.
int pico_attention_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout,
                       const float* lse, void* dq, void* dk, void* dv, float* delta, float* dq_accum,
                       const PicoAttnParams* p, int64_t do_batch_stride, int64_t do_row_stride,
                       int64_t dq_batch_stride, int64_t dq_row_stride, int64_t dk_batch_stride,
                       int64_t dk_row_stride, int64_t dv_batch_stride, int64_t dv_row_stride,
                       cudaStream_t stream);

#ifdef __cplusplus
}
#endif
