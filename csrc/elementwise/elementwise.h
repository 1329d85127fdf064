// C entry points of the memory-bound kernels (normalisation, rotary embedding, SwiGLU,
// cross-entropy, AdamW, embedding, fp8 block quantisation). Device pointers throughout;
// 0 on success, message in pico_last_error() otherwise. bf16 tensors are passed as void*.
#pragma once
#include <cuda_runtime.h>

#include "../runtime/symm.h"
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- RMSNorm ---------------------------------------------------------------------------
// h = x (+ residual); y = h * rsqrt(mean(h^2)+eps) * w.  h_out (optional) receives h when a
// residual is given. rstd (optional) receives the per-row statistic for the backward.
int pico_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* h_out,
                     float* rstd, int rows, int H, float eps, cudaStream_t stream);
// Rows of fp32 scratch (each H wide) that pico_rmsnorm_bwd needs in dw_partial.
int pico_rmsnorm_bwd_num_partials(void);
// dh = d(norm)/dh (+ dres);  dw (fp32 and/or bf16, = or +=) = sum_rows dy*h*rstd.
int pico_rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd,
                     const void* dres, void* dh, float* dw_partial, float* dw_f32, void* dw_bf16,
                     int accumulate, int rows, int H, cudaStream_t stream);

// ---- RoPE (half-split, in place) ---------------------------------------------------------
// x: rows x (nheads*d) with `row_stride` elements between rows; position of row r is
// pos_offset + (r % seq). cos/sin: fp32 [max_pos, d/2]. sign=+1 forward, -1 backward.
int pico_rope_inplace(void* x, int64_t row_stride, int rows, int seq, int pos_offset, int nheads,
                      int d, const float* cos, const float* sin, int sign, cudaStream_t stream);

// ---- SwiGLU ------------------------------------------------------------------------------
// gu: [rows, 2*I] (gate | up, row stride ld_gu); y[rows, I] = silu(gate) * up.
// rows_dev (optional, device): when given, only min(rows, *rows_dev) rows are processed - for buffers
// whose row count is known only on the device; the remaining rows of the output are left untouched.
int pico_swiglu_fwd(const void* gu, int64_t ld_gu, void* y, int rows, int I, const int* rows_dev,
                    cudaStream_t stream);
// dgu[rows, 2*I] from dy[rows, I] and the saved gu
int pico_swiglu_bwd(const void* dy, const void* gu, int64_t ld_gu, void* dgu, int64_t ld_dgu,
                    int rows, int I, const int* rows_dev, cudaStream_t stream);

// ---- cross entropy on a vocabulary shard ---------------------------------------------------
// stats[row] = {max_j l[row,j], sum_j exp(l - max), l[row,target] or 0 if target is not in
// [vocab_start, vocab_start+V)}. logits bf16 [rows, V] with row stride ldl.
int pico_ce_stats(const void* logits, int64_t ldl, const int64_t* targets, float* stats, int rows,
                  int V, int vocab_start, cudaStream_t stream);
// Given the (already reduced over shards) stats: loss[row] = log(sum) + max - target_logit and,
// when dlogits != NULL, dlogits = (softmax - onehot) * grad_scale (may alias logits).
int pico_ce_loss_grad(const void* logits, int64_t ldl, const int64_t* targets, const float* stats,
                      float* loss, void* dlogits, int64_t ldd, float grad_scale, int rows, int V,
                      int vocab_start, cudaStream_t stream);

// Vocabulary-parallel form without a collective call: every rank writes the triples of its shard
// into block my_rank of the [world][rows][3] fp32 table of all ranks (`dst`, symmetric memory) and
// raises flag [slot][my_rank] = epoch; pico_ce_loss_grad_gathered waits (bounded) for all world
// flags, merges the world triples of each row in rank order (max, rescaled sum, sum) and proceeds
// like pico_ce_loss_grad.
int pico_ce_stats_push(const void* logits, int64_t ldl, const int64_t* targets, int rows, int V,
                       int vocab_start, PicoPeerTable dst, PicoPeerTable flags, int world, int my_rank,
                       int slot, uint32_t epoch, cudaStream_t stream);
int pico_ce_loss_grad_gathered(const void* logits, int64_t ldl, const int64_t* targets,
                               const float* gathered_stats, float* loss, void* dlogits, int64_t ldd,
                               float grad_scale, int rows, int V, int vocab_start,
                               const uint32_t* local_flags, int world, int slot, uint32_t epoch,
                               uint32_t timeout_ms, cudaStream_t stream);

// ---- AdamW over flat buffers ----------------------------------------------------------------
// p (bf16) / master (fp32, optional) / g (fp32) / m, v (fp32), n elements. Decoupled weight
// decay as torch.optim.AdamW. g is multiplied by grad_scale first and zeroed afterwards when
// zero_grad != 0.
int pico_adamw(void* p_bf16, float* master, float* g, float* m, float* v, int64_t n, float lr,
               float beta1, float beta2, float eps, float weight_decay, float bias_corr1,
               float bias_corr2, float grad_scale, int zero_grad, cudaStream_t stream);

// ---- embedding -------------------------------------------------------------------------------
// out[row] = W[ids[row]-vocab_start] or 0 when the id is outside this vocabulary shard.
int pico_embedding_fwd(const void* W, const int64_t* ids, void* out, int rows, int H, int Vlocal,
                       int vocab_start, cudaStream_t stream);
// dW[ids[row]-vocab_start] += dout[row] (fp32 accumulation)
int pico_embedding_bwd(const void* dout, const int64_t* ids, float* dW, int rows, int H, int Vlocal,
                       int vocab_start, cudaStream_t stream);

// ---- mixture-of-experts routing (moe_route.cu) -----------------------------------------------
// Router: logits bf16 [T, E] (row stride ldl, E <= 256) -> probs fp32 [T, E] (softmax), the k experts
// with the largest probs (+ bias[e] when bias != NULL; ties to the lower index) in idx int32 [T, k],
// their un-biased probabilities in w fp32 [T, k] (divided by their sum when renorm != 0 and k > 1),
// and counts[e] += rows routed to e (int32 [E], zeroed by the caller). k <= 8.
int pico_moe_route(const void* logits, int64_t ldl, const float* bias, float* probs, int32_t* idx, float* w,
                   int32_t* counts, int T, int E, int k, int renorm, cudaStream_t stream);
// dlogits fp32 [T, E] from dw fp32 [T, k] and, optionally, a dense gradient dprobs fp32 [T, E].
int pico_moe_route_bwd(const float* probs, const int32_t* idx, const float* w, const float* dw,
                       const float* dprobs, float* dlogits, int T, int E, int k, int renorm, cudaStream_t stream);
// pos[r] = number of earlier routed rows with the same expert (idx int32 [R], row order); when
// row_of_slot != NULL (int32 [E * C], -1 on entry) row_of_slot[e * C + pos] = r for pos < C.
int pico_moe_slots(const int32_t* idx, int R, int E, int C, int32_t* pos, int32_t* row_of_slot,
                   cudaStream_t stream);
// y[t] = sum_j [pos[t,j] < C] w[t,j] * out[idx[t,j] * C + pos[t,j]] (out bf16 [E*C, d], y bf16 [T, d]).
int pico_moe_combine(const void* out, const int32_t* idx, const int32_t* pos, const float* w, void* y, int T,
                     int k, int C, int d, cudaStream_t stream);
// dout[s] = w[row] * dy[row / k] and dw[row] = <dy[row / k], out[s]> with row = row_of_slot[s]
// (dout[s] = 0 for empty slots; dw fp32 [T*k] zeroed by the caller).
int pico_moe_combine_bwd(const void* dy, const void* out, const int32_t* row_of_slot, const float* w, void* dout,
                         float* dw, int64_t slots, int k, int d, cudaStream_t stream);

// ---- merge of two partial attention results (disjoint key sets) ------------------------------
// out = out_a * exp(lse_a - lse) + out_b * exp(lse_b - lse), lse = log(exp(lse_a) + exp(lse_b)).
// out_a fp32 (a_is_f32) or bf16, out_b bf16, all [B, S, H, D] contiguous; out fp32 (may be out_a);
// lse tensors fp32 [B, H, S] (lse may be lse_a).
int pico_attn_merge(const void* out_a, int a_is_f32, const float* lse_a, const void* out_b, const float* lse_b,
                    float* out, float* lse, int B, int S, int H, int D, cudaStream_t stream);

// ---- misc ---------------------------------------------------------------------------------
// dst_f32 += src_bf16 (n elements); used to fold bf16 gradients into fp32 accumulators.
int pico_accumulate_bf16_into_f32(const void* src, float* dst, int64_t n, cudaStream_t stream);
// x (bf16, n elements, contiguous) *= *scale_dev, skipped entirely when the device scalar is 1
int pico_scale_unless_one(void* x_bf16, int64_t n, const float* scale_dev, cudaStream_t stream);
// writes a buffer larger than L2 (cache flush between timed iterations)
int pico_fill_u32(void* dst, uint32_t value, int64_t n_words, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
