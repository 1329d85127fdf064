// ZeRO-1 optimizer step fused with its collectives: gradient reduce-scatter, AdamW on this rank's
// shard, and the parameter all-gather happen in one kernel through NVLink peer memory.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../runtime/symm.h"

#ifdef __cplusplus
extern "C" {
#endif

// Every rank holds a flat fp32 gradient buffer and a flat bf16 parameter buffer of the same
// layout in symmetric memory (`grads`, `params`: base pointer per rank). This rank owns elements
// [shard_start, shard_start + shard_len) and keeps their AdamW state (m, v, optional fp32 master
// copy) locally. The kernel
//   1. waits (bounded) until flag [ready_slot][r] >= epoch for every rank r (its backward is done),
//   2. for each owned element sums the gradients of all ranks in rank order (peer loads, fp32,
//      deterministic), scales by grad_scale, applies AdamW,
//   3. stores the updated bf16 value into the parameter buffer of every rank (peer stores).
// The caller then raises / waits on a "done" flag before it clears its gradient buffer and starts
// the next forward pass. shard_start and shard_len must be multiples of 8.
int pico_zero1_adamw(PicoPeerTable grads, PicoPeerTable params, float* m, float* v, float* master,
                     int64_t shard_start, int64_t shard_len, int world, int my_rank, float lr, float beta1,
                     float beta2, float eps, float weight_decay, float bias_corr1, float bias_corr2,
                     float grad_scale, const uint32_t* local_flags, int ready_slot, uint32_t epoch,
                     uint32_t timeout_ms, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
