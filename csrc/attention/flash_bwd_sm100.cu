// Flash attention backward for sm_100a on tcgen05 tensor cores.
//
// One CTA owns a block of 128 keys of one (batch, kv head); K_j and V_j stay resident in shared
// memory and the dK_j / dV_j accumulators stay in tensor memory while the CTA walks every query
// block (and every query head of the group, for grouped-query attention) that can see those keys:
//
//   S  = Q_i K_j^T            dP = dO_i V_j^T                     (tensor cores -> TMEM)
//   P  = exp(S*scale - lse)   dS = P * (dP - delta) * scale       (one thread per query row)
//   dV_j += P^T dO_i          dK_j += dS^T Q_i                    (TMEM accumulators)
//   dQ_i += dS K_j            -> fp32 tile, TMA reduce-add into the global dQ accumulator
//
// P and dS are written once, as bf16, into swizzled shared memory and serve as the K-major A
// operand of the dQ GEMM and, read transposed through an MN-major descriptor, of the dV / dK
// GEMMs; Q_i and dO_i tiles are likewise read in both orientations, so nothing is transposed by
// copying. delta = rowsum(dO * O) comes from a small pre-pass; the dQ accumulator is converted to
// bf16 by a post-pass.
//
// Roles: warp 8 (one thread) issues all TMA loads and tcgen05.mma; warps 0-7 do the softmax
// arithmetic and all epilogues. Every wait is bounded.
#include <cuda_bf16.h>
#include <math_constants.h>

#include <cstring>

#include "../common/host.h"
#include "../common/ptx.cuh"
#include "attention.h"

namespace pico {

constexpr int kBM = 128;   // query rows per step
constexpr int kBN = 128;   // keys per CTA
constexpr int kBwdSoftmaxThreads = 256;   // two threads per query row, 64 key columns each
constexpr int kBwdThreads = kBwdSoftmaxThreads + 32;
constexpr float kBwdLog2e = 1.4426950408889634f;

template <int D>
struct BwdCfg {
  static constexpr int kTile = 128 * D * 2;                 // one bf16 [128, D] tile
  static constexpr int kStages = (D == 64) ? 2 : 1;         // Q_i / dO_i ring depth
  static constexpr int kPds = 2 * 128 * 128 * 2;            // P and dS tiles
  // fp32 dQ staging tile: its own buffer for head_dim 64 (so the reduce-add of one step can still
  // be reading it while the next step writes P/dS); aliases P/dS for head_dim 128 (no room)
  static constexpr int kStagingOwn = (D == 64) ? 128 * D * 4 : 0;
  static constexpr int kTiles = 2 * kTile + kStages * 2 * kTile + kPds + kStagingOwn;
  static constexpr int kNumBars = 1 + 2 * kStages + 4;      // kv, qdo_full/qdo_empty per stage, sdp_full, pds_ready, dq_full, s_free
  static constexpr int kSmemBytes = kTiles + kNumBars * 8 + 16 + 1024;
  static constexpr int kPanels = D / 64;
  // TMEM columns: [0,128) S then dQ, [128,256) dP, [256,256+D) dV, [256+D, 256+2D) dK
  static constexpr int kTmemCols = 512;
};

struct BwdMaps {
  CUtensorMap q, k, v, dout, dq_accum;
};

__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                                  float* __restrict__ delta, PicoAttnParams p, int64_t do_batch_stride,
                                  int64_t do_row_stride) {
  // head_dim / 8 adjacent lanes per (batch, row, head), 16 bytes of each operand per lane; the
  // heads of a row are contiguous, so a warp reads one 512-byte run of each tensor
  const int gsz = p.head_dim >> 3;            // 8 or 16 lanes per item
  const int per_warp = 32 / gsz;
  const int64_t total = (int64_t)p.batch * p.seq_q * p.heads;
  const int lane = threadIdx.x & 31;
  const int sub = lane / gsz, li = lane % gsz;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t w = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5; w * per_warp < total; w += warps) {
    const int64_t item = w * per_warp + sub;
    float acc = 0.f;
    int h = 0, row = 0, b = 0;
    if (item < total) {
      h = (int)(item % p.heads);
      const int64_t t = item / p.heads;
      row = (int)(t % p.seq_q);
      b = (int)(t / p.seq_q);
      const uint4 ov = *reinterpret_cast<const uint4*>(out + b * p.o_batch_stride + row * p.o_row_stride +
                                                      h * p.head_dim + li * 8);
      const uint4 dv = *reinterpret_cast<const uint4*>(dout + b * do_batch_stride + row * do_row_stride +
                                                      h * p.head_dim + li * 8);
      const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&ov);
      const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&dv);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = __bfloat1622float2(o2[i]);
        const float2 g = __bfloat1622float2(d2[i]);
        acc += a.x * g.x + a.y * g.y;
      }
    }
    for (int off = gsz >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (item < total && li == 0) delta[((int64_t)b * p.heads + h) * p.seq_q + row] = acc;
  }
}

__global__ void attn_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq,
                                       PicoAttnParams p, int64_t dq_batch_stride, int64_t dq_row_stride) {
  const int hd = p.heads * p.head_dim;
  const int64_t nvec = (int64_t)p.batch * p.seq_q * hd / 8;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e = i * 8;
    const int col = (int)(e % hd);
    const int64_t t = e / hd;
    const int row = (int)(t % p.seq_q);
    const int b = (int)(t / p.seq_q);
    const float4 a = reinterpret_cast<const float4*>(acc + e)[0];
    const float4 c = reinterpret_cast<const float4*>(acc + e)[1];
    uint4 o;
    o.x = pack_bf16x2(a.x, a.y);
    o.y = pack_bf16x2(a.z, a.w);
    o.z = pack_bf16x2(c.x, c.y);
    o.w = pack_bf16x2(c.z, c.w);
    *reinterpret_cast<uint4*>(dq + b * dq_batch_stride + row * dq_row_stride + col) = o;
  }
}

// uniform yes/no across the 256 softmax threads (they share named barriers afterwards)
__device__ __forceinline__ int all_agree_128(bool ok) {
  int all_ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "barrier.cta.red.and.pred q, 1, 256, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t"
      "}\n"
      : "=r"(all_ok)
      : "r"((int)ok)
      : "memory");
  return all_ok;
}

template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
flash_bwd_kernel(const __grid_constant__ BwdMaps maps, const float* __restrict__ lse,
                 const float* __restrict__ delta, __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv,
                 const PicoAttnParams p, int64_t dk_batch_stride, int64_t dk_row_stride,
                 int64_t dv_batch_stride, int64_t dv_row_stride, int* status) {
  using Cfg = BwdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + Cfg::kTile;
  uint8_t* sQ = sV + Cfg::kTile;                          // [stage]
  uint8_t* sdO = sQ + Cfg::kStages * Cfg::kTile;          // [stage]
  uint8_t* sP = sdO + Cfg::kStages * Cfg::kTile;
  uint8_t* sdS = sP + 128 * 128 * 2;
  uint8_t* staging = (D == 64) ? sdS + 128 * 128 * 2 : sP;  // fp32 dQ tile
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kTiles);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;
  uint64_t* qdo_empty = qdo_full + Cfg::kStages;
  uint64_t* sdp_full = qdo_empty + Cfg::kStages;
  uint64_t* pds_ready = sdp_full + 1;
  uint64_t* dq_full = pds_ready + 1;
  uint64_t* s_free = dq_full + 1;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(s_free + 1);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // blocks are dispatched x-fastest: under a causal mask key block 0 has the most query blocks to
  // walk, so every (head, batch) of the heavy key blocks starts before any light one
  const int kv_block = blockIdx.z;
  const int kv_head = blockIdx.x;
  const int batch = blockIdx.y;
  const int group = p.heads / p.kv_heads;
  const int k0 = kv_block * kBN;
  const int num_q_blocks = (p.seq_q + kBM - 1) / kBM;
  // first query block that can see any key of this block
  int i_min = 0;
  if (p.causal) {
    const int first_key_pos = p.k_pos0 + k0;
    const int need = first_key_pos - p.q_pos0 - (kBM - 1);   // q0 >= need
    i_min = need <= 0 ? 0 : (need + kBM - 1) / kBM;
  }
  const int nqb = max(0, num_q_blocks - i_min);
  const int total = nqb * group;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(pds_ready, kBwdSoftmaxThreads);
    mbar_init(dq_full, 1);
    mbar_init(s_free, kBwdSoftmaxThreads);
    *abort_word = 0;
    mbar_fence_init();
    tma_prefetch_desc(&maps.q);
    tma_prefetch_desc(&maps.k);
    tma_prefetch_desc(&maps.v);
    tma_prefetch_desc(&maps.dout);
    tma_prefetch_desc(&maps.dq_accum);
  }
  if (warp == 8) {
    tmem_alloc(tmem_ptr_smem, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const uint32_t tmem_s = tmem_base;              // S, later dQ
  const uint32_t tmem_dp = tmem_base + 128;
  const uint32_t tmem_dv = tmem_base + 256;
  const uint32_t tmem_dk = tmem_base + 256 + D;
  // head_dim 64 leaves room for a separate dQ accumulator, so S/dP of the next step can be issued
  // while the dQ tile of this step is still being drained; head_dim 128 reuses the S columns
  const uint32_t tmem_dq = (D == 64) ? tmem_base + 384 : tmem_s;

  if (warp == 8) {
    if (lane == 0 && total > 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);   // S, dP: both operands K-major
      constexpr uint32_t idesc_t = umma_idesc_bf16(128, D, 1, 1);     // dV, dK: both operands MN-major
      constexpr uint32_t idesc_q = umma_idesc_bf16(128, D, 0, 1);     // dQ: A K-major, B MN-major
      auto load_qdo = [&](int it) {
        const int st = it % Cfg::kStages;
        const int g = it / nqb;
        const int qrow0 = (i_min + it % nqb) * kBM;
        const int head = kv_head * group + g;
        mbar_arrive_expect_tx(&qdo_full[st], 2 * Cfg::kTile);
#pragma unroll
        for (int pn = 0; pn < Cfg::kPanels; ++pn) {
          tma_load_4d(sQ + st * Cfg::kTile + pn * 16384, &maps.q, &qdo_full[st], pn * 64, head, qrow0, batch);
          tma_load_4d(sdO + st * Cfg::kTile + pn * 16384, &maps.dout, &qdo_full[st], pn * 64, head, qrow0, batch);
        }
      };
      mbar_arrive_expect_tx(kv_full, 2 * Cfg::kTile);
#pragma unroll
      for (int pn = 0; pn < Cfg::kPanels; ++pn) {
        tma_load_4d(sK + pn * 16384, &maps.k, kv_full, pn * 64, kv_head, k0, batch);
        tma_load_4d(sV + pn * 16384, &maps.v, kv_full, pn * 64, kv_head, k0, batch);
      }
      load_qdo(0);
      if (Cfg::kStages > 1 && total > 1) load_qdo(1);
      bool ok = mbar_wait(kv_full, 0, abort_word, status, 2000);
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      const uint32_t p_addr = smem_u32(sP), ds_addr = smem_u32(sdS);
      // S = Q K^T and dP = dO V^T of step `it`
      auto issue_sdp = [&](int it) -> bool {
        const int st = it % Cfg::kStages;
        if (!mbar_wait(&qdo_full[st], (it / Cfg::kStages) & 1, abort_word, status, 2020)) return false;
        if (D != 64 && it >= 1 && !mbar_wait(s_free, (it - 1) & 1, abort_word, status, 2030)) return false;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQ + st * Cfg::kTile);
        const uint32_t do_addr = smem_u32(sdO + st * Cfg::kTile);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          tc_mma_f16_ss(tmem_s, umma_smem_desc(q_addr + off, 16, 1024), umma_smem_desc(k_addr + off, 16, 1024),
                        idesc_s, kk != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          tc_mma_f16_ss(tmem_dp, umma_smem_desc(do_addr + off, 16, 1024), umma_smem_desc(v_addr + off, 16, 1024),
                        idesc_s, kk != 0 ? 1u : 0u);
        }
        tc_commit(sdp_full);
        return true;
      };
      if (ok) ok = issue_sdp(0);
      for (int it = 0; it < total && ok; ++it) {
        const int st = it % Cfg::kStages;
        if (!mbar_wait(pds_ready, it & 1, abort_word, status, 2040)) break;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQ + st * Cfg::kTile);
        const uint32_t do_addr = smem_u32(sdO + st * Cfg::kTile);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {   // contraction over the 128 query rows, 16 per step
          tc_mma_f16_ss(tmem_dv, umma_smem_desc(p_addr + kk * 2048, 16384, 1024),
                        umma_smem_desc(do_addr + kk * 2048, 16384, 1024), idesc_t, (it | kk) != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          tc_mma_f16_ss(tmem_dk, umma_smem_desc(ds_addr + kk * 2048, 16384, 1024),
                        umma_smem_desc(q_addr + kk * 2048, 16384, 1024), idesc_t, (it | kk) != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {   // contraction over the 128 keys
          const uint32_t a_off = (kk >> 2) * 16384 + (kk & 3) * 32;
          tc_mma_f16_ss(tmem_dq, umma_smem_desc(ds_addr + a_off, 16, 1024),
                        umma_smem_desc(k_addr + kk * 2048, 16384, 1024), idesc_q, kk != 0 ? 1u : 0u);
        }
        tc_commit(&qdo_empty[st]);
        tc_commit(dq_full);
        if (Cfg::kStages > 1) {
          // next step's S/dP first (its operands are already resident), then refill this stage
          if (it + 1 < total && !issue_sdp(it + 1)) break;
          if (it + 2 < total) {
            if (!mbar_wait(&qdo_empty[st], (it / Cfg::kStages) & 1, abort_word, status, 2050)) break;
            load_qdo(it + 2);
          }
        } else if (it + 1 < total) {
          if (!mbar_wait(&qdo_empty[0], it & 1, abort_word, status, 2050)) break;
          load_qdo(it + 1);
          if (!issue_sdp(it + 1)) break;
        }
      }
    }
  } else {
    // warps w and w+4 share TMEM lane quarter w%4 (rows) and split the columns in halves
    const int half = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const int et = threadIdx.x;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const float scale_log2 = p.sm_scale * kBwdLog2e;
    bool alive = true;
    for (int it = 0; it < total; ++it) {
      const int g = it / nqb;
      const int q0 = (i_min + it % nqb) * kBM;
      const int head = kv_head * group + g;
      const int q_idx = q0 + row;
      const bool valid = q_idx < p.seq_q;
      const int q_pos = p.q_pos0 + q_idx;
      float lse_log2 = CUDART_INF_F, delta_r = 0.f;
      if (valid) {
        const int64_t off = ((int64_t)batch * p.heads + head) * p.seq_q + q_idx;
        const float l = lse[off];
        lse_log2 = (l == -CUDART_INF_F) ? CUDART_INF_F : l * kBwdLog2e;
        delta_r = delta[off];
      }
      // keys with index >= k_limit are invisible to this row (0 for rows that are out of range or
      // saw no key at all in the forward pass)
      int k_limit = p.seq_k;
      if (p.causal) k_limit = min(k_limit, q_pos - p.k_pos0 + 1);
      if (!valid || lse_log2 == CUDART_INF_F) k_limit = 0;
      if (!all_agree_128(mbar_wait(sdp_full, it & 1, abort_word, status, 2100))) {
        alive = false;
        break;
      }
      tc_fence_after();
      uint8_t* prow = sP + row * 128;
      uint8_t* dsrow = sdS + row * 128;
#pragma unroll 1
      for (int c = 2 * half; c < 2 * half + 2; ++c) {
        uint32_t sv[32], dpv[32];
        tmem_ld_32x32b_x32(tmem_s + lane_base + c * 32, sv);
        tmem_ld_32x32b_x32(tmem_dp + lane_base + c * 32, dpv);
        tmem_ld_wait();
        float pr[32], ds[32];
        // columns [0, lim) of this chunk are visible to this query row (branch-free masking)
        const int lim = k_limit - (k0 + c * 32);
        const float neg_lse = (lse_log2 == CUDART_INF_F) ? 0.f : -lse_log2;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float e = exp2f(fmaf(__uint_as_float(sv[i]), scale_log2, neg_lse));
          const float pv = i < lim ? e : 0.f;
          pr[i] = pv;
          ds[i] = pv * (__uint_as_float(dpv[i]) - delta_r) * p.sm_scale;
        }
        uint8_t* ppanel = prow + (c >> 1) * 16384;
        uint8_t* dpanel = dsrow + (c >> 1) * 16384;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int chunk = ((c & 1) * 4 + q4) ^ (row & 7);
          uint4 o;
          o.x = pack_bf16x2(pr[8 * q4 + 0], pr[8 * q4 + 1]);
          o.y = pack_bf16x2(pr[8 * q4 + 2], pr[8 * q4 + 3]);
          o.z = pack_bf16x2(pr[8 * q4 + 4], pr[8 * q4 + 5]);
          o.w = pack_bf16x2(pr[8 * q4 + 6], pr[8 * q4 + 7]);
          *reinterpret_cast<uint4*>(ppanel + (chunk << 4)) = o;
          o.x = pack_bf16x2(ds[8 * q4 + 0], ds[8 * q4 + 1]);
          o.y = pack_bf16x2(ds[8 * q4 + 2], ds[8 * q4 + 3]);
          o.z = pack_bf16x2(ds[8 * q4 + 4], ds[8 * q4 + 5]);
          o.w = pack_bf16x2(ds[8 * q4 + 6], ds[8 * q4 + 7]);
          *reinterpret_cast<uint4*>(dpanel + (chunk << 4)) = o;
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(pds_ready);
      // ---- dQ tile of this step: TMEM -> fp32 staging -> reduce-add into the global accumulator
      if (!all_agree_128(mbar_wait(dq_full, it & 1, abort_word, status, 2200))) {
        alive = false;
        break;
      }
      tc_fence_after();
      if (D == 64 && it > 0) {
        if (et == 0) tma_store_wait_read<0>();
        named_barrier_sync(2, kBwdSoftmaxThreads);
      }
#pragma unroll 1
      for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_dq + lane_base + c * 32, v);
        tmem_ld_wait();
        uint8_t* srow = staging + c * 16384 + row * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<uint4*>(srow + ((j ^ (row & 7)) << 4)) =
              make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
      }
      tc_fence_before();
      mbar_arrive(s_free);
      fence_proxy_async_smem();
      named_barrier_sync(2, kBwdSoftmaxThreads);
      if (et == 0) {
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c)
          tma_reduce_add_4d(&maps.dq_accum, staging + c * 16384, c * 32, head, q0, batch);
        tma_store_commit();
        // with a private staging buffer the read-out may overlap the next step's P/dS phase;
        // it only has to finish before the staging tile is written again
        if (D != 64) tma_store_wait_read<0>();
      }
      if (D != 64) named_barrier_sync(2, kBwdSoftmaxThreads);
    }
    // ---- dK / dV of this key block
    if (alive) {
      const int kidx = k0 + row;
      const bool valid_key = kidx < p.seq_k;
      __nv_bfloat16* dk_row = dk + (int64_t)batch * dk_batch_stride + (int64_t)kidx * dk_row_stride + kv_head * D;
      __nv_bfloat16* dv_row = dv + (int64_t)batch * dv_batch_stride + (int64_t)kidx * dv_row_stride + kv_head * D;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const uint32_t src = which == 0 ? tmem_dv : tmem_dk;
        __nv_bfloat16* dst = which == 0 ? dv_row : dk_row;
#pragma unroll 1
        for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
          uint32_t v[32];
          if (total > 0) {
            tmem_ld_32x32b_x32(src + lane_base + c * 32, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0u;
          }
          if (valid_key) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(v[8 * q4 + 0]), __uint_as_float(v[8 * q4 + 1]));
              o.y = pack_bf16x2(__uint_as_float(v[8 * q4 + 2]), __uint_as_float(v[8 * q4 + 3]));
              o.z = pack_bf16x2(__uint_as_float(v[8 * q4 + 4]), __uint_as_float(v[8 * q4 + 5]));
              o.w = pack_bf16x2(__uint_as_float(v[8 * q4 + 6]), __uint_as_float(v[8 * q4 + 7]));
              *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = o;
            }
          }
        }
      }
    }
    if (et == 0) tma_store_wait<0>();
  }

  if (*abort_word) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int D>
static int launch_bwd(const void* q, const void* k, const void* v, const void* dout, const float* lse,
                      void* dk, void* dv, const float* delta, float* dq_accum, const PicoAttnParams* p,
                      int64_t do_batch_stride, int64_t do_row_stride, int64_t dk_batch_stride,
                      int64_t dk_row_stride, int64_t dv_batch_stride, int64_t dv_row_stride,
                      cudaStream_t stream) {
  using Cfg = BwdCfg<D>;
  BwdMaps maps;
  const CUtensorMapDataType bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  int rc = pico_host::make_tmap_bshd(&maps.q, q, bf, 2, D, p->heads, p->seq_q, p->batch, p->q_row_stride * 2,
                                     p->q_batch_stride * 2, 64, kBM);
  if (rc) return rc;
  rc = pico_host::make_tmap_bshd(&maps.k, k, bf, 2, D, p->kv_heads, p->seq_k, p->batch, p->k_row_stride * 2,
                                 p->k_batch_stride * 2, 64, kBN);
  if (rc) return rc;
  rc = pico_host::make_tmap_bshd(&maps.v, v, bf, 2, D, p->kv_heads, p->seq_k, p->batch, p->v_row_stride * 2,
                                 p->v_batch_stride * 2, 64, kBN);
  if (rc) return rc;
  rc = pico_host::make_tmap_bshd(&maps.dout, dout, bf, 2, D, p->heads, p->seq_q, p->batch, do_row_stride * 2,
                                 do_batch_stride * 2, 64, kBM);
  if (rc) return rc;
  const uint64_t acc_row = (uint64_t)p->heads * D * 4;
  rc = pico_host::make_tmap_bshd(&maps.dq_accum, dq_accum, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, D, p->heads,
                                 p->seq_q, p->batch, acc_row, acc_row * p->seq_q, 32, kBM);
  if (rc) return rc;
  auto kern = flash_bwd_kernel<D>;
  static int attr_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (attr_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) {
      pico_host::set_error("attention bwd: cudaFuncSetAttribute(%d): %s", Cfg::kSmemBytes, cudaGetErrorString(e));
      return (int)e;
    }
    attr_dev = dev;
  }
  dim3 grid(p->kv_heads, p->batch, (p->seq_k + kBN - 1) / kBN);
  kern<<<grid, kBwdThreads, Cfg::kSmemBytes, stream>>>(maps, lse, delta, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv,
                                                      *p, dk_batch_stride, dk_row_stride, dv_batch_stride,
                                                      dv_row_stride, pico_status_buffer());
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    pico_host::set_error("attention bwd launch: %s", cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

}  // namespace pico

extern "C" int pico_attention_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                  const float* lse, void* dq, void* dk, void* dv, float* delta, float* dq_accum,
                                  const PicoAttnParams* p, int64_t do_batch_stride, int64_t do_row_stride,
                                  int64_t dq_batch_stride, int64_t dq_row_stride, int64_t dk_batch_stride,
                                  int64_t dk_row_stride, int64_t dv_batch_stride, int64_t dv_row_stride,
                                  cudaStream_t stream) {
  using namespace pico;
  if (p->batch <= 0 || p->seq_q <= 0 || p->seq_k <= 0 || p->heads <= 0) return 0;
  if (p->head_dim != 64 && p->head_dim != 128) {
    pico_host::set_error("attention: head_dim %d not supported (64 or 128)", p->head_dim);
    return -2;
  }
  if (p->heads % p->kv_heads != 0) {
    pico_host::set_error("attention: heads (%d) must be a multiple of kv_heads (%d)", p->heads, p->kv_heads);
    return -2;
  }
  const int64_t rows = (int64_t)p->batch * p->seq_q * p->heads;
  const int sms = pico_host::num_sms();
  {
    int64_t blocks = (rows * (p->head_dim / 8) + 255) / 256;
    if (blocks > sms * 16) blocks = sms * 16;
    attn_delta_kernel<<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)out, (const __nv_bfloat16*)dout, delta,
                                                      *p, do_batch_stride, do_row_stride);
  }
  cudaError_t e = cudaMemsetAsync(dq_accum, 0, sizeof(float) * rows * p->head_dim, stream);
  if (e != cudaSuccess) {
    pico_host::set_error("attention bwd: memset: %s", cudaGetErrorString(e));
    return (int)e;
  }
  int rc;
  if (p->head_dim == 64)
    rc = launch_bwd<64>(q, k, v, dout, lse, dk, dv, delta, dq_accum, p, do_batch_stride, do_row_stride,
                        dk_batch_stride, dk_row_stride, dv_batch_stride, dv_row_stride, stream);
  else
    rc = launch_bwd<128>(q, k, v, dout, lse, dk, dv, delta, dq_accum, p, do_batch_stride, do_row_stride,
                         dk_batch_stride, dk_row_stride, dv_batch_stride, dv_row_stride, stream);
  if (rc) return rc;
  {
    int64_t nvec = rows * p->head_dim / 8;
    int64_t blocks = (nvec + 255) / 256;
    if (blocks > sms * 16) blocks = sms * 16;
    attn_dq_convert_kernel<<<(int)blocks, 256, 0, stream>>>(dq_accum, (__nv_bfloat16*)dq, *p, dq_batch_stride,
                                                           dq_row_stride);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    pico_host::set_error("attention bwd: %s", cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}
