// Flash attention forward for sm_100a: S = Q K^T and O += P V run on tcgen05 tensor cores with
// the accumulators in tensor memory; Q, K and V tiles arrive by TMA (128-byte swizzle); the
// online softmax runs in registers, one thread per query row.
//
// One CTA handles 128 query rows of one (batch, head) and walks the key/value sequence in blocks
// of 128:
//   warp 8 (one thread)  : TMA loads of Q once and of K/V blocks into a 2-stage ring, and all
//                          tcgen05.mma issue: S(j) = Q K_j^T, then O += P_j V_j once P_j is ready
//   warps 0-7 (256 thr.) : tcgen05.ld the S row, scale, mask, online-softmax update, write P_j as
//                          bf16 into swizzled shared memory (the A operand of the second GEMM),
//                          rescale the O accumulator in TMEM when the running maximum moved,
//                          final normalisation and store of O and the log-sum-exp
// Two CTAs fit on an SM for head_dim 64 (each allocates 256 TMEM columns), so one CTA's softmax
// overlaps the other's tensor-core work without intra-CTA software pipelining.
//
// Every wait is bounded (see common/ptx.cuh); a CTA that gives up frees its TMEM and returns.
#include <cuda_bf16.h>
#include <math_constants.h>

#include <cstdlib>
#include <cstring>

#include "../common/host.h"
#include "../common/ptx.cuh"
#include "attention.h"

namespace pico {

constexpr int kBlockM = 128;
constexpr int kBlockN = 128;
constexpr int kSoftmaxThreads = 256;   // two threads per query row, 64 key columns each
constexpr int kFwdThreads = kSoftmaxThreads + 32;
constexpr float kLog2e = 1.4426950408889634f;
// only rescale the accumulator when the running max grew by more than this (log2 units);
// smaller drifts are absorbed by the fp32 range of the un-normalised probabilities
constexpr float kRescaleThreshold = 8.0f;

template <int D>
struct FwdCfg {
  static constexpr int kQBytes = kBlockM * D * 2;
  static constexpr int kKVBytes = kBlockN * D * 2;       // one K or V tile
  static constexpr int kPBytes = kBlockM * kBlockN * 2;  // P tile, bf16
  static constexpr int kStages = 2;
  static constexpr int kTiles = kQBytes + 2 * kStages * kKVBytes + kPBytes;
  static constexpr int kNumBars = 1 + 3 * kStages + 3;   // q, k_full/v_full/kv_empty per stage, s_full, p_ready, pv_done
  // no alignment slack: the kernel has no static shared memory, so the dynamic window starts on a
  // 1024-byte boundary (checked at run time); this keeps two CTAs per SM for head_dim 64
  static constexpr int kSmemBytes = kTiles + 256;
  static constexpr int kTmemCols = 256;                  // S: 128 columns, O: D (<= 128) columns
  static constexpr int kPanels = D / 64;                 // 64-element (128-byte) column panels of Q/K/V
};

struct FwdMaps {
  CUtensorMap q, k, v;
};

template <int D>
__global__ void __launch_bounds__(kFwdThreads, (D == 64) ? 2 : 1)
flash_fwd_kernel(const __grid_constant__ FwdMaps maps, __nv_bfloat16* __restrict__ out,
                 float* __restrict__ lse, const PicoAttnParams p, int* status) {
  using Cfg = FwdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if ((smem_u32(smem) & 1023u) != 0) {   // swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) report_error(status, PICO_ERR_BOUNDS, 1999, (int)(smem_u32(smem) & 1023u));
    return;
  }
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Cfg::kQBytes;                       // [stage]
  uint8_t* sV = sK + Cfg::kStages * Cfg::kKVBytes;       // [stage]
  uint8_t* sP = sV + Cfg::kStages * Cfg::kKVBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kTiles);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* v_full = k_full + Cfg::kStages;
  uint64_t* kv_empty = v_full + Cfg::kStages;
  uint64_t* s_full = kv_empty + Cfg::kStages;
  uint64_t* p_ready = s_full + 1;
  uint64_t* pv_done = p_ready + 1;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(pv_done + 1);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // heavy (late) query tiles first so the causal triangle balances across the grid
  const int num_q_tiles = (p.seq_q + kBlockM - 1) / kBlockM;
  const int q_tile = num_q_tiles - 1 - (int)blockIdx.x;
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int kv_head = head / (p.heads / p.kv_heads);
  const int q0 = q_tile * kBlockM;

  // key blocks this tile needs: all of them, or (causal) those that start at or before the last
  // query position of the tile
  int num_kv = (p.seq_k + kBlockN - 1) / kBlockN;
  if (p.causal) {
    const int last_q_pos = p.q_pos0 + min(q0 + kBlockM, p.seq_q) - 1;
    const int visible = last_q_pos - p.k_pos0 + 1;       // keys [0, visible) may be attended
    num_kv = visible <= 0 ? 0 : min(num_kv, (visible + kBlockN - 1) / kBlockN);
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_ready, kSoftmaxThreads);
    mbar_init(pv_done, 1);
    *abort_word = 0;
    mbar_fence_init();
    tma_prefetch_desc(&maps.q);
    tma_prefetch_desc(&maps.k);
    tma_prefetch_desc(&maps.v);
  }
  if (warp == 8) {
    tmem_alloc(tmem_ptr_smem, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const uint32_t tmem_s = tmem_base;          // columns [0, 128)
  const uint32_t tmem_o = tmem_base + 128;    // columns [128, 128 + D)
  const bool tracing = p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
  int trace_n = 0;
#define PICO_STAMP(base)                                                             \
  do {                                                                               \
    if (tracing && trace_n < 250) p.trace[(base) + trace_n++] = global_timer_ns();   \
  } while (0)

  if (warp == 8) {
    // ------------------------------------------------------------ TMA + MMA issue (one thread)
    if (lane == 0 && num_kv > 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(kBlockM, kBlockN, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc_bf16(kBlockM, D, 0, 1);
      auto load_kv = [&](int j) {
        const int s = j & 1;
        uint8_t* k_dst = sK + s * Cfg::kKVBytes;
        uint8_t* v_dst = sV + s * Cfg::kKVBytes;
        mbar_arrive_expect_tx(&k_full[s], Cfg::kKVBytes);
#pragma unroll
        for (int pn = 0; pn < Cfg::kPanels; ++pn)
          tma_load_4d(k_dst + pn * 16384, &maps.k, &k_full[s], pn * 64, kv_head, j * kBlockN, batch);
        mbar_arrive_expect_tx(&v_full[s], Cfg::kKVBytes);
#pragma unroll
        for (int pn = 0; pn < Cfg::kPanels; ++pn)
          tma_load_4d(v_dst + pn * 16384, &maps.v, &v_full[s], pn * 64, kv_head, j * kBlockN, batch);
      };
      mbar_arrive_expect_tx(q_full, Cfg::kQBytes);
#pragma unroll
      for (int pn = 0; pn < Cfg::kPanels; ++pn)
        tma_load_4d(sQ + pn * 16384, &maps.q, q_full, pn * 64, head, q0, batch);
      load_kv(0);
      bool ok = mbar_wait(q_full, 0, abort_word, status, 1000);
      for (int j = 0; j < num_kv && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        PICO_STAMP(0);
        if (!mbar_wait(&k_full[s], ph, abort_word, status, 1020)) break;
        PICO_STAMP(0);
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQ);
        const uint32_t k_addr = smem_u32(sK + s * Cfg::kKVBytes);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          tc_mma_f16_ss(tmem_s, umma_smem_desc(q_addr + off, 16, 1024),
                        umma_smem_desc(k_addr + off, 16, 1024), idesc_s, kk != 0 ? 1u : 0u);
        }
        tc_commit(s_full);
        // prefetch the next K/V block while the softmax of this one runs; its stage was last read by
        // the P V product of block j-1, which has had the whole S(j) issue to finish
        if (j + 1 < num_kv) {
          if (j + 1 >= 2 &&
              !mbar_wait(&kv_empty[(j + 1) & 1], (((j + 1) >> 1) - 1) & 1, abort_word, status, 1010)) {
            ok = false;
            break;
          }
          load_kv(j + 1);
        }
        PICO_STAMP(0);
        if (!mbar_wait(p_ready, j & 1, abort_word, status, 1030)) break;
        PICO_STAMP(0);
        if (!mbar_wait(&v_full[s], ph, abort_word, status, 1040)) break;
        tc_fence_after();
        const uint32_t p_addr = smem_u32(sP);
        const uint32_t v_addr = smem_u32(sV + s * Cfg::kKVBytes);
#pragma unroll
        for (int kk = 0; kk < kBlockN / 16; ++kk) {
          const uint32_t a_off = (kk >> 2) * 16384 + (kk & 3) * 32;
          tc_mma_f16_ss(tmem_o, umma_smem_desc(p_addr + a_off, 16, 1024),
                        umma_smem_desc(v_addr + kk * 2048, 16384, 1024), idesc_o,
                        (j | kk) != 0 ? 1u : 0u);
        }
        tc_commit(&kv_empty[s]);
        tc_commit(pv_done);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax + epilogue (256 threads)
    // warps w and w+4 share TMEM lane quarter w%4 (rows) and split the 128 key columns in halves
    const int half = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    float* xchg = reinterpret_cast<float*>(sP);   // [2][128] floats, valid while no P tile is live
    const bool valid_row = (q0 + row) < p.seq_q;
    const int q_pos = p.q_pos0 + q0 + row;
    const float scale_log2 = p.sm_scale * kLog2e;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    float m_run = -CUDART_INF_F;   // running max of the scaled scores (log2 units)
    float l_run = 0.f;
    bool alive = true;
    for (int j = 0; j < num_kv; ++j) {
      if (threadIdx.x == 0) PICO_STAMP(512);
      const bool ok = mbar_wait(s_full, j & 1, abort_word, status, 1100);
      if (threadIdx.x == 0) PICO_STAMP(512);
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
      if (!all_ok) {
        alive = false;
        break;
      }
      tc_fence_after();
      const int k_base = j * kBlockN;
      const bool need_mask = (p.causal && (p.k_pos0 + k_base + kBlockN - 1 > p.q_pos0 + q0)) ||
                             (k_base + kBlockN > p.seq_k);
      // S values of this thread's 64 columns are read from TMEM once and stay in registers for
      // both the maximum and the exponentials (branch-free inner loops: the mask is applied with
      // selects, and only on blocks that need it)
      float mx = -CUDART_INF_F;
      // keys with index >= k_limit are invisible to this row
      int k_limit = p.seq_k;
      if (p.causal) k_limit = min(k_limit, q_pos - p.k_pos0 + 1);
      uint32_t sv[2][32];
      tmem_ld_32x32b_x32(tmem_s + lane_base + (2 * half) * 32, sv[0]);
      tmem_ld_32x32b_x32(tmem_s + lane_base + (2 * half + 1) * 32, sv[1]);
      tmem_ld_wait();
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, m2 = -CUDART_INF_F, m3 = -CUDART_INF_F;
        if (need_mask) {
          const int lim = k_limit - (k_base + (2 * half + cc) * 32);   // columns [0, lim) are visible
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            m0 = fmaxf(m0, i + 0 < lim ? __uint_as_float(sv[cc][i + 0]) : -CUDART_INF_F);
            m1 = fmaxf(m1, i + 1 < lim ? __uint_as_float(sv[cc][i + 1]) : -CUDART_INF_F);
            m2 = fmaxf(m2, i + 2 < lim ? __uint_as_float(sv[cc][i + 2]) : -CUDART_INF_F);
            m3 = fmaxf(m3, i + 3 < lim ? __uint_as_float(sv[cc][i + 3]) : -CUDART_INF_F);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            m0 = fmaxf(m0, __uint_as_float(sv[cc][i + 0]));
            m1 = fmaxf(m1, __uint_as_float(sv[cc][i + 1]));
            m2 = fmaxf(m2, __uint_as_float(sv[cc][i + 2]));
            m3 = fmaxf(m3, __uint_as_float(sv[cc][i + 3]));
          }
        }
        mx = fmaxf(mx, fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)));
      }
      mx *= scale_log2;   // scale > 0, so the maximum commutes with the scaling
      // combine with the other half of the row (the P buffer is idle here: the previous P V
      // product completed before this S tile was signalled)
      xchg[half * 128 + row] = mx;
      named_barrier_sync(3, kSoftmaxThreads);
      mx = fmaxf(mx, xchg[(half ^ 1) * 128 + row]);
      named_barrier_sync(3, kSoftmaxThreads);   // both halves have read before P overwrites the area
      if (threadIdx.x == 0) PICO_STAMP(512);
      const float m_new = fmaxf(m_run, mx);
      const bool grow = (m_new - m_run > kRescaleThreshold) || (m_run == -CUDART_INF_F);
      const float m_use = grow ? m_new : m_run;
      const float alpha = (m_run == -CUDART_INF_F) ? 0.f : exp2f(m_run - m_use);
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
        for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_o + lane_base + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st_32x32b_x32(tmem_o + lane_base + c * 32, v);
        }
        tmem_st_wait();
      }
      l_run *= alpha;
      m_run = m_use;
      // pass 2: probabilities -> bf16 P tile in shared memory, row sum
      float sum = 0.f;
      uint8_t* prow = sP + row * 128;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = 2 * half + cc;
        const uint32_t (&v)[32] = sv[cc];
        float pr[32];
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
        // exp2(s*scale - m) as one fused multiply-add per element; a row that has seen no key yet
        // (m = -inf) gets offset 0 and is masked entirely through lim = 0
        const float neg_m = (m_run == -CUDART_INF_F) ? 0.f : -m_run;
        if (need_mask || m_run == -CUDART_INF_F) {
          const int lim = (m_run == -CUDART_INF_F) ? 0 : k_limit - (k_base + c * 32);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float e = exp2f(fmaf(__uint_as_float(v[i]), scale_log2, neg_m));
            pr[i] = i < lim ? e : 0.f;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) pr[i] = exp2f(fmaf(__uint_as_float(v[i]), scale_log2, neg_m));
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          s0 += pr[i + 0];
          s1 += pr[i + 1];
          s2 += pr[i + 2];
          s3 += pr[i + 3];
        }
        sum += (s0 + s1) + (s2 + s3);
        uint8_t* panel = prow + (c >> 1) * 16384;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 o;
          o.x = pack_bf16x2(pr[8 * q4 + 0], pr[8 * q4 + 1]);
          o.y = pack_bf16x2(pr[8 * q4 + 2], pr[8 * q4 + 3]);
          o.z = pack_bf16x2(pr[8 * q4 + 4], pr[8 * q4 + 5]);
          o.w = pack_bf16x2(pr[8 * q4 + 6], pr[8 * q4 + 7]);
          const int chunk = (c & 1) * 4 + q4;
          *reinterpret_cast<uint4*>(panel + ((chunk ^ (row & 7)) << 4)) = o;
        }
      }
      l_run += sum;
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_ready);
      if (threadIdx.x == 0) PICO_STAMP(512);
    }
    // ---- epilogue
    if (alive) {
      bool ok = true;
      if (num_kv > 0) ok = mbar_wait(pv_done, (num_kv - 1) & 1, abort_word, status, 1200);
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
      if (all_ok) {
        tc_fence_after();
        xchg[half * 128 + row] = l_run;
        named_barrier_sync(3, kSoftmaxThreads);
        l_run += xchg[(half ^ 1) * 128 + row];
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        __nv_bfloat16* orow =
            out + (int64_t)batch * p.o_batch_stride + (int64_t)(q0 + row) * p.o_row_stride + head * D;
#pragma unroll 1
        for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
          uint32_t v[32];
          if (num_kv > 0) {
            tmem_ld_32x32b_x32(tmem_o + lane_base + c * 32, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0u;
          }
          if (valid_row) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(v[8 * q4 + 0]) * inv, __uint_as_float(v[8 * q4 + 1]) * inv);
              o.y = pack_bf16x2(__uint_as_float(v[8 * q4 + 2]) * inv, __uint_as_float(v[8 * q4 + 3]) * inv);
              o.z = pack_bf16x2(__uint_as_float(v[8 * q4 + 4]) * inv, __uint_as_float(v[8 * q4 + 5]) * inv);
              o.w = pack_bf16x2(__uint_as_float(v[8 * q4 + 6]) * inv, __uint_as_float(v[8 * q4 + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) = o;
            }
          }
        }
        if (valid_row && lse != nullptr && half == 0) {
          const float val = l_run > 0.f ? (m_run + log2f(l_run)) / kLog2e : -CUDART_INF_F;
          lse[((int64_t)batch * p.heads + head) * p.seq_q + q0 + row] = val;
        }
      }
    }
  }

  // ---------------------------------------------------------------------- teardown
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
static int launch_fwd(const void* q, const void* k, const void* v, void* out, float* lse,
                      const PicoAttnParams* p, cudaStream_t stream) {
  using Cfg = FwdCfg<D>;
  FwdMaps maps;
  int rc = pico_host::make_tmap_bshd(&maps.q, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, D, p->heads, p->seq_q,
                                     p->batch, p->q_row_stride * 2, p->q_batch_stride * 2, 64, kBlockM);
  if (rc) return rc;
  rc = pico_host::make_tmap_bshd(&maps.k, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, D, p->kv_heads, p->seq_k,
                                 p->batch, p->k_row_stride * 2, p->k_batch_stride * 2, 64, kBlockN);
  if (rc) return rc;
  rc = pico_host::make_tmap_bshd(&maps.v, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, D, p->kv_heads, p->seq_k,
                                 p->batch, p->v_row_stride * 2, p->v_batch_stride * 2, 64, kBlockN);
  if (rc) return rc;
  auto kern = flash_fwd_kernel<D>;
  static int attr_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (attr_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) {
      pico_host::set_error("attention fwd: cudaFuncSetAttribute(%d): %s", Cfg::kSmemBytes, cudaGetErrorString(e));
      return (int)e;
    }
    attr_dev = dev;
  }
  dim3 grid((p->seq_q + kBlockM - 1) / kBlockM, p->heads, p->batch);
  kern<<<grid, kFwdThreads, Cfg::kSmemBytes, stream>>>(maps, (__nv_bfloat16*)out, lse, *p, pico_status_buffer());
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    pico_host::set_error("attention fwd launch: %s", cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

// two query tiles per CTA, softmax of one overlapping the tensor-core work of the other
// (flash_fwd_pingpong_sm100.cu)
int launch_fwd_pingpong(const void* q, const void* k, const void* v, void* out, float* lse,
                        const PicoAttnParams* p, cudaStream_t stream);

}  // namespace pico

extern "C" int pico_attention_fwd(const void* q, const void* k, const void* v, void* out, float* lse,
                                  const PicoAttnParams* p, cudaStream_t stream) {
  if (p->batch <= 0 || p->seq_q <= 0 || p->heads <= 0) return 0;
  if (p->heads % p->kv_heads != 0) {
    pico_host::set_error("attention: heads (%d) must be a multiple of kv_heads (%d)", p->heads, p->kv_heads);
    return -2;
  }
  if ((p->o_row_stride % 8) != 0 || (p->o_batch_stride % 8) != 0 || (reinterpret_cast<uintptr_t>(out) & 15)) {
    pico_host::set_error("attention: output must be 16-byte aligned with strides that are multiples of 8");
    return -2;
  }
  // PICO_ATTN_FWD=single selects the one-tile-per-CTA kernel of this file (A/B comparisons)
  static const bool single = [] {
    const char* e = getenv("PICO_ATTN_FWD");
    return e != nullptr && strcmp(e, "single") == 0;
  }();
  if (!single && (p->head_dim == 64 || p->head_dim == 128))
    return pico::launch_fwd_pingpong(q, k, v, out, lse, p, stream);
  if (p->head_dim == 64) return pico::launch_fwd<64>(q, k, v, out, lse, p, stream);
  if (p->head_dim == 128) return pico::launch_fwd<128>(q, k, v, out, lse, p, stream);
  pico_host::set_error("attention: head_dim %d not supported (64 or 128)", p->head_dim);
  return -2;
}
