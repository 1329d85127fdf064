// Flash attention forward for sm_100a, two query tiles per CTA ("ping-pong").
//
// One CTA owns 256 query rows of one (batch, head) as two 128-row tiles A and B and walks the
// key/value sequence in blocks of 128. While the softmax of one tile runs on the CUDA cores the
// tensor cores work on the other tile, so neither unit waits for the other inside the CTA:
//
//   warps 0-3  : softmax of tile A  (one thread per query row, all 128 key columns of the block)
//   warps 4-7  : softmax of tile B
//   warp  8    : tcgen05.mma issue (one thread): S_t(j) = Q_t K_j^T and O_t += P_t(j) V_j
//   warp  9    : TMA loads (one thread): Q tiles once, K and V blocks into rings
//
// Tensor memory: S_A | S_B (128 fp32 columns each) | O_A | O_B (head_dim columns each) and, for
// head_dim 64, Q_A | Q_B (32 columns each). A softmax thread owns a whole row, so the row maximum
// and sum need no exchange between threads; it reads its S row from tensor memory twice (maximum,
// then exponentials) instead of holding 128 values in registers.
//
// Shared-memory bandwidth is what the tensor cores run out of first with tiles this small, so
// operands are kept in tensor memory where possible: P_t(j) is written as packed bf16 pairs over the
// first 64 columns of S_t and is the TMEM A operand of O_t += P_t V_j; for head_dim 64 the query
// tile is stored to tensor memory once by the softmax threads and is the TMEM A operand of every
// S_t = Q_t K_j^T. Only K_j and V_j are read from shared memory then.
// The accumulator is rescaled lazily: only when the running maximum grew by more than 2^8, which
// the fp32 range of the un-normalised probabilities absorbs.
//
// Issue order of the MMA thread (the tensor pipe executes in order):
//   S_A(0) | S_B(0) PV_A(0) S_A(1) | PV_B(0) S_B(1) | PV_A(1) S_A(2) | ...
// The commit after S_t(j+1) also covers PV_t(j): when the softmax of tile t sees S_t(j+1) it may
// overwrite P_t and rescale O_t.
//
// Every wait is bounded (common/ptx.cuh); a CTA that gives up frees its TMEM and returns.
#include <cuda_bf16.h>
#include <math_constants.h>

#include <cstring>
#include <type_traits>

#include "../common/host.h"
#include "../common/ptx.cuh"
#include "attention.h"

namespace pico {
namespace pp {

constexpr int kTileM = 128;            // rows of one query tile
constexpr int kCtaM = 2 * kTileM;      // rows per CTA
constexpr int kBlockN = 128;
constexpr int kGroupThreads = 128;
constexpr int kThreads = 2 * kGroupThreads + 64;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;

template <int D>
struct Cfg {
  static constexpr int kQBytes = kTileM * D * 2;          // one query tile
  static constexpr int kKVBytes = kBlockN * D * 2;        // one K or V block
  static constexpr int kPBytes = kTileM * kBlockN * 2;    // one P tile
  static constexpr bool kQInTmem = (D == 64);              // no TMEM columns left for it at head_dim 128
  static constexpr int kKStages = (D == 64) ? 4 : 2;
  static constexpr int kVStages = (D == 64) ? 4 : 2;
  static constexpr int kTiles = (kQInTmem ? 0 : 2 * kQBytes) + (kKStages + kVStages) * kKVBytes;
  // q_full[2] (TMA, or 128 softmax threads when Q goes to TMEM), k_full/k_empty[kKStages],
  // v_full/v_empty[kVStages], s_full[2], p_ready[2], o_done[2]
  static constexpr int kNumBars = 2 + 2 * kKStages + 2 * kVStages + 6;
  static constexpr int kSmemBytes = kTiles + kNumBars * 8 + 16;
  static constexpr int kTmemCols = 512;
  static constexpr int kPanels = D / 64;
};

struct Maps {
  CUtensorMap q, k, v;
};

// number of key blocks a tile whose last valid row is `last_row` (index in the local sequence) needs
__device__ __forceinline__ int blocks_needed(const PicoAttnParams& p, int first_row, int last_row) {
  if (last_row < first_row) return 0;
  int n = (p.seq_k + kBlockN - 1) / kBlockN;
  if (p.causal) {
    const int visible = p.q_pos0 + last_row - p.k_pos0 + 1;
    n = visible <= 0 ? 0 : min(n, (visible + kBlockN - 1) / kBlockN);
  }
  return n;
}

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
flash_fwd_pingpong_kernel(const __grid_constant__ Maps maps, const __nv_bfloat16* __restrict__ q_ptr,
                          __nv_bfloat16* __restrict__ out,
                          float* __restrict__ lse, const PicoAttnParams p, int* status) {
  using C = Cfg<D>;
  extern __shared__ uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {   // swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) report_error(status, PICO_ERR_BOUNDS, 2999, (int)(smem_u32(smem) & 1023u));
    return;
  }
  uint8_t* sQ = smem;                                   // [2] (absent when Q lives in TMEM)
  uint8_t* sK = sQ + (C::kQInTmem ? 0 : 2 * C::kQBytes);   // [kKStages]
  uint8_t* sV = sK + C::kKStages * C::kKVBytes;         // [kVStages]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kTiles);
  uint64_t* q_full = bars;
  uint64_t* k_full = q_full + 2;
  uint64_t* k_empty = k_full + C::kKStages;
  uint64_t* v_full = k_empty + C::kKStages;
  uint64_t* v_empty = v_full + C::kVStages;
  uint64_t* s_full = v_empty + C::kVStages;
  uint64_t* p_ready = s_full + 2;
  uint64_t* o_done = p_ready + 2;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(o_done + 2);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // heavy (late) query tiles first so the causal triangle balances across the grid
  const int num_q = (p.seq_q + kCtaM - 1) / kCtaM;
  // blocks are dispatched x-fastest: every (head, batch) of the heaviest query block starts before
  // any lighter block, so the tail of the grid consists of the shortest CTAs
  const int q_blk = num_q - 1 - (int)blockIdx.z;
  const int head = blockIdx.x;
  const int batch = blockIdx.y;
  const int kv_head = head / (p.heads / p.kv_heads);
  const int q0 = q_blk * kCtaM;

  const int n0 = blocks_needed(p, q0, min(q0 + kTileM, p.seq_q) - 1);              // key blocks of tile A
  const int n1 = blocks_needed(p, q0 + kTileM, min(q0 + kCtaM, p.seq_q) - 1);      // ... of tile B
  const int n_max = max(n0, n1);

  if (threadIdx.x == 0) {
    for (int t = 0; t < 2; ++t) {
      mbar_init(&q_full[t], C::kQInTmem ? kGroupThreads : 1);
      mbar_init(&s_full[t], 1);
      mbar_init(&p_ready[t], kGroupThreads);
      mbar_init(&o_done[t], 1);
    }
    for (int s = 0; s < C::kKStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < C::kVStages; ++s) {
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    *abort_word = 0;
    mbar_fence_init();
    tma_prefetch_desc(&maps.q);
    tma_prefetch_desc(&maps.k);
    tma_prefetch_desc(&maps.v);
  }
  if (warp == 8) {
    tmem_alloc(tmem_ptr_smem, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  // optional timeline of the first CTA (performance debugging): SM clock stamps, 256 per role;
  // roles: 0 = softmax A (thread 0), 1 = softmax B (thread 128), 2 = MMA issue
  const bool tracing = p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
  int trace_n = 0;
#define PP_STAMP(role)                                                                          \
  do {                                                                                          \
    if (tracing && trace_n < 256) p.trace[(role) * 256 + trace_n++] = (unsigned long long)clock64(); \
  } while (0)

  if (warp == 9) {
    // ---------------------------------------------------------------------------- TMA loads
    if (lane == 0 && n_max > 0) {
      for (int t = 0; t < 2; ++t) {
        if ((t == 0 ? n0 : n1) == 0 || C::kQInTmem) continue;
        mbar_arrive_expect_tx(&q_full[t], C::kQBytes);
#pragma unroll
        for (int pn = 0; pn < C::kPanels; ++pn)
          tma_load_4d(sQ + t * C::kQBytes + pn * 16384, &maps.q, &q_full[t], pn * 64, head, q0 + t * kTileM, batch);
      }
      for (int j = 0; j < n_max; ++j) {
        const int ks = j % C::kKStages, vs = j % C::kVStages;
        if (j >= C::kKStages &&
            !mbar_wait(&k_empty[ks], ((j / C::kKStages) - 1) & 1, abort_word, status, 2010))
          break;
        mbar_arrive_expect_tx(&k_full[ks], C::kKVBytes);
#pragma unroll
        for (int pn = 0; pn < C::kPanels; ++pn)
          tma_load_4d(sK + ks * C::kKVBytes + pn * 16384, &maps.k, &k_full[ks], pn * 64, kv_head, j * kBlockN, batch);
        if (j >= C::kVStages &&
            !mbar_wait(&v_empty[vs], ((j / C::kVStages) - 1) & 1, abort_word, status, 2011))
          break;
        mbar_arrive_expect_tx(&v_full[vs], C::kKVBytes);
#pragma unroll
        for (int pn = 0; pn < C::kPanels; ++pn)
          tma_load_4d(sV + vs * C::kKVBytes + pn * 16384, &maps.v, &v_full[vs], pn * 64, kv_head, j * kBlockN, batch);
      }
    }
  } else if (warp == 8) {
    // ---------------------------------------------------------------------------- MMA issue
    // This thread is the pacemaker of the CTA: everything it does between two products delays
    // both softmax groups, so the tile index is a compile-time constant (no indexed local arrays)
    // and ready barriers are only polled when this is the first reader of a block.
    if (lane == 0 && n_max > 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(kTileM, kBlockN, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc_bf16(kTileM, D, 0, 1);
      bool ok = true;
      // S_t(j) = Q_t K_j^T into S_t's columns; releases K_j after its last reader
      auto issue_s = [&](auto tc, int j) {
        constexpr int t = decltype(tc)::value;
        const int ks = j % C::kKStages;
        // the first tile that reads K_j waits for it to land
        if ((t == 0 || j >= n0) && !mbar_wait(&k_full[ks], (j / C::kKStages) & 1, abort_word, status, 2020)) {
          ok = false;
          return;
        }
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQ + t * C::kQBytes);
        const uint32_t k_addr = smem_u32(sK + ks * C::kKVBytes);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          if (C::kQInTmem)   // 16 bf16 of K per step = 8 packed columns of the query tile
            tc_mma_f16_ts(tmem_base + t * kBlockN, tmem_base + 2 * kBlockN + 2 * D + t * (D / 2) + kk * 8,
                          umma_smem_desc(k_addr + off, 16, 1024), idesc_s, kk != 0 ? 1u : 0u);
          else
            tc_mma_f16_ss(tmem_base + t * kBlockN, umma_smem_desc(q_addr + off, 16, 1024),
                          umma_smem_desc(k_addr + off, 16, 1024), idesc_s, kk != 0 ? 1u : 0u);
        }
        tc_commit(&s_full[t]);
        if (t == 1 || j >= n1) tc_commit(&k_empty[ks]);   // last reader of K_j
      };
      // O_t += P_t(j) V_j, then S_t(j+1) (or the completion signal of the tile)
      auto issue_pv = [&](auto tc, int j) {
        constexpr int t = decltype(tc)::value;
        const int vs = j % C::kVStages;
        if ((t == 0 || j >= n0) && !mbar_wait(&v_full[vs], (j / C::kVStages) & 1, abort_word, status, 2040)) {
          ok = false;
          return;
        }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sV + vs * C::kKVBytes);
        const uint32_t o_tmem = tmem_base + 2 * kBlockN + t * D;
        const uint32_t p_tmem = tmem_base + t * kBlockN;   // packed bf16 pairs over S_t's first 64 columns
#pragma unroll
        for (int kk = 0; kk < kBlockN / 16; ++kk)
          tc_mma_f16_ts(o_tmem, p_tmem + kk * 8, umma_smem_desc(v_addr + kk * 2048, 16384, 1024), idesc_o,
                        (j | kk) != 0 ? 1u : 0u);
        if (t == 1 || j >= n1) tc_commit(&v_empty[vs]);  // last reader of V_j
        if (j + 1 < (t == 0 ? n0 : n1))
          issue_s(tc, j + 1);
        else
          tc_commit(&o_done[t]);
      };
      using T0 = std::integral_constant<int, 0>;
      using T1 = std::integral_constant<int, 1>;
      // Start the two tiles half a period apart: S_B(0) is issued only when P_A(0) is ready, so the
      // softmax of one tile runs while the other tile's products execute. Started together the
      // two softmax groups would stay in lock-step, compete for the exponential unit, and then both
      // wait for the tensor cores.
      const bool both = n0 > 0 && n1 > 0;
      if (n0 > 0) {
        ok = mbar_wait(&q_full[0], 0, abort_word, status, 2000);
        if (ok) issue_s(T0{}, 0);
      } else {
        ok = mbar_wait(&q_full[1], 0, abort_word, status, 2001);
        if (ok) issue_s(T1{}, 0);
      }
      for (int j = 0; j < n_max && ok; ++j) {
        if (j < n0) {
          if (!mbar_wait(&p_ready[0], j & 1, abort_word, status, 2030)) break;
          if (both && j == 0) {   // delayed first product of tile B (see above)
            if (!mbar_wait(&q_full[1], 0, abort_word, status, 2001)) break;
            issue_s(T1{}, 0);
            if (!ok) break;
          }
          issue_pv(T0{}, j);
          if (!ok) break;
        }
        if (j < n1) {
          if (!mbar_wait(&p_ready[1], j & 1, abort_word, status, 2031)) break;
          issue_pv(T1{}, j);
        }
      }
    }
  } else {
    // ---------------------------------------------------------------------------- softmax + epilogue
    const int t = warp >> 2;                        // tile of this group
    const int row = (warp & 3) * 32 + lane;         // row inside the tile = TMEM lane
    const int q_row = q0 + t * kTileM + row;        // row in the local query sequence
    const bool valid_row = q_row < p.seq_q;
    const int q_pos = p.q_pos0 + q_row;
    const float scale_log2 = p.sm_scale * kLog2e;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tmem_s = tmem_base + t * kBlockN + lane_base;
    const uint32_t tmem_o = tmem_base + 2 * kBlockN + t * D + lane_base;
    const int n_mine = t == 0 ? n0 : n1;
    if (C::kQInTmem && n_mine > 0) {
      // this thread's query row (64 bf16 = 32 packed columns) -> tensor memory, once
      uint32_t qv[32];
      if (valid_row) {
        const uint4* src = reinterpret_cast<const uint4*>(q_ptr + (int64_t)batch * p.q_batch_stride +
                                                         (int64_t)q_row * p.q_row_stride + head * D);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint4 v4 = __ldg(src + i);
          qv[4 * i + 0] = v4.x;
          qv[4 * i + 1] = v4.y;
          qv[4 * i + 2] = v4.z;
          qv[4 * i + 3] = v4.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) qv[i] = 0u;
      }
      tmem_st_32x32b_x32(tmem_base + 2 * kBlockN + 2 * D + t * (D / 2) + lane_base, qv);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&q_full[t]);
    }
    float m_run = -CUDART_INF_F;   // running max of the scaled scores (log2 units)
    float l_run = 0.f;
    bool alive = true;
    // keys with index >= k_limit are invisible to this row
    int k_limit = p.seq_k;
    if (p.causal) k_limit = min(k_limit, q_pos - p.k_pos0 + 1);
    for (int j = 0; j < n_mine; ++j) {
      if ((threadIdx.x & 127) == 0) PP_STAMP(t);
      // warp-uniform outcome: the lanes of a warp stay together through the shuffles below
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[t], j & 1, abort_word, status, 2100 + t))) {
        alive = false;
        break;
      }
      tc_fence_after();
      if ((threadIdx.x & 127) == 0) PP_STAMP(t);
      const int k_base = j * kBlockN;
      const bool need_mask =
          (p.causal && (p.k_pos0 + k_base + kBlockN - 1 > p.q_pos0 + q0 + t * kTileM)) || (k_base + kBlockN > p.seq_k);
      // the whole S row (128 fp32) comes into registers with four loads in flight and one wait
      uint32_t sv[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(tmem_s + c * 32, sv[c]);
      tmem_ld_wait();
      if ((threadIdx.x & 127) == 0) PP_STAMP(t);
      // ---- masking: on the few blocks that need it (diagonal, ragged end) invisible scores become
      // -inf in place, so the arithmetic below exists only once in the instruction stream
      // (exp2(-inf) = 0; the kernel is large enough for instruction fetch to matter)
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int lim = k_limit - (k_base + c * 32);   // columns [0, lim) of the chunk are visible
#pragma unroll
          for (int i = 0; i < 32; ++i)
            sv[c][i] = i < lim ? sv[c][i] : __float_as_uint(-CUDART_INF_F);
        }
      }
      // ---- row maximum
      float mx;
      {
        float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, m2 = -CUDART_INF_F, m3 = -CUDART_INF_F;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            m0 = fmaxf(m0, __uint_as_float(sv[c][i + 0]));
            m1 = fmaxf(m1, __uint_as_float(sv[c][i + 1]));
            m2 = fmaxf(m2, __uint_as_float(sv[c][i + 2]));
            m3 = fmaxf(m3, __uint_as_float(sv[c][i + 3]));
          }
        }
        mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
      }
      mx *= scale_log2;   // scale > 0, so the maximum commutes with the scaling (-inf stays -inf)
      const float m_new = fmaxf(m_run, mx);
      const bool grow = (m_new - m_run > kRescaleThreshold) || (m_run == -CUDART_INF_F);
      const float m_use = grow ? m_new : m_run;
      const float alpha = (m_run == -CUDART_INF_F) ? 0.f : exp2f(m_run - m_use);
      // PV_t(j-1) completed before S_t(j) was signalled, so O_t is quiescent here
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_o + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st_32x32b_x32(tmem_o + c * 32, v);
        }
        tmem_st_wait();
      }
      l_run *= alpha;
      m_run = m_use;
      // ---- probabilities -> packed bf16 P over the first 64 columns of S_t, row sum
      // exp2(s*scale - m) is one fused multiply-add per element; a row that has seen no key yet
      // (m = -inf) uses offset 0: all its scores are -inf and give 0
      const float neg_m = (m_run == -CUDART_INF_F) ? 0.f : -m_run;
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
      // P only overwrites S columns 0..63 (chunks 0 and 1), so chunks 2 and 3 are dropped after the
      // maximum and read again while chunks 0 and 1 are exponentiated; this keeps the live register
      // count under the limit of this launch configuration
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if (c == 1) tmem_ld_32x32b_x32(tmem_s + 2 * 32, sv[2]);
        if (c == 2) {
          tmem_ld_wait();
          tmem_ld_32x32b_x32(tmem_s + 3 * 32, sv[3]);
        }
        if (c == 3) tmem_ld_wait();
        if (c >= 2 && need_mask) {   // the reloaded chunks come unmasked
          const int lim = k_limit - (k_base + c * 32);
#pragma unroll
          for (int i = 0; i < 32; ++i)
            sv[c][i] = i < lim ? sv[c][i] : __float_as_uint(-CUDART_INF_F);
        }
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float e0 = exp2f(fmaf(__uint_as_float(sv[c][i + 0]), scale_log2, neg_m));
          const float e1 = exp2f(fmaf(__uint_as_float(sv[c][i + 1]), scale_log2, neg_m));
          const float e2 = exp2f(fmaf(__uint_as_float(sv[c][i + 2]), scale_log2, neg_m));
          const float e3 = exp2f(fmaf(__uint_as_float(sv[c][i + 3]), scale_log2, neg_m));
          s0 += e0;
          s1 += e1;
          s2 += e2;
          s3 += e3;
          pk[i / 2] = pack_bf16x2(e0, e1);
          pk[i / 2 + 1] = pack_bf16x2(e2, e3);
        }
        // every S column of chunks 0 and 1 is already in registers, so P may overwrite them
        tmem_st_32x32b_x16(tmem_s + c * 16, pk);
      }
      l_run += (s0 + s1) + (s2 + s3);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_ready[t]);
      if ((threadIdx.x & 127) == 0) PP_STAMP(t);
    }
    // ---- epilogue: normalise and store this thread's output row
    if (alive) {
      bool ok = true;
      if (n_mine > 0) ok = mbar_wait(&o_done[t], 0, abort_word, status, 2200 + t);
      if (ok) {
        tc_fence_after();
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        __nv_bfloat16* orow =
            out + (int64_t)batch * p.o_batch_stride + (int64_t)q_row * p.o_row_stride + head * D;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t v[32];
          if (n_mine > 0) {
            tmem_ld_32x32b_x32(tmem_o + c * 32, v);
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
        if (valid_row && lse != nullptr) {
          const float val = l_run > 0.f ? (m_run + log2f(l_run)) / kLog2e : -CUDART_INF_F;
          lse[((int64_t)batch * p.heads + head) * p.seq_q + q_row] = val;
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
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int D>
static int launch(const void* q, const void* k, const void* v, void* out, float* lse, const PicoAttnParams* p,
                  cudaStream_t stream) {
  using C = Cfg<D>;
  Maps maps;
  int rc = pico_host::make_tmap_bshd(&maps.q, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, D, p->heads, p->seq_q,
                                     p->batch, p->q_row_stride * 2, p->q_batch_stride * 2, 64, kTileM);
  if (rc) return rc;
  rc = pico_host::make_tmap_bshd(&maps.k, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, D, p->kv_heads, p->seq_k,
                                 p->batch, p->k_row_stride * 2, p->k_batch_stride * 2, 64, kBlockN);
  if (rc) return rc;
  rc = pico_host::make_tmap_bshd(&maps.v, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, D, p->kv_heads, p->seq_k,
                                 p->batch, p->v_row_stride * 2, p->v_batch_stride * 2, 64, kBlockN);
  if (rc) return rc;
  auto kern = flash_fwd_pingpong_kernel<D>;
  static int attr_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (attr_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) {
      pico_host::set_error("attention fwd: cudaFuncSetAttribute(%d): %s", C::kSmemBytes, cudaGetErrorString(e));
      return (int)e;
    }
    attr_dev = dev;
  }
  dim3 grid(p->heads, p->batch, (p->seq_q + kCtaM - 1) / kCtaM);
  kern<<<grid, kThreads, C::kSmemBytes, stream>>>(maps, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, lse, *p,
                                                  pico_status_buffer());
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    pico_host::set_error("attention fwd launch: %s", cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

}  // namespace pp
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
  if (p->head_dim == 64) return pico::pp::launch<64>(q, k, v, out, lse, p, stream);
  if (p->head_dim == 128) return pico::pp::launch<128>(q, k, v, out, lse, p, stream);
  pico_host::set_error("attention: head_dim %d not supported (64 or 128)", p->head_dim);
  return -2;
}
