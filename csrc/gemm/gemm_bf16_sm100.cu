// Persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   D[M,N] (=|+=) op(A)[M,K] * op(B)[K,N]        fp32 accumulation in tensor memory
//
// One CTA per SM walks output tiles of 128 x BN. Roles:
//   warp 0    : TMA producer  - streams 64-deep K slices of A and B into a ring of shared
//                               memory stages (128-byte swizzle), one mbarrier per stage
//   warp 1    : MMA issuer    - one elected thread issues tcgen05.mma (128 x BN x 16) per
//                               K step; accumulators live in TMEM, double buffered so the
//                               epilogue of tile i overlaps the main loop of tile i+1
//   warps 2-5 : epilogue      - tcgen05.ld the accumulator, convert, stage in swizzled
//                               shared memory, TMA store (or TMA reduce-add for D +=)
//
// Operand layouts (all row-major with a leading dimension in elements):
//   a_mn_major = 0 : A stored [M, K]  (K contiguous)      - activations in a forward linear
//   a_mn_major = 1 : A stored [K, M]  (M contiguous)      - dY in a weight-gradient GEMM
//   b_mn_major = 0 : B stored [N, K]  (K contiguous)      - nn.Linear weight in forward
//   b_mn_major = 1 : B stored [K, N]  (N contiguous)      - weight in dgrad, X in wgrad
// so forward, dgrad and wgrad of a bias-free linear all run without a transpose copy.
//
// Ragged M, N, K are handled by TMA (zero fill on load, clipping on store); the only
// requirement is 16-byte aligned base pointers and leading dimensions.
#include <cuda_bf16.h>

#include <cstring>

#include "../common/host.h"
#include "../common/ptx.cuh"
#include "../runtime/flags.cuh"
#include "gemm.h"

namespace pico {

constexpr int BM = 128;
constexpr int BK = 64;          // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int kNumEpilogueThreads = 128;
constexpr int kNumThreads = 64 + kNumEpilogueThreads;
constexpr int kStagingBytes = 128 * 128;  // 128 rows x 128 bytes
constexpr int kNumStaging = 2;

template <int BN>
struct GemmCfg {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kSmemTiles = kStages * kStageBytes + kNumStaging * kStagingBytes;
  // barriers: full[kStages], empty[kStages], tmem_full[2], tmem_empty[2] + tmem ptr + abort
  static constexpr int kSmemBytes = kSmemTiles + (2 * kStages + 4) * 8 + 16 + 1024;
  static constexpr int kTmemCols = (2 * BN <= 512) ? ((2 * BN < 32) ? 32 : 2 * BN) : 512;
};

enum OutMode : int { OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ACC = 2 };

// Output tensor maps: one per destination. A plain GEMM uses m[0]; a GEMM fused with a
// reduce-scatter stores row block b of the output through m[b], which addresses rank b's
// staging buffer (peer memory over NVLink).
struct DMaps {
  CUtensorMap m[PICO_MAX_PEERS];
};

// Collective fusion parameters (all zero = plain GEMM).
struct GemmComm {
  // all-gather -> GEMM: the rows of A arrive in equal blocks, block b written by rank b into
  // this GPU's gather buffer; tiles of block b are loaded only after flag [a_slot][b] >= a_epoch
  const uint32_t* a_flags;
  int a_slot;
  uint32_t a_epoch;
  int a_skip_block;       // this rank's own block: already in place, never waited for
  // Row geometry shared by both fusions: the M rows are `pieces` of blk_rows rows; piece p belongs
  // to block p % num_blocks (the rank that wrote it / that receives it) and is the (p / num_blocks)-th
  // piece of that block. One piece per block is the plain "rank r owns rows [r*m, (r+1)*m)" split;
  // several pieces per block is a [batch, sequence] tensor whose sequence is split over the ranks.
  int blk_rows;           // 0 = no collective fusion
  int num_blocks;
  int first_block;        // tile order starts with this block (own rows / the neighbour's rows)
  int scatter;            // GEMM -> reduce-scatter: rows of block b are stored through DMaps::m[b]
  unsigned long long timeout_ns;
  // grouped GEMM (experts of a mixture-of-experts layer), see PicoGemmGroups in gemm.h
  const int* tile_group;  // row-grouped mode: group of every 128-row tile of A / D (-1 = skip)
  int b_group_rows;       //   rows of one group's matrix inside the stacked B
  const int* seg_start;   // reduction-grouped mode: group g reduces over rows [seg_start[g], seg_start[g+1])
  int num_groups;
};

struct TileCoord {
  int m, n;
};

// What one persistent-loop iteration works on. Plain GEMM: the whole K range of output tile
// (m, n). Row-grouped: the same, with B taken from group `grp`. Reduction-grouped: output tile
// (m, n) of group `grp` (stacked along the rows of D), reduced over that group's K blocks.
struct TileWork {
  int m, n, grp, kb0, kb1;
  bool skip;
};

// Grouped rasterisation: consecutive tile indices (= CTAs running at the same time) cover a
// compact block of the output so A and B slices are shared through L2.
__device__ __forceinline__ TileCoord tile_coord(int tile, int num_m, int num_n) {
  constexpr int kGroup = 16;
  int tiles_per_group = kGroup * num_n;
  int g = tile / tiles_per_group;
  int first_m = g * kGroup;
  int gsize = min(kGroup, num_m - first_m);
  int r = tile - g * tiles_per_group;
  TileCoord c;
  c.m = first_m + r % gsize;
  c.n = r / gsize;
  return c;
}

// Order in which the m-tiles of a collective-fused GEMM are visited: all pieces of block
// first_block, then those of first_block + 1, ... (wrapping), so the rows that are available
// first (or wanted first by a peer) are computed first. lm: logical m-tile index.
__device__ __forceinline__ int block_first_m(int lm, int num_m, const GemmComm& comm) {
  const int tpp = comm.blk_rows / BM;                       // tiles per piece
  const int per_block = num_m / comm.num_blocks;            // tiles per block (all its pieces)
  const int o = lm / per_block;
  const int rem = lm - o * per_block;
  const int piece_of_block = rem / tpp;
  const int j = rem - piece_of_block * tpp;
  int blk = comm.first_block + o;
  if (blk >= comm.num_blocks) blk -= comm.num_blocks;
  return (piece_of_block * comm.num_blocks + blk) * tpp + j;
}

__device__ __forceinline__ TileWork tile_work(int tile, int num_m, int num_n, int num_kb,
                                              const GemmComm& comm) {
  TileWork w;
  w.grp = 0;
  w.kb0 = 0;
  w.kb1 = num_kb;
  w.skip = false;
  if (comm.seg_start != nullptr) {
    const int per_group = num_m * num_n;
    w.grp = tile / per_group;
    TileCoord c = tile_coord(tile - w.grp * per_group, num_m, num_n);
    w.m = c.m;
    w.n = c.n;
    w.kb0 = __ldg(comm.seg_start + w.grp) / BK;
    w.kb1 = __ldg(comm.seg_start + w.grp + 1) / BK;
    w.skip = w.kb1 <= w.kb0;
    return w;
  }
  TileCoord c = tile_coord(tile, num_m, num_n);
  w.m = comm.blk_rows > 0 ? block_first_m(c.m, num_m, comm) : c.m;
  w.n = c.n;
  if (comm.tile_group != nullptr) {
    w.grp = __ldg(comm.tile_group + c.m);
    w.skip = w.grp < 0;
  }
  return w;
}

template <int BN, int A_MN, int B_MN, int OUT>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ DMaps dmaps, const GemmComm comm, int M, int N, int K,
                 int* status) {
  using Cfg = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment is required by the 128-byte swizzle atoms
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* stage_base = smem;
  uint8_t* staging = smem + Cfg::kStages * Cfg::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::kSmemTiles);
  uint64_t* empty_bar = full_bar + Cfg::kStages;
  uint64_t* tmem_full = empty_bar + Cfg::kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (M + BM - 1) / BM;
  const int num_n = (N + BN - 1) / BN;
  const int num_tiles = num_m * num_n * (comm.seg_start != nullptr ? comm.num_groups : 1);
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 1);
    }
    *abort_word = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&dmaps.m[0]);
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr_smem, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint64_t ready_pieces = 0;  // per block (8 bits each): pieces of A known to have arrived
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const TileWork tw = tile_work(tile, num_m, num_n, num_kb, comm);
        if (tw.skip) continue;
        const int m0 = tw.m * BM, n0 = tw.n * BN;
        // row-grouped mode: this tile's B is group grp's block of the stacked matrix
        const int b_off = comm.tile_group != nullptr ? tw.grp * comm.b_group_rows : 0;
        if (comm.a_flags != nullptr) {
          const int piece = m0 / comm.blk_rows;
          const int blk = piece % comm.num_blocks;
          // the writer reports its pieces in order: piece k of a block is there once progress > k
          const uint32_t need = min(piece / comm.num_blocks + 1, 254);
          if (blk != comm.a_skip_block && ((ready_pieces >> (8 * blk)) & 0xFFu) < need) {
            if (!wait_flag_ge(comm.a_flags + comm.a_slot * PICO_MAX_PEERS + blk,
                              flag_value(comm.a_flags, comm.a_slot, comm.a_epoch, need), comm.timeout_ns, status,
                              500 + blk)) {
              *abort_word = 1;
              break;
            }
            ready_pieces = (ready_pieces & ~(0xFFull << (8 * blk))) | ((uint64_t)need << (8 * blk));
            // the rows were written by another GPU; order the flag observation before the
            // bulk-copy engine's reads of them
            asm volatile("fence.proxy.async;" ::: "memory");
          }
        }
        for (int kb = tw.kb0; kb < tw.kb1; ++kb) {
          if (!mbar_wait(&empty_bar[s], phase ^ 1, abort_word, status, 100 + s)) {
            ok = false;
            break;
          }
          uint8_t* sa = stage_base + s * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kABytes;
          mbar_arrive_expect_tx(&full_bar[s], Cfg::kStageBytes);
          const int k0 = kb * BK;
          if (A_MN == 0) {
            tma_load_2d(sa, &tmap_a, &full_bar[s], k0, m0);  // box 64(K) x 128(M)
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)  // boxes 64(M) x 64(K)
              tma_load_2d(sa + j * (64 * BK * 2), &tmap_a, &full_bar[s], m0 + j * 64, k0);
          }
          if (B_MN == 0) {
            tma_load_2d(sb, &tmap_b, &full_bar[s], k0, n0 + b_off);  // box 64(K) x BN
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)  // boxes 64(N) x 64(K)
              tma_load_2d(sb + j * (64 * BK * 2), &tmap_b, &full_bar[s], n0 + j * 64, k0 + b_off);
          }
          if (++s == Cfg::kStages) {
            s = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN, B_MN);
      int s = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const TileWork tw = tile_work(tile, num_m, num_n, num_kb, comm);
        if (tw.skip) continue;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_word, status, 200 + acc)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = tw.kb0; kb < tw.kb1; ++kb) {
          if (!mbar_wait(&full_bar[s], phase, abort_word, status, 300 + s)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(stage_base + s * Cfg::kStageBytes);
          const uint32_t sb = sa + Cfg::kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major: step 32 bytes inside the swizzle row; MN-major: step 16 k-rows.
            uint64_t da = A_MN == 0 ? umma_smem_desc(sa + k * (UMMA_K * 2), 16, 1024)
                                    : umma_smem_desc(sa + k * (UMMA_K * 128), 64 * BK * 2, 1024);
            uint64_t db = B_MN == 0 ? umma_smem_desc(sb + k * (UMMA_K * 2), 16, 1024)
                                    : umma_smem_desc(sb + k * (UMMA_K * 128), 64 * BK * 2, 1024);
            tc_mma_f16_ss(d_tmem, da, db, idesc, ((kb - tw.kb0) | k) != 0 ? 1u : 0u);
          }
          tc_commit(&empty_bar[s]);  // stage reusable once these MMAs have read it
          if (++s == Cfg::kStages) {
            s = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        tc_commit(&tmem_full[acc]);  // accumulator complete
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int et = threadIdx.x - 64;             // 0..127
    const int quarter = warp & 3;                 // TMEM lane quarter this warp may access
    const int row = quarter * 32 + lane;          // row of the tile owned by this thread
    constexpr int kColsPerChunk = (OUT == OUT_BF16) ? 64 : 32;  // 128 bytes of output per row
    constexpr int kChunks = BN / kColsPerChunk;
    int acc = 0;
    uint32_t acc_phase = 0;
    int buf = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const TileWork tw = tile_work(tile, num_m, num_n, num_kb, comm);
      if (tw.skip) continue;
      int m0 = tw.m * BM;
      if (comm.seg_start != nullptr) m0 += tw.grp * M;   // groups are stacked along the rows of D
      const int n0 = tw.n * BN;
      const CUtensorMap* tmap_d = &dmaps.m[0];
      if (comm.scatter) {
        const int piece = m0 / comm.blk_rows;
        const int dest = piece % comm.num_blocks;
        tmap_d = &dmaps.m[dest];
        m0 = (piece / comm.num_blocks) * comm.blk_rows + (m0 - piece * comm.blk_rows);
      }
      bool ok = mbar_wait(&tmem_full[acc], acc_phase, abort_word, status, 400 + acc);
      // uniform decision for the four epilogue warps (they share named barriers below)
      int all_ok;
      asm volatile(
          "{\n\t"
          ".reg .pred p, q;\n\t"
          "setp.ne.b32 p, %1, 0;\n\t"
          "barrier.cta.red.and.pred q, 2, 128, p;\n\t"
          "selp.u32 %0, 1, 0, q;\n\t"
          "}\n"
          : "=r"(all_ok)
          : "r"((int)ok)
          : "memory");
      if (!all_ok) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < kChunks; ++c) {
        // skip column chunks that are entirely out of range (uniform across threads)
        if (n0 + c * kColsPerChunk >= N) break;
        uint8_t* sbuf = staging + buf * kStagingBytes;
        if (et == 0) tma_store_wait_read<kNumStaging - 1>();
        named_barrier_sync(1, kNumEpilogueThreads);
        uint8_t* srow = sbuf + row * 128;
        if (OUT == OUT_BF16) {
          uint32_t v0[32], v1[32];
          tmem_ld_32x32b_x32(t_row + c * 64, v0);
          tmem_ld_32x32b_x32(t_row + c * 64 + 32, v1);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v0[8 * j + 0]), __uint_as_float(v0[8 * j + 1]));
            o.y = pack_bf16x2(__uint_as_float(v0[8 * j + 2]), __uint_as_float(v0[8 * j + 3]));
            o.z = pack_bf16x2(__uint_as_float(v0[8 * j + 4]), __uint_as_float(v0[8 * j + 5]));
            o.w = pack_bf16x2(__uint_as_float(v0[8 * j + 6]), __uint_as_float(v0[8 * j + 7]));
            *reinterpret_cast<uint4*>(srow + ((j ^ (row & 7)) << 4)) = o;
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v1[8 * j + 0]), __uint_as_float(v1[8 * j + 1]));
            o.y = pack_bf16x2(__uint_as_float(v1[8 * j + 2]), __uint_as_float(v1[8 * j + 3]));
            o.z = pack_bf16x2(__uint_as_float(v1[8 * j + 4]), __uint_as_float(v1[8 * j + 5]));
            o.w = pack_bf16x2(__uint_as_float(v1[8 * j + 6]), __uint_as_float(v1[8 * j + 7]));
            *reinterpret_cast<uint4*>(srow + (((j + 4) ^ (row & 7)) << 4)) = o;
          }
        } else {
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_row + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 o = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            *reinterpret_cast<uint4*>(srow + ((j ^ (row & 7)) << 4)) = o;
          }
        }
        fence_proxy_async_smem();
        named_barrier_sync(1, kNumEpilogueThreads);
        if (et == 0) {
          if (OUT == OUT_F32_ACC)
            tma_reduce_add_2d(tmap_d, sbuf, n0 + c * kColsPerChunk, m0);
          else
            tma_store_2d(tmap_d, sbuf, n0 + c * kColsPerChunk, m0);
          tma_store_commit();
        }
        buf ^= 1;
      }
      // accumulator drained: hand it back to the MMA warp
      tc_fence_before();
      named_barrier_sync(1, kNumEpilogueThreads);
      if (et == 0) mbar_arrive(&tmem_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if (et == 0) tma_store_wait<0>();
  }

  // ---------------------------------------------------------------------- teardown
  if (*abort_word) {
    // give copies that were already issued time to land before shared memory goes away
    uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int BN, int A_MN, int B_MN, int OUT>
static int launch(const void* A, const void* B, void* D, int M, int N, int K, int lda, int ldb,
                  int ldd, int max_ctas, const PicoGemmComm* pc, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  using pico_host::Swizzle;
  CUtensorMap ta, tb;
  DMaps dm;
  GemmComm comm;
  memset(&comm, 0, sizeof(comm));
  int rc;
  if (A_MN == 0)
    rc = pico_host::make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, (uint64_t)lda * 2,
                                 64, BM, Swizzle::B128);
  else
    rc = pico_host::make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, (uint64_t)lda * 2,
                                 64, 64, Swizzle::B128);
  if (rc) return rc;
  const bool row_grouped = pc && pc->tile_group != nullptr;
  const bool red_grouped = pc && pc->seg_start != nullptr;
  if (row_grouped || red_grouped) {
    if (pc->num_groups <= 0 || (row_grouped && red_grouped) || pc->d_num_dest > 0 || pc->a_flags != nullptr) {
      pico_host::set_error("grouped gemm: one grouping mode, at least one group, no collective fusion");
      return -2;
    }
    if (row_grouped && (A_MN != 0 || pc->b_group_rows != (B_MN == 0 ? N : K) || (B_MN == 1 && K % BK != 0))) {
      pico_host::set_error("row-grouped gemm: need K-major A, one [N,K] or [K,N] matrix per group and K %% %d == 0", BK);
      return -2;
    }
    if (red_grouped && (A_MN != 1 || B_MN != 1 || M % BM != 0)) {
      pico_host::set_error("reduction-grouped gemm: need MN-major A and B and M %% %d == 0", BM);
      return -2;
    }
  }
  const int b_rows_total = row_grouped ? pc->num_groups * pc->b_group_rows : (B_MN == 0 ? N : K);
  if (B_MN == 0)
    rc = pico_host::make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, b_rows_total, (uint64_t)ldb * 2,
                                 64, BN, Swizzle::B128);
  else
    rc = pico_host::make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, b_rows_total, (uint64_t)ldb * 2,
                                 64, 64, Swizzle::B128);
  if (rc) return rc;
  const bool scatter = pc && pc->d_num_dest > 0;
  const bool gather = pc && pc->a_flags != nullptr;
  const int num_dest = scatter ? pc->d_num_dest : 1;
  if (num_dest > PICO_MAX_PEERS) {
    pico_host::set_error("gemm: %d destinations exceed the maximum of %d", num_dest, PICO_MAX_PEERS);
    return -2;
  }
  if (scatter || gather) {
    const int nb = pc->num_blocks;
    if (A_MN != 0 || pc->blk_rows <= 0 || pc->blk_rows % BM != 0 || nb < 1 || nb > PICO_MAX_PEERS ||
        M % (pc->blk_rows * nb) != 0 || (scatter && nb != num_dest) || (scatter && gather) ||
        pc->first_block < 0 || pc->first_block >= nb) {
      pico_host::set_error("collective gemm: need K-major A, pieces of a multiple of %d rows, M (%d) = pieces x "
                           "blocks (%d) x %d rows, and one direction per launch", BM, M, nb, pc->blk_rows);
      return -2;
    }
    comm.blk_rows = pc->blk_rows;
    comm.num_blocks = nb;
    comm.first_block = pc->first_block;
    comm.scatter = scatter ? 1 : 0;
  }
  const int d_rows = scatter ? M / num_dest : (red_grouped ? pc->num_groups * M : M);
  for (int b = 0; b < num_dest; ++b) {
    void* dptr = (pc && pc->d_num_dest > 0) ? pc->d_ptrs[b] : D;
    if (OUT == OUT_BF16)
      rc = pico_host::make_tmap_2d(&dm.m[b], dptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, d_rows,
                                   (uint64_t)ldd * 2, 64, BM, Swizzle::B128);
    else
      rc = pico_host::make_tmap_2d(&dm.m[b], dptr, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, N, d_rows,
                                   (uint64_t)ldd * 4, 32, BM, Swizzle::B128);
    if (rc) return rc;
  }
  for (int b = num_dest; b < PICO_MAX_PEERS; ++b) dm.m[b] = dm.m[0];
  if (gather) {
    comm.a_flags = pc->a_flags;
    comm.a_slot = pc->a_slot;
    comm.a_epoch = pc->a_epoch;
    comm.a_skip_block = pc->a_skip_block;
  }
  if (pc) {
    comm.timeout_ns = (unsigned long long)pc->timeout_ms * 1000000ull;
    comm.tile_group = pc->tile_group;
    comm.b_group_rows = pc->b_group_rows;
    comm.seg_start = pc->seg_start;
    comm.num_groups = pc->num_groups;
  }

  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, OUT>;
  static bool attr_set = false;  // per template instantiation
  static int attr_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set || attr_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
    if (e != cudaSuccess) {
      pico_host::set_error("cudaFuncSetAttribute(smem=%d): %s", Cfg::kSmemBytes,
                           cudaGetErrorString(e));
      return (int)e;
    }
    attr_set = true;
    attr_dev = dev;
  }
  const int num_tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * (red_grouped ? pc->num_groups : 1);
  int ctas = pico_host::num_sms();
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  if (num_tiles < ctas) ctas = num_tiles;
  kern<<<ctas, kNumThreads, Cfg::kSmemBytes, stream>>>(ta, tb, dm, comm, M, N, K, pico_status_buffer());
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    pico_host::set_error("gemm launch: %s", cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

template <int BN>
static int dispatch_bn(const void* A, const void* B, void* D, int M, int N, int K, int lda, int ldb,
                       int ldd, int a_mn, int b_mn, int out_mode, int max_ctas, const PicoGemmComm* pc,
                       cudaStream_t st) {
#define PICO_CASE(AM, BMJ, OM)                                                                   \
  if (a_mn == AM && b_mn == BMJ && out_mode == OM)                                               \
    return launch<BN, AM, BMJ, OM>(A, B, D, M, N, K, lda, ldb, ldd, max_ctas, pc, st);
  PICO_CASE(0, 0, OUT_BF16)
  PICO_CASE(0, 1, OUT_BF16)
  PICO_CASE(1, 1, OUT_BF16)
  PICO_CASE(1, 0, OUT_BF16)
  PICO_CASE(0, 0, OUT_F32)
  PICO_CASE(0, 1, OUT_F32)
  PICO_CASE(1, 1, OUT_F32)
  PICO_CASE(1, 1, OUT_F32_ACC)
  PICO_CASE(0, 0, OUT_F32_ACC)
#undef PICO_CASE
  pico_host::set_error("unsupported gemm variant a_mn=%d b_mn=%d out=%d", a_mn, b_mn, out_mode);
  return -10;
}

}  // namespace pico

extern "C" int pico_gemm_bf16_ex(const void* A, const void* B, void* D, int M, int N, int K, int lda,
                                 int ldb, int ldd, int a_mn_major, int b_mn_major, int out_mode,
                                 int max_ctas, const PicoGemmComm* comm, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  // Narrow outputs waste less of the tile with a smaller BN.
  if (N <= 64)
    return pico::dispatch_bn<64>(A, B, D, M, N, K, lda, ldb, ldd, a_mn_major, b_mn_major, out_mode,
                                 max_ctas, comm, stream);
  // ... and so do problems with no more 128 x 128 tiles than the device has SMs (one wave either way).
  if (N <= 128 || ((N + 127) / 128) * ((M + 127) / 128) <= pico_host::num_sms())
    return pico::dispatch_bn<128>(A, B, D, M, N, K, lda, ldb, ldd, a_mn_major, b_mn_major,
                                  out_mode, max_ctas, comm, stream);
  return pico::dispatch_bn<256>(A, B, D, M, N, K, lda, ldb, ldd, a_mn_major, b_mn_major, out_mode,
                                max_ctas, comm, stream);
}

extern "C" int pico_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, int lda,
                              int ldb, int ldd, int a_mn_major, int b_mn_major, int out_mode,
                              int max_ctas, cudaStream_t stream) {
  return pico_gemm_bf16_ex(A, B, D, M, N, K, lda, ldb, ldd, a_mn_major, b_mn_major, out_mode,
                           max_ctas, nullptr, stream);
}
