#include "tp_comm.h"

#include <cuda_bf16.h>

#include "../common/host.h"
#include "../elementwise/norm_kernels.cuh"
#include "../runtime/flags.cuh"

namespace pico {

__global__ void push_rows_kernel(const uint4* __restrict__ src, PicoPeerTable dst, PicoPeerTable flags,
                                 int world, int my_rank, int num_pieces, int64_t nvec_piece, int slot,
                                 uint32_t epoch, unsigned int* counter, int skip_self) {
  // piece p of the source (nvec_piece vectors) is piece p * world + my_rank of the destination.
  // (Reporting the pieces one by one, each behind a grid-wide rendezvous, was measured slower than
  // one pass over everything with a single flag at the end: 286 vs 271 ms per step at 4 GPUs.)
  const int64_t nvec = (int64_t)num_pieces * nvec_piece;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec;
       i += (int64_t)gridDim.x * blockDim.x) {
    const uint4 v = src[i];
    const int64_t p = i / nvec_piece;
    const int64_t o = (p * world + my_rank) * nvec_piece + (i - p * nvec_piece);
    if (skip_self == 2) {
      reinterpret_cast<uint4*>(dst.ptr[my_rank])[o] = v;
    } else {
      for (int r = 0; r < world; ++r)
        if (!(skip_self && r == my_rank)) reinterpret_cast<uint4*>(dst.ptr[r])[o] = v;
    }
  }
  if (skip_self != 2) raise_flags_when_grid_done(counter, flags, world, my_rank, slot, epoch);
}

// Block o of src goes into slot `my_rank` of rank o's staging buffer, for o < num_dst; the flag is
// raised on every rank of the group (also on those that received nothing), so all ranks stay in
// step with the epoch protocol.
__global__ void scatter_rows_kernel(const uint4* __restrict__ src, PicoPeerTable dst, PicoPeerTable flags,
                                    int world, int my_rank, int num_dst, int64_t nvec_block, int64_t nvec_piece,
                                    int slot, uint32_t epoch, unsigned int* counter) {
  // the source is a sequence of pieces (nvec_piece vectors); piece p goes to destination
  // p % num_dst as that destination's (p / num_dst)-th piece
  const int64_t total = (int64_t)num_dst * nvec_block;
  const int64_t base = (int64_t)my_rank * nvec_block;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t p = i / nvec_piece;
    const int o = (int)(p % num_dst);
    const int64_t j = (p / num_dst) * nvec_piece + (i - p * nvec_piece);
    reinterpret_cast<uint4*>(dst.ptr[o])[base + j] = src[i];
  }
  raise_flags_when_grid_done(counter, flags, world, my_rank, slot, epoch);
}

__global__ void slot_sum_kernel(const uint4* __restrict__ staging, int world, int first_slot, int64_t nvec,
                                const uint4* __restrict__ addend, uint4* __restrict__ out,
                                const uint32_t* local_flags, int slot, uint32_t epoch,
                                uint64_t timeout_ns, int* status) {
  if (!wait_slot_all(local_flags, slot, world, epoch, timeout_ns, status, 700)) return;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec;
       i += (int64_t)gridDim.x * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = first_slot; s < world; ++s) {
      float f[8];
      unpack8(staging[(int64_t)s * nvec + i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    if (addend) {
      float f[8];
      unpack8(addend[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    out[i] = pack8(acc);
  }
}

constexpr int kMaxDev = 64;
unsigned int* g_counters[kMaxDev] = {nullptr};

// One zero-initialised word per device for the "last CTA" detection; created on first use.
static unsigned int* grid_counter() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
  if (!g_counters[dev]) {
    unsigned int* p = nullptr;
    // words 0..63: one per kernel kind; words 64..319: one per piece of a push; words 320..575: the
    // same for pushes that leave this rank's own buffer out (they run on a stream of their own and
    // may overlap an ordinary push)
    if (cudaMalloc(&p, 576 * sizeof(unsigned int)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 576 * sizeof(unsigned int));
    g_counters[dev] = p;
  }
  return g_counters[dev];
}

}  // namespace pico

using namespace pico;

static int check_world(const char* what, int world, int slot) {
  if (world < 1 || world > PICO_MAX_PEERS || slot < 0 || slot >= PICO_FLAG_SLOTS) {
    pico_host::set_error("%s: world %d / flag slot %d out of range", what, world, slot);
    return -2;
  }
  return 0;
}

extern "C" int pico_push_rows(const void* src, PicoPeerTable dst, PicoPeerTable flags, int world,
                              int my_rank, int rows, int cols, int piece_rows, int slot, uint32_t epoch,
                              int skip_self, cudaStream_t stream) {
  if (int rc = check_world("push_rows", world, slot)) return rc;
  const int64_t n = (int64_t)rows * cols;
  if (piece_rows <= 0) piece_rows = rows;
  if (n % 8 != 0 || rows % piece_rows != 0 || ((int64_t)piece_rows * cols) % 8 != 0 || rows / piece_rows > 254) {
    pico_host::set_error("push_rows: rows*cols and piece_rows*cols must be multiples of 8, rows a multiple of "
                         "piece_rows, at most 254 pieces");
    return -2;
  }
  unsigned int* counter = grid_counter();
  if (!counter) return -1;
  const int64_t nvec_piece = (int64_t)piece_rows * cols / 8;
  int grid = (int)((n / 8 + 255) / 256);
  const int cap = pico_host::num_sms() * 4;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  push_rows_kernel<<<grid, 256, 0, stream>>>((const uint4*)src, dst, flags, world, my_rank, rows / piece_rows,
                                             nvec_piece, slot, epoch, counter + (skip_self == 1 ? 320 : 64), skip_self);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("push_rows: %s", cudaGetErrorString(e));
  return (int)e;
}

extern "C" int pico_slot_sum(const void* staging, int world, int rows, int cols, const void* addend,
                             void* out, const uint32_t* local_flags, int slot, uint32_t epoch,
                             uint32_t timeout_ms, cudaStream_t stream) {
  return pico_slot_sum_from(staging, world, 0, rows, cols, addend, out, local_flags, slot, epoch, timeout_ms,
                            stream);
}

extern "C" int pico_scatter_rows(const void* src, PicoPeerTable dst, PicoPeerTable flags, int world,
                                 int my_rank, int num_dst, int rows, int cols, int piece_rows, int slot,
                                 uint32_t epoch, cudaStream_t stream) {
  if (int rc = check_world("scatter_rows", world, slot)) return rc;
  const int64_t n = (int64_t)rows * cols;
  if (piece_rows <= 0) piece_rows = rows;
  if (n % 8 != 0 || num_dst < 0 || num_dst > world || rows % piece_rows != 0 ||
      ((int64_t)piece_rows * cols) % 8 != 0) {
    pico_host::set_error("scatter_rows: rows*cols and piece_rows*cols must be multiples of 8, rows a multiple of "
                         "piece_rows, 0 <= num_dst <= world");
    return -2;
  }
  unsigned int* counter = grid_counter();
  if (!counter) return -1;
  const int64_t nvec = n / 8;
  int grid = (int)((nvec * num_dst + 255) / 256);
  const int cap = pico_host::num_sms() * 4;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  scatter_rows_kernel<<<grid, 256, 0, stream>>>((const uint4*)src, dst, flags, world, my_rank, num_dst, nvec,
                                                (int64_t)piece_rows * cols / 8, slot, epoch, counter + 2);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("scatter_rows: %s", cudaGetErrorString(e));
  return (int)e;
}

extern "C" int pico_slot_sum_from(const void* staging, int world, int first_slot, int rows, int cols,
                                  const void* addend, void* out, const uint32_t* local_flags, int slot,
                                  uint32_t epoch, uint32_t timeout_ms, cudaStream_t stream) {
  if (int rc = check_world("slot_sum", world, slot)) return rc;
  if (first_slot < 0 || first_slot > world) {
    pico_host::set_error("slot_sum: first slot %d out of range", first_slot);
    return -2;
  }
  const int64_t n = (int64_t)rows * cols;
  if (n % 8 != 0) {
    pico_host::set_error("slot_sum: rows*cols must be a multiple of 8");
    return -2;
  }
  const int64_t nvec = n / 8;
  int grid = (int)((nvec + 255) / 256);
  const int cap = pico_host::num_sms() * 8;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  slot_sum_kernel<<<grid, 256, 0, stream>>>((const uint4*)staging, world, first_slot, nvec, (const uint4*)addend,
                                            (uint4*)out, local_flags, slot, epoch,
                                            (uint64_t)timeout_ms * 1000000ull, pico_status_buffer());
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) pico_host::set_error("slot_sum: %s", cudaGetErrorString(e));
  return (int)e;
}
