// Symmetric memory between the GPUs of one NVLink domain, and the flag primitives the fused
// compute+collective kernels synchronise with.
//
// A symmetric buffer is one cudaMalloc'd region per rank whose IPC handle has been opened by
// every peer, so a kernel on any rank can load from / store to the same offset on any other
// rank through plain pointers (NVLink peer access). Kernels receive a PeerTable with the base
// pointer of the buffer on every rank of the group.
//
// Flags are 32-bit epoch counters in a symmetric buffer: slot s of rank r holds one word per
// source rank. A rank signals by storing a new, larger epoch into its own word on every peer
// (release, system scope); a consumer waits (acquire, system scope, bounded) until the words it
// needs reach the epoch. Epochs only grow, so flags are never cleared.
//
// The flag buffer of a rank is PICO_FLAG_BYTES long: the flag words, then one "epoch base" word
// per slot. Every kernel adds the base word of its slot (read from its own rank's buffer) to the
// epoch it is launched with. Outside CUDA graphs the host keeps a mirror of the base and passes
// the difference, so nothing changes; a captured graph ends with pico_epoch_base_add, which moves
// the base past the epochs the graph used, so the same graph can be replayed any number of times.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define PICO_MAX_PEERS 8
#define PICO_FLAG_SLOTS 256
#define PICO_FLAG_BYTES ((PICO_FLAG_SLOTS * PICO_MAX_PEERS + PICO_FLAG_SLOTS) * 4)
#define PICO_MAX_EPOCH_DELTAS 256

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
  void* ptr[PICO_MAX_PEERS];
} PicoPeerTable;

typedef struct {
  int n;
  int slot[PICO_MAX_EPOCH_DELTAS];
  uint32_t delta[PICO_MAX_EPOCH_DELTAS];
} PicoEpochDeltas;

// cudaMalloc `bytes` (zero-filled) and export its IPC handle (64 bytes).
int pico_symm_alloc(size_t bytes, void** ptr, unsigned char* handle64);
// Map a peer's buffer into this process. The pointer stays valid until pico_symm_close.
int pico_symm_open(const unsigned char* handle64, void** ptr);
int pico_symm_close(void* ptr);
int pico_symm_free(void* ptr);

// Store `epoch` into word [slot][my_rank] of the flag buffer of every rank in `flags`.
int pico_signal_peers(PicoPeerTable flags, int world, int my_rank, int slot, uint32_t epoch,
                      cudaStream_t stream);
// Wait until words [slot][src] of the local flag buffer are >= epoch for every src in
// [0, world). Gives up after timeout_ms (error code 2 in the status words); returns normally.
int pico_wait_flags(const uint32_t* local_flags, int world, int slot, uint32_t epoch,
                    uint32_t timeout_ms, cudaStream_t stream);

// base[slot[i]] += delta[i] in the epoch-base words of this rank's flag buffer (stream ordered).
int pico_epoch_base_add(uint32_t* local_flags, const PicoEpochDeltas* deltas, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
