// Peer-memory runtime: symmetric buffers shared between the GPUs of one node through CUDA IPC, and
// collectives that move data with plain peer loads/stores over NVLink from inside the kernel.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

namespace mk {

constexpr int PEER_MAX = 8;            // ranks per node
constexpr int PEER_MAX_BLOCKS = 128;   // CTAs taking part in a collective
// flag area per rank: PEER_MAX_BLOCKS * (PEER_MAX + 1) unsigned ints (per-CTA arrival slots + local epoch)
constexpr size_t PEER_FLAG_BYTES = PEER_MAX_BLOCKS * (PEER_MAX + 1) * sizeof(unsigned int);

struct PeerPtrs {
  void* data[PEER_MAX];
  unsigned int* flags[PEER_MAX];
};

// cudaMalloc + zero fill + IPC handle (64 bytes)
cudaError_t peer_alloc(size_t bytes, void** ptr, char* handle64);
cudaError_t peer_open(const char* handle64, void** ptr);
cudaError_t peer_close(void* ptr);
cudaError_t peer_free(void* ptr);

// In-place sum over `world` ranks of n elements (fp32 or bf16, summed in fp32, scaled by `scale`).
// Two-shot: every rank reduces its 1/world slice from all peers, then stores the result into every peer.
// Cross-rank ordering uses per-CTA epoch flags in symmetric memory with bounded waits: a rank that does not see its
// peers within `wait_seconds` sets *err = 16 and leaves.  The limit is the tolerated skew between ranks (a slow data
// loader, a rank writing a checkpoint), not a liveness check: dead ranks are the host watchdog's business.
cudaError_t peer_allreduce(const PeerPtrs& p, int world, int rank, long long n, int is_bf16, float scale,
                           double wait_seconds, int* err, cudaStream_t s);

}  // namespace mk
