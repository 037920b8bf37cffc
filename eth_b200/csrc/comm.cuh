// Peer-memory substrate and fused communication kernels (see comm.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ethb {

constexpr int kMaxPeers = 8;

// Pointers of one symmetric allocation as seen from this process: ptrs[r] is rank r's copy.
struct PeerPtrs {
  void* ptrs[kMaxPeers];
};

// ---- symmetric allocation through CUDA IPC -----------------------------------------------
// Allocates `bytes` with cudaMalloc (zero-filled) and returns the 64-byte IPC handle in `handle`.
cudaError_t peer_alloc(size_t bytes, void** ptr, unsigned char handle[64]);
cudaError_t peer_open(const unsigned char handle[64], void** ptr);
cudaError_t peer_close(void* ptr);
cudaError_t peer_free(void* ptr);

// ---- cross-GPU barrier over a flag array ------------------------------------------------------
// flags: symmetric int32 [world] per rank. Rank r writes `epoch` into flags[peer][r] on every peer
// and waits until its own flags[*] all reached `epoch`. Bounded; reports through `status`.
cudaError_t peer_barrier(const PeerPtrs& flags, int rank, int world, int epoch, int* status,
                         cudaStream_t st);

// ---- one-shot all-reduce of a symmetric buffer, optionally fused with the optimizer ------------
struct ReduceArgs {
  PeerPtrs bufs;        // symmetric gradient buckets (each rank's own packed bucket)
  PeerPtrs flags;       // symmetric int32 [world] arrival flags
  int rank, world;
  int epoch;            // strictly increasing per use of `flags`
  int64_t n;            // elements
  int dtype;            // element type of the buckets
  float scale;          // multiply the sum by this (gradient normalisation)
  void* out;            // reduced result, local (may alias bufs.ptrs[rank]); dtype out_dtype
  int out_dtype;
  float* norm_acc;      // optional: [0] += sum(out^2), [1] = non-finite flag
  float norm_weight;    // weight applied to this bucket's sum of squares (0 to skip)
  int* status;
};
cudaError_t peer_allreduce(const ReduceArgs& a, cudaStream_t st);

}  // namespace ethb
