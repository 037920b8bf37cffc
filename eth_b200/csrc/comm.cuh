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

// ---- two-shot in-place all-reduce of gradient pieces, without device-side waiting ---------------
// The gradients of a bucket are a list of pieces (rows x run elements, row stride `stride`, at
// element offset `off`) that sit at the SAME offsets in every rank's symmetric gradient buffer.
// Rank r sums, for its 1 / world share of every piece, the values of all ranks (peer loads, fp32,
// rank order), scales, and stores the result into every rank's buffer (peer stores): a
// reduce-scatter followed by an all-gather that uses both NVLink directions and never packs.
// The kernel itself waits for nobody. Synchronisation is done by `peer_flags`, a one-warp kernel
// small enough to share an SM with a resident GEMM CTA, so that a rank waiting for a peer does
// not keep compute kernels off the SMs:
//   peer_flags(signal arrive, wait arrive)  ->  peer_reduce_pieces (ends with signal done)
//   ... and before the gradients are consumed:  peer_flags(wait done).
// Flag block of one process group (int32, symmetric): [0, 8) arrive, [8, 16) done, [16] counter.
constexpr int kFlagArrive = 0;
constexpr int kFlagDone = kMaxPeers;
constexpr int kFlagCounter = 2 * kMaxPeers;
struct PieceReduceArgs {
  PeerPtrs bases;          // per rank: address that piece offsets are relative to
  PeerPtrs flags;          // per rank: the group's flag block
  const int64_t* pieces;   // device, [num_pieces][4] = element offset, rows, run, stride (run % 8 == 0)
  int num_pieces;
  int rank, world, epoch;
  int dtype;               // kF32 / kF16 / kBF16
  float scale;
};
cudaError_t peer_reduce_pieces(const PieceReduceArgs& a, cudaStream_t st);
// signal_base / wait_base: flag offset (kFlagArrive / kFlagDone) or -1 to skip that half.
cudaError_t peer_flags(const PeerPtrs& flags, int rank, int world, int epoch, int signal_base,
                       int wait_base, int* status, cudaStream_t st);

// ---- pipeline transfers through peer memory ---------------------------------------------------
// A stage boundary moves rectangles of activations (or gradients) from the ranks of one stage into
// ring slots that the ranks of the next stage own. The payload travels as 2-D device-to-device
// copies on a copy stream (`peer_copy_2d`: rows x width bytes, independent pitches), so no SM takes
// part; afterwards the sender posts the micro-batch's sequence number to one flag per receiver
// (`flags_post`, ordered behind the copies by the stream), and the receiver's compute stream waits
// on its flags with a one-warp kernel (`flags_wait`, bounded: `limit_scale` times the wait limit)
// before the first kernel that reads the slot.
struct FlagList {
  int* ptrs[2 * kMaxPeers];   // flag words, in this process' address space (local or peer-mapped)
  int count;
};
cudaError_t peer_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                         size_t rows, cudaStream_t st);
cudaError_t flags_post(const FlagList& flags, int value, cudaStream_t st);
cudaError_t flags_wait(const FlagList& flags, int value, int limit_scale, int* status, cudaStream_t st);

}  // namespace ethb
