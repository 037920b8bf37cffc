// Peer-memory substrate: symmetric buffers exchanged through CUDA IPC handles, a bounded
// cross-GPU flag barrier, and a one-shot all-reduce kernel over peer pointers that fuses the
// gradient normalisation, the dtype cast and the squared-norm / non-finite reduction that the
// optimizer needs. All device-side waits are bounded and report through a status word.
//
// Flag array layout (int32, symmetric, zero-initialised), W = world size:
//   [0, W)     arrival flags   - flags[r] on rank q is written by rank r
//   [W, 2W)    release flags   - same, for "I have finished reading your buffer"
//   [2W]       local block counter
#include "comm.cuh"
#include "gemm_sm100.cuh"
#include "sm100_common.cuh"

namespace ethb {

cudaError_t peer_alloc(size_t bytes, void** ptr, unsigned char handle[64]) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return e;
  e = cudaMemset(*ptr, 0, bytes);
  if (e != cudaSuccess) return e;
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, *ptr);
  if (e != cudaSuccess) return e;
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle, &h, 64);
  return cudaDeviceSynchronize();
}
cudaError_t peer_open(const unsigned char handle[64], void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}
cudaError_t peer_close(void* ptr) { return cudaIpcCloseMemHandle(ptr); }
cudaError_t peer_free(void* ptr) { return cudaFree(ptr); }

namespace {

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Spin until *p >= target; false (and status set) on timeout.
__device__ __forceinline__ bool wait_flag_ge(const int* p, int target, int* status) {
  if (ld_acquire_sys(p) >= target) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (ld_acquire_sys(p) < target) {
    if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > ETHB_WAIT_NS) {
      if (status) atomicCAS(status, 0, kStatusTimeoutPeerFlag);
      return false;
    }
  }
  return true;
}

__global__ void __launch_bounds__(32, 1) flags_post_kernel(FlagList flags, int value) {
  if (threadIdx.x < flags.count) {
    __threadfence_system();
    st_release_sys(flags.ptrs[threadIdx.x], value);
  }
}

// Waits up to `limit_scale` wait limits per flag; the first flag that gives up records the status.
__global__ void __launch_bounds__(32, 1) flags_wait_kernel(FlagList flags, int value, int limit_scale, int* status) {
  if (threadIdx.x >= flags.count) return;
  for (int round = 0; round < limit_scale; ++round)
    if (wait_flag_ge(flags.ptrs[threadIdx.x], value, round + 1 == limit_scale ? status : nullptr)) return;
}

__global__ void peer_barrier_kernel(PeerPtrs flags, int rank, int world, int epoch, int* status) {
  const int p = threadIdx.x;
  if (p < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<int*>(flags.ptrs[p]) + rank, epoch);
    wait_flag_ge(reinterpret_cast<const int*>(flags.ptrs[rank]) + p, epoch, status);
  }
}

template <typename T>
__device__ __forceinline__ void ld8(const T* p, float (&f)[8]) {
  if constexpr (sizeof(T) == 2) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    const T* h = reinterpret_cast<const T*>(&u);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = HalfTraits<T>::to_f(h[i]);
  } else {
    float4 a = reinterpret_cast<const float4*>(p)[0];
    float4 b = reinterpret_cast<const float4*>(p)[1];
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
}
template <typename T>
__device__ __forceinline__ void st8(T* p, const float (&f)[8]) {
  if constexpr (sizeof(T) == 2) {
    uint4 u;
    T* h = reinterpret_cast<T*>(&u);
#pragma unroll
    for (int i = 0; i < 8; ++i) h[i] = HalfTraits<T>::from_f(f[i]);
    *reinterpret_cast<uint4*>(p) = u;
  } else {
    reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
  }
}

// One-shot all-reduce: every rank pulls every peer's bucket through NVLink, sums in fp32 in a
// fixed rank order (so all ranks produce bit-identical results), scales, casts and stores
// locally, and accumulates the squared norm of what it stored.
template <typename T, typename O>
__global__ void peer_allreduce_kernel(ReduceArgs a) {
  __shared__ float red[32];
  __shared__ int ok_s;
  int* my_flags = reinterpret_cast<int*>(a.flags.ptrs[a.rank]);
  const int W = a.world;
  // ---- arrival: my bucket is complete (stream order); tell every peer, then wait for all.
  if (blockIdx.x == 0 && threadIdx.x < W) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<int*>(a.flags.ptrs[threadIdx.x]) + a.rank, a.epoch);
  }
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < W) {
    if (!wait_flag_ge(my_flags + threadIdx.x, a.epoch, a.status)) ok_s = 0;
  }
  __syncthreads();
  float ssq = 0.f;
  bool bad = false;
  if (ok_s) {
    const int64_t nvec = a.n >> 3;
    O* out = reinterpret_cast<O*>(a.out);
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int r = 0; r < W; ++r) {
        float v[8];
        ld8(reinterpret_cast<const T*>(a.bufs.ptrs[r]) + i * 8, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += v[j];
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        acc[j] *= a.scale;
        bad |= !isfinite(acc[j]);
        ssq += acc[j] * acc[j];
      }
      st8(out + i * 8, acc);
    }
    // tail (n not a multiple of 8)
    for (int64_t i = (nvec << 3) + blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
         i < a.n; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
      float s = 0.f;
      for (int r = 0; r < W; ++r)
        s += HalfTraits<T>::to_f(reinterpret_cast<const T*>(a.bufs.ptrs[r])[i]);
      s *= a.scale;
      bad |= !isfinite(s);
      ssq += s * s;
      out[i] = HalfTraits<O>::from_f(s);
    }
  }
  if (a.norm_acc) {
    // block reduction of ssq
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
    if (lane == 0) red[warp] = ssq;
    __syncthreads();
    if (warp == 0) {
      float r = lane < nw ? red[lane] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
      if (lane == 0 && a.norm_weight != 0.f) atomicAdd(a.norm_acc, r * a.norm_weight);
    }
    if (bad) a.norm_acc[1] = 1.0f;
  }
  // ---- release: the last block of this rank tells every peer that their buckets are no longer
  // being read here, then waits for the same from all peers, so that when this kernel has
  // finished on a rank, nobody reads that rank's bucket any more.
  __syncthreads();
  __shared__ int last_s;
  if (threadIdx.x == 0) {
    __threadfence();
    const int done = atomicAdd(my_flags + 2 * W, 1);
    last_s = (done == static_cast<int>(gridDim.x) - 1);
  }
  __syncthreads();
  if (last_s) {
    if (threadIdx.x == 0) my_flags[2 * W] = 0;
    if (threadIdx.x < W) {
      __threadfence_system();
      st_release_sys(reinterpret_cast<int*>(a.flags.ptrs[threadIdx.x]) + W + a.rank, a.epoch);
      wait_flag_ge(my_flags + W + threadIdx.x, a.epoch, a.status);
    }
  }
}

// One warp: optionally tell every peer `epoch` at flags[peer][signal_base + rank], optionally wait
// (bounded) until flags[rank][wait_base + p] >= epoch for every p.
__global__ void __launch_bounds__(32, 1)
peer_flags_kernel(PeerPtrs flags, int rank, int world, int epoch, int signal_base, int wait_base, int* status) {
  const int p = threadIdx.x;
  if (p >= world) return;
  if (signal_base >= 0) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<int*>(flags.ptrs[p]) + signal_base + rank, epoch);
  }
  if (wait_base >= 0)
    wait_flag_ge(reinterpret_cast<const int*>(flags.ptrs[rank]) + wait_base + p, epoch, status);
}

template <typename T>
__global__ void __launch_bounds__(256)
peer_reduce_pieces_kernel(PieceReduceArgs a) {
  const int W = a.world;
  const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t nthr = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int j = 0; j < a.num_pieces; ++j) {
    const int64_t off = a.pieces[j * 4 + 0], rows = a.pieces[j * 4 + 1];
    const int64_t run = a.pieces[j * 4 + 2], stride = a.pieces[j * 4 + 3];
    const int64_t vpr = run >> 3;                 // 8-element vectors per row
    const int64_t nvec = rows * vpr;
    const int64_t per = (nvec + W - 1) / W;       // this rank's share of the piece
    const int64_t lo = a.rank * per;
    const int64_t hi = lo + per < nvec ? lo + per : nvec;
    for (int64_t i = lo + tid; i < hi; i += nthr) {
      const int64_t row = i / vpr;
      const int64_t e = off + row * stride + (i - row * vpr) * 8;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int r = 0; r < W; ++r) {
        float v[8];
        ld8(reinterpret_cast<const T*>(a.bases.ptrs[r]) + e, v);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] += v[k];
      }
      if (a.scale != 1.0f) {
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] *= a.scale;
      }
      for (int d = 0; d < W; ++d) st8(reinterpret_cast<T*>(a.bases.ptrs[d]) + e, acc);
    }
  }
  // the last block to finish publishes "my share is in your buffer, and I no longer read yours"
  __shared__ int last_s;
  int* my_flags = reinterpret_cast<int*>(a.flags.ptrs[a.rank]);
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int done = atomicAdd(my_flags + kFlagCounter, 1);
    last_s = (done == static_cast<int>(gridDim.x) - 1);
  }
  __syncthreads();
  if (last_s) {
    if (threadIdx.x == 0) my_flags[kFlagCounter] = 0;
    if (threadIdx.x < W) {
      __threadfence_system();
      st_release_sys(reinterpret_cast<int*>(a.flags.ptrs[threadIdx.x]) + kFlagDone + a.rank, a.epoch);
    }
  }
}

}  // namespace

cudaError_t peer_flags(const PeerPtrs& flags, int rank, int world, int epoch, int signal_base,
                       int wait_base, int* status, cudaStream_t st) {
  if (world > kMaxPeers || world < 1) return cudaErrorInvalidValue;
  peer_flags_kernel<<<1, 32, 0, st>>>(flags, rank, world, epoch, signal_base, wait_base, status);
  count_launch();
  return cudaGetLastError();
}

cudaError_t peer_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                         size_t rows, cudaStream_t st) {
  if (rows == 0 || width_bytes == 0) return cudaSuccess;
  if (width_bytes > dst_pitch || width_bytes > src_pitch) return cudaErrorInvalidValue;
  if (rows == 1 || (dst_pitch == width_bytes && src_pitch == width_bytes))
    return cudaMemcpyAsync(dst, src, width_bytes * rows, cudaMemcpyDeviceToDevice, st);
  return cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, cudaMemcpyDeviceToDevice, st);
}

cudaError_t flags_post(const FlagList& flags, int value, cudaStream_t st) {
  if (flags.count < 1 || flags.count > 2 * kMaxPeers) return cudaErrorInvalidValue;
  flags_post_kernel<<<1, 32, 0, st>>>(flags, value);
  count_launch();
  return cudaGetLastError();
}

cudaError_t flags_wait(const FlagList& flags, int value, int limit_scale, int* status, cudaStream_t st) {
  if (flags.count < 1 || flags.count > 2 * kMaxPeers || limit_scale < 1 || limit_scale > 64) return cudaErrorInvalidValue;
  flags_wait_kernel<<<1, 32, 0, st>>>(flags, value, limit_scale, status);
  count_launch();
  return cudaGetLastError();
}

cudaError_t peer_reduce_pieces(const PieceReduceArgs& a, cudaStream_t st) {
  if (a.world > kMaxPeers || a.world < 1 || a.num_pieces <= 0 || a.pieces == nullptr) return cudaErrorInvalidValue;
  // enough blocks to keep NVLink busy in both directions, few enough to leave SMs to compute kernels
  const int grid = 148 * 2;
  if (a.dtype == kBF16) peer_reduce_pieces_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(a);
  else if (a.dtype == kF16) peer_reduce_pieces_kernel<__half><<<grid, 256, 0, st>>>(a);
  else if (a.dtype == kF32) peer_reduce_pieces_kernel<float><<<grid, 256, 0, st>>>(a);
  else return cudaErrorInvalidValue;
  count_launch();
  return cudaGetLastError();
}

cudaError_t peer_barrier(const PeerPtrs& flags, int rank, int world, int epoch, int* status,
                         cudaStream_t st) {
  if (world > kMaxPeers) return cudaErrorInvalidValue;
  peer_barrier_kernel<<<1, 32, 0, st>>>(flags, rank, world, epoch, status);
  count_launch();
  return cudaGetLastError();
}

cudaError_t peer_allreduce(const ReduceArgs& a, cudaStream_t st) {
  if (a.world > kMaxPeers || a.world < 1 || a.n <= 0) return cudaErrorInvalidValue;
  int64_t blocks = (a.n / 8 + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  if (blocks < 1) blocks = 1;
  const int grid = static_cast<int>(blocks);
#define ETHB_AR(T, O) peer_allreduce_kernel<T, O><<<grid, 256, 0, st>>>(a)
  if (a.dtype == kBF16) {
    if (a.out_dtype == kBF16) ETHB_AR(__nv_bfloat16, __nv_bfloat16);
    else if (a.out_dtype == kF32) ETHB_AR(__nv_bfloat16, float);
    else return cudaErrorInvalidValue;
  } else if (a.dtype == kF16) {
    if (a.out_dtype == kF16) ETHB_AR(__half, __half);
    else if (a.out_dtype == kF32) ETHB_AR(__half, float);
    else return cudaErrorInvalidValue;
  } else {
    if (a.out_dtype == kF32) ETHB_AR(float, float);
    else return cudaErrorInvalidValue;
  }
#undef ETHB_AR
  count_launch();
  return cudaGetLastError();
}

}  // namespace ethb
