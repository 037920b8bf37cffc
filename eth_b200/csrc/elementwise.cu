// Bandwidth-bound kernels of the GPT stage program. All use 128-bit accesses, fp32 math and
// grids sized against the 148 SMs of a B200; none of them allocates.
#include "elementwise.cuh"
#include "gemm_sm100.cuh"
#include "sm100_common.cuh"

namespace ethb {
namespace {

constexpr int kSMs = 148;

template <typename T> struct Vec8 {  // 8 x 16-bit = 16 bytes, or 8 x fp32 = 32 bytes
  T v[8];
};
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]) {
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
__device__ __forceinline__ void store8(T* p, const float (&f)[8]) {
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

// 8 packed 16-bit values held in a register quad -> floats (the fused LayerNorm backward keeps rows
// packed between its two phases). Only meaningful for 16-bit T.
template <typename T>
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  if constexpr (sizeof(T) == 2) {
    const T* h = reinterpret_cast<const T*>(&u);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = HalfTraits<T>::to_f(h[i]);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = 0.f;
  }
}

// Eight elements as they sit in memory: 4 registers for 16-bit types, 8 for fp32.
template <typename T, int N>
__device__ __forceinline__ void load_raw8(const T* p, float (&raw)[N]) {
  if constexpr (sizeof(T) == 2) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    raw[0] = __uint_as_float(u.x); raw[1] = __uint_as_float(u.y);
    raw[2] = __uint_as_float(u.z); raw[3] = __uint_as_float(u.w);
  } else {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    raw[0] = a.x; raw[1] = a.y; raw[2] = a.z; raw[3] = a.w;
    raw[4] = b.x; raw[5] = b.y; raw[6] = b.z; raw[7] = b.w;
  }
}
template <typename T, int N>
__device__ __forceinline__ void unpack_raw8(const float (&raw)[N], float (&f)[8]) {
  if constexpr (sizeof(T) == 2) {
    unpack8<T>(make_uint4(__float_as_uint(raw[0]), __float_as_uint(raw[1]), __float_as_uint(raw[2]),
                          __float_as_uint(raw[3])), f);
  } else {
#pragma unroll
    for (int q = 0; q < 8; ++q) f[q] = raw[q];
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum; `red` is a 32-float shared buffer. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = (lane < nw) ? red[lane] : 0.f;
  return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = (lane < nw) ? red[lane] : -INFINITY;
  return warp_max(r);
}

#define ETHB_DISPATCH(dtype, T, ...)                                  \
  do {                                                                 \
    if ((dtype) == kBF16) { using T = __nv_bfloat16; __VA_ARGS__; }    \
    else if ((dtype) == kF16) { using T = __half; __VA_ARGS__; }       \
    else { using T = float; __VA_ARGS__; }                             \
  } while (0)

// =============================================================================================
// LayerNorm
// =============================================================================================
// One CTA per row; each thread keeps ITERS 8-element slices of the row in registers.
template <typename T, int kLnMaxIter>
__global__ void ln_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gamma,
                              const T* __restrict__ beta, T* __restrict__ y,
                              float* __restrict__ mean, float* __restrict__ rstd, int rows,
                              int hidden, float eps) {
  __shared__ float red[32];
  const int nvec = hidden >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + static_cast<int64_t>(row) * hidden;
    float v[kLnMaxIter][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kLnMaxIter; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < nvec) {
        load8(xr + c * 8, v[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) s += v[i][j];
      }
    }
    const float mu = block_sum(s, red) / hidden;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < kLnMaxIter; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { float d = v[i][j] - mu; q += d * d; }
      }
    }
    const float rs = rsqrtf(block_sum(q, red) / hidden + eps);
    if (threadIdx.x == 0) { mean[row] = mu; rstd[row] = rs; }
    T* yr = y + static_cast<int64_t>(row) * hidden;
#pragma unroll
    for (int i = 0; i < kLnMaxIter; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < nvec) {
        float g[8], b[8], o[8];
        load8(gamma + c * 8, g);
        load8(beta + c * 8, b);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mu) * rs * g[j] + b[j];
        store8(yr + c * 8, o);
      }
    }
  }
}

// Warp-per-row forward for 16-bit rows of 256 * VPL elements (VPL <= 16). A lane keeps VPL 16-byte
// pieces of the row packed in registers (lane l owns pieces l, l + 32, ...: a warp reads 512
// contiguous bytes per instruction), so mean and variance need only warp shuffles: no block barrier
// sits between a row's load and its store, and with 8 independent warps per CTA the loads of some
// rows always overlap the arithmetic of others. gamma / beta (a few KB) are re-read per row: they stay
// in L1, and keeping them out of the register file lets two CTAs (16 warps) share an SM.
template <typename T, int VPL>
__global__ void __launch_bounds__(256, VPL > 8 ? 1 : 2)
ln_fwd_warp_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                   T* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd, int rows,
                   float eps) {
  constexpr int kHidden = VPL * 256;
  const int lane = threadIdx.x & 31;
  const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int nwarps = gridDim.x * (blockDim.x >> 5);
  // A warp walks its rows with the next row's loads already in flight while it reduces and stores
  // the current one (the grid is two CTAs per SM, not one warp per row).
  uint4 raw[VPL], nxt[VPL];
  if (warp < rows) {
    const T* xr = x + static_cast<int64_t>(warp) * kHidden;
#pragma unroll
    for (int i = 0; i < VPL; ++i) nxt[i] = *reinterpret_cast<const uint4*>(xr + (lane + 32 * i) * 8);
  }
  for (int row = warp; row < rows; row += nwarps) {
#pragma unroll
    for (int i = 0; i < VPL; ++i) raw[i] = nxt[i];
    if (row + nwarps < rows) {
      const T* xn = x + static_cast<int64_t>(row + nwarps) * kHidden;
#pragma unroll
      for (int i = 0; i < VPL; ++i) nxt[i] = *reinterpret_cast<const uint4*>(xn + (lane + 32 * i) * 8);
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      float v[8];
      unpack8<T>(raw[i], v);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += v[j];
    }
    const float mu = warp_sum(s) * (1.0f / kHidden);
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      float v[8];
      unpack8<T>(raw[i], v);
#pragma unroll
      for (int j = 0; j < 8; ++j) { const float d = v[j] - mu; q += d * d; }
    }
    const float rs = rsqrtf(warp_sum(q) * (1.0f / kHidden) + eps);
    if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
    T* yr = y + static_cast<int64_t>(row) * kHidden;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      float v[8], gv[8], bv[8], o[8];
      unpack8<T>(raw[i], v);
      load8(gamma + (lane + 32 * i) * 8, gv);
      load8(beta + (lane + 32 * i) * 8, bv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (v[j] - mu) * rs * gv[j] + bv[j];
      store8(yr + (lane + 32 * i) * 8, o);
    }
  }
}

// Backward. One pass over dy and x: thread t of a CTA owns columns [8t, 8t + 8) of every row the CTA
// visits (blockDim.x = hidden / 8), so the dgamma / dbeta column sums stay in registers for the
// whole kernel and dx needs only two block-wide reductions per batch of R rows (sum(dy*gamma) and
// sum(dy*gamma*xhat) of each row). A CTA keeps its R rows as packed 16-bit registers between the
// reduction and the dx pass. Each CTA writes one slab of partial column sums; reduce_parts_kernel
// adds the slabs. Rows wider than 8192 elements use the two-kernel fallback below.
template <typename T, int R>
__global__ void __launch_bounds__(R == 5 ? 256 : (R == 4 ? 512 : 1024), R == 5 ? 2 : 1)
ln_bwd_fused_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
                    const float* __restrict__ mean, const float* __restrict__ rstd,
                    const T* __restrict__ dres, T* __restrict__ dx, float* __restrict__ ws, int rows,
                    int hidden, int add_to_ws) {
  __shared__ float red[2][R][32];
  __shared__ float tot[2][R];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5, nwarps = blockDim.x >> 5;
  const int c0 = t * 8;
  float g[8];
  load8(gamma + c0, g);
  float dg[8] = {0, 0, 0, 0, 0, 0, 0, 0}, db[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int r0 = blockIdx.x * R; r0 < rows; r0 += gridDim.x * R) {
    // everything a batch needs from memory is requested up front (the residual gradient too): one
    // memory latency per batch, R * 3 independent 16-byte loads per thread in flight
    uint4 xr[R], dyr[R], rr[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int r = r0 + i;
      if (r < rows) {
        xr[i] = *reinterpret_cast<const uint4*>(x + static_cast<int64_t>(r) * hidden + c0);
        dyr[i] = *reinterpret_cast<const uint4*>(dy + static_cast<int64_t>(r) * hidden + c0);
        rr[i] = dres != nullptr ? *reinterpret_cast<const uint4*>(dres + static_cast<int64_t>(r) * hidden + c0)
                                : make_uint4(0, 0, 0, 0);
      } else {
        xr[i] = make_uint4(0, 0, 0, 0);
        dyr[i] = make_uint4(0, 0, 0, 0);
        rr[i] = make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int i = 0; i < R; ++i) {
      float xv[8], dv[8];
      unpack8<T>(xr[i], xv);
      unpack8<T>(dyr[i], dv);
      // per-row statistics are re-read where they are used (broadcast loads, L1 hits)
      const float mu_i = r0 + i < rows ? mean[r0 + i] : 0.f, rs_i = r0 + i < rows ? rstd[r0 + i] : 0.f;
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float w = dv[j] * g[j];
        s1 += w;
        s2 += w * (xv[j] - mu_i) * rs_i;
      }
      s1 = warp_sum(s1);
      s2 = warp_sum(s2);
      if (lane == 0) {
        red[0][i][warp] = s1;
        red[1][i][warp] = s2;
      }
    }
    __syncthreads();
    if (t < 2 * R) {
      const int which = t / R, i = t % R;
      float a = 0.f;
      for (int w = 0; w < nwarps; ++w) a += red[which][i][w];
      tot[which][i] = a / hidden;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int r = r0 + i;
      if (r >= rows) break;
      // The rows are unpacked again here on purpose: carrying R * 16 floats across the barrier
      // instead of R * 8 packed registers would spill. The empty asm hides the packed values'
      // provenance from the optimiser so that it cannot reuse the first unpacking.
      asm volatile("" : "+r"(xr[i].x), "+r"(xr[i].y), "+r"(xr[i].z), "+r"(xr[i].w));
      asm volatile("" : "+r"(dyr[i].x), "+r"(dyr[i].y), "+r"(dyr[i].z), "+r"(dyr[i].w));
      float xv[8], dv[8], o[8];
      unpack8<T>(xr[i], xv);
      unpack8<T>(dyr[i], dv);
      const float m1 = tot[0][i], m2 = tot[1][i];
      const float mu_i = mean[r], rs_i = rstd[r];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = (xv[j] - mu_i) * rs_i;
        o[j] = (dv[j] * g[j] - m1 - xh * m2) * rs_i;
        dg[j] += dv[j] * xh;
        db[j] += dv[j];
      }
      if (dres != nullptr) {   // gradient arriving through the residual branch
        float rv[8];
        unpack8<T>(rr[i], rv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += rv[j];
      }
      store8(dx + static_cast<int64_t>(r) * hidden + c0, o);
    }
  }
  float* wg = ws + static_cast<int64_t>(blockIdx.x) * hidden + c0;
  float* wb = ws + static_cast<int64_t>(gridDim.x + blockIdx.x) * hidden + c0;
  if (add_to_ws) {   // the slabs persist over micro-batches and are reduced once per step
    const float4 a0 = reinterpret_cast<const float4*>(wg)[0], a1 = reinterpret_cast<const float4*>(wg)[1];
    const float4 b0 = reinterpret_cast<const float4*>(wb)[0], b1 = reinterpret_cast<const float4*>(wb)[1];
    dg[0] += a0.x; dg[1] += a0.y; dg[2] += a0.z; dg[3] += a0.w;
    dg[4] += a1.x; dg[5] += a1.y; dg[6] += a1.z; dg[7] += a1.w;
    db[0] += b0.x; db[1] += b0.y; db[2] += b0.z; db[3] += b0.w;
    db[4] += b1.x; db[5] += b1.y; db[6] += b1.z; db[7] += b1.w;
  }
  *reinterpret_cast<float4*>(wg) = make_float4(dg[0], dg[1], dg[2], dg[3]);
  *reinterpret_cast<float4*>(wg + 4) = make_float4(dg[4], dg[5], dg[6], dg[7]);
  *reinterpret_cast<float4*>(wb) = make_float4(db[0], db[1], db[2], db[3]);
  *reinterpret_cast<float4*>(wb + 4) = make_float4(db[4], db[5], db[6], db[7]);
}

// Fallback for very wide rows, two kernels.
//  (1) dx: one warp per row, no block-level synchronisation. Two passes over the row: the first
//      accumulates sum(dy*gamma) and sum(dy*gamma*xhat), the second recomputes the terms (the row is
//      L1/L2 resident by then) and writes dx.
//  (2) dgamma / dbeta partials: a (32 x 8) CTA owns 256 columns and a slab of rows; each thread keeps
//      8 column sums in registers and the 8 row-lanes are combined through shared memory. A last
//      small kernel sums the slabs (reduce_parts_kernel).
template <typename T>
__global__ void ln_bwd_dx_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                 const T* __restrict__ gamma, const float* __restrict__ mean,
                                 const float* __restrict__ rstd, const T* __restrict__ dres,
                                 T* __restrict__ dx, int rows, int hidden) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int nvec = hidden >> 3;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows;
       row += gridDim.x * warps_per_block) {
    const int64_t off = static_cast<int64_t>(row) * hidden;
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
    for (int c = lane; c < nvec; c += 32) {
      float xv[8], dyv[8], g[8];
      load8(x + off + c * 8, xv);
      load8(dy + off + c * 8, dyv);
      load8(gamma + c * 8, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float w = dyv[j] * g[j];
        s1 += w;
        s2 += w * (xv[j] - mu) * rs;
      }
    }
    const float m1 = warp_sum(s1) / hidden;
    const float m2 = warp_sum(s2) / hidden;
    for (int c = lane; c < nvec; c += 32) {
      float xv[8], dyv[8], g[8], o[8];
      load8(x + off + c * 8, xv);
      load8(dy + off + c * 8, dyv);
      load8(gamma + c * 8, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (dyv[j] * g[j] - m1 - (xv[j] - mu) * rs * m2) * rs;
      if (dres != nullptr) {
        float rv[8];
        load8(dres + off + c * 8, rv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += rv[j];
      }
      store8(dx + off + c * 8, o);
    }
  }
}

template <typename T>
__global__ void ln_bwd_param_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                    const float* __restrict__ mean, const float* __restrict__ rstd,
                                    float* __restrict__ ws, int rows, int hidden) {
  __shared__ float sg[8][256 + 8];
  __shared__ float sb[8][256 + 8];
  const int c0 = (blockIdx.x * 32 + threadIdx.x) * 8;
  const int parts = gridDim.y;
  const int per = (rows + parts - 1) / parts;
  const int r0 = per * blockIdx.y, r1 = min(rows, r0 + per);
  float dg[8] = {0, 0, 0, 0, 0, 0, 0, 0}, db[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (c0 < hidden) {
    for (int r = r0 + threadIdx.y; r < r1; r += 8) {
      float xv[8], dyv[8];
      load8(x + static_cast<int64_t>(r) * hidden + c0, xv);
      load8(dy + static_cast<int64_t>(r) * hidden + c0, dyv);
      const float mu = mean[r], rs = rstd[r];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        dg[j] += dyv[j] * (xv[j] - mu) * rs;
        db[j] += dyv[j];
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    sg[threadIdx.y][threadIdx.x * 8 + j] = dg[j];
    sb[threadIdx.y][threadIdx.x * 8 + j] = db[j];
  }
  __syncthreads();
  const int t = threadIdx.y * 32 + threadIdx.x;
  const int c = blockIdx.x * 256 + t;
  if (c < hidden) {
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) { a += sg[k][t]; b += sb[k][t]; }
    ws[static_cast<int64_t>(blockIdx.y) * hidden + c] = a;
    ws[static_cast<int64_t>(parts + blockIdx.y) * hidden + c] = b;
  }
}

// out[c] (+)= sum_p ws[p, c]   for two stacked workspaces (dgamma | dbeta) or one (colsum).
// CTA = 32 columns x 8 part-lanes: each thread adds every 8th slab, shared memory adds the lanes.
template <typename G>
__global__ void reduce_parts_kernel(float* __restrict__ ws, G* __restrict__ out0,
                                    G* __restrict__ out1, int parts, int cols, int accumulate, int clear = 0) {
  __shared__ float sa[8][33], sb[8][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float a = 0.f, b = 0.f;
  if (c < cols) {
    for (int p = threadIdx.y; p < parts; p += 8) {
      a += ws[static_cast<int64_t>(p) * cols + c];
      if (out1) b += ws[static_cast<int64_t>(parts + p) * cols + c];
      if (clear) {   // persistent slabs start the next step from zero
        ws[static_cast<int64_t>(p) * cols + c] = 0.f;
        if (out1) ws[static_cast<int64_t>(parts + p) * cols + c] = 0.f;
      }
    }
  }
  sa[threadIdx.y][threadIdx.x] = a;
  sb[threadIdx.y][threadIdx.x] = b;
  __syncthreads();
  if (threadIdx.y != 0 || c >= cols) return;
#pragma unroll
  for (int k = 1; k < 8; ++k) {
    a += sa[k][threadIdx.x];
    b += sb[k][threadIdx.x];
  }
  if (accumulate) {
    a += HalfTraits<G>::to_f(out0[c]);
    if (out1) b += HalfTraits<G>::to_f(out1[c]);
  }
  out0[c] = HalfTraits<G>::from_f(a);
  if (out1) out1[c] = HalfTraits<G>::from_f(b);
}

// =============================================================================================
// bias + GeLU, dropout + residual
// =============================================================================================
template <typename T>
__global__ void bias_gelu_fwd_kernel(const T* __restrict__ x, const T* __restrict__ bias,
                                     T* __restrict__ y, int64_t nvec, int cvec) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float a[8], b[8], o[8];
    load8(x + i * 8, a);
    if (bias) load8(bias + (i % cvec) * 8, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = gelu_tanh(a[j] + (bias ? b[j] : 0.f));
    store8(y + i * 8, o);
  }
}
template <typename T>
__global__ void bias_gelu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                     const T* __restrict__ bias, T* __restrict__ dx, int64_t nvec,
                                     int cvec) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float a[8], b[8], d[8], o[8];
    load8(x + i * 8, a);
    load8(dy + i * 8, d);
    if (bias) load8(bias + (i % cvec) * 8, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = d[j] * gelu_tanh_grad(a[j] + (bias ? b[j] : 0.f));
    store8(dx + i * 8, o);
  }
}

template <typename T>
__global__ void bias_dropout_add_kernel(const T* __restrict__ x, const T* __restrict__ bias,
                                        const T* __restrict__ residual, T* __restrict__ out,
                                        int64_t nvec, int cvec, float p, uint64_t seed,
                                        uint64_t offset) {
  const float inv_keep = p > 0.f ? 1.0f / (1.0f - p) : 1.0f;
  constexpr int kVecRegs = sizeof(T) == 2 ? 4 : 8;
  // U vectors per thread and step: all loads of a step are issued before any arithmetic, so a
  // thread has 2 * U independent 16-byte requests in flight instead of two
  constexpr int U = 4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  // column of vector i0 and its advance per vector, kept incrementally: a 64-bit `i % cvec` per
  // vector would cost more instructions than the rest of the loop body
  const int col_step = static_cast<int>(stride % cvec);
  int col0 = static_cast<int>((blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) % cvec);
  for (int64_t i0 = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i0 < nvec; i0 += stride * U) {
    float a[U][kVecRegs], r[U][kVecRegs];      // kept as loaded (packed for 16-bit types)
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < nvec) {
        load_raw8(x + i * 8, a[u]);
        if (residual) load_raw8(residual + i * 8, r[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = i0 + u * stride;
      if (i >= nvec) break;
      float av[8], rv[8], b[8], o[8];
      unpack_raw8<T>(a[u], av);
      if (residual) unpack_raw8<T>(r[u], rv);
      if (bias) load8(bias + col0 * 8, b);
      col0 += col_step;
      if (col0 >= cvec) col0 -= cvec;
      bool keep[8];
      if (p > 0.f) keep8(seed, offset, i, p, keep);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float v = av[j] + (bias ? b[j] : 0.f);
        if (p > 0.f) v = keep[j] ? v * inv_keep : 0.f;
        o[j] = v + (residual ? rv[j] : 0.f);
      }
      store8(out + i * 8, o);
    }
  }
}
template <typename T>
__global__ void dropout_bwd_kernel(const T* __restrict__ dy, T* __restrict__ dx, int64_t nvec,
                                   float p, uint64_t seed, uint64_t offset) {
  const float inv_keep = 1.0f / (1.0f - p);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float d[8], o[8];
    load8(dy + i * 8, d);
    bool keep[8];
    keep8(seed, offset, i, p, keep);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = keep[j] ? d[j] * inv_keep : 0.f;
    store8(dx + i * 8, o);
  }
}

// dropout backward fused with the column sums of its result (the bias gradient of the preceding
// row-parallel GEMM): thread t of a CTA owns columns [8t, 8t + 8) of every row the CTA visits and
// keeps their sums in registers; one slab of partial sums per CTA, added by reduce_parts_kernel.
template <typename T>
__global__ void dropout_bwd_colsum_kernel(const T* __restrict__ dy, T* __restrict__ dx,
                                          float* __restrict__ ws, int64_t rows, int cols, float p,
                                          uint64_t seed, uint64_t offset, int add_to_ws) {
  const float inv_keep = 1.0f / (1.0f - p);
  const int cvec = cols >> 3;
  const int t = threadIdx.x;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  constexpr int U = 8;
  for (int64_t r0 = static_cast<int64_t>(blockIdx.x) * U; r0 < rows; r0 += static_cast<int64_t>(gridDim.x) * U) {
    uint4 raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (r0 + u < rows) raw[u] = *reinterpret_cast<const uint4*>(dy + ((r0 + u) * cvec + t) * 8);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (r0 + u >= rows) break;
      const int64_t i = (r0 + u) * cvec + t;
      float d[8], o[8];
      unpack8<T>(raw[u], d);
      bool keep[8];
      keep8(seed, offset, i, p, keep);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j] = keep[j] ? d[j] * inv_keep : 0.f;
        acc[j] += o[j];
      }
      store8(dx + i * 8, o);
    }
  }
  float* w = ws + static_cast<int64_t>(blockIdx.x) * cols + t * 8;
  if (add_to_ws) {
    const float4 a0 = reinterpret_cast<const float4*>(w)[0], a1 = reinterpret_cast<const float4*>(w)[1];
    acc[0] += a0.x; acc[1] += a0.y; acc[2] += a0.z; acc[3] += a0.w;
    acc[4] += a1.x; acc[5] += a1.y; acc[6] += a1.z; acc[7] += a1.w;
  }
  *reinterpret_cast<float4*>(w) = make_float4(acc[0], acc[1], acc[2], acc[3]);
  *reinterpret_cast<float4*>(w + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
}

// =============================================================================================
// column sums
// =============================================================================================
// CTA (32 x 8): 32 lanes cover 256 consecutive columns (8 each), 8 row-lanes stride over the rows
// of this CTA's row slab. grid = (col blocks, parts).
template <typename T>
__global__ void colsum_partial_kernel(const T* __restrict__ x, float* __restrict__ ws,
                                      int64_t rows, int cols) {
  __shared__ float sm[8][256 + 8];
  const int c0 = (blockIdx.x * 32 + threadIdx.x) * 8;
  const int parts = gridDim.y;
  const int64_t per = (rows + parts - 1) / parts;
  const int64_t r0 = per * blockIdx.y, r1 = min(rows, r0 + per);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (c0 < cols) {
    for (int64_t r = r0 + threadIdx.y; r < r1; r += 8) {
      float v[8];
      load8(x + r * cols + c0, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) sm[threadIdx.y][threadIdx.x * 8 + j] = acc[j];
  __syncthreads();
  const int t = threadIdx.y * 32 + threadIdx.x;  // 0..255
  const int c = blockIdx.x * 256 + t;
  if (c < cols) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) s += sm[k][t];
    ws[static_cast<int64_t>(blockIdx.y) * cols + c] = s;
  }
}

// =============================================================================================
// softmax family: one CTA (128 threads) per row, three passes over an L2-resident row.
// =============================================================================================
template <typename T>
__global__ void softmax_fwd_kernel(const T* __restrict__ x, const uint8_t* __restrict__ mask,
                                   T* __restrict__ y, int heads, int sq, int sk, float scale,
                                   int mode, int mask_batch) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const int q = static_cast<int>(row % sq);
  const int64_t bh = row / sq;
  const int64_t b = bh / heads;
  const T* xr = x + row * sk;
  T* yr = y + row * sk;
  const uint8_t* mr = nullptr;
  if (mode == 2) mr = mask + ((mask_batch == 1 ? 0 : b) * sq + q) * static_cast<int64_t>(sk);
  const int limit = (mode == 1) ? q + 1 : sk;
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < limit; c += blockDim.x) {
    float v = HalfTraits<T>::to_f(xr[c]) * scale;
    if (mr && mr[c]) v = -10000.0f;
    mx = fmaxf(mx, v);
  }
  mx = block_max(mx, red);
  float sum = 0.f;
  for (int c = threadIdx.x; c < limit; c += blockDim.x) {
    float v = HalfTraits<T>::to_f(xr[c]) * scale;
    if (mr && mr[c]) v = -10000.0f;
    sum += __expf(v - mx);
  }
  sum = block_sum(sum, red);
  const float inv = 1.0f / sum;
  for (int c = threadIdx.x; c < sk; c += blockDim.x) {
    float o = 0.f;
    if (c < limit) {
      float v = HalfTraits<T>::to_f(xr[c]) * scale;
      if (mr && mr[c]) v = -10000.0f;
      o = __expf(v - mx) * inv;
    }
    yr[c] = HalfTraits<T>::from_f(o);
  }
}
template <typename T>
__global__ void softmax_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ y,
                                   T* __restrict__ dx, int sq, int sk, float scale, int mode) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const int q = static_cast<int>(row % sq);
  const int limit = (mode == 1) ? q + 1 : sk;
  const T* dyr = dy + row * sk;
  const T* yr = y + row * sk;
  T* dxr = dx + row * sk;
  float dot = 0.f;
  for (int c = threadIdx.x; c < limit; c += blockDim.x)
    dot += HalfTraits<T>::to_f(dyr[c]) * HalfTraits<T>::to_f(yr[c]);
  dot = block_sum(dot, red);
  for (int c = threadIdx.x; c < sk; c += blockDim.x) {
    float o = 0.f;
    if (c < limit) {
      const float yy = HalfTraits<T>::to_f(yr[c]);
      o = scale * yy * (HalfTraits<T>::to_f(dyr[c]) - dot);
    }
    dxr[c] = HalfTraits<T>::from_f(o);
  }
}

// =============================================================================================
// embedding
// =============================================================================================
template <typename T>
__global__ void embedding_fwd_kernel(const int64_t* __restrict__ tokens, const T* __restrict__ word,
                                     const T* __restrict__ pos, T* __restrict__ out, int64_t ntok,
                                     int seq, int hidden, int v0, int v1, int add_pos) {
  const int nvec = hidden >> 3;
  for (int64_t t = blockIdx.x; t < ntok; t += gridDim.x) {
    const int64_t tok = tokens[t];
    const bool mine = tok >= v0 && tok < v1;
    const T* wr = word + (mine ? (tok - v0) : 0) * hidden;
    const T* pr = pos + static_cast<int64_t>(t % seq) * hidden;
    T* orow = out + t * hidden;
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
      float w[8] = {0, 0, 0, 0, 0, 0, 0, 0}, pv[8];
      if (mine) load8(wr + c * 8, w);
      if (add_pos) {
        load8(pr + c * 8, pv);
#pragma unroll
        for (int j = 0; j < 8; ++j) w[j] += pv[j];
      }
      store8(orow + c * 8, w);
    }
  }
}
template <typename G>
__device__ __forceinline__ void atomic_add_g(G* p, float v) {
  if constexpr (sizeof(G) == 4) atomicAdd(p, v);
  else atomicAdd(p, HalfTraits<G>::from_f(v));
}
template <typename T, typename G>
__global__ void embedding_bwd_kernel(const int64_t* __restrict__ tokens, const T* __restrict__ dout,
                                     G* __restrict__ dword, G* __restrict__ dpos, int64_t ntok,
                                     int seq, int hidden, int v0, int v1, int add_pos) {
  for (int64_t t = blockIdx.x; t < ntok; t += gridDim.x) {
    const int64_t tok = tokens[t];
    const bool mine = tok >= v0 && tok < v1;
    const T* drow = dout + t * hidden;
    G* wr = dword + (mine ? (tok - v0) : 0) * hidden;
    G* pr = dpos ? dpos + static_cast<int64_t>(t % seq) * hidden : nullptr;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float d = HalfTraits<T>::to_f(drow[c]);
      if (mine) atomic_add_g(wr + c, d);
      if (add_pos && pr) atomic_add_g(pr + c, d);
    }
  }
}

// =============================================================================================
// vocab-parallel cross entropy
// =============================================================================================
template <typename T>
__global__ void ce_stats_kernel(const T* __restrict__ logits, const int64_t* __restrict__ targets,
                                float* __restrict__ stats, int64_t rows, int vl, int64_t ld,
                                int v0) {
  __shared__ float red[32];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* lr = logits + row * ld;
    const int nvec = vl >> 3;
    // online (max, sum) per thread, merged across the block
    float mx = -INFINITY, sum = 0.f;
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
      float v[8];
      load8(lr + c * 8, v);
      float m8 = v[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) m8 = fmaxf(m8, v[j]);
      const float nm = fmaxf(mx, m8);
      float s8 = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) s8 += __expf(v[j] - nm);
      sum = sum * __expf(mx - nm) + s8;
      mx = nm;
    }
    const float gm = block_max(mx, red);
    const float contrib = (mx == -INFINITY) ? 0.f : sum * __expf(mx - gm);
    const float gs = block_sum(contrib, red);
    if (threadIdx.x == 0) {
      const int64_t t = targets[row] - v0;
      const float tl = (t >= 0 && t < vl) ? HalfTraits<T>::to_f(lr[t]) : 0.f;
      stats[row * 3 + 0] = gm;
      stats[row * 3 + 1] = gs;
      stats[row * 3 + 2] = tl;
    }
    __syncthreads();
  }
}
__global__ void ce_combine_kernel(const float* __restrict__ all, float* __restrict__ loss,
                                  float* __restrict__ gmax, float* __restrict__ gsum, int64_t rows,
                                  int world) {
  const int64_t r = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (r >= rows) return;
  float m = -INFINITY;
  for (int w = 0; w < world; ++w) m = fmaxf(m, all[(w * rows + r) * 3]);
  float s = 0.f, t = 0.f;
  for (int w = 0; w < world; ++w) {
    const float* p = all + (w * rows + r) * 3;
    s += p[1] * __expf(p[0] - m);
    t += p[2];
  }
  gmax[r] = m;
  gsum[r] = s;
  loss[r] = __logf(s) + m - t;
}
template <typename T>
__global__ void ce_bwd_kernel(T* __restrict__ logits, const int64_t* __restrict__ targets,
                              const float* __restrict__ gmax, const float* __restrict__ gsum,
                              const float* __restrict__ dloss, int64_t rows, int vl, int64_t ld,
                              int v0) {
  const int nvec = vl >> 3;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    T* lr = logits + row * ld;
    const float m = gmax[row], inv = 1.0f / gsum[row], g = dloss[row];
    const int64_t t = targets[row] - v0;
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
      float v[8];
      load8(lr + c * 8, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float sm = __expf(v[j] - m) * inv;
        if (c * 8 + j == t) sm -= 1.0f;
        v[j] = sm * g;
      }
      store8(lr + c * 8, v);
    }
  }
}

// =============================================================================================
// optimizer
// =============================================================================================
template <typename G>
__global__ void grad_norm_kernel(const G* __restrict__ g, int64_t n, float inv_scale,
                                 float* __restrict__ acc, int head) {
  __shared__ float red[32];
  float s = 0.f;
  bool bad = false;
  // `head` leading elements (fewer than 8) bring the pointer to a 16-byte boundary: a range of a
  // flat buffer may start anywhere, the vector loop below needs aligned addresses
  if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < head) {
    const float u = HalfTraits<G>::to_f(g[threadIdx.x]) * inv_scale;
    bad |= !isfinite(u);
    s += u * u;
  }
  g += head;
  n -= head;
  const int64_t nvec = n >> 3;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float v[8];
    load8(g + i * 8, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float u = v[j] * inv_scale;
      bad |= !isfinite(u);
      s += u * u;
    }
  }
  for (int64_t i = (nvec << 3) + blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float u = HalfTraits<G>::to_f(g[i]) * inv_scale;
    bad |= !isfinite(u);
    s += u * u;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(acc, s);
  if (bad) acc[1] = 1.0f;
}

template <typename P, typename G>
__global__ void adam_kernel(AdamArgs a) {
  const float found_inf = a.ctrl ? a.ctrl[1] : 0.f;
  if (found_inf != 0.f) return;  // overflow: the whole step is skipped on every rank
  // ctrl[0] holds the sum of squares of the raw (loss-scaled, not yet normalised) gradients;
  // ctrl[2], when used, the factor that turns a raw gradient into the true one
  // (loss normalisation / loss scale), so neither value ever has to visit the host.
  const float inv_scale = (a.ctrl && a.scale_from_ctrl) ? a.ctrl[2] : a.inv_scale;
  float clip = 1.0f;
  if (a.ctrl && a.max_norm > 0.f) {
    const float norm = sqrtf(a.ctrl[0]) * inv_scale;
    clip = fminf(1.0f, a.max_norm / (norm + 1.0e-6f));
  }
  const float gscale = inv_scale * clip;
  P* param = reinterpret_cast<P*>(a.param);
  const G* grad = reinterpret_cast<const G*>(a.grad);
  const float step = a.lr / a.bias_correction1;
  const float inv_bc2 = 1.0f / sqrtf(a.bias_correction2);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < a.n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float g = HalfTraits<G>::to_f(grad[i]) * gscale;
    float p = a.master[i];
    if (!a.adamw) g += a.weight_decay * p;
    const float m = a.beta1 * a.exp_avg[i] + (1.0f - a.beta1) * g;
    const float v = a.beta2 * a.exp_avg_sq[i] + (1.0f - a.beta2) * g * g;
    a.exp_avg[i] = m;
    a.exp_avg_sq[i] = v;
    const float denom = sqrtf(v) * inv_bc2 + a.eps;
    if (a.adamw) p *= (1.0f - a.lr * a.weight_decay);
    p -= step * (m / denom);
    a.master[i] = p;
    if (reinterpret_cast<void*>(param) != reinterpret_cast<void*>(a.master))
      param[i] = HalfTraits<P>::from_f(p);
  }
}

template <typename S, typename D>
__global__ void strided_copy_kernel(const CopySegment* __restrict__ segs, float scale) {
  const CopySegment s = segs[blockIdx.y];
  const int64_t total = s.rows * s.run;
  const S* src = reinterpret_cast<const S*>(s.src);
  D* dst = reinterpret_cast<D*>(s.dst);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / s.run, c = i - r * s.run;
    dst[r * s.dst_stride + c] =
        HalfTraits<D>::from_f(HalfTraits<S>::to_f(src[r * s.src_stride + c]) * scale);
  }
}
template <typename T>
__global__ void scale_kernel(T* __restrict__ x, int64_t n, float scale) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    x[i] = HalfTraits<T>::from_f(HalfTraits<T>::to_f(x[i]) * scale);
}

__global__ void synthetic_batch_kernel(int64_t* __restrict__ tokens, int64_t* __restrict__ labels,
                                       float* __restrict__ loss_mask,
                                       const int64_t* __restrict__ sample_ids, int nsamples,
                                       int seq, int vocab) {
  const int64_t n = static_cast<int64_t>(nsamples) * seq;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t s = sample_ids[i / seq], pos = i % seq;
    int64_t t = (s * 1103515245LL + pos * 12345LL) % vocab;
    if (t < 0) t += vocab;
    tokens[i] = t;
    if (labels) {
      int64_t l = (s * 1103515245LL + (pos + 1) * 12345LL) % vocab;
      if (l < 0) l += vocab;
      labels[i] = l;
    }
    loss_mask[i] = ((s + pos) % 4 != 0) ? 1.0f : 0.0f;
  }
}

inline int grid_for(int64_t work_items, int threads, int per_sm = 8) {
  int64_t blocks = (work_items + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(kSMs) * per_sm;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}
// (iterations, threads) so that iterations * threads * 8 >= hidden with <= 512 threads when possible
inline void ln_shape(int hidden, int& iters, int& threads) {
  const int nvec = hidden / 8;
  iters = nvec <= 512 ? 1 : (nvec <= 1024 ? 2 : 4);
  threads = ((nvec + iters - 1) / iters + 31) / 32 * 32;
  if (threads < 32) threads = 32;
}
#define ETHB_LN_ITERS(iters, I, ...)                  \
  do {                                                 \
    if ((iters) == 1) { constexpr int I = 1; __VA_ARGS__; }      \
    else if ((iters) == 2) { constexpr int I = 2; __VA_ARGS__; } \
    else { constexpr int I = 4; __VA_ARGS__; }                   \
  } while (0)

}  // namespace

// ---------------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------------
cudaError_t layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y,
                          float* mean, float* rstd, int rows, int hidden, float eps, int dtype,
                          cudaStream_t st) {
  if (hidden % 8 != 0 || hidden / 8 > 4 * 1024) return cudaErrorInvalidValue;
  if (dtype != kF32 && hidden % 256 == 0 && hidden / 256 <= 16 && hidden / 256 >= 1) {
    // warp per row, 8 warps per CTA, at most two CTAs per SM: every warp walks several rows
    const int grid = (rows + 7) / 8 < 2 * kSMs ? (rows + 7) / 8 : 2 * kSMs;
#define ETHB_LN_WARP(V)                                                                          \
  case V:                                                                                         \
    if (dtype == kBF16)                                                                           \
      ln_fwd_warp_kernel<__nv_bfloat16, V><<<grid, 256, 0, st>>>(                                 \
          (const __nv_bfloat16*)x, (const __nv_bfloat16*)gamma, (const __nv_bfloat16*)beta,       \
          (__nv_bfloat16*)y, mean, rstd, rows, eps);                                              \
    else                                                                                          \
      ln_fwd_warp_kernel<__half, V><<<grid, 256, 0, st>>>((const __half*)x, (const __half*)gamma, \
                                                          (const __half*)beta, (__half*)y, mean,  \
                                                          rstd, rows, eps);                       \
    count_launch();                                                                               \
    return cudaGetLastError();
    switch (hidden / 256) {
      ETHB_LN_WARP(1) ETHB_LN_WARP(2) ETHB_LN_WARP(3) ETHB_LN_WARP(4) ETHB_LN_WARP(5) ETHB_LN_WARP(6)
      ETHB_LN_WARP(8) ETHB_LN_WARP(10) ETHB_LN_WARP(12) ETHB_LN_WARP(16)
      default: break;   // other widths: the CTA-per-row kernel below
    }
#undef ETHB_LN_WARP
  }
  int iters, threads;
  ln_shape(hidden, iters, threads);
  const int grid = rows < kSMs * 16 ? rows : kSMs * 16;
  ETHB_DISPATCH(dtype, T, ETHB_LN_ITERS(iters, I,
                (ln_fwd_kernel<T, I><<<grid, threads, 0, st>>>(
                    (const T*)x, (const T*)gamma, (const T*)beta, (T*)y, mean, rstd, rows, hidden,
                    eps))));
  count_launch();
  return cudaGetLastError();
}

// Rows per batch of the fused backward, chosen so that the packed rows fit the register budget of
// a CTA of hidden / 8 threads.
static int ln_bwd_rows_per_batch(int hidden) {
  const int threads = hidden / 8;
  return threads <= 256 ? 5 : (threads <= 512 ? 4 : 2);
}
bool ln_bwd_fused_ok(int hidden, int dtype) {
  return dtype != kF32 && hidden % 256 == 0 && hidden <= 8192;
}

int ln_bwd_parts(int rows, int hidden, int dtype) {
  if (ln_bwd_fused_ok(hidden, dtype)) {
    const int r = ln_bwd_rows_per_batch(hidden);
    const int threads = hidden / 8;
    const int per_sm = threads <= 256 ? 2 : 1;
    int p = (rows + r - 1) / r;
    if (p > kSMs * per_sm) p = kSMs * per_sm;
    return p < 1 ? 1 : p;
  }
  int p = rows / 64;
  if (p < 1) p = 1;
  if (p > 96) p = 96;
  return p;
}

cudaError_t layernorm_bwd(const void* dy, const void* x, const void* gamma, const float* mean,
                          const float* rstd, const void* dres, void* dx, void* dgamma, void* dbeta,
                          float* ws, int rows, int hidden, int dtype, int grad_dtype, int accumulate,
                          cudaStream_t st, int ws_mode) {
  if (hidden % 8 != 0 || hidden / 8 > 4 * 1024) return cudaErrorInvalidValue;
  if (ws_mode != kWsImmediate && !ln_bwd_fused_ok(hidden, dtype)) return cudaErrorInvalidValue;
  const int parts = ln_bwd_parts(rows, hidden, dtype);
  dim3 rgrid((hidden + 31) / 32), rblock(32, 8);
  if (ln_bwd_fused_ok(hidden, dtype)) {
    const int threads = hidden / 8;
    const int r = ln_bwd_rows_per_batch(hidden);
#define ETHB_LN_BWD(R)                                                                              \
  ETHB_DISPATCH(dtype, T,                                                                           \
                (ln_bwd_fused_kernel<T, R><<<parts, threads, 0, st>>>(                              \
                    (const T*)dy, (const T*)x, (const T*)gamma, mean, rstd, (const T*)dres, (T*)dx, ws, rows, \
                    hidden, ws_mode != kWsImmediate)))
    if (r == 5) { ETHB_LN_BWD(5); } else if (r == 4) { ETHB_LN_BWD(4); } else { ETHB_LN_BWD(2); }
#undef ETHB_LN_BWD
    if (ws_mode == kWsAccumulate) {   // the column sums stay in the slabs until a later call flushes them
      count_launch();
      return cudaGetLastError();
    }
    ETHB_DISPATCH(grad_dtype, G,
                  (reduce_parts_kernel<G><<<rgrid, rblock, 0, st>>>(ws, (G*)dgamma, (G*)dbeta, parts, hidden,
                                                                    accumulate, ws_mode == kWsFlush)));
    count_launch(2);
    return cudaGetLastError();
  }
  const int warps = 4;
  int grid = (rows + warps - 1) / warps;
  if (grid > kSMs * 16) grid = kSMs * 16;
  ETHB_DISPATCH(dtype, T,
                (ln_bwd_dx_kernel<T><<<grid, warps * 32, 0, st>>>((const T*)dy, (const T*)x, (const T*)gamma,
                                                                  mean, rstd, (const T*)dres, (T*)dx, rows,
                                                                  hidden)));
  dim3 pgrid((hidden + 255) / 256, parts), pblock(32, 8);
  ETHB_DISPATCH(dtype, T,
                (ln_bwd_param_kernel<T><<<pgrid, pblock, 0, st>>>((const T*)dy, (const T*)x, mean, rstd, ws,
                                                                  rows, hidden)));
  ETHB_DISPATCH(grad_dtype, G,
                (reduce_parts_kernel<G><<<rgrid, rblock, 0, st>>>(ws, (G*)dgamma, (G*)dbeta, parts, hidden,
                                                                  accumulate)));
  count_launch(3);
  return cudaGetLastError();
}

cudaError_t bias_gelu_fwd(const void* x, const void* bias, void* y, int64_t rows, int cols,
                          int dtype, cudaStream_t st) {
  if (cols % 8) return cudaErrorInvalidValue;
  const int64_t nvec = rows * cols / 8;
  ETHB_DISPATCH(dtype, T,
                (bias_gelu_fwd_kernel<T><<<grid_for(nvec, 256), 256, 0, st>>>(
                    (const T*)x, (const T*)bias, (T*)y, nvec, cols / 8)));
  count_launch();
  return cudaGetLastError();
}
cudaError_t bias_gelu_bwd(const void* dy, const void* x, const void* bias, void* dx, int64_t rows,
                          int cols, int dtype, cudaStream_t st) {
  if (cols % 8) return cudaErrorInvalidValue;
  const int64_t nvec = rows * cols / 8;
  ETHB_DISPATCH(dtype, T,
                (bias_gelu_bwd_kernel<T><<<grid_for(nvec, 256), 256, 0, st>>>(
                    (const T*)dy, (const T*)x, (const T*)bias, (T*)dx, nvec, cols / 8)));
  count_launch();
  return cudaGetLastError();
}

cudaError_t bias_dropout_add_fwd(const void* x, const void* bias, const void* residual, void* out,
                                 int64_t rows, int cols, float p, uint64_t seed, uint64_t offset,
                                 int dtype, cudaStream_t st) {
  if (cols % 8) return cudaErrorInvalidValue;
  const int64_t nvec = rows * cols / 8;
  ETHB_DISPATCH(dtype, T,
                (bias_dropout_add_kernel<T><<<grid_for(nvec, 256), 256, 0, st>>>(
                    (const T*)x, (const T*)bias, (const T*)residual, (T*)out, nvec, cols / 8, p,
                    seed, offset)));
  count_launch();
  return cudaGetLastError();
}
cudaError_t dropout_bwd(const void* dy, void* dx, int64_t rows, int cols, float p, uint64_t seed,
                        uint64_t offset, int dtype, cudaStream_t st) {
  if (cols % 8) return cudaErrorInvalidValue;
  const int64_t nvec = rows * cols / 8;
  ETHB_DISPATCH(dtype, T,
                (dropout_bwd_kernel<T><<<grid_for(nvec, 256), 256, 0, st>>>((const T*)dy, (T*)dx,
                                                                            nvec, p, seed, offset)));
  count_launch();
  return cudaGetLastError();
}

int dropout_bwd_colsum_parts(int64_t rows, int cols, int dtype) {
  if (dtype == kF32 || cols % 256 != 0 || cols > 8192) return 0;   // not fusable: use the separate kernels
  int64_t p = (rows + 7) / 8;
  const int cap = kSMs * (cols / 8 <= 256 ? 4 : (cols / 8 <= 512 ? 2 : 1));
  if (p > cap) p = cap;
  return static_cast<int>(p < 1 ? 1 : p);
}
cudaError_t dropout_bwd_colsum(const void* dy, void* dx, void* bias_grad, float* ws, int64_t rows,
                               int cols, float p, uint64_t seed, uint64_t offset, int dtype,
                               int grad_dtype, int accumulate, cudaStream_t st, int ws_mode) {
  const int parts = dropout_bwd_colsum_parts(rows, cols, dtype);
  if (parts <= 0) return cudaErrorInvalidValue;
  ETHB_DISPATCH(dtype, T,
                (dropout_bwd_colsum_kernel<T><<<parts, cols / 8, 0, st>>>((const T*)dy, (T*)dx, ws, rows, cols,
                                                                         p, seed, offset, ws_mode != kWsImmediate)));
  if (ws_mode == kWsAccumulate) {
    count_launch();
    return cudaGetLastError();
  }
  ETHB_DISPATCH(grad_dtype, G,
                (reduce_parts_kernel<G><<<dim3((cols + 31) / 32), dim3(32, 8), 0, st>>>(
                    ws, (G*)bias_grad, (G*)nullptr, parts, cols, accumulate, ws_mode == kWsFlush)));
  count_launch(2);
  return cudaGetLastError();
}

int colsum_parts(int64_t rows) {
  int64_t p = (rows + 63) / 64;
  if (p > 64) p = 64;
  if (p < 1) p = 1;
  return static_cast<int>(p);
}
cudaError_t colsum(const void* x, void* out, float* ws, int64_t rows, int cols, int dtype,
                   int out_dtype, int accumulate, cudaStream_t st) {
  if (cols % 8) return cudaErrorInvalidValue;
  const int parts = colsum_parts(rows);
  dim3 grid((cols + 255) / 256, parts), block(32, 8);
  ETHB_DISPATCH(dtype, T,
                (colsum_partial_kernel<T><<<grid, block, 0, st>>>((const T*)x, ws, rows, cols)));
  ETHB_DISPATCH(out_dtype, G,
                (reduce_parts_kernel<G><<<dim3((cols + 31) / 32), dim3(32, 8), 0, st>>>(
                    ws, (G*)out, (G*)nullptr, parts, cols, accumulate)));
  count_launch(2);
  return cudaGetLastError();
}

cudaError_t softmax_fwd(const void* x, const uint8_t* mask, void* y, int64_t batches, int heads,
                        int sq, int sk, float scale, int mode, int mask_batch, int dtype,
                        cudaStream_t st) {
  const int64_t rows = batches * heads * sq;
  if (rows <= 0 || rows > 0x7fffffffLL) return cudaErrorInvalidValue;
  ETHB_DISPATCH(dtype, T,
                (softmax_fwd_kernel<T><<<static_cast<unsigned>(rows), 128, 0, st>>>(
                    (const T*)x, mask, (T*)y, heads, sq, sk, scale, mode, mask_batch)));
  count_launch();
  return cudaGetLastError();
}
cudaError_t softmax_bwd(const void* dy, const void* y, void* dx, int64_t rows, int sq, int sk,
                        float scale, int mode, int dtype, cudaStream_t st) {
  if (rows <= 0 || rows > 0x7fffffffLL) return cudaErrorInvalidValue;
  ETHB_DISPATCH(dtype, T,
                (softmax_bwd_kernel<T><<<static_cast<unsigned>(rows), 128, 0, st>>>(
                    (const T*)dy, (const T*)y, (T*)dx, sq, sk, scale, mode)));
  count_launch();
  return cudaGetLastError();
}

cudaError_t embedding_fwd(const int64_t* tokens, const void* word, const void* pos, void* out,
                          int64_t ntok, int seq, int hidden, int vocab_start, int vocab_end,
                          int add_pos, int dtype, cudaStream_t st) {
  if (hidden % 8) return cudaErrorInvalidValue;
  const int grid = ntok < kSMs * 16 ? static_cast<int>(ntok) : kSMs * 16;
  ETHB_DISPATCH(dtype, T,
                (embedding_fwd_kernel<T><<<grid, 128, 0, st>>>(tokens, (const T*)word,
                                                               (const T*)pos, (T*)out, ntok, seq,
                                                               hidden, vocab_start, vocab_end,
                                                               add_pos)));
  count_launch();
  return cudaGetLastError();
}
cudaError_t embedding_bwd(const int64_t* tokens, const void* dout, void* dword, void* dpos,
                          int64_t ntok, int seq, int hidden, int vocab_start, int vocab_end,
                          int add_pos, int dtype, int grad_dtype, cudaStream_t st) {
  const int grid = ntok < kSMs * 16 ? static_cast<int>(ntok) : kSMs * 16;
  ETHB_DISPATCH(dtype, T, ETHB_DISPATCH(grad_dtype, G,
                (embedding_bwd_kernel<T, G><<<grid, 256, 0, st>>>(tokens, (const T*)dout, (G*)dword,
                                                                  (G*)dpos, ntok, seq, hidden,
                                                                  vocab_start, vocab_end,
                                                                  add_pos))));
  count_launch();
  return cudaGetLastError();
}

cudaError_t ce_local_stats(const void* logits, const int64_t* targets, float* stats, int64_t rows,
                           int vocab_local, int64_t ld, int vocab_start, int dtype,
                           cudaStream_t st) {
  if (vocab_local % 8 || ld % 8) return cudaErrorInvalidValue;
  const int grid = rows < kSMs * 8 ? static_cast<int>(rows) : kSMs * 8;
  ETHB_DISPATCH(dtype, T,
                (ce_stats_kernel<T><<<grid, 256, 0, st>>>((const T*)logits, targets, stats, rows,
                                                          vocab_local, ld, vocab_start)));
  count_launch();
  return cudaGetLastError();
}
cudaError_t ce_combine(const float* stats_all, float* loss, float* gmax, float* gsum, int64_t rows,
                       int world, cudaStream_t st) {
  ce_combine_kernel<<<static_cast<unsigned>((rows + 255) / 256), 256, 0, st>>>(stats_all, loss, gmax,
                                                                              gsum, rows, world);
  count_launch();
  return cudaGetLastError();
}
cudaError_t ce_bwd(void* logits, const int64_t* targets, const float* gmax, const float* gsum,
                   const float* dloss, int64_t rows, int vocab_local, int64_t ld, int vocab_start,
                   int dtype, cudaStream_t st) {
  if (vocab_local % 8 || ld % 8) return cudaErrorInvalidValue;
  const int grid = rows < kSMs * 8 ? static_cast<int>(rows) : kSMs * 8;
  ETHB_DISPATCH(dtype, T,
                (ce_bwd_kernel<T><<<grid, 256, 0, st>>>((T*)logits, targets, gmax, gsum, dloss, rows,
                                                        vocab_local, ld, vocab_start)));
  count_launch();
  return cudaGetLastError();
}

cudaError_t grad_norm_sq(const void* grad, int64_t n, int grad_dtype, float inv_scale, float* acc,
                         cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  const int esize = grad_dtype == kF32 ? 4 : 2;
  const uintptr_t addr = reinterpret_cast<uintptr_t>(grad);
  if (addr % esize != 0) return cudaErrorMisalignedAddress;
  int64_t head = static_cast<int64_t>(((16 - (addr & 15)) & 15) / esize);
  if (head > n) head = n;
  ETHB_DISPATCH(grad_dtype, G,
                (grad_norm_kernel<G><<<grid_for(n / 8 + 1, 256, 4), 256, 0, st>>>((const G*)grad, n,
                                                                                  inv_scale, acc, static_cast<int>(head))));
  count_launch();
  return cudaGetLastError();
}

cudaError_t fused_adam(const AdamArgs& a, cudaStream_t st) {
  if (a.n <= 0) return cudaSuccess;
  const int grid = grid_for(a.n, 256, 8);
  ETHB_DISPATCH(a.param_dtype, P, ETHB_DISPATCH(a.grad_dtype, G,
                (adam_kernel<P, G><<<grid, 256, 0, st>>>(a))));
  count_launch();
  return cudaGetLastError();
}

cudaError_t strided_copy_scale(const CopySegment* segs_dev, int nsegs, int64_t max_elems,
                               float scale, int src_dtype, int dst_dtype, cudaStream_t st) {
  if (nsegs <= 0) return cudaSuccess;
  int gx = grid_for(max_elems, 256, 4);
  dim3 grid(gx, nsegs);
  ETHB_DISPATCH(src_dtype, S, ETHB_DISPATCH(dst_dtype, D,
                (strided_copy_kernel<S, D><<<grid, 256, 0, st>>>(segs_dev, scale))));
  count_launch();
  return cudaGetLastError();
}
cudaError_t scale_inplace(void* x, int64_t n, float scale, int dtype, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  ETHB_DISPATCH(dtype, T,
                (scale_kernel<T><<<grid_for(n, 256, 8), 256, 0, st>>>((T*)x, n, scale)));
  count_launch();
  return cudaGetLastError();
}

cudaError_t synthetic_batch(int64_t* tokens, int64_t* labels, float* loss_mask,
                            const int64_t* sample_ids, int nsamples, int seq, int vocab,
                            cudaStream_t st) {
  const int64_t n = static_cast<int64_t>(nsamples) * seq;
  synthetic_batch_kernel<<<grid_for(n, 256, 4), 256, 0, st>>>(tokens, labels, loss_mask, sample_ids,
                                                              nsamples, seq, vocab);
  count_launch();
  return cudaGetLastError();
}

}  // namespace ethb

// ================================================================================================
// Allocation-free column sums (see no_alloc.h): same kernels as `colsum`, partial sums in a
// fixed device array owned by the library.
// ================================================================================================
#include "no_alloc.h"

#include <mutex>

namespace {

// parts x cols floats; 64 x 16384 x 4 B = 4 MiB per GPU that loads the library
static __device__ __align__(256) float g_colsum_scratch[ETHB_COLSUM_NOALLOC_MAX_PARTS * ETHB_COLSUM_NOALLOC_MAX_COLS];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_scratch_mutex;

// Device address of the scratch array on the current device. In host code the array's name is only
// a handle for the runtime; the address a kernel can use comes from cudaGetSymbolAddress, queried
// once per device with that device current.
cudaError_t scratch_for_current_device(float** ptr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_colsum_scratch);
    if (e != cudaSuccess) return e;
    g_scratch_addr[dev] = static_cast<float*>(p);
  }
  *ptr = g_scratch_addr[dev];
  return cudaSuccess;
}

}  // namespace

extern "C" int ethb_colsum_noalloc(const void* x, void* out, int64_t rows, int32_t cols, int32_t dtype,
                                   int32_t out_dtype, int32_t accumulate, void* cuda_stream) {
  using namespace ethb;
  if (x == nullptr || out == nullptr || rows <= 0 || cols <= 0 || cols % 8 != 0) return ETHB_NOALLOC_BAD_ARGUMENT;
  if (dtype < 0 || dtype > 2 || out_dtype < 0 || out_dtype > 2) return ETHB_NOALLOC_BAD_ARGUMENT;
  // the kernel reads x with 16-byte vector loads (rows stay aligned because cols % 8 == 0)
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0) return ETHB_NOALLOC_BAD_ARGUMENT;
  if (cols > ETHB_COLSUM_NOALLOC_MAX_COLS) return ETHB_NOALLOC_TOO_LARGE;
  const int parts = colsum_parts(rows);
  if (parts > ETHB_COLSUM_NOALLOC_MAX_PARTS) return ETHB_NOALLOC_TOO_LARGE;
  float* ws = nullptr;
  cudaError_t e = scratch_for_current_device(&ws);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = colsum(x, out, ws, rows, cols, dtype, out_dtype, accumulate, static_cast<cudaStream_t>(cuda_stream));
  return static_cast<int>(e);
}

extern "C" const char* ethb_noalloc_strerror(int code) {
  if (code == 0) return "success";
  if (code == ETHB_NOALLOC_BAD_ARGUMENT)
    return "bad argument: null pointer, x not 16-byte aligned, non-positive size, cols not a multiple of 8, or "
           "unknown dtype code";
  if (code == ETHB_NOALLOC_TOO_LARGE)
    return "problem exceeds the built-in scratch array (cols <= 16384 and at most 64 row partitions)";
  if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
  return "unknown error code";
}
