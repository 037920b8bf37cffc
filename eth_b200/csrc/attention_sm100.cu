// Causal flash attention for sm_100a on tcgen05 tensor cores with TMEM accumulators.
//
// Forward. One CTA owns 256 query rows (two 128-row tiles) of one (batch, head) and streams the
// key/value tiles once for both:
//   warp 0      TMA producer: Q (once), then K_j / V_j tiles into a ring of shared-memory stages.
//   warp 1      MMA issuer:   S_t = Q_t K_j^T  (operands in shared memory, accumulator in TMEM),
//               O_t += P_t V_j (P_t read from TMEM, V_j from shared memory as an MN-major operand).
//   warps 2-5   softmax of query tile 0, warps 6-9 softmax of query tile 1: one thread per query
//               row; tcgen05.ld the scores, online softmax in the exp2 domain, write P back to
//               TMEM as packed 16-bit (aliasing the score columns) and rescale the O accumulator
//               only when the running maximum grew by more than 2^8 (exact after the final
//               normalisation, and it keeps TMEM read-modify-write traffic rare).
// The two query tiles ping-pong: while one tile's softmax runs on the CUDA cores, the tensor
// core executes the other tile's MMAs.
//
// TMEM map (512 columns): S_0/P_0 [0,128)  S_1/P_1 [128,256)  O_0 [256,256+D)  O_1 [384,384+D).
//
// Backward is two kernels (see the second half of this file): one per key/value tile that
// produces dK and dV, one per query tile that produces dQ. Both recompute the scores.
#include "attention_sm100.cuh"
#include "gemm_sm100.cuh"
#include "sm100_common.cuh"

#include <cstdio>
#include <mutex>

namespace ethb {

cudaError_t make_tmap_2d_16bit(CUtensorMap* map, const void* base, int dtype, uint64_t inner,
                               uint64_t outer, uint64_t ld, uint32_t box_inner,
                               uint32_t box_outer);

namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr int kTile = 128;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* m, uint64_t* bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)),
        "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                              const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) ==
            cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(sym);
  });
  return fn;
}

// 4-D map over a [batch, seq, heads, head_dim] view: dims {d, seq, heads, batch}, box {64, rows, 1, 1}.
cudaError_t make_tmap_bshd(CUtensorMap* map, const void* base, int dtype, int d, int seq, int heads,
                           int batch, const int64_t strides[3], int box_rows) {
  EncodeFn fn = encode_fn();
  if (!fn) return cudaErrorNotSupported;
  ensure_thread_context();
  if (reinterpret_cast<uintptr_t>(base) & 15) return cudaErrorMisalignedAddress;
  for (int i = 0; i < 3; ++i)
    if ((strides[i] * 2) % 16 != 0) return cudaErrorMisalignedAddress;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(seq),
                        static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(batch)};
  // strides[] = (batch, seq, heads) element strides
  cuuint64_t gstr[3] = {static_cast<cuuint64_t>(strides[1]) * 2,
                        static_cast<cuuint64_t>(strides[2]) * 2,
                        static_cast<cuuint64_t>(strides[0]) * 2};
  cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                       : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                  4, const_cast<void*>(base), dims, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    fprintf(stderr, "[eth_b200] cuTensorMapEncodeTiled failed (%d): base=%p dims={%llu,%llu,%llu,%llu} "
            "strides(bytes)={%llu,%llu,%llu} box_rows=%d\n", static_cast<int>(r), base,
            (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)dims[2],
            (unsigned long long)dims[3], (unsigned long long)gstr[0], (unsigned long long)gstr[1],
            (unsigned long long)gstr[2], box_rows);
  ETHB_RETURN_IF(r != CUDA_SUCCESS, cudaErrorInvalidValue, "cuTensorMapEncodeTiled (4-D)");
  return cudaSuccess;
}

__device__ __forceinline__ uint32_t pack_pair(float a, float b, int dtype) {
  return pack2(a, b, dtype);
}

// ==============================================================================================
// forward
// ==============================================================================================
template <int D> struct FwdCfg {
  static constexpr int kHalves = D / 64;
  static constexpr int kQBytes = 2 * kHalves * 16384;       // two query tiles
  // K and V tiles travel through one ring of equal slots in the order K_0 V_0 K_1 V_1 ...: a K
  // slot is free again as soon as both score MMAs of its tile are done, a whole iteration before
  // the V slot of the same tile, so five slots keep the loads a full iteration ahead of their use.
  static constexpr int kSlotBytes = kHalves * 16384;
  static constexpr int kSlots = (D == 128) ? 5 : 8;
  static constexpr int kSmemBytes = kQBytes + kSlots * kSlotBytes + 1024 + 256;
  static constexpr int kThreads = 320;
};

struct FwdBarriers {
  uint64_t q_full;
  uint64_t kv_full[8];
  uint64_t kv_empty[8];
  uint64_t s_full[2];
  uint64_t p_half[8];     // [tile * 4 + quarter]: 32 more P columns of a tile are written
  uint64_t o_done[2];
  uint32_t tmem_base;
  uint32_t pad;
};

template <int D, int DT>
__global__ void __launch_bounds__(320, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                const __grid_constant__ CUtensorMap tv, const AttnArgs p) {
  using C = FwdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + C::kQBytes;
  FwdBarriers* bars = reinterpret_cast<FwdBarriers*>(sKV + C::kSlots * C::kSlotBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // 1-D grid, dispatched in index order: all (head, batch) pairs of the heaviest (latest) query
  // block first, the lightest last, so that the causal triangle balances across the SMs and the
  // last CTAs to start are the short ones
  const int bh = blockIdx.x % (p.heads * p.batch), slot = blockIdx.x / (p.heads * p.batch);
  const int head = bh % p.heads, batch = bh / p.heads;
  const int q_blocks = gridDim.x / (p.heads * p.batch);
  const int qb = p.causal ? (q_blocks - 1 - slot) : slot;
  const int kv_tiles = (p.seq_k + kTile - 1) / kTile;
  int n_t[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int qt = 2 * qb + t;
    if (qt * kTile >= p.seq_q) n_t[t] = 0;
    else n_t[t] = p.causal ? min(qt + 1, kv_tiles) : kv_tiles;
  }
  const int n = max(n_t[0], n_t[1]);

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < C::kSlots; ++s) {
      mbar_init(&bars->kv_full[s], 1);
      mbar_init(&bars->kv_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&bars->s_full[t], 1);
      for (int q = 0; q < 4; ++q) mbar_init(&bars->p_half[4 * t + q], 4);   // one arrival per softmax warp
      mbar_init(&bars->o_done[t], 1);
    }
    fence_mbar_init();
    prefetch_tmap(&tq);
    prefetch_tmap(&tk);
    prefetch_tmap(&tv);
  }
  if (warp == 1) tmem_alloc(&bars->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (elect_one()) {
      mbar_expect_tx(&bars->q_full, C::kQBytes);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int h = 0; h < C::kHalves; ++h)
          tma_load_4d(sQ + (t * C::kHalves + h) * 16384, &tq, &bars->q_full, h * 64,
                      (2 * qb + t) * kTile, head, batch);
      int slot = 0;
      uint32_t phase = 0;
      for (int i = 0; i < 2 * n; ++i) {   // item 2j is K_j, item 2j + 1 is V_j
        if (!mbar_wait(&bars->kv_empty[slot], phase ^ 1, p.status, kStatusTimeoutEmpty)) break;
        uint8_t* dst = sKV + slot * C::kSlotBytes;
        mbar_expect_tx(&bars->kv_full[slot], C::kSlotBytes);
#pragma unroll
        for (int h = 0; h < C::kHalves; ++h)
          tma_load_4d(dst + h * 16384, (i & 1) ? &tv : &tk, &bars->kv_full[slot], h * 64, (i >> 1) * kTile, head,
                      batch);
        if (++slot == C::kSlots) { slot = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      const int fmt = DT == kBF16 ? 1 : 0;
      const uint32_t idesc_qk = make_idesc_f16(fmt, 0, 0, 128, 128);
      const uint32_t idesc_pv = make_idesc_f16(fmt, 0, 1, 128, D);
      bool ok = mbar_wait(&bars->q_full, 0, p.status, kStatusTimeoutFull);
      // One thread issues every MMA, so the issue path is kept short: descriptors of the tile
      // origins are built once, each MMA only adds a constant to them.
      const uint64_t dq0 = make_smem_desc_sw128(smem_u32(sQ), 16, 1024);
      const uint64_t dk0 = make_smem_desc_sw128(smem_u32(sKV), 16, 1024);
      const uint64_t dv0 = make_smem_desc_sw128(smem_u32(sKV), 16384, 1024);
      auto issue_qk = [&](int t, int slot) {
        const uint64_t dq = desc_advance(dq0, t * C::kHalves * 16384);
        const uint64_t dk = desc_advance(dk0, slot * C::kSlotBytes);
#pragma unroll
        for (int h = 0; h < C::kHalves; ++h)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_f16(tmem_base + t * 128, desc_advance(dq, h * 16384 + k * 32),
                       desc_advance(dk, h * 16384 + k * 32), idesc_qk, (h | k) != 0 ? 1u : 0u);
        tc_commit(&bars->s_full[t]);
      };
      // O_t += P_t V_j in two halves of the key range: the first four MMAs start as soon as the
      // softmax warps have written P columns 0-63, while they still compute columns 64-127.
      auto issue_pv = [&](int t, int slot, int j) {
        const uint64_t dv = desc_advance(dv0, slot * C::kSlotBytes);
        bool got = true;
#pragma unroll
        for (int half = 0; half < 4 && got; ++half) {
          got = mbar_wait(&bars->p_half[4 * t + half], j & 1, p.status, kStatusTimeoutTmemFull);
          tc_fence_after();
          if (!got) break;
#pragma unroll
          for (int k = half * 2; k < half * 2 + 2; ++k)
            tc_mma_f16_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + k * 8,
                          desc_advance(dv, k * 2048), idesc_pv, (j | k) != 0 ? 1u : 0u);
        }
        if (got) tc_commit(&bars->o_done[t]);
        return got;
      };
      // ring position of item i (K_j is item 2j, V_j item 2j + 1)
      auto wait_item = [&](int i) {
        const bool got = mbar_wait(&bars->kv_full[i % C::kSlots], (i / C::kSlots) & 1, p.status, kStatusTimeoutFull);
        tc_fence_after();
        return got;
      };
      if (ok && n > 0) {
        ok = wait_item(0);
        if (ok) {
          if (n_t[0] > 0) issue_qk(0, 0);
          if (n_t[1] > 0) issue_qk(1, 0);
          tc_commit(&bars->kv_empty[0]);
        }
      }
      for (int j = 0; j < n && ok; ++j) {
        const int vslot = (2 * j + 1) % C::kSlots, kslot = (2 * j + 2) % C::kSlots;
        ok = wait_item(2 * j + 1);
        if (!ok) break;
        if (j < n_t[0]) {
          ok = issue_pv(0, vslot, j);
          if (!ok) break;
        }
        if (j + 1 < n) {
          ok = wait_item(2 * j + 2);
          if (!ok) break;
        }
        if (j + 1 < n_t[0]) issue_qk(0, kslot);
        if (j < n_t[1]) {
          ok = issue_pv(1, vslot, j);
          if (!ok) break;
        }
        tc_commit(&bars->kv_empty[vslot]);
        if (j + 1 < n_t[1]) issue_qk(1, kslot);
        if (j + 1 < n) tc_commit(&bars->kv_empty[kslot]);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax + epilogue
    const int t = (warp - 2) >> 2;       // query tile of this warpgroup
    const int quarter = warp & 3;        // TMEM lane quarter
    const int r_local = quarter * 32 + lane;
    const int qt = 2 * qb + t;
    const int q_row = qt * kTile + r_local;
    const uint32_t lane_bits = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem_base + t * 128 + lane_bits;
    const uint32_t o_addr = tmem_base + 256 + t * 128 + lane_bits;
    const float sl2 = p.scale * kLog2e;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    const int nt = n_t[t];
    for (int j = 0; j < nt && ok; ++j) {
      ok = mbar_wait(&bars->s_full[t], j & 1, p.status, kStatusTimeoutTmemFull);
      if (!ok) break;
      tc_fence_after();
      const bool diag = p.causal && (j == qt);
      const bool tail = (j + 1) * kTile > p.seq_k;
      const int col_limit_tail = p.seq_k - j * kTile;  // valid columns in a tail tile
      // One TMEM read of the whole 128-column score row: the four loads are issued back to back
      // and waited for once, so their latency overlaps.
      uint32_t r[4][32];
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(s_addr + c * 32, r[c]);
      tmem_ld_wait();
      if (diag || tail) {   // rare: the diagonal tile of a causal row block, or a ragged last tile
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = c * 32 + i;
            if ((diag && col > r_local) || (tail && col >= col_limit_tail)) r[c][i] = 0xff800000u;  // -inf
          }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        mx0 = fmaxf(mx0, __uint_as_float(r[0][i]));
        mx1 = fmaxf(mx1, __uint_as_float(r[1][i]));
        mx2 = fmaxf(mx2, __uint_as_float(r[2][i]));
        mx3 = fmaxf(mx3, __uint_as_float(r[3][i]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      const float m_new = fmaxf(m_run, mx * sl2);
      if (j == 0) {
        m_run = m_new;
      } else {
        const bool need = m_new > m_run + kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {
          const float m_upd = need ? m_new : m_run;
          const float alpha = exp2f(m_run - m_upd);
          l_run *= alpha;
          m_run = m_upd;
          // PV_{j-1} must have landed before O is touched
          ok = mbar_wait(&bars->o_done[t], (j - 1) & 1, p.status, kStatusTimeoutTmemFull);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < D / 16; ++c) {
            uint32_t o16[16];
            tmem_ld_32x32b_x16(o_addr + c * 16, o16);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) o16[i] = __float_as_uint(__uint_as_float(o16[i]) * alpha);
            tmem_st_32x32b_x16(o_addr + c * 16, o16);
          }
          tmem_st_wait();
        }
      }
      // P = exp2(s * scale_log2 - m), packed to 16 bit into the first 64 score columns
      float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = exp2f(fmaf(__uint_as_float(r[c][2 * i]), sl2, -m_run));
          const float p1 = exp2f(fmaf(__uint_as_float(r[c][2 * i + 1]), sl2, -m_run));
          ls0 += p0;
          ls1 += p1;
          pk[i] = pack_pair(p0, p1, DT);
        }
        tmem_st_32x32b_x16(s_addr + c * 16, pk);
        {   // a quarter of the key range is complete: hand it to the MMA warp
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->p_half[4 * t + c]);
        }
      }
      const float lsum = ls0 + ls1;
      l_run += lsum;
    }
    if (ok && nt > 0) {
      ok = mbar_wait(&bars->o_done[t], (nt - 1) & 1, p.status, kStatusTimeoutTmemFull);
      tc_fence_after();
    }
    ok = __all_sync(0xffffffffu, ok);
    if (ok && nt > 0) {
      const float inv_l = 1.0f / l_run;
      const bool row_ok = q_row < p.seq_q;
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.o) + batch * p.o_strides[0] +
                       static_cast<int64_t>(q_row) * p.o_strides[1] + head * p.o_strides[2];
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32b_x32(o_addr + c * 32, r);
        tmem_ld_wait();
        if (row_ok) {
          uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_pair(__uint_as_float(r[q * 8 + 0]) * inv_l, __uint_as_float(r[q * 8 + 1]) * inv_l, DT);
            o.y = pack_pair(__uint_as_float(r[q * 8 + 2]) * inv_l, __uint_as_float(r[q * 8 + 3]) * inv_l, DT);
            o.z = pack_pair(__uint_as_float(r[q * 8 + 4]) * inv_l, __uint_as_float(r[q * 8 + 5]) * inv_l, DT);
            o.w = pack_pair(__uint_as_float(r[q * 8 + 6]) * inv_l, __uint_as_float(r[q * 8 + 7]) * inv_l, DT);
            dst[q] = o;
          }
        }
      }
      if (row_ok)
        p.lse[(static_cast<int64_t>(batch) * p.heads + head) * p.seq_q + q_row] =
            (m_run + log2f(l_run)) * kLn2;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int D, int DT>
cudaError_t launch_fwd(const AttnArgs& a, cudaStream_t st) {
  using C = FwdCfg<D>;
  CUtensorMap tq, tk, tv;
  cudaError_t e;
  e = make_tmap_bshd(&tq, a.q, a.dtype, D, a.seq_q, a.heads, a.batch, a.q_strides, kTile);
  if (e != cudaSuccess) return e;
  e = make_tmap_bshd(&tk, a.k, a.dtype, D, a.seq_k, a.heads, a.batch, a.k_strides, kTile);
  if (e != cudaSuccess) return e;
  e = make_tmap_bshd(&tv, a.v, a.dtype, D, a.seq_k, a.heads, a.batch, a.v_strides, kTile);
  if (e != cudaSuccess) return e;
  static bool attr = false;
  if (!attr) {
    e = cudaFuncSetAttribute(attn_fwd_kernel<D, DT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             C::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr = true;
  }
  const int q_blocks = (a.seq_q + 2 * kTile - 1) / (2 * kTile);
  attn_fwd_kernel<D, DT><<<q_blocks * a.heads * a.batch, C::kThreads, C::kSmemBytes, st>>>(tq, tk, tv, a);
  count_launch();
  return cudaGetLastError();
}


// ==============================================================================================
// backward
// ==============================================================================================
// Shared by both backward kernels: 2 resident 128-row tiles + a 2-stage ring of streamed tile
// pairs, processed in 64-row/column sub-tiles that ping-pong between two TMEM score buffers:
//   buffer b: S at columns [128b, 128b+64), dP at [128b+64, 128b+128); the 16-bit P / dS that
//   feed the next MMAs alias the first 32 columns of S / dP. Accumulators start at column 256.
template <int D> struct BwdCfg {
  static constexpr int kHalves = D / 64;
  static constexpr int kTileBytes = kHalves * 16384;        // one 128-row tile
  static constexpr int kResidentBytes = 2 * kTileBytes;
  static constexpr int kStages = 2;
  static constexpr int kStageBytes = 2 * kTileBytes;
  static constexpr int kAuxBytes = 2 * 2 * 2 * 64 * 4;      // [wg][parity][lse|delta][64]
  static constexpr int kSmemBytes = kResidentBytes + kStages * kStageBytes + kAuxBytes + 1024 + 256;
  static constexpr int kThreads = 320;
};

struct BwdBarriers {
  uint64_t res_full;
  uint64_t st_full[2];
  uint64_t st_empty[2];
  uint64_t s_full[2];
  uint64_t p_full[2];
  uint64_t done;
  uint64_t qdo_full;      // dQ kernel: the Q and dO rows of the tile sit in TMEM
  uint64_t p_early[2];    // dQ kernel: the first 16 of each warpgroup's 32 dS columns are written
  uint32_t tmem_base;
  uint32_t pad;
};

__device__ __forceinline__ void wg_bar_sync(int wg) {
  asm volatile("bar.sync %0, 128;" ::"r"(wg + 1) : "memory");
}

// delta[b,h,s] = sum_d dO * O. A (b, s, h) row of head_dim elements is covered by head_dim / 8
// adjacent lanes with one 16-byte load each per tensor (head_dim is 64 or 128: 8 or 16 lanes); a
// thread takes kDeltaRows rows, strided by the grid, and issues all their loads before any
// arithmetic, so 2 * kDeltaRows requests are in flight per thread.
constexpr int kDeltaRows = 4;
__global__ void __launch_bounds__(256) attn_delta_kernel(const AttnArgs p) {
  const int lanes = p.head_dim >> 3;                        // lanes per row (power of two, <= 16)
  const int rows_per_block = blockDim.x / lanes;
  const int64_t total = static_cast<int64_t>(p.batch) * p.seq_q * p.heads;
  const int sub = threadIdx.x / lanes, vec = threadIdx.x % lanes;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * rows_per_block;
  const int64_t row0 = static_cast<int64_t>(blockIdx.x) * rows_per_block + sub;
  uint4 ov[kDeltaRows], gv[kDeltaRows];
#pragma unroll
  for (int u = 0; u < kDeltaRows; ++u) {
    const int64_t row = row0 + u * stride;
    if (row < total) {
      const int h = static_cast<int>(row % p.heads);
      const int64_t bs = row / p.heads;
      const int s = static_cast<int>(bs % p.seq_q);
      const int b = static_cast<int>(bs / p.seq_q);
      ov[u] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.o) + b * p.o_strides[0] +
                                              static_cast<int64_t>(s) * p.o_strides[1] + h * p.o_strides[2] + vec * 8);
      gv[u] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.d_o) + b * p.do_strides[0] +
                                              static_cast<int64_t>(s) * p.do_strides[1] + h * p.do_strides[2] + vec * 8);
    } else {
      ov[u] = make_uint4(0, 0, 0, 0);
      gv[u] = make_uint4(0, 0, 0, 0);
    }
  }
#pragma unroll
  for (int u = 0; u < kDeltaRows; ++u) {
    const uint32_t ow[4] = {ov[u].x, ov[u].y, ov[u].z, ov[u].w}, gw[4] = {gv[u].x, gv[u].y, gv[u].z, gv[u].w};
    float acc = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = unpack2(ow[e], p.dtype), d = unpack2(gw[e], p.dtype);
      acc += a.x * d.x + a.y * d.y;
    }
    for (int off = lanes >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    const int64_t row = row0 + u * stride;
    if (vec == 0 && row < total) {
      const int h = static_cast<int>(row % p.heads);
      const int64_t bs = row / p.heads;
      p.delta[(static_cast<int64_t>(bs / p.seq_q) * p.heads + h) * p.seq_q + (bs % p.seq_q)] = acc;
    }
  }
}

// ---- dK / dV: persistent CTAs over (key/value tile, head, batch) --------------------------------
// One CTA per SM walks a static list of tiles, heaviest first (under the causal mask key tile j
// meets q_tiles - j query tiles), handed out round by round in alternating CTA order, with
// j = tile / (heads * batch).
// TMEM, the barriers and the tensor-map prefetch are set up once per CTA instead of once per tile;
// barrier parities therefore run on counters that persist across tiles (`it`: tiles done by this
// CTA, `sbase`: query tiles streamed so far). No CTA-wide barrier
// separates the tiles: the loads and first score MMAs of the next tile overlap the accumulator stores
// of the current one.
template <int D, int DT>
__global__ void __launch_bounds__(320, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                     const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                     const AttnArgs p) {
  using C = BwdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + C::kTileBytes;
  uint8_t* sStage = smem + C::kResidentBytes;  // stage: [Q tile | dO tile]
  float* sAux = reinterpret_cast<float*>(sStage + C::kStages * C::kStageBytes);
  BwdBarriers* bars = reinterpret_cast<BwdBarriers*>(reinterpret_cast<uint8_t*>(sAux) + C::kAuxBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tiles = (p.seq_q + kTile - 1) / kTile;
  const int kv_tiles = (p.seq_k + kTile - 1) / kTile;
  const int hb = p.heads * p.batch;
  const int total_tiles = kv_tiles * hb;

  if (threadIdx.x == 0) {
    mbar_init(&bars->res_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->st_full[s], 1);
      mbar_init(&bars->st_empty[s], 1);
      mbar_init(&bars->s_full[s], 1);
      mbar_init(&bars->p_full[s], 8);      // both softmax warpgroups work on every sub-tile, one arrival per warp
    }
    mbar_init(&bars->done, 1);
    fence_mbar_init();
    prefetch_tmap(&tq); prefetch_tmap(&tk); prefetch_tmap(&tv); prefetch_tmap(&tdo);
  }
  if (warp == 1) tmem_alloc(&bars->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  int p_stage = 0;           // producer: ring position of the next query-tile stage (persists across tiles)
  uint32_t p_phase = 0;
  int sbase = 0;             // query tiles streamed by this CTA before the current tile

  // Round r hands out tiles [r * grid, (r + 1) * grid), heaviest first, in alternating direction
  // (CTA 0 gets the heaviest tile of an even round and the lightest of an odd one), so the tile
  // weights of a CTA add up to nearly the same total everywhere; `it` counts the tiles this CTA
  // has processed (barrier parities run on it).
  for (int round = 0, it = 0; round * static_cast<int>(gridDim.x) < total_tiles; ++round) {
  const int tile = round * gridDim.x + ((round & 1) ? gridDim.x - 1 - blockIdx.x : blockIdx.x);
  if (tile >= total_tiles) continue;             // only in the last round
  const int j = tile / hb;                       // key/value tile
  const int head = (tile % hb) % p.heads, batch = (tile % hb) / p.heads;
  const int i0 = p.causal ? j : 0;
  const int nq = max(q_tiles - i0, 0);
  const int U = 2 * nq;
  if (warp == 0) {
    if (elect_one()) {
      // the resident K / V buffers are free once every MMA of the previous tile has completed; the
      // loads of this tile then run while the other warps still store the previous accumulators
      bool free_kv = it == 0 || mbar_wait(&bars->done, (it - 1) & 1, p.status, kStatusTimeoutTmemFull);
      if (free_kv) {
        mbar_expect_tx(&bars->res_full, C::kResidentBytes);
#pragma unroll
        for (int h = 0; h < C::kHalves; ++h) {
          tma_load_4d(sK + h * 16384, &tk, &bars->res_full, h * 64, j * kTile, head, batch);
          tma_load_4d(sV + h * 16384, &tv, &bars->res_full, h * 64, j * kTile, head, batch);
        }
      }
      int stage = p_stage;
      uint32_t phase = p_phase;
      for (int t = 0; t < nq && free_kv; ++t) {
        if (!mbar_wait(&bars->st_empty[stage], phase ^ 1, p.status, kStatusTimeoutEmpty)) break;
        uint8_t* sq = sStage + stage * C::kStageBytes;
        uint8_t* sdo = sq + C::kTileBytes;
        mbar_expect_tx(&bars->st_full[stage], C::kStageBytes);
#pragma unroll
        for (int h = 0; h < C::kHalves; ++h) {
          tma_load_4d(sq + h * 16384, &tq, &bars->st_full[stage], h * 64, (i0 + t) * kTile, head, batch);
          tma_load_4d(sdo + h * 16384, &tdo, &bars->st_full[stage], h * 64, (i0 + t) * kTile, head, batch);
        }
        if (++stage == 2) { stage = 0; phase ^= 1; }
      }
    }
    // every lane tracks the ring position, whichever lane is elected next time
    p_phase ^= static_cast<uint32_t>(((p_stage + nq) >> 1) & 1);
    p_stage = (p_stage + nq) & 1;
  } else if (warp == 1) {
    if (elect_one()) {
      const int fmt = DT == kBF16 ? 1 : 0;
      const uint32_t idesc_s = make_idesc_f16(fmt, 0, 0, 128, 64);
      const uint32_t idesc_acc = make_idesc_f16(fmt, 0, 1, 128, D);
      // One thread issues every MMA and the score MMAs are short (N = 64), so the issue path must
      // stay short too: tile-origin descriptors are built once, each MMA adds a constant.
      const uint64_t dK0 = make_smem_desc_sw128(smem_u32(sK), 16, 1024);
      const uint64_t dV0 = make_smem_desc_sw128(smem_u32(sV), 16, 1024);
      const uint64_t dQk0 = make_smem_desc_sw128(smem_u32(sStage), 16, 1024);          // K-major view
      const uint64_t dQm0 = make_smem_desc_sw128(smem_u32(sStage), 16384, 1024);       // MN-major view
      auto issue_sdp = [&](int u) {
        const int stage = (sbase + (u >> 1)) & 1, sub = u & 1, b = u & 1;
        const uint64_t dQ = desc_advance(dQk0, stage * C::kStageBytes + sub * 8192);
        const uint64_t dDO = desc_advance(dQ, C::kTileBytes);
#pragma unroll
        for (int h = 0; h < C::kHalves; ++h)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_f16(tmem_base + b * 128, desc_advance(dK0, h * 16384 + k * 32),
                       desc_advance(dQ, h * 16384 + k * 32), idesc_s, (h | k) != 0 ? 1u : 0u);
#pragma unroll
        for (int h = 0; h < C::kHalves; ++h)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_f16(tmem_base + b * 128 + 64, desc_advance(dV0, h * 16384 + k * 32),
                       desc_advance(dDO, h * 16384 + k * 32), idesc_s, (h | k) != 0 ? 1u : 0u);
        tc_commit(&bars->s_full[b]);
      };
      bool ok = mbar_wait(&bars->res_full, it & 1, p.status, kStatusTimeoutFull);
      if (ok && U > 0) {
        ok = mbar_wait(&bars->st_full[sbase & 1], (sbase >> 1) & 1, p.status, kStatusTimeoutFull);
        tc_fence_after();
        if (ok) { issue_sdp(0); issue_sdp(1); }
      }
      for (int u = 0; u < U && ok; ++u) {
        const int b = u & 1, stage = (sbase + (u >> 1)) & 1, sub = u & 1;
        ok = mbar_wait(&bars->p_full[b], (sbase + (u >> 1)) & 1, p.status, kStatusTimeoutTmemFull);
        if (!ok) break;
        tc_fence_after();
        const uint64_t dQ = desc_advance(dQm0, stage * C::kStageBytes + sub * 8192);
        const uint64_t dDO = desc_advance(dQ, C::kTileBytes);
        // queries 0-31 of P / dS sit at columns [0, 16) of their buffer, queries 32-63 at [32, 48)
#pragma unroll
        for (int k = 0; k < 4; ++k)   // dV += P^T dO
          tc_mma_f16_ts(tmem_base + 256, tmem_base + b * 128 + (k >> 1) * 32 + (k & 1) * 8,
                        desc_advance(dDO, k * 2048), idesc_acc, (u | k) != 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 4; ++k)   // dK += dS^T Q
          tc_mma_f16_ts(tmem_base + 384, tmem_base + b * 128 + 64 + (k >> 1) * 32 + (k & 1) * 8,
                        desc_advance(dQ, k * 2048), idesc_acc, (u | k) != 0 ? 1u : 0u);
        if (sub == 1) tc_commit(&bars->st_empty[stage]);
        if (u + 2 < U) {
          const int u2 = u + 2;
          if ((u2 & 1) == 0) {
            const int sq = sbase + (u2 >> 1);
            ok = mbar_wait(&bars->st_full[sq & 1], (sq >> 1) & 1, p.status, kStatusTimeoutFull);
            if (!ok) break;
            tc_fence_after();
          }
          issue_sdp(u2);
        }
      }
      tc_commit(&bars->done);
    }
  } else {
    const int wg = (warp - 2) >> 2;      // sub-tile parity handled by this warpgroup
    const int quarter = warp & 3;
    const int r_local = quarter * 32 + lane;     // key/value row inside the tile
    const int wg_tid = threadIdx.x - 64 - wg * 128;
    const uint32_t lane_bits = static_cast<uint32_t>(quarter * 32) << 16;
    const float sl2 = p.scale * kLog2e;
    const float* lse_bh = p.lse + (static_cast<int64_t>(batch) * p.heads + head) * p.seq_q;
    const float* delta_bh = p.delta + (static_cast<int64_t>(batch) * p.heads + head) * p.seq_q;
    bool ok = true;
    // Both warpgroups work on every 64-query sub-tile, each on 32 of its columns (see the dQ kernel),
    // so the softmax of a sub-tile takes half as long and hides under the score MMAs of the other
    // buffer; each warpgroup overwrites only columns it has read itself. The lse / delta values of a
    // query tile are staged once per tile and warpgroup (its 2 x 32 columns), one tile ahead: the
    // global loads for tile t + 1 are issued before tile t is processed and parked in shared memory
    // after it, so their latency is never waited for.
    const int a_sub = (wg_tid >> 5) & 1, a_col = wg_tid & 31;
    auto aux_query = [&](int t) { return (i0 + t) * kTile + a_sub * 64 + wg * 32 + a_col; };
    auto aux_slot = [&](int t) { return sAux + ((wg * 2 + (t & 1)) * 2) * 64; };   // [lse 2 x 32 | delta 2 x 32]
    if (wg_tid < 64 && nq > 0) {
      const int qi = aux_query(0);
      const bool in = qi < p.seq_q;
      aux_slot(0)[wg_tid] = in ? lse_bh[qi] * kLog2e : INFINITY;
      aux_slot(0)[64 + wg_tid] = in ? delta_bh[qi] : 0.f;
    }
    for (int t = 0; t < nq && ok; ++t) {
      wg_bar_sync(wg);                 // tile t's values are staged; everyone has left tile t - 1
      float next_lse = INFINITY, next_delta = 0.f;
      if (wg_tid < 64 && t + 1 < nq) {
        const int qi = aux_query(t + 1);
        if (qi < p.seq_q) {
          next_lse = lse_bh[qi] * kLog2e;
          next_delta = delta_bh[qi];
        }
      }
      const int i = i0 + t;
      const bool diag = p.causal && (i == j);
#pragma unroll 1
      for (int sub = 0; sub < 2 && ok; ++sub) {
        const float* a_lse = aux_slot(t) + sub * 32;
        const float* a_del = a_lse + 64;
        const uint32_t s_addr = tmem_base + sub * 128 + wg * 32 + lane_bits;
        const uint32_t dp_addr = s_addr + 64;
        ok = mbar_wait(&bars->s_full[sub], (sbase + t) & 1, p.status, kStatusTimeoutTmemFull);
        if (!ok) break;
        tc_fence_after();
        uint32_t rs[32], rd[32];
        __syncwarp();
        tmem_ld_32x32b_x32(s_addr, rs);
        tmem_ld_32x32b_x32(dp_addr, rd);
        tmem_ld_wait();
        uint32_t pk[16], dk[16];
        // lse / delta come as 16-byte broadcast loads (four query columns each); only the tile on
        // the diagonal pays for the causal mask
#pragma unroll
        for (int y = 0; y < 8; ++y) {
          const float4 l4 = *reinterpret_cast<const float4*>(a_lse + 4 * y);
          const float4 e4 = *reinterpret_cast<const float4*>(a_del + 4 * y);
          const float lv[4] = {l4.x, l4.y, l4.z, l4.w}, ev[4] = {e4.x, e4.y, e4.z, e4.w};
          float pv[4];
#pragma unroll
          for (int c = 0; c < 4; ++c) pv[c] = exp2f(fmaf(__uint_as_float(rs[4 * y + c]), sl2, -lv[c]));
          if (diag) {
            const int ql = sub * 64 + wg * 32 + 4 * y;     // query row inside the 128-row tile
#pragma unroll
            for (int c = 0; c < 4; ++c)
              if (r_local > ql + c) pv[c] = 0.f;
          }
          float dv[4];
#pragma unroll
          for (int c = 0; c < 4; ++c) dv[c] = pv[c] * (__uint_as_float(rd[4 * y + c]) - ev[c]);
          pk[2 * y] = pack_pair(pv[0], pv[1], DT);
          pk[2 * y + 1] = pack_pair(pv[2], pv[3], DT);
          dk[2 * y] = pack_pair(dv[0], dv[1], DT);
          dk[2 * y + 1] = pack_pair(dv[2], dv[3], DT);
        }
        tmem_st_32x32b_x16(s_addr, pk);
        tmem_st_32x32b_x16(dp_addr, dk);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_full[sub]);   // one arrival per warp
      }
      if (wg_tid < 64 && t + 1 < nq) {
        aux_slot(t + 1)[wg_tid] = next_lse;
        aux_slot(t + 1)[64 + wg_tid] = next_delta;
      }
    }
    // epilogue: warpgroup 0 stores dV, warpgroup 1 stores dK * scale
    if (ok) ok = mbar_wait(&bars->done, it & 1, p.status, kStatusTimeoutTmemFull);
    ok = __all_sync(0xffffffffu, ok);
    if (ok && U > 0) {
      tc_fence_after();
      const int kv_row = j * kTile + r_local;
      const bool row_ok = kv_row < p.seq_k;
      const int64_t* st = wg == 0 ? p.dv_strides : p.dk_strides;
      uint16_t* orow = reinterpret_cast<uint16_t*>(wg == 0 ? p.dv : p.dk) + batch * st[0] +
                       static_cast<int64_t>(kv_row) * st[1] + head * st[2];
      const float mul = wg == 0 ? 1.0f : p.scale;
      const uint32_t acc_addr = tmem_base + 256 + wg * 128 + lane_bits;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32b_x32(acc_addr + c * 32, r);
        tmem_ld_wait();
        if (row_ok) {
          uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_pair(__uint_as_float(r[q * 8 + 0]) * mul, __uint_as_float(r[q * 8 + 1]) * mul, DT);
            o.y = pack_pair(__uint_as_float(r[q * 8 + 2]) * mul, __uint_as_float(r[q * 8 + 3]) * mul, DT);
            o.z = pack_pair(__uint_as_float(r[q * 8 + 4]) * mul, __uint_as_float(r[q * 8 + 5]) * mul, DT);
            o.w = pack_pair(__uint_as_float(r[q * 8 + 6]) * mul, __uint_as_float(r[q * 8 + 7]) * mul, DT);
            dst[q] = o;
          }
        }
      }
    }
  }
  // End of tile, without a CTA-wide barrier: the roles meet again only through the mbarriers. The
  // producer waits for `done` before it refills K / V; the first dV / dK MMAs of the next tile
  // (which overwrite the accumulators) wait for that tile's first P, and a softmax warp writes that
  // only after it has stored its part of these accumulators.
  sbase += nq;
  ++it;
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) break;   // a wait gave up: stop
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---- dQ: persistent CTAs over (query tile, head, batch) -----------------------------------------
// Like the dK / dV kernel: one CTA per SM, tiles heaviest first (query tile i meets i + 1 key tiles
// under the causal mask) handed out round by round in alternating CTA order, TMEM and barriers set
// up once, parities on counters that persist across tiles (`it`, `sbase`), and no CTA-wide barrier
// between tiles: the Q / dO loads and first score MMAs of the next tile overlap the dQ store.
template <int D, int DT>
__global__ void __launch_bounds__(320, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                   const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                   const AttnArgs p) {
  using C = BwdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = smem + C::kTileBytes;
  uint8_t* sStage = smem + C::kResidentBytes;  // stage: [K tile | V tile]
  BwdBarriers* bars = reinterpret_cast<BwdBarriers*>(sStage + C::kStages * C::kStageBytes + C::kAuxBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hb = p.heads * p.batch;
  const int q_tiles_total = (p.seq_q + kTile - 1) / kTile;
  const int kv_tiles = (p.seq_k + kTile - 1) / kTile;
  const int total_tiles = q_tiles_total * hb;

  if (threadIdx.x == 0) {
    mbar_init(&bars->res_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->st_full[s], 1);
      mbar_init(&bars->st_empty[s], 1);
      mbar_init(&bars->s_full[s], 1);
      mbar_init(&bars->p_full[s], 8);      // both softmax warpgroups work on every sub-tile, one arrival per warp
      mbar_init(&bars->p_early[s], 8);
    }
    mbar_init(&bars->done, 1);
    mbar_init(&bars->qdo_full, 8);         // one arrival per softmax warp
    fence_mbar_init();
    prefetch_tmap(&tq); prefetch_tmap(&tk); prefetch_tmap(&tv); prefetch_tmap(&tdo);
  }
  if (warp == 1) tmem_alloc(&bars->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  int p_stage = 0;           // producer: ring position of the next key/value stage (persists across tiles)
  uint32_t p_phase = 0;
  int sbase = 0;             // key/value tiles streamed by this CTA before the current tile

  for (int round = 0, it = 0; round * static_cast<int>(gridDim.x) < total_tiles; ++round) {
  const int tile = round * gridDim.x + ((round & 1) ? gridDim.x - 1 - blockIdx.x : blockIdx.x);
  if (tile >= total_tiles) continue;             // only in the last round
  const int slot = tile / hb;
  const int head = (tile % hb) % p.heads, batch = (tile % hb) / p.heads;
  const int i = p.causal ? (q_tiles_total - 1 - slot) : slot;  // query tile, heavy first
  const int nkv = p.causal ? min(i + 1, kv_tiles) : kv_tiles;
  const int U = 2 * nkv;
  if (warp == 0) {
    if (elect_one()) {
      // Q / dO are free once every MMA of the previous tile has completed
      const bool free_q = it == 0 || mbar_wait(&bars->done, (it - 1) & 1, p.status, kStatusTimeoutTmemFull);
      if (free_q) {
        mbar_expect_tx(&bars->res_full, C::kResidentBytes);
#pragma unroll
        for (int h = 0; h < C::kHalves; ++h) {
          tma_load_4d(sQ + h * 16384, &tq, &bars->res_full, h * 64, i * kTile, head, batch);
          tma_load_4d(sDO + h * 16384, &tdo, &bars->res_full, h * 64, i * kTile, head, batch);
        }
      }
      int stage = p_stage;
      uint32_t phase = p_phase;
      for (int t = 0; t < nkv && free_q; ++t) {
        if (!mbar_wait(&bars->st_empty[stage], phase ^ 1, p.status, kStatusTimeoutEmpty)) break;
        uint8_t* sk = sStage + stage * C::kStageBytes;
        uint8_t* sv = sk + C::kTileBytes;
        mbar_expect_tx(&bars->st_full[stage], C::kStageBytes);
#pragma unroll
        for (int h = 0; h < C::kHalves; ++h) {
          tma_load_4d(sk + h * 16384, &tk, &bars->st_full[stage], h * 64, t * kTile, head, batch);
          tma_load_4d(sv + h * 16384, &tv, &bars->st_full[stage], h * 64, t * kTile, head, batch);
        }
        if (++stage == 2) { stage = 0; phase ^= 1; }
      }
    }
    // every lane tracks the ring position, whichever lane is elected next time
    p_phase ^= static_cast<uint32_t>(((p_stage + nkv) >> 1) & 1);
    p_stage = (p_stage + nkv) & 1;
  } else if (warp == 1) {
    if (elect_one()) {
      const int fmt = DT == kBF16 ? 1 : 0;
      const uint32_t idesc_s = make_idesc_f16(fmt, 0, 0, 128, 64);
      const uint32_t idesc_acc = make_idesc_f16(fmt, 0, 1, 128, D);
      // short issue path: tile-origin descriptors once, constants added per MMA
      const uint64_t dKk0 = make_smem_desc_sw128(smem_u32(sStage), 16, 1024);          // K-major view
      const uint64_t dKm0 = make_smem_desc_sw128(smem_u32(sStage), 16384, 1024);       // MN-major view
      // Q and dO are A operands read from TMEM (columns [384, 448) and [448, 512), staged there by
      // the softmax warps): a score MMA then reads only its 2 KB B operand from shared memory, where
      // with both operands in shared memory the N = 64 MMAs ran into the 128 B/clk of the SM.
      auto issue_sdp = [&](int u) {
        const int stage = (sbase + (u >> 1)) & 1, sub = u & 1, b = u & 1;
        const uint64_t dK = desc_advance(dKk0, stage * C::kStageBytes + sub * 8192);
        const uint64_t dV = desc_advance(dK, C::kTileBytes);
#pragma unroll
        for (int h = 0; h < C::kHalves; ++h)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_f16_ts(tmem_base + b * 128, tmem_base + 384 + (h * 4 + k) * 8,
                          desc_advance(dK, h * 16384 + k * 32), idesc_s, (h | k) != 0 ? 1u : 0u);
#pragma unroll
        for (int h = 0; h < C::kHalves; ++h)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_f16_ts(tmem_base + b * 128 + 64, tmem_base + 448 + (h * 4 + k) * 8,
                          desc_advance(dV, h * 16384 + k * 32), idesc_s, (h | k) != 0 ? 1u : 0u);
        tc_commit(&bars->s_full[b]);
      };
      bool ok = mbar_wait(&bars->qdo_full, it & 1, p.status, kStatusTimeoutFull);
      if (ok && U > 0) {
        ok = mbar_wait(&bars->st_full[sbase & 1], (sbase >> 1) & 1, p.status, kStatusTimeoutFull);
        tc_fence_after();
        if (ok) { issue_sdp(0); issue_sdp(1); }
      }
      for (int u = 0; u < U && ok; ++u) {
        const int b = u & 1, stage = (sbase + (u >> 1)) & 1, sub = u & 1;
        // dQ += dS K; keys 0-31 of dS sit at columns [0, 16), keys 32-63 at [32, 48). The first 16
        // keys of each warpgroup (k-steps 0 and 2) are handed over before the other 16 (1 and 3).
        const uint64_t dK = desc_advance(dKm0, stage * C::kStageBytes + sub * 8192);
        ok = mbar_wait(&bars->p_early[b], (sbase + (u >> 1)) & 1, p.status, kStatusTimeoutTmemFull);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 4; k += 2)
          tc_mma_f16_ts(tmem_base + 256, tmem_base + b * 128 + 64 + (k >> 1) * 32 + (k & 1) * 8,
                        desc_advance(dK, k * 2048), idesc_acc, (u | k) != 0 ? 1u : 0u);
        ok = mbar_wait(&bars->p_full[b], (sbase + (u >> 1)) & 1, p.status, kStatusTimeoutTmemFull);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 1; k < 4; k += 2)
          tc_mma_f16_ts(tmem_base + 256, tmem_base + b * 128 + 64 + (k >> 1) * 32 + (k & 1) * 8,
                        desc_advance(dK, k * 2048), idesc_acc, 1u);
        if (sub == 1) tc_commit(&bars->st_empty[stage]);
        if (u + 2 < U) {
          const int u2 = u + 2;
          if ((u2 & 1) == 0) {
            const int sq = sbase + (u2 >> 1);
            ok = mbar_wait(&bars->st_full[sq & 1], (sq >> 1) & 1, p.status, kStatusTimeoutFull);
            if (!ok) break;
            tc_fence_after();
          }
          issue_sdp(u2);
        }
      }
      tc_commit(&bars->done);
    }
  } else {
    const int wg = (warp - 2) >> 2;
    const int quarter = warp & 3;
    const int r_local = quarter * 32 + lane;     // query row inside the tile
    const int q_row = i * kTile + r_local;
    const bool row_ok = q_row < p.seq_q;
    const uint32_t lane_bits = static_cast<uint32_t>(quarter * 32) << 16;
    const float sl2 = p.scale * kLog2e;
    const int64_t bh = (static_cast<int64_t>(batch) * p.heads + head) * p.seq_q;
    const float lse2 = row_ok ? p.lse[bh + q_row] * kLog2e : INFINITY;
    const float delta = row_ok ? p.delta[bh + q_row] : 0.f;
    bool ok = true;
    // Stage the tile's rows as TMEM operands: warpgroup 0 copies the Q rows, warpgroup 1 the dO rows,
    // one thread per row, out of the 128-byte-swizzled tiles the TMA wrote (16-byte chunk c of row r
    // sits at chunk c ^ (r & 7)); element d of a row lands in TMEM column d / 2 of the operand.
    ok = mbar_wait(&bars->res_full, it & 1, p.status, kStatusTimeoutFull);
    if (ok) {
      const uint8_t* src = (wg == 0 ? sQ : sDO) + r_local * 128;
      const uint32_t dst = tmem_base + 384 + wg * 64 + lane_bits;
      __syncwarp();
#pragma unroll
      for (int h = 0; h < C::kHalves; ++h)
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          uint32_t v[16];
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            const int c = g * 4 + c4;
            const uint4 x = *reinterpret_cast<const uint4*>(src + h * 16384 + ((c ^ (r_local & 7)) << 4));
            v[c4 * 4 + 0] = x.x; v[c4 * 4 + 1] = x.y; v[c4 * 4 + 2] = x.z; v[c4 * 4 + 3] = x.w;
          }
          tmem_st_32x32b_x16(dst + h * 32 + g * 16, v);
        }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->qdo_full);
    }
    // Both warpgroups work on every 64-key sub-tile, each on 32 of its columns: the time from
    // "scores ready" to "dS ready" halves, so it fits under the score MMAs of the other buffer and
    // the tensor core seldom waits for it. A warpgroup writes its 16-bit dS over the first half of
    // the dP columns it has just read (its own input), never over the other warpgroup's.
    for (int u = 0; u < U && ok; ++u) {
      const int t = u >> 1, sub = u & 1;
      const uint32_t s_addr = tmem_base + sub * 128 + wg * 32 + lane_bits;
      const uint32_t dp_addr = s_addr + 64;
      ok = mbar_wait(&bars->s_full[sub], (sbase + t) & 1, p.status, kStatusTimeoutTmemFull);
      if (!ok) break;
      tc_fence_after();
      const bool diag = p.causal && (t == i);
      const int kv0 = t * kTile + sub * 64 + wg * 32;   // first key index of this warpgroup's columns
      const bool ragged = kv0 + 32 > p.seq_k;
      uint32_t rs[32], rd[32];
      __syncwarp();
      tmem_ld_32x32b_x32(s_addr, rs);
      tmem_ld_32x32b_x32(dp_addr, rd);
      tmem_ld_wait();
      uint32_t dk[16];
      const float neg_lse = -lse2;
#pragma unroll
      for (int part = 0; part < 2; ++part) {   // 16 keys at a time, handed over as soon as they are written
        if (!(diag || ragged)) {   // the common case carries no mask
#pragma unroll
          for (int x = part * 8; x < part * 8 + 8; ++x) {
            const float p0 = exp2f(fmaf(__uint_as_float(rs[2 * x]), sl2, neg_lse));
            const float p1 = exp2f(fmaf(__uint_as_float(rs[2 * x + 1]), sl2, neg_lse));
            dk[x] = pack_pair(p0 * (__uint_as_float(rd[2 * x]) - delta), p1 * (__uint_as_float(rd[2 * x + 1]) - delta),
                              DT);
          }
        } else {
#pragma unroll
          for (int x = part * 8; x < part * 8 + 8; ++x) {
            const int col = 2 * x;
            const int kl = sub * 64 + wg * 32 + col;      // key row inside the 128-row tile
            float p0 = exp2f(fmaf(__uint_as_float(rs[2 * x]), sl2, neg_lse));
            float p1 = exp2f(fmaf(__uint_as_float(rs[2 * x + 1]), sl2, neg_lse));
            if ((diag && kl > r_local) || (ragged && kv0 + col >= p.seq_k)) p0 = 0.f;
            if ((diag && kl + 1 > r_local) || (ragged && kv0 + col + 1 >= p.seq_k)) p1 = 0.f;
            dk[x] = pack_pair(p0 * (__uint_as_float(rd[2 * x]) - delta), p1 * (__uint_as_float(rd[2 * x + 1]) - delta),
                              DT);
          }
        }
        if (part == 0) {
          tmem_st_32x32b_x8(dp_addr, dk);
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->p_early[sub]);
        }
      }
      tmem_st_32x32b_x8(dp_addr + 8, dk + 8);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_full[sub]);   // one arrival per warp
    }
    if (ok) ok = mbar_wait(&bars->done, it & 1, p.status, kStatusTimeoutTmemFull);
    ok = __all_sync(0xffffffffu, ok);
    if (ok && U > 0) {
      tc_fence_after();
      // each warpgroup stores half of the head dimension
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.dq) + batch * p.dq_strides[0] +
                       static_cast<int64_t>(q_row) * p.dq_strides[1] + head * p.dq_strides[2];
      const uint32_t acc_addr = tmem_base + 256 + lane_bits;
#pragma unroll 1
      for (int c = wg * (D / 64); c < (wg + 1) * (D / 64); ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32b_x32(acc_addr + c * 32, r);
        tmem_ld_wait();
        if (row_ok) {
          uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_pair(__uint_as_float(r[q * 8 + 0]) * p.scale, __uint_as_float(r[q * 8 + 1]) * p.scale, DT);
            o.y = pack_pair(__uint_as_float(r[q * 8 + 2]) * p.scale, __uint_as_float(r[q * 8 + 3]) * p.scale, DT);
            o.z = pack_pair(__uint_as_float(r[q * 8 + 4]) * p.scale, __uint_as_float(r[q * 8 + 5]) * p.scale, DT);
            o.w = pack_pair(__uint_as_float(r[q * 8 + 6]) * p.scale, __uint_as_float(r[q * 8 + 7]) * p.scale, DT);
            dst[q] = o;
          }
        }
      }
    }
  }
  // End of tile, without a CTA-wide barrier: the producer waits for `done` before it reloads Q / dO;
  // the first dQ MMAs of the next tile (which overwrite the accumulator) wait for that tile's first
  // dS, and a softmax warp writes that only after it has stored its part of this accumulator.
  sbase += nkv;
  ++it;
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) break;   // a wait gave up: stop
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// SMs of the current device (persistent kernels launch one CTA per SM).
static int attn_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

template <int D, int DT>
cudaError_t launch_bwd(const AttnArgs& a, cudaStream_t st) {
  using C = BwdCfg<D>;
  CUtensorMap tq, tk, tv, tdo;
  ETHB_TRY(make_tmap_bshd(&tq, a.q, a.dtype, D, a.seq_q, a.heads, a.batch, a.q_strides, kTile), "bwd tensor map q");
  ETHB_TRY(make_tmap_bshd(&tk, a.k, a.dtype, D, a.seq_k, a.heads, a.batch, a.k_strides, kTile), "bwd tensor map k");
  ETHB_TRY(make_tmap_bshd(&tv, a.v, a.dtype, D, a.seq_k, a.heads, a.batch, a.v_strides, kTile), "bwd tensor map v");
  ETHB_TRY(make_tmap_bshd(&tdo, a.d_o, a.dtype, D, a.seq_q, a.heads, a.batch, a.do_strides, kTile), "bwd tensor map dO");
  static bool attr = false;
  if (!attr) {
    ETHB_TRY(cudaFuncSetAttribute(attn_bwd_dkdv_kernel<D, DT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  C::kSmemBytes), "bwd smem attribute dkdv");
    ETHB_TRY(cudaFuncSetAttribute(attn_bwd_dq_kernel<D, DT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  C::kSmemBytes), "bwd smem attribute dq");
    attr = true;
  }
  const int64_t rows = static_cast<int64_t>(a.batch) * a.seq_q * a.heads;
  for (int i = 0; i < 3; ++i)
    ETHB_RETURN_IF(a.o_strides[i] % 8 != 0 || a.do_strides[i] % 8 != 0, cudaErrorMisalignedAddress,
                   "attention backward: strides of o / d_o must be multiples of 8 elements");
  ETHB_RETURN_IF((reinterpret_cast<uintptr_t>(a.o) & 15) != 0 || (reinterpret_cast<uintptr_t>(a.d_o) & 15) != 0,
                 cudaErrorMisalignedAddress, "attention backward: o / d_o must be 16-byte aligned");
  {
    const int rows_per_block = 256 / (a.head_dim / 8);
    const int64_t blocks = (rows + static_cast<int64_t>(rows_per_block) * kDeltaRows - 1) / (rows_per_block * kDeltaRows);
    attn_delta_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(a);
  }
  {
    const int tiles = ((a.seq_k + kTile - 1) / kTile) * a.heads * a.batch;
    const int sms = attn_sm_count();
    attn_bwd_dkdv_kernel<D, DT><<<tiles < sms ? tiles : sms, C::kThreads, C::kSmemBytes, st>>>(tq, tk, tv, tdo, a);
  }
  {
    const int tiles = ((a.seq_q + kTile - 1) / kTile) * a.heads * a.batch;
    const int sms = attn_sm_count();
    attn_bwd_dq_kernel<D, DT><<<tiles < sms ? tiles : sms, C::kThreads, C::kSmemBytes, st>>>(tq, tk, tv, tdo, a);
  }
  count_launch(3);
  ETHB_TRY(cudaGetLastError(), "bwd kernel launch");
  return cudaSuccess;
}

}  // namespace

cudaError_t attention_fwd(const AttnArgs& a, cudaStream_t st) {
  if (a.dtype != kF16 && a.dtype != kBF16) return cudaErrorInvalidValue;
  if (a.causal && a.seq_q != a.seq_k) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(a.o) & 15) || a.o_strides[1] % 8 || a.o_strides[2] % 8 ||
      a.o_strides[0] % 8)
    return cudaErrorMisalignedAddress;
  // one instantiation per element type: conversions in the softmax loops compile to one instruction
  const bool bf = a.dtype == kBF16;
  if (a.head_dim == 128) return bf ? launch_fwd<128, kBF16>(a, st) : launch_fwd<128, kF16>(a, st);
  if (a.head_dim == 64) return bf ? launch_fwd<64, kBF16>(a, st) : launch_fwd<64, kF16>(a, st);
  return cudaErrorInvalidValue;
}

cudaError_t attention_bwd(const AttnArgs& a, cudaStream_t st) {
  ETHB_RETURN_IF(a.dtype != kF16 && a.dtype != kBF16, cudaErrorInvalidValue, "attention dtype");
  ETHB_RETURN_IF(a.causal && a.seq_q != a.seq_k, cudaErrorInvalidValue, "causal needs seq_q == seq_k");
  const void* outs[3] = {a.dq, a.dk, a.dv};
  const int64_t* strs[3] = {a.dq_strides, a.dk_strides, a.dv_strides};
  for (int i = 0; i < 3; ++i) {
    if (reinterpret_cast<uintptr_t>(outs[i]) & 15) return cudaErrorMisalignedAddress;
    for (int k = 0; k < 3; ++k)
      if (strs[i][k] % 8) return cudaErrorMisalignedAddress;
  }
  const bool bf = a.dtype == kBF16;
  if (a.head_dim == 128) return bf ? launch_bwd<128, kBF16>(a, st) : launch_bwd<128, kF16>(a, st);
  if (a.head_dim == 64) return bf ? launch_bwd<64, kBF16>(a, st) : launch_bwd<64, kF16>(a, st);
  ETHB_RETURN_IF(true, cudaErrorInvalidValue, "head_dim must be 64 or 128");
}

}  // namespace ethb
