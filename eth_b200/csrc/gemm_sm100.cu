// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   D[M,N] = epilogue( alpha * sum_k A(m,k) * B(n,k) )
//
// Two kernels share the epilogue. The single-CTA kernel (also the one that carries the fused
// tensor-parallel all-reduce) is described here; the CTA-pair kernel further down computes
// 256 x BN tiles with `cta_group::2` MMAs and is the default for plain GEMMs.
//
// One CTA per SM walks a static list of 128 x BN output tiles. Inside a CTA:
//   warp 0   : TMA producer  - streams 128x64 / BNx64 operand tiles through a ring of shared
//              memory stages (128-byte swizzle), signalling `full[stage]` by transaction count.
//   warp 1   : MMA issuer    - one elected lane issues tcgen05.mma (M=128, N=BN, K=16) four times
//              per stage into one of two TMEM accumulators, then tcgen05.commit releases the
//              stage (`empty[stage]`) and, after the last k-block, publishes the accumulator
//              (`tmem_full[acc]`).
//   warps 2-9: epilogue      - tcgen05.ld the accumulator (lane == output row), apply
//              bias / residual / GeLU / GeLU-grad / accumulate, convert and store. While they
//              drain accumulator `acc`, the MMA warp already fills `acc ^ 1`.
//
// Both operands may be K-major ([rows, K]) or MN-major ([K, rows]); that covers the three GEMMs
// of a linear layer (forward, data-gradient, weight-gradient) without materialising transposes.
// With `comm.world > 1` the epilogue additionally all-reduces the output tiles across the GPUs
// of a tensor-parallel group through peer memory (see the GemmComm notes in gemm_sm100.cuh).
#include "gemm_sm100.cuh"
#include "sm100_common.cuh"

#include <atomic>
#include <mutex>
#include <unordered_map>

namespace ethb {

static std::atomic<int64_t> g_launches{0};
int64_t launch_count() { return g_launches.load(); }
void count_launch(int n) { g_launches.fetch_add(n); }
static std::atomic<int> g_gemm_variant{0};
void set_gemm_variant(int v) { g_gemm_variant.store(v); }
static std::atomic<int> g_tail_split{1};
void set_gemm_tail_split(int on) { g_tail_split.store(on); }
static thread_local const char* g_error_detail = "";
const char* last_error_detail() { return g_error_detail; }
void set_error_detail(const char* where) { g_error_detail = where; }
// Driver entry points (cuTensorMapEncodeTiled) need a context bound to the calling thread; a
// fresh thread (e.g. the autograd engine's) has none until its first runtime call.
void ensure_thread_context() {
  static thread_local bool ready = false;
  if (!ready) {
    cudaFree(nullptr);
    ready = true;
  }
}

namespace {

constexpr int BM = 128;
constexpr int BK = 64;                 // 64 x 2 bytes = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kThreads = 352;          // producer warp, MMA warp, 8 epilogue warps, publisher warp
constexpr int kPublisherWarp = 10;
constexpr int kEpiThreads = 256;       // two warps per TMEM lane quarter; they split a tile's columns
constexpr int kGroupM = 16;            // band height (in tiles) of the L2-friendly rasterisation

template <int BN> struct Cfg {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BN;  // two accumulators
  static constexpr int kEpiBytes = 8 * 4096;  // per-epilogue-warp 32 x 128 B transpose buffer (fused all-reduce)
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/ + kEpiBytes;
};

struct Barriers {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t pub_count;   // fused all-reduce: epilogue-warp arrivals after storing a partial tile
  uint32_t rpub_count;  // fused all-reduce: epilogue-warp arrivals after reducing an owned tile
  uint32_t pad;
};

// Monotonic arrival counters between the epilogue warps and the publisher thread (an mbarrier's
// parity could only tell phases apart while the publisher lags by at most one tile).
__device__ __forceinline__ void warp_arrive(uint32_t* counter, int lane) {
  __syncwarp();
  if (lane == 0) {
    __threadfence_block();
    atomicAdd_block(counter, 1u);
  }
}
__device__ __forceinline__ bool counter_reached(const uint32_t* counter, uint32_t target) {
  if (*reinterpret_cast<const volatile uint32_t*>(counter) < target) return false;
  __threadfence_block();
  return true;
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_band = kGroupM * tiles_n;
  const int band = tile / per_band;
  const int r = tile - band * per_band;
  const int rows = min(kGroupM, tiles_m - band * kGroupM);
  tn = r / rows;
  tm = band * kGroupM + (r - tn * rows);
}

// The it-th tile of CTA `cta` in a grid of G CTAs. Plain GEMM and fused all-reduce walk the
// rasterised tile list with stride G. In reduce-scatter mode (W | G) the tile must lie in the row
// block of its owner (cta + it) % W: within one `it` the CTAs cta = W * j + r cover, for every
// owner, the G / W consecutive tiles it * (G / W) + j of that owner's block.
__device__ __forceinline__ bool sched_tile(const GemmArgs& p, int cta, int G, int it, int tiles_m,
                                           int tiles_n, int& tm, int& tn) {
  if (p.comm.world > 1 && p.comm.mode == 1) {
    const int W = p.comm.world;
    const int rows_per = tiles_m / W;
    const int vp = it * (G / W) + cta / W;
    if (vp >= rows_per * tiles_n) return false;
    tile_coords(vp, rows_per, tiles_n, tm, tn);
    tm += ((cta + it) % W) * rows_per;
    return true;
  }
  const int tile = cta + it * G;
  if (tile >= tiles_m * tiles_n) return false;
  tile_coords(tile, tiles_m, tiles_n, tm, tn);
  if (p.comm.world > 1 && p.comm.mode == 2)   // all-gather: rows this rank already holds come first
    tm = (tm + p.comm.rank * (tiles_m / p.comm.world)) % tiles_m;
  return true;
}

// ---- all-gather mode --------------------------------------------------------------------------
// flags[r] (ints, symmetric): [kAgUnitFlags + row / 8] = epoch once the 8-row unit starting at `row`
// of r's operand buffer has been written by the rank that owns those rows.
constexpr int kAgUnitRows = 8;
constexpr int kAgUnitFlags = 64;
__device__ __forceinline__ int sched_count(const GemmArgs& p, int cta, int G, int tiles_m, int tiles_n) {
  if (p.comm.world > 1 && p.comm.mode == 1) {
    const int W = p.comm.world;
    const int per = (tiles_m / W) * tiles_n, step = G / W, first = cta / W;
    return first < per ? (per - first + step - 1) / step : 0;
  }
  const int num = tiles_m * tiles_n;
  return cta < num ? (num - cta + G - 1) / G : 0;
}

__device__ __forceinline__ void epi_bar_sync() {
  asm volatile("bar.sync 1, 256;" ::: "memory");
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
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

// Staging layout of one 128 x BN partial tile: 16-byte pieces ordered [chunk of 32 columns][piece
// 0..3][row], so that a warp-wide store or load of one piece of 32 consecutive rows is 512
// contiguous bytes (NVLink-friendly when the owner is a peer).
__device__ __forceinline__ int64_t stage_piece_offset(int c, int q, int row_in_tile) {
  return (static_cast<int64_t>(c * 4 + q) * BM + row_in_tile) * 8;  // in 16-bit elements
}

// Sum the `world` staged partials of one owned tile, add bias / residual, and write the result
// into every rank's output. Called by the 256 epilogue threads (row = lane of a TMEM quarter, two
// warps per quarter take half of the columns each). Results go
// through a per-warp shared-memory transpose so that global stores are 128-byte row segments.
template <int BN>
__device__ __forceinline__ void comm_reduce_tile(const GemmArgs& p, int tm, int tn, int slot, int slots,
                                                 int quarter, int col_half, int lane, uint8_t* warp_buf,
                                                 bool from_tmem = false, uint32_t taddr = 0) {
  const GemmComm& cm = p.comm;
  const int row_in_tile = quarter * 32 + lane;
  const int row = tm * BM + row_in_tile;
  const bool row_ok = row < p.M;
  const uint16_t* base = reinterpret_cast<const uint16_t*>(cm.stage[cm.rank]) +
                         static_cast<int64_t>(slot) * (BM * BN);
  const int64_t src_stride = static_cast<int64_t>(slots) * (BM * BN);
#pragma unroll 1
  for (int cp = col_half * (BN / 128); cp < (col_half + 1) * (BN / 128); ++cp) {
    if (tn * BN + cp * 64 >= p.N) break;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int c = cp * 2 + half;
      const int col0 = tn * BN + c * 32;
      float v[32];
      if (from_tmem) {   // this rank's own partial is still in the accumulator (warp-wide load)
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0.f;
      }
#pragma unroll 2
      for (int s = 0; s < cm.world; ++s) {
        if (from_tmem && s == cm.rank) continue;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 u = __ldcg(reinterpret_cast<const uint4*>(base + s * src_stride +
                                                                 stage_piece_offset(c, q, row_in_tile)));
          const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = unpack2(w[e], p.ab_dtype);
            v[q * 8 + e * 2] += f.x;
            v[q * 8 + e * 2 + 1] += f.y;
          }
        }
      }
      if (p.bias != nullptr && col0 < p.N) {
        const uint4* bp = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.bias) + col0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (col0 + q * 8 < p.N) {
            const uint4 b = __ldg(bp + q);
            const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = unpack2(bw[e], p.ab_dtype);
              v[q * 8 + e * 2] += f.x;
              v[q * 8 + e * 2 + 1] += f.y;
            }
          }
        }
      }
      if (p.drop_p > 0.f && col0 < p.N) {   // after the reduction: one rank draws the mask for all
        const float inv_keep = 1.0f / (1.0f - p.drop_p);
        const int64_t vec0 = (static_cast<int64_t>(row) * p.N + col0) >> 3;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          bool keep[8];
          keep8(p.drop_seed, p.drop_offset, vec0 + q, p.drop_p, keep);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[q * 8 + e] = keep[e] ? v[q * 8 + e] * inv_keep : 0.f;
        }
      }
      if (row_ok && p.aux_mode == kAuxAdd && col0 < p.N) {
        const uint4* ap = reinterpret_cast<const uint4*>(
            reinterpret_cast<const uint16_t*>(p.aux) +
            static_cast<int64_t>(cm.mode == 1 ? row - cm.rank * (p.M / cm.world) : row) * p.ldaux + col0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (col0 + q * 8 < p.N) {
            const uint4 a = __ldg(ap + q);
            const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = unpack2(aw[e], p.ab_dtype);
              v[q * 8 + e * 2] += f.x;
              v[q * 8 + e * 2 + 1] += f.y;
            }
          }
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 o;
        o.x = pack2(v[q * 8 + 0], v[q * 8 + 1], p.ab_dtype);
        o.y = pack2(v[q * 8 + 2], v[q * 8 + 3], p.ab_dtype);
        o.z = pack2(v[q * 8 + 4], v[q * 8 + 5], p.ab_dtype);
        o.w = pack2(v[q * 8 + 6], v[q * 8 + 7], p.ab_dtype);
        const int piece = half * 4 + q;   // 16-byte piece inside this row's 128-byte segment
        *reinterpret_cast<uint4*>(warp_buf + lane * 128 + ((piece ^ (lane & 7)) * 16)) = o;
      }
    }
    __syncwarp();
    // 8 lanes cover one row's 128 bytes; 4 rows per store instruction
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rl = i * 4 + (lane >> 3);
      const int piece = lane & 7;
      const uint4 o = *reinterpret_cast<const uint4*>(warp_buf + rl * 128 + ((piece ^ (rl & 7)) * 16));
      const int grow = tm * BM + quarter * 32 + rl;
      const int gcol = tn * BN + cp * 64 + piece * 8;
      if (grow < p.M && gcol < p.N) {
        if (cm.mode == 1) {   // reduce-scatter: the owner keeps its rows, nothing goes back to the peers
          *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(cm.out[cm.rank]) +
                                    static_cast<int64_t>(grow - cm.rank * (p.M / cm.world)) * p.ldd + gcol) = o;
        } else {
          for (int dst = 0; dst < cm.world; ++dst)
            *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(cm.out[dst]) +
                                      static_cast<int64_t>(grow) * p.ldd + gcol) = o;
        }
      }
    }
    __syncwarp();
  }
}

// Epilogue for 16-bit outputs that are only written (no accumulate): the same math as
// `epilogue_tile`, but rows leave -- and the `aux` operand arrives -- through a per-warp 4 KB
// shared-memory transpose, so that every global load / store instruction of a warp moves four
// whole 128-byte row segments instead of 32 scattered 16-byte pieces. `row0` is the first of the
// warp's 32 rows; columns are handled 64 at a time.
template <int BN>
__device__ __forceinline__ void epilogue_tile_staged(const GemmArgs& p, uint32_t taddr, int row0,
                                                     int lane, int n_base, int c_begin, int c_end,
                                                     uint8_t* warp_buf) {
  auto slot = [&](int r, int piece) { return warp_buf + r * 128 + ((piece ^ (r & 7)) * 16); };
#pragma unroll 1
  for (int cp = c_begin / 2; cp < c_end / 2; ++cp) {
    const int gc0 = n_base + cp * 64;
    if (gc0 >= p.N) break;  // uniform across the warp
    if (p.aux_mode != kAuxNone) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rl = i * 4 + (lane >> 3), piece = lane & 7;
        const int grow = row0 + rl, gcol = gc0 + piece * 8;
        uint4 a = make_uint4(0, 0, 0, 0);
        if (grow < p.M && gcol < p.N)
          a = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.aux) +
                                                   static_cast<int64_t>(grow) * p.ldaux + gcol));
        *reinterpret_cast<uint4*>(slot(rl, piece)) = a;
      }
      __syncwarp();
    }
    float v[2][32];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int col0 = gc0 + half * 32;
      uint32_t r[32];
      __syncwarp();
      tmem_ld_32x32b_x32(taddr + (cp * 2 + half) * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) v[half][j] = __uint_as_float(r[j]) * p.alpha;
      if (p.bias != nullptr) {
        const uint4* bp = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.bias) + col0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (col0 + q * 8 < p.N) {
            const uint4 b = __ldg(bp + q);
            const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = unpack2(bw[e], p.ab_dtype);
              v[half][q * 8 + e * 2] += f.x;
              v[half][q * 8 + e * 2 + 1] += f.y;
            }
          }
        }
      }
      if (p.drop_p > 0.f) {
        const float inv_keep = 1.0f / (1.0f - p.drop_p);
        const int64_t vec0 = (static_cast<int64_t>(row0 + lane) * p.N + col0) >> 3;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          bool keep[8];
          keep8(p.drop_seed, p.drop_offset, vec0 + q, p.drop_p, keep);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[half][q * 8 + e] = keep[e] ? v[half][q * 8 + e] * inv_keep : 0.f;
        }
      }
      if (p.aux_mode != kAuxNone) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 a = *reinterpret_cast<const uint4*>(slot(lane, half * 4 + q));
          const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = unpack2(aw[e], p.ab_dtype);
            if (p.aux_mode == kAuxAdd) {
              v[half][q * 8 + e * 2] += f.x;
              v[half][q * 8 + e * 2 + 1] += f.y;
            } else {
              v[half][q * 8 + e * 2] *= gelu_tanh_grad(f.x);
              v[half][q * 8 + e * 2 + 1] *= gelu_tanh_grad(f.y);
            }
          }
        }
      }
    }
    __syncwarp();
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      void* out = which == 0 ? p.D : p.D2;
      if (out == nullptr) break;
      const int odt = which == 0 ? p.d_dtype : p.ab_dtype;
#pragma unroll
      for (int half = 0; half < 2; ++half)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float w[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) w[e] = which == 0 ? v[half][q * 8 + e] : gelu_tanh(v[half][q * 8 + e]);
          uint4 o;
          o.x = pack2(w[0], w[1], odt);
          o.y = pack2(w[2], w[3], odt);
          o.z = pack2(w[4], w[5], odt);
          o.w = pack2(w[6], w[7], odt);
          *reinterpret_cast<uint4*>(slot(lane, half * 4 + q)) = o;
        }
      __syncwarp();
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rl = i * 4 + (lane >> 3), piece = lane & 7;
        const int grow = row0 + rl, gcol = gc0 + piece * 8;
        if (grow < p.M && gcol < p.N)
          *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(out) + static_cast<int64_t>(grow) * p.ldd + gcol) =
              *reinterpret_cast<const uint4*>(slot(rl, piece));
      }
      __syncwarp();
    }
  }
}

// Drain one 128 x BN accumulator (this thread owns TMEM lane == output row `row`) through the
// fused epilogue: alpha, bias, residual / GeLU-gradient, accumulate, convert, optional GeLU copy.
// `n_base` is the first output column of the tile; [c_begin, c_end) selects 32-column chunks of it.
template <int BN>
__device__ __forceinline__ void epilogue_tile(const GemmArgs& p, uint32_t taddr, int row, int n_base,
                                              int c_begin = 0, int c_end = BN / 32) {
  const bool row_ok = row < p.M;
  const int out_is_f32 = (p.d_dtype == kF32);
#pragma unroll 1
  for (int c = c_begin; c < c_end; ++c) {
    const int col0 = n_base + c * 32;
    if (col0 >= p.N) break;  // uniform across the warp
    uint32_t r[32];
    __syncwarp();
    tmem_ld_32x32b_x32(taddr + c * 32, r);
    tmem_ld_wait();
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
    if (p.bias != nullptr) {
      const uint4* bp = reinterpret_cast<const uint4*>(
          reinterpret_cast<const uint16_t*>(p.bias) + col0);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (col0 + q * 8 < p.N) {
          uint4 b = __ldg(bp + q);
          const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float2 f = unpack2(bw[e], p.ab_dtype);
            v[q * 8 + e * 2] += f.x;
            v[q * 8 + e * 2 + 1] += f.y;
          }
        }
      }
    }
    if (p.drop_p > 0.f) {
      const float inv_keep = 1.0f / (1.0f - p.drop_p);
      const int64_t vec0 = (static_cast<int64_t>(row) * p.N + col0) >> 3;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        bool keep[8];
        keep8(p.drop_seed, p.drop_offset, vec0 + q, p.drop_p, keep);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[q * 8 + e] = keep[e] ? v[q * 8 + e] * inv_keep : 0.f;
      }
    }
    if (row_ok) {
      if (p.aux_mode != kAuxNone) {
        const uint4* ap = reinterpret_cast<const uint4*>(
            reinterpret_cast<const uint16_t*>(p.aux) + static_cast<int64_t>(row) * p.ldaux +
            col0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (col0 + q * 8 < p.N) {
            uint4 a = __ldg(ap + q);
            const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float2 f = unpack2(aw[e], p.ab_dtype);
              if (p.aux_mode == kAuxAdd) {
                v[q * 8 + e * 2] += f.x;
                v[q * 8 + e * 2 + 1] += f.y;
              } else {
                v[q * 8 + e * 2] *= gelu_tanh_grad(f.x);
                v[q * 8 + e * 2 + 1] *= gelu_tanh_grad(f.y);
              }
            }
          }
        }
      }
      if (out_is_f32) {
        float4* dp = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.D) +
                                               static_cast<int64_t>(row) * p.ldd + col0);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          if (col0 + q * 4 < p.N) {
            float4 o = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
            if (p.accumulate) {
              float4 old = dp[q];
              o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
            }
            dp[q] = o;
          }
        }
      } else {
        uint4* dp = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.D) +
                                             static_cast<int64_t>(row) * p.ldd + col0);
        uint4* d2p = p.D2 ? reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.D2) +
                                                     static_cast<int64_t>(row) * p.ldd + col0)
                          : nullptr;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (col0 + q * 8 < p.N) {
            if (p.accumulate) {
              uint4 old = dp[q];
              const uint32_t ow[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float2 f = unpack2(ow[e], p.d_dtype);
                v[q * 8 + e * 2] += f.x;
                v[q * 8 + e * 2 + 1] += f.y;
              }
            }
            uint4 o;
            o.x = pack2(v[q * 8 + 0], v[q * 8 + 1], p.d_dtype);
            o.y = pack2(v[q * 8 + 2], v[q * 8 + 3], p.d_dtype);
            o.z = pack2(v[q * 8 + 4], v[q * 8 + 5], p.d_dtype);
            o.w = pack2(v[q * 8 + 6], v[q * 8 + 7], p.d_dtype);
            dp[q] = o;
            if (d2p) {
              uint4 g;
              g.x = pack2(gelu_tanh(v[q * 8 + 0]), gelu_tanh(v[q * 8 + 1]), p.ab_dtype);
              g.y = pack2(gelu_tanh(v[q * 8 + 2]), gelu_tanh(v[q * 8 + 3]), p.ab_dtype);
              g.z = pack2(gelu_tanh(v[q * 8 + 4]), gelu_tanh(v[q * 8 + 5]), p.ab_dtype);
              g.w = pack2(gelu_tanh(v[q * 8 + 6]), gelu_tanh(v[q * 8 + 7]), p.ab_dtype);
              d2p[q] = g;
            }
          }
        }
      }
    }
  }
}

// Tile schedule of one CTA as the fused all-reduce sees it. `vcta` numbers the CTAs of the grid; in
// the CTA-pair kernel each CTA of a pair is its own virtual CTA (it publishes and reduces the
// 128-row half tiles it computes). Ownership alternates along a CTA's tile list: tile index `it`
// belongs to rank (okey + it) % W, where okey is the CTA number -- or the pair number, so that
// both halves of a pair's tile have one owner and the pair can order its tiles by owner.
struct CommSched {
  int vcta, G, tiles_m, tiles_n;   // tiles_m in 128-row units
  bool pair;
  int pair_index, num_pairs, cta_in_pair;
  __device__ __forceinline__ int count(const GemmArgs& p) const {
    if (pair) {
      const int n2 = ((tiles_m + 1) / 2) * tiles_n;
      return pair_index < n2 ? (n2 - pair_index + num_pairs - 1) / num_pairs : 0;
    }
    return sched_count(p, vcta, G, tiles_m, tiles_n);
  }
  __device__ __forceinline__ bool tile(const GemmArgs& p, int it, int& tm, int& tn) const {
    if (pair) {
      const int tiles_m2 = (tiles_m + 1) / 2;
      const int t2 = pair_index + it * num_pairs;
      if (t2 >= tiles_m2 * tiles_n) return false;
      int tm2;
      tile_coords(t2, tiles_m2, tiles_n, tm2, tn);
      tm = 2 * tm2 + cta_in_pair;
      return true;
    }
    return sched_tile(p, vcta, G, it, tiles_m, tiles_n, tm, tn);
  }
  __device__ __forceinline__ int okey() const { return pair ? pair_index : vcta; }
  __device__ __forceinline__ int owner(int it, int W) const { return (okey() + it) % W; }
};

// Number of tiles of a list of n_my tiles that rank `me` owns, and the index of the first one.
__device__ __forceinline__ int comm_owned(int okey, int n_my, int W, int me, int* first = nullptr) {
  const int f = ((me - okey) % W + W) % W;
  if (first) *first = f;
  return n_my > f ? (n_my - f + W - 1) / W : 0;
}

// Processing order of a CTA's tile list in all-reduce mode: the j-th tile processed is list index
// comm_order(j). Tiles owned by rank me+1 come first, then me+2, ..., and this rank's own tiles
// last. Every rank therefore pushes its partials of a peer's tiles while that peer is still busy
// with other ranks' tiles, and by the time a rank reaches its own tiles the peers' partials have
// long landed in its staging area: it adds them to the accumulator it just computed and sends the
// result out, so only that one transfer is left after the last MMA. Other modes keep list order.
__device__ __forceinline__ int comm_order(const GemmComm& cm, int okey, int n_my, int j) {
  if (cm.mode != 0) return j;
  const int W = cm.world;
  for (int g = 1; g <= W; ++g) {
    int first;
    const int cnt = comm_owned(okey, n_my, W, (cm.rank + g) % W, &first);
    if (j < cnt) return first + j * W;
    j -= cnt;
  }
  return n_my;
}

// Publisher of the fused all-reduce / reduce-scatter (one thread). System-scope fences wait for every
// outstanding NVLink store of the SM (microseconds); the epilogue warps therefore never fence: they
// bump a shared-memory counter after the stores of a tile and carry on, and this thread issues the
// (cumulative) fence and writes the flags. `pub_count` counts partial tiles pushed to their owner
// (all tiles in reduce-scatter mode, where a rank also stages its own), `rpub_count` owned tiles
// whose result has been written.
__device__ __forceinline__ void comm_publisher(const GemmArgs& p, const CommSched& cs, Barriers* bars) {
  const GemmComm& cm = p.comm;
  const int W = cm.world, me = cm.rank;
  const bool ordered = cm.mode == 0;
  const int n_my = cs.count(p);
  int first_owned;
  const int n_red = comm_owned(cs.okey(), n_my, W, me, &first_owned);
  const int n_push = ordered ? n_my - n_red : n_my;
  int pa = 0, pr = 0;
  uint64_t t0 = globaltimer_ns();
  while (pa < n_push || pr < n_red) {
    bool progressed = false;
    if (pa < n_push && counter_reached(&bars->pub_count, (kEpiThreads / 32) * (pa + 1))) {
      const int it = ordered ? comm_order(cm, cs.okey(), n_my, pa) : pa;
      const int o = cs.owner(it, W);
      if (o != me) {
        __threadfence_system();
        st_release_sys(cm.flags[o] + (cs.vcta + it * cs.G) * kGemmMaxPeers + me, cm.epoch);
      }
      ++pa;
      progressed = true;
    }
    if (pr < n_red && counter_reached(&bars->rpub_count, (kEpiThreads / 32) * (pr + 1))) {
      const int it = first_owned + pr * W;   // own tiles are processed in list order in every mode
      __threadfence_system();
      for (int d = 0; d < W; ++d)
        if (d != me)
          st_release_sys(cm.flags[d] + cm.max_tiles * kGemmMaxPeers + (cs.vcta + it * cs.G), cm.epoch);
      ++pr;
      progressed = true;
    }
    if (progressed) {
      t0 = globaltimer_ns();
    } else {
      __nanosleep(64);
      if (globaltimer_ns() - t0 > ETHB_WAIT_NS) {
        if (p.status) atomicCAS(p.status, 0, kStatusTimeoutGridFlag);
        break;
      }
    }
  }
}

// Epilogue of the fused all-reduce / reduce-scatter (the 8 epilogue warps of a CTA). Every CTA
// reduces 1 / W of what it computes. Publishing (fence + flag) is left to the publisher thread.
//   all-reduce: tiles are processed in `comm_order`. A peer's tile: the accumulator goes to the
//     owner's staging area. An own tile: wait (bounded; normally not at all) for the peers'
//     partials, add them to the accumulator and write the result into every rank's output.
//   reduce-scatter: list order; every partial, the own one too, is staged, and owned tiles are
//     reduced from the staging area as soon as the peers' flags are seen.
template <int BN>
__device__ __forceinline__ void comm_epilogue(const GemmArgs& p, const CommSched& cs, Barriers* bars,
                                              uint32_t tmem_base, uint8_t* epi_smem, int warp, int lane) {
  const GemmComm& cm = p.comm;
  const int quarter = warp & 3;
  const int col_half = (warp - 2) >> 2;
  const int row_in_tile = quarter * 32 + lane;
  const int tid_e = threadIdx.x - 64;
  const int W = cm.world, me = cm.rank;
  const bool ordered = cm.mode == 0;
  const int slots = (cs.tiles_m * cs.tiles_n + W - 1) / W + cs.G;
  int* my_flags = cm.flags[me];
  __shared__ int s_ready;
  const int n_my = cs.count(p);
  // staging slot of the it-th tile of this CTA inside its owner's area: slots are per CTA
  auto slot_of = [&](int it) { return cs.vcta + (it / W) * cs.G; };
  auto release_acc = [&](int acc) {
    tc_fence_before();
    if (cs.pair)
      mbar_arrive_cluster(mapa_shared(smem_u32(&bars->tmem_empty[acc]), 0));
    else
      mbar_arrive(&bars->tmem_empty[acc]);
  };
  int red = 0, drained = 0;
  bool ok = true;
  auto reduce_one = [&](int it) {
    int rtm, rtn;
    if (cs.tile(p, it, rtm, rtn))
      comm_reduce_tile<BN>(p, rtm, rtn, slot_of(it), slots, quarter, col_half, lane,
                           epi_smem + (warp - 2) * 4096);
    warp_arrive(&bars->rpub_count, lane);
  };
  for (int j = 0; j < n_my && ok; ++j) {
    const int it = ordered ? comm_order(cm, cs.okey(), n_my, j) : j;
    const int owner = cs.owner(it, W), slot = slot_of(it);
    const int acc = j & 1;
    const uint32_t acc_phase = (j >> 1) & 1;
    if (!mbar_wait(&bars->tmem_full[acc], acc_phase, p.status, kStatusTimeoutTmemFull)) {
      ok = false;
      break;
    }
    tc_fence_after();
    const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
    if (ordered && owner == me) {
      // own tile: accumulator + the peers' staged partials -> every rank's output
      const int t2 = cs.vcta + it * cs.G;
      if (tid_e == 0) s_ready = 1;
      epi_bar_sync();
      if (tid_e < W && tid_e != me && !wait_flag_ge(my_flags + t2 * kGemmMaxPeers + tid_e, cm.epoch, p.status))
        s_ready = 0;
      epi_bar_sync();
      if (!s_ready) {
        ok = false;
        break;
      }
      int rtm, rtn;
      if (cs.tile(p, it, rtm, rtn))
        comm_reduce_tile<BN>(p, rtm, rtn, slot, slots, quarter, col_half, lane, epi_smem + (warp - 2) * 4096,
                             true, taddr);
      release_acc(acc);
      warp_arrive(&bars->rpub_count, lane);
      continue;
    }
    // this rank's partial tile -> the owner's staging area (a peer store unless owned)
    uint16_t* dst = reinterpret_cast<uint16_t*>(cm.stage[owner]) +
                    (static_cast<int64_t>(me) * slots + slot) * (BM * BN);
#pragma unroll 1
    for (int c = col_half * (BN / 64); c < (col_half + 1) * (BN / 64); ++c) {
      uint32_t r[32];
      __syncwarp();
      tmem_ld_32x32b_x32(taddr + c * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 o;
        o.x = pack2(__uint_as_float(r[q * 8 + 0]) * p.alpha, __uint_as_float(r[q * 8 + 1]) * p.alpha, p.ab_dtype);
        o.y = pack2(__uint_as_float(r[q * 8 + 2]) * p.alpha, __uint_as_float(r[q * 8 + 3]) * p.alpha, p.ab_dtype);
        o.z = pack2(__uint_as_float(r[q * 8 + 4]) * p.alpha, __uint_as_float(r[q * 8 + 5]) * p.alpha, p.ab_dtype);
        o.w = pack2(__uint_as_float(r[q * 8 + 6]) * p.alpha, __uint_as_float(r[q * 8 + 7]) * p.alpha, p.ab_dtype);
        *reinterpret_cast<uint4*>(dst + stage_piece_offset(c, q, row_in_tile)) = o;
      }
    }
    warp_arrive(&bars->pub_count, lane);
    release_acc(acc);
    if (ordered) continue;
    drained = j + 1;
    // reduce-scatter, opportunistic: reduce owned tiles whose peer partials have all arrived
    while (red < drained) {
      if (cs.owner(red, W) != me) { ++red; continue; }
      const int t2 = cs.vcta + red * cs.G;
      if (tid_e == 0) {
        int ready = 1;
        for (int s = 0; s < W; ++s)
          if (s != me && ld_acquire_sys(my_flags + t2 * kGemmMaxPeers + s) < cm.epoch) ready = 0;
        s_ready = ready;
      }
      epi_bar_sync();
      const int ready = s_ready;
      epi_bar_sync();
      if (!ready) break;
      reduce_one(red);
      ++red;
    }
  }
  // reduce-scatter drain: remaining owned tiles, now with (bounded) blocking waits
  while (!ordered && ok && red < n_my) {
    if (cs.owner(red, W) == me) {
      const int t2 = cs.vcta + red * cs.G;
      if (tid_e < W && tid_e != me)
        wait_flag_ge(my_flags + t2 * kGemmMaxPeers + tid_e, cm.epoch, p.status);
      epi_bar_sync();
      reduce_one(red);
    }
    ++red;
  }
  // the tiles owned by peers must have landed in this rank's output before the kernel ends
  for (int i = tid_e; i < n_my && ok; i += kEpiThreads) {
    if (cs.owner(i, W) != me)
      wait_flag_ge(my_flags + cm.max_tiles * kGemmMaxPeers + (cs.vcta + i * cs.G), cm.epoch, p.status);
  }
}

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a,
                    const __grid_constant__ CUtensorMap tma_b, const GemmArgs p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment is required by the 128-byte swizzle atoms.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  Barriers* bars = reinterpret_cast<Barriers*>(smem + C::kStages * C::kStageBytes);
  uint8_t* epi_smem = smem + C::kStages * C::kStageBytes + 256;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int k_blocks = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tmem_full[a], 1);
      mbar_init(&bars->tmem_empty[a], kEpiThreads);
    }
    bars->pub_count = 0;
    bars->rpub_count = 0;
    fence_mbar_init();
    prefetch_tmap(&tma_a);
    prefetch_tmap(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, C::kTmemCols);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int tm, tn;
      const int n_my = sched_count(p, blockIdx.x, gridDim.x, tiles_m, tiles_n);
      for (int j = 0; ok && j < n_my; ++j) {
        // fused all-reduce: tiles owned by peers first, this rank's own tiles last
        const int it = p.comm.world > 1 ? comm_order(p.comm, blockIdx.x, n_my, j) : j;
        if (!sched_tile(p, blockIdx.x, gridDim.x, it, tiles_m, tiles_n, tm, tn)) break;
        const int m0 = tm * BM, n0 = tn * BN;
        if (p.comm.world > 1 && p.comm.mode == 2 && tm / (tiles_m / p.comm.world) != p.comm.rank) {
          // rows gathered from a peer: all 16 eight-row units of this 128-row block must have landed
          const int* uf = p.comm.flags[p.comm.rank] + kAgUnitFlags + tm * (BM / kAgUnitRows);
          const uint64_t t0 = globaltimer_ns();
          for (int u = 0; u < BM / kAgUnitRows && ok; ++u) {
            uint32_t spins = 0;
            while (ld_acquire_sys(uf + u) < p.comm.epoch) {
              if ((++spins & 0x3f) == 0 && globaltimer_ns() - t0 > ETHB_WAIT_NS) {
                if (p.status) atomicCAS(p.status, 0, kStatusTimeoutGridFlag);
                ok = false;
                break;
              }
            }
          }
          if (!ok) break;
          asm volatile("fence.proxy.async;" ::: "memory");   // generic-proxy stores -> TMA (async proxy) reads
        }
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, p.status, kStatusTimeoutEmpty)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * C::kStageBytes;
          uint8_t* sb = sa + C::kABytes;
          mbar_expect_tx(&bars->full[stage], C::kStageBytes);
          if (!p.a_mn) {
            tma_load_2d(sa, &tma_a, &bars->full[stage], kb * BK, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * 8192, &tma_a, &bars->full[stage], m0 + j * 64, kb * BK);
          }
          if (!p.b_mn) {
            tma_load_2d(sb, &tma_b, &bars->full[stage], kb * BK, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * 8192, &tma_b, &bars->full[stage], n0 + j * 64, kb * BK);
          }
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc =
          make_idesc_f16(p.ab_dtype == kBF16 ? 1 : 0, p.a_mn, p.b_mn, BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const int n_my = sched_count(p, blockIdx.x, gridDim.x, tiles_m, tiles_n);
      for (int it = 0; it < n_my && ok; ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&bars->tmem_empty[acc], acc_phase ^ 1, p.status, kStatusTimeoutTmemEmpty)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&bars->full[stage], phase, p.status, kStatusTimeoutFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * C::kStageBytes);
          const uint32_t sb = sa + C::kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = p.a_mn ? make_smem_desc_sw128(sa + k * 2048, 8192, 1024)
                                       : make_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t db = p.b_mn ? make_smem_desc_sw128(sb + k * 2048, 8192, 1024)
                                       : make_smem_desc_sw128(sb + k * 32, 16, 1024);
            tc_mma_f16(tmem_d, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(&bars->empty[stage]);
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
        tc_commit(&bars->tmem_full[acc]);
      }
    }
  } else if (warp == kPublisherWarp && p.comm.world > 1 && p.comm.mode == 2) {
    // ---------------------------------------------- gather warp (all-gather of A, push model)
    // One warp per CTA copies 8-row units of THIS rank's row block into every peer's operand buffer
    // (posted NVLink stores need no round trip, unlike loads), in increasing row order -- the order
    // in which the peers' tile schedules need them -- and then raises the unit's flag on the peer.
    // A slot of the operand ring is rewritten RING calls later; by then the peer has finished with
    // it, because every call needs the peer's block of the previous call to complete.
    const GemmComm& cm = p.comm;
    const int W = cm.world, me = cm.rank;
    const int rows_per = p.M / W;
    const int units = rows_per / kAgUnitRows;
    const int row_vecs = p.K / 8;                               // 16-byte pieces per row
    const uint16_t* from = reinterpret_cast<const uint16_t*>(cm.stage[me]);
    int pending = 0;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
      const int row0 = me * rows_per + u * kAgUnitRows;
      const int total = kAgUnitRows * row_vecs;
      for (int base = 0; base < total; base += 32 * 16) {
        uint4 v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int idx = base + j * 32 + lane;
          if (idx < total) {
            const int r = idx / row_vecs, c = idx - r * row_vecs;
            v[j] = *reinterpret_cast<const uint4*>(from + static_cast<int64_t>(row0 + r) * p.lda + c * 8);
          }
        }
        for (int d = 0; d < W; ++d) {
          if (d == me) continue;
          uint16_t* to = reinterpret_cast<uint16_t*>(cm.stage[d]);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int idx = base + j * 32 + lane;
            if (idx < total) {
              const int r = idx / row_vecs, c = idx - r * row_vecs;
              *reinterpret_cast<uint4*>(to + static_cast<int64_t>(row0 + r) * p.lda + c * 8) = v[j];
            }
          }
        }
      }
      // a system-scope fence waits for all outstanding NVLink stores: raise the flags of two units at a time
      ++pending;
      if (pending == 2 || u + static_cast<int>(gridDim.x) >= units) {
        __syncwarp();
        if (lane == 0) {
          __threadfence_system();
          for (int q = 0; q < pending; ++q) {
            const int uq = u - q * static_cast<int>(gridDim.x);
            for (int d = 0; d < W; ++d)
              if (d != me)
                st_release_sys(cm.flags[d] + kAgUnitFlags + (me * rows_per) / kAgUnitRows + uq, cm.epoch);
          }
        }
        pending = 0;
      }
    }
  } else if (warp == kPublisherWarp) {
    if (p.comm.world > 1 && elect_one()) {
      const CommSched cs{static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x), tiles_m, tiles_n, false, 0, 0, 0};
      comm_publisher(p, cs, bars);
    }
  } else if (p.comm.world > 1 && p.comm.mode != 2) {
    const CommSched cs{static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x), tiles_m, tiles_n, false, 0, 0, 0};
    comm_epilogue<BN>(p, cs, bars, tmem_base, epi_smem, warp, lane);
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lane quarter this warp may access
    const int row_in_tile = quarter * 32 + lane;
    bool ok = true;
    int tm, tn;
    for (int it = 0; sched_tile(p, blockIdx.x, gridDim.x, it, tiles_m, tiles_n, tm, tn); ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (ok && !mbar_wait(&bars->tmem_full[acc], acc_phase, p.status, kStatusTimeoutTmemFull))
        ok = false;
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      const int col_half = (warp - 2) >> 2;
      epilogue_tile<BN>(p, taddr, tm * BM + row_in_tile, tn * BN, col_half * (BN / 64), (col_half + 1) * (BN / 64));
      tc_fence_before();
      mbar_arrive(&bars->tmem_empty[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------
// CTA-pair variant: a cluster of two CTAs computes one 256 x BN tile. Each CTA loads its own 128
// rows of A and its own half (BN/2 rows) of the B tile, so every byte of B is fetched from L2 once
// per pair instead of once per CTA; the even CTA issues `tcgen05.mma.cta_group::2` (M = 256), which
// reads both CTAs' shared memory and writes 128 accumulator rows into each CTA's TMEM. Barriers:
//   full[s]       leader only; transaction bytes of both CTAs' loads
//   empty[s]      in both CTAs; signalled by the leader's multicast commit
//   tmem_full[a]  in both CTAs; multicast commit after the last k-block
//   tmem_empty[a] leader only; all 512 epilogue threads of the pair arrive on it
// ------------------------------------------------------------------------------------------
template <int BN> struct PairCfg {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = (BN / 2) * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 6 : 8;
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kEpiBytes = 8 * 4096;   // per-epilogue-warp 32 x 128 B transpose buffer
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256 + kEpiBytes;
};

constexpr int kPairThreads = 352;      // producer warp, MMA warp, 8 epilogue warps, publisher warp
constexpr int kPairEpiThreads = 256;

// Tile list of the CTA-pair kernel. The last `tail_split` tiles of the rasterised list are executed
// as two 256 x (BN / 2) halves each: when the last wave of full tiles would leave most pairs idle,
// the halves spread it over twice as many pairs and it takes about half as long.
struct PairTile {
  int tm, tn, n_off, half;
};
__device__ __forceinline__ bool pair_tile(int v, int num_tiles, int tail_split, int tiles_m, int tiles_n,
                                          int half_width, PairTile& t) {
  const int full = num_tiles - tail_split;
  if (v >= full + 2 * tail_split) return false;
  int tile = v;
  t.n_off = 0;
  t.half = 0;
  if (v >= full) {
    const int h = v - full;
    tile = full + (h >> 1);
    t.n_off = (h & 1) * half_width;
    t.half = 1;
  }
  tile_coords(tile, tiles_m, tiles_n, t.tm, t.tn);
  return true;
}

template <int BN>
__global__ void __launch_bounds__(kPairThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tma_a,
                         const __grid_constant__ CUtensorMap tma_b,
                         const __grid_constant__ CUtensorMap tma_b_half, const GemmArgs p,
                         const int tail_split) {
  using C = PairCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  Barriers* bars = reinterpret_cast<Barriers*>(smem + C::kStages * C::kStageBytes);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();      // 0 = leader, 1 = peer
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tmem_full[a], 1);
      mbar_init(&bars->tmem_empty[a], 2 * kPairEpiThreads);
    }
    bars->pub_count = 0;
    bars->rpub_count = 0;
    fence_mbar_init();
    prefetch_tmap(&tma_a);
    prefetch_tmap(&tma_b);
  }
  if (warp == 1) tmem_alloc_pair(&bars->tmem_base, C::kTmemCols);
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      PairTile t;
      const bool fused = p.comm.world > 1;   // tiles owned by peers first, own tiles last (no tail split then)
      const int n_list = pair < num_tiles ? (num_tiles - pair + num_pairs - 1) / num_pairs : 0;
      for (int j = 0; ok; ++j) {
        if (fused && j >= n_list) break;
        const int v = pair + (fused ? comm_order(p.comm, pair, n_list, j) : j) * num_pairs;
        if (!pair_tile(v, num_tiles, tail_split, tiles_m, tiles_n, BN / 2, t)) break;
        const int m0 = t.tm * 2 * BM + static_cast<int>(cta) * BM;
        // this CTA's share of the B tile: BN / 2 rows of a full tile, BN / 4 rows of a half tile
        const int n0 = t.tn * BN + t.n_off + static_cast<int>(cta) * (t.half ? BN / 4 : BN / 2);
        const uint32_t stage_tx = t.half ? C::kABytes + C::kBBytes / 2 : C::kStageBytes;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, p.status, kStatusTimeoutEmpty)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * C::kStageBytes;
          uint8_t* sb = sa + C::kABytes;
          if (cta == 0) mbar_expect_tx(&bars->full[stage], 2 * stage_tx);
          const uint32_t full_leader = mapa_shared(smem_u32(&bars->full[stage]), 0);
          if (!p.a_mn) {
            tma_load_2d_pair(sa, &tma_a, full_leader, kb * BK, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d_pair(sa + j * 8192, &tma_a, full_leader, m0 + j * 64, kb * BK);
          }
          if (!p.b_mn) {
            tma_load_2d_pair(sb, t.half ? &tma_b_half : &tma_b, full_leader, kb * BK, n0);
          } else {
            const int chunks = t.half ? BN / 256 : BN / 128;
            for (int j = 0; j < chunks; ++j)
              tma_load_2d_pair(sb + j * 8192, &tma_b, full_leader, n0 + j * 64, kb * BK);
          }
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
      }
      // Every load issued above has been consumed once the slots it used are free again; wait for
      // that so that no commit arrives in this CTA's shared memory after it has exited.
      for (int i = 0; i < C::kStages && ok; ++i) {
        if (!mbar_wait(&bars->empty[stage], phase ^ 1, p.status, kStatusTimeoutEmpty)) ok = false;
        if (++stage == C::kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (cta == 0 && elect_one()) {
      const uint32_t idesc_full = make_idesc_f16(p.ab_dtype == kBF16 ? 1 : 0, p.a_mn, p.b_mn, 2 * BM, BN);
      const uint32_t idesc_half = make_idesc_f16(p.ab_dtype == kBF16 ? 1 : 0, p.a_mn, p.b_mn, 2 * BM, BN / 2);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      PairTile t;
      for (int v = pair; ok && pair_tile(v, num_tiles, tail_split, tiles_m, tiles_n, BN / 2, t); v += num_pairs, ++it) {
        const uint32_t idesc = t.half ? idesc_half : idesc_full;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&bars->tmem_empty[acc], acc_phase ^ 1, p.status, kStatusTimeoutTmemEmpty)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&bars->full[stage], phase, p.status, kStatusTimeoutFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * C::kStageBytes);
          const uint32_t sb = sa + C::kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = p.a_mn ? make_smem_desc_sw128(sa + k * 2048, 8192, 1024)
                                       : make_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t db = p.b_mn ? make_smem_desc_sw128(sb + k * 2048, 8192, 1024)
                                       : make_smem_desc_sw128(sb + k * 32, 16, 1024);
            tc_mma_f16_pair(tmem_d, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit_pair(&bars->empty[stage], 3);
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit_pair(&bars->tmem_full[acc], 3);
      }
    }
  } else if (warp == kPublisherWarp) {
    if (p.comm.world > 1 && elect_one()) {
      const CommSched cs{static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x), (p.M + BM - 1) / BM, tiles_n,
                         true, pair, num_pairs, static_cast<int>(cta)};
      comm_publisher(p, cs, bars);
    }
  } else if (p.comm.world > 1) {
    // ------------------------------------------------------------------ fused all-reduce epilogue: every CTA of
    // the pair publishes and reduces the 128-row half tiles it computes, as its own virtual CTA
    const CommSched cs{static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x), (p.M + BM - 1) / BM, tiles_n,
                       true, pair, num_pairs, static_cast<int>(cta)};
    comm_epilogue<BN>(p, cs, bars, tmem_base, smem + C::kStages * C::kStageBytes + 256, warp, lane);
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9, both CTAs)
    // A warp may only touch the TMEM lane quarter (warp % 4); two warps share each quarter and
    // split the tile's columns, which halves the drain time of an accumulator.
    const int quarter = warp & 3;
    const int col_half = (warp - 2) >> 2;
    const int row_in_tile = quarter * 32 + lane;
    // The transpose costs shared-memory bandwidth that the MMAs also need, so it is used only where
    // the direct path is slower: a second output or an `aux` operand.
    const bool staged = p.d_dtype != kF32 && !p.accumulate && (p.D2 != nullptr || p.aux_mode != kAuxNone);
    uint8_t* epi_smem = smem + C::kStages * C::kStageBytes + 256;
    int it = 0;
    PairTile t;
    for (int v = pair; pair_tile(v, num_tiles, tail_split, tiles_m, tiles_n, BN / 2, t); v += num_pairs, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait_relaxed(&bars->tmem_full[acc], acc_phase, p.status, kStatusTimeoutTmemFull)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      const int row_base = t.tm * 2 * BM + static_cast<int>(cta) * BM;
      // 32-column chunks of the accumulator for this warp: half of the tile's (or half tile's) columns
      const int chunks = t.half ? BN / 128 : BN / 64;
      const int n_base = t.tn * BN + t.n_off;
      if (staged)
        epilogue_tile_staged<BN>(p, taddr, row_base + quarter * 32, lane, n_base, col_half * chunks,
                                 (col_half + 1) * chunks, epi_smem + (warp - 2) * 4096);
      else
        epilogue_tile<BN>(p, taddr, row_base + row_in_tile, n_base, col_half * chunks, (col_half + 1) * chunks);
      tc_fence_before();
      mbar_arrive_cluster(mapa_shared(smem_u32(&bars->tmem_empty[acc]), 0));
    }
  }

  // Neither CTA may free its TMEM or exit while its partner can still touch its shared memory,
  // barriers or accumulators.
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, C::kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                              const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(sym);
  });
  return fn;
}

}  // namespace

// 2-D tensor map over a 16-bit matrix: `inner` contiguous elements, `outer` rows of stride `ld`
// elements, box {box_inner, box_outer}, 128-byte swizzle, zero fill outside the tensor.
cudaError_t make_tmap_2d_16bit(CUtensorMap* map, const void* base, int dtype, uint64_t inner,
                               uint64_t outer, uint64_t ld, uint32_t box_inner,
                               uint32_t box_outer) {
  EncodeFn fn = get_encode_fn();
  if (!fn) return cudaErrorNotSupported;
  ensure_thread_context();
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld * 2) % 16 != 0)
    return cudaErrorMisalignedAddress;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                       : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                  2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

namespace {

int device_sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return sms;
}

template <int BN>
cudaError_t launch(const GemmArgs& a, cudaStream_t stream) {
  using C = Cfg<BN>;
  CUtensorMap ta, tb;
  cudaError_t e;
  if (!a.a_mn)
    e = make_tmap_2d_16bit(&ta, a.A, a.ab_dtype, a.K, a.M, a.lda, BK, BM);
  else
    e = make_tmap_2d_16bit(&ta, a.A, a.ab_dtype, a.M, a.K, a.lda, 64, BK);
  if (e != cudaSuccess) return e;
  if (!a.b_mn)
    e = make_tmap_2d_16bit(&tb, a.B, a.ab_dtype, a.K, a.N, a.ldb, BK, BN);
  else
    e = make_tmap_2d_16bit(&tb, a.B, a.ab_dtype, a.N, a.K, a.ldb, 64, BK);
  if (e != cudaSuccess) return e;

  static bool attr_set = false;
  if (!attr_set) {
    e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             C::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  const int tiles = ((a.M + BM - 1) / BM) * ((a.N + BN - 1) / BN);
  int sms = a.sm_count > 0 ? a.sm_count : device_sm_count();
  int grid = tiles < sms ? tiles : sms;
  if (a.comm.world > 1 && a.comm.mode == 2) {
    ETHB_RETURN_IF(a.M % (BM * a.comm.world) != 0 || a.a_mn, cudaErrorInvalidValue,
                   "fused all-gather GEMM: M must be a multiple of 128 * world and A row-major");
  } else if (a.comm.world > 1) {
    const int W = a.comm.world;
    if (a.comm.mode == 1) {   // reduce-scatter: the schedule needs W | grid and whole row blocks per rank
      ETHB_RETURN_IF(a.M % (BM * W) != 0, cudaErrorInvalidValue, "fused reduce-scatter: M must be a multiple of 128 * world");
      grid = grid / W * W;
      ETHB_RETURN_IF(grid <= 0, cudaErrorInvalidValue, "fused reduce-scatter: fewer SMs than ranks");
    }
    const int64_t slots = (tiles + W - 1) / W + grid;
    ETHB_RETURN_IF(tiles + grid > a.comm.max_tiles, cudaErrorInvalidValue, "fused collective GEMM: more tiles than flags");
    ETHB_RETURN_IF(slots * W * BM * BN > a.comm.stage_elems, cudaErrorInvalidValue,
                   "fused collective GEMM: staging area too small");
  }
  gemm_tcgen05_kernel<BN><<<grid, kThreads, C::kSmemBytes, stream>>>(ta, tb, a);
  count_launch();
  return cudaGetLastError();
}

// How many CTA pairs the device can keep resident at once (a pair needs two SMs of one
// cluster-capable group; parts with an odd number of usable SMs per group fit fewer than SMs / 2).
template <int BN>
int resident_pairs() {
  static int pairs = -1;
  if (pairs >= 0) return pairs;
  using C = PairCfg<BN>;
  if (cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           C::kSmemBytes) != cudaSuccess) {
    cudaGetLastError();
    return pairs = 0;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * (device_sm_count() / 2));
  cfg.blockDim = dim3(kPairThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_tcgen05_pair_kernel<BN>, &cfg) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  const int cap = device_sm_count() / 2;
  return pairs = (n < cap ? n : cap);
}

template <int BN>
cudaError_t launch_pair(const GemmArgs& a, cudaStream_t stream) {
  using C = PairCfg<BN>;
  CUtensorMap ta, tb;
  cudaError_t e;
  if (!a.a_mn)
    e = make_tmap_2d_16bit(&ta, a.A, a.ab_dtype, a.K, a.M, a.lda, BK, BM);
  else
    e = make_tmap_2d_16bit(&ta, a.A, a.ab_dtype, a.M, a.K, a.lda, 64, BK);
  if (e != cudaSuccess) return e;
  if (!a.b_mn)
    e = make_tmap_2d_16bit(&tb, a.B, a.ab_dtype, a.K, a.N, a.ldb, BK, BN / 2);
  else
    e = make_tmap_2d_16bit(&tb, a.B, a.ab_dtype, a.N, a.K, a.ldb, 64, BK);
  if (e != cudaSuccess) return e;
  CUtensorMap tbh = tb;   // B rows of one CTA for a half tile (K-major B only; MN-major reuses `tb`)
  if (!a.b_mn) {
    e = make_tmap_2d_16bit(&tbh, a.B, a.ab_dtype, a.K, a.N, a.ldb, BK, BN / 4);
    if (e != cudaSuccess) return e;
  }
  static bool attr_set = false;
  if (!attr_set) {
    e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             C::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  const int tiles = ((a.M + 2 * BM - 1) / (2 * BM)) * ((a.N + BN - 1) / BN);
  const int max_pairs = a.sm_count > 0 ? (a.sm_count / 2 < resident_pairs<BN>() ? a.sm_count / 2 : resident_pairs<BN>())
                                       : resident_pairs<BN>();
  if (max_pairs <= 0) return cudaErrorLaunchOutOfResources;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  if (a.comm.world > 1) {
    const int W = a.comm.world;
    const int half_tiles = 2 * tiles;
    const int64_t slots = (half_tiles + W - 1) / W + 2 * pairs;
    ETHB_RETURN_IF(a.comm.mode != 0, cudaErrorInvalidValue, "CTA-pair kernel: only the all-reduce mode is fused");
    ETHB_RETURN_IF(half_tiles + 2 * pairs > a.comm.max_tiles, cudaErrorInvalidValue,
                   "fused all-reduce: more tiles than flags");
    ETHB_RETURN_IF(slots * W * BM * BN > a.comm.stage_elems, cudaErrorInvalidValue,
                   "fused all-reduce: staging area too small");
  }
  // Split the tiles of a last wave that fills at most half of the pairs into 256 x 128 halves.
  int tail_split = 0;
  if (BN == 256 && a.comm.world <= 1 && g_tail_split.load() && tiles > pairs) {
    const int rest = tiles % pairs;
    if (rest > 0 && 2 * rest <= pairs) tail_split = rest;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(kPairThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel<BN>, ta, tb, tbh, a, tail_split);
  count_launch();
  return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace

cudaError_t gemm_tcgen05(const GemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0) return cudaErrorInvalidValue;
  if (a.N % 8 != 0 || a.ldd % 8 != 0) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(a.D) & 15) != 0) return cudaErrorMisalignedAddress;
  if (a.ab_dtype != kF16 && a.ab_dtype != kBF16) return cudaErrorInvalidValue;
  if (a.drop_p != 0.f)
    ETHB_RETURN_IF(!(a.drop_p > 0.f && a.drop_p < 1.f) || a.aux_mode == kAuxGeluGrad || a.D2 != nullptr ||
                       a.accumulate || (a.comm.world > 1 && a.comm.mode != 0),
                   cudaErrorInvalidValue, "epilogue dropout: needs 0 < p < 1 and a plain or residual-add epilogue");
  if (a.comm.world > 1) {
    ETHB_RETURN_IF(a.comm.world > kGemmMaxPeers, cudaErrorInvalidValue, "fused all-reduce: too many peers");
    ETHB_RETURN_IF(a.comm.mode != 2 && (a.d_dtype != a.ab_dtype || a.accumulate || a.D2 != nullptr ||
                                        a.aux_mode == kAuxGeluGrad),
                   cudaErrorInvalidValue, "fused all-reduce: unsupported epilogue");
  }
  const int variant = g_gemm_variant.load();
  if ((a.comm.world <= 1 || a.comm.mode == 0) && variant >= 3)
    return variant == 3 ? launch_pair<128>(a, stream) : launch_pair<256>(a, stream);
  if (variant == 1) return launch<128>(a, stream);
  if (variant == 2 && a.N > 128) return launch<256>(a, stream);
  // Plain GEMMs wider than one 128-column tile run on CTA pairs (256 x 256 tiles): measured faster
  // than either single-CTA tile on every shape of the GPT layers.
  if (variant == 0 && (a.comm.world <= 1 || a.comm.mode == 0) && a.N > 128 && a.M > 128 &&
      resident_pairs<256>() > 0)
    return launch_pair<256>(a, stream);
  // Pick the tile width that minimises (waves x cost per wave).
  const int sms = a.sm_count > 0 ? a.sm_count : device_sm_count();
  const int tm = (a.M + BM - 1) / BM;
  const long t256 = static_cast<long>(tm) * ((a.N + 255) / 256);
  const long t128 = static_cast<long>(tm) * ((a.N + 127) / 128);
  const double c256 = static_cast<double>((t256 + sms - 1) / sms) * 2.0;
  const double c128 = static_cast<double>((t128 + sms - 1) / sms) * 1.08;
  if (a.N > 128 && c256 <= c128) return launch<256>(a, stream);
  return launch<128>(a, stream);
}

}  // namespace ethb
