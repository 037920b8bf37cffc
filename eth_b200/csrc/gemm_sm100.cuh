// C ABI of the tcgen05 GEMM family (see gemm_sm100.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ethb {

// Epilogue of D = alpha * (A x B^T) [+ bias] [op aux] [+ D]:
enum GemmAuxMode : int {
  kAuxNone = 0,
  kAuxAdd = 1,       // value += aux[row, col]                 (residual add)
  kAuxGeluGrad = 2,  // value *= gelu'(aux[row, col])          (dgrad of GEMM-2 fused with dGeLU)
};

constexpr int kGemmMaxPeers = 8;

// Tensor-parallel all-reduce fused into the GEMM epilogue (world > 1). Every pointer array holds
// the addresses of the same symmetric allocation on each rank of the tensor-parallel group:
//   stage[r] : r's staging area for partial tiles, [source rank][owned slot][128 x BN] 16-bit
//   out[r]   : r's copy of the reduced result D (row stride GemmArgs::ldd)
//   flags[r] : r's int32 flags: arrive[tile * kGemmMaxPeers + source] then done[tile] at
//              offset max_tiles * kGemmMaxPeers
// Tiles are owned round-robin along each CTA's tile list. All-reduce: every rank first computes the
// tiles its peers own and stores those partials into the owners' staging areas, then its own tiles,
// whose accumulators it sums in fp32 with the partials that have arrived meanwhile, applies
// bias / residual, and writes the result into every rank's `out`. `epoch` must increase with every
// call that uses the same flags.
struct GemmComm {
  int world, rank, epoch, max_tiles;
  void* stage[kGemmMaxPeers];
  void* out[kGemmMaxPeers];
  int* flags[kGemmMaxPeers];
  int64_t stage_elems;  // capacity of one rank's staging area in 16-bit elements
  // 0: all-reduce (every rank receives the full [M, N] result).
  // 1: reduce-scatter along rows: rank r receives rows [r * M / world, (r + 1) * M / world) of the sum
  //    in its own `out[rank]` buffer of M / world rows; M must be a multiple of 128 * world. Tiles of a
  //    rank's row block are owned by that rank, so reduced data never crosses NVLink a second time.
  // 2: all-gather of A, then a plain GEMM. `stage[r]` is rank r's [M, K] operand buffer (row stride
  //    lda) in which rank r has filled its own row block [r * M / world, (r + 1) * M / world) before
  //    the call; the kernel pushes that block into every peer's buffer over NVLink (8 rows per step,
  //    plain peer stores, one flag per step) while the MMAs already work on the local rows, and
  //    computes the full [M, N] product with the usual epilogue; tiles of a peer's rows wait for
  //    those rows only. `out` is unused. M must be a multiple of 128 * world. A buffer may be reused
  //    for this mode after two further calls on the same flags.
  int mode;
};

struct GemmArgs {
  // problem: D[M,N] = sum_k A(m,k) * B(n,k)
  int M, N, K;
  // operand layouts in global memory (16-bit elements, fp16 or bf16):
  //   a_mn == 0: A is [M, K] with K contiguous, row stride lda.   a_mn == 1: A is [K, M], M contiguous.
  //   b_mn == 0: B is [N, K] with K contiguous, row stride ldb.   b_mn == 1: B is [K, N], N contiguous.
  const void* A; int64_t lda; int a_mn;
  const void* B; int64_t ldb; int b_mn;
  int ab_dtype;  // kF16 or kBF16
  // outputs
  void* D; int64_t ldd; int d_dtype;  // kF32 / kF16 / kBF16
  void* D2;                          // optional gelu(value) output, same ld and dtype as A/B
  const void* bias;                  // optional [N], ab_dtype
  const void* aux; int64_t ldaux; int aux_mode;  // optional [M,N], ab_dtype
  int accumulate;                    // D += value instead of D = value
  // Optional dropout of (alpha * acc + bias), applied before `aux` is added (aux_mode none or
  // add): the bias-dropout-add of a transformer sub-block in the epilogue of its output GEMM. The
  // mask is that of a contiguous [M, N] tensor (sm100_common.cuh: keep8); needs N % 8 == 0.
  float drop_p;                      // 0 = no dropout
  unsigned long long drop_seed, drop_offset;
  float alpha;
  int* status;                       // device status word (0 == ok)
  int sm_count;                      // CTAs to launch at most (0 = all SMs)
  GemmComm comm;                     // comm.world <= 1: plain GEMM
};

// Returns cudaSuccess or the launch/encode error. Never allocates.
cudaError_t gemm_tcgen05(const GemmArgs& args, cudaStream_t stream);
// Kernel choice for plain GEMMs: 0 = automatic, 1 / 2 = one CTA per 128 x 128 / 128 x 256 tile,
// 3 / 4 = CTA pair per 256 x 128 / 256 x 256 tile. Meant for tests and benchmarks.
void set_gemm_variant(int v);
// Splitting of a sparsely filled last wave of the CTA-pair kernel into half tiles (default on).
void set_gemm_tail_split(int on);

// Where the last failing launcher of this thread gave up (empty if none).
void ensure_thread_context();
const char* last_error_detail();
void set_error_detail(const char* where);
#define ETHB_RETURN_IF(cond, err, where) \
  do { if (cond) { ::ethb::set_error_detail(where); return (err); } } while (0)
#define ETHB_TRY(expr, where) \
  do { cudaError_t e__ = (expr); if (e__ != cudaSuccess) { ::ethb::set_error_detail(where); return e__; } } while (0)

// Number of kernel launches made by this library since load (for bench accounting).
int64_t launch_count();
void count_launch(int n = 1);

}  // namespace ethb
