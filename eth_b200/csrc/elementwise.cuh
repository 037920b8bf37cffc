// C++ launchers of the bandwidth-bound kernels (LayerNorm, GeLU, dropout-add, softmax family,
// embedding, cross-entropy, column sums, optimizer, gradient pack/unpack). All take raw device
// pointers and a stream, never allocate, and return the launch error.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ethb {

// ---- LayerNorm (fp32 statistics; x/y/gamma/beta share one 16-bit or fp32 dtype) -----------
cudaError_t layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y,
                          float* mean, float* rstd, int rows, int hidden, float eps, int dtype,
                          cudaStream_t st);
// What happens to the per-CTA partial column sums ("slabs") that a kernel leaves in its workspace:
//   kWsImmediate   slabs are overwritten and summed into the output by a second launch right away;
//   kWsAccumulate  the kernel ADDS its partials to the slabs and nothing else happens: the caller
//                  keeps one zero-initialised workspace per op across the micro-batches of a step,
//                  which takes the second launch off the critical path of every backward;
//   kWsFlush       as kWsAccumulate, then the slabs are summed into the output and cleared
//                  (the last micro-batch of a step).
enum WorkspaceMode : int { kWsImmediate = 0, kWsAccumulate = 1, kWsFlush = 2 };

// Workspace: `ws` holds 2 * ln_bwd_parts(rows, hidden, dtype) * hidden floats (partial dgamma |
// partial dbeta).
int ln_bwd_parts(int rows, int hidden, int dtype);
// Whether the one-kernel backward (and with it kWsAccumulate / kWsFlush) handles this width and type.
bool ln_bwd_fused_ok(int hidden, int dtype);
// `dres` (may be null): a gradient of the same shape that is added to dx, i.e. the gradient that
// reaches the LayerNorm input through the residual branch.
cudaError_t layernorm_bwd(const void* dy, const void* x, const void* gamma, const float* mean,
                          const float* rstd, const void* dres, void* dx, void* dgamma, void* dbeta,
                          float* ws, int rows, int hidden, int dtype, int grad_dtype, int accumulate,
                          cudaStream_t st, int ws_mode = kWsImmediate);

// ---- bias + GeLU(tanh) ----------------------------------------------------------------------
cudaError_t bias_gelu_fwd(const void* x, const void* bias, void* y, int64_t rows, int cols,
                          int dtype, cudaStream_t st);
cudaError_t bias_gelu_bwd(const void* dy, const void* x, const void* bias, void* dx, int64_t rows,
                          int cols, int dtype, cudaStream_t st);

// ---- out = residual + dropout(x + bias) ------------------------------------------------------
// The keep-mask is a pure function of (seed, offset, element index), so backward regenerates it.
cudaError_t bias_dropout_add_fwd(const void* x, const void* bias, const void* residual, void* out,
                                 int64_t rows, int cols, float p, uint64_t seed, uint64_t offset,
                                 int dtype, cudaStream_t st);
cudaError_t dropout_bwd(const void* dy, void* dx, int64_t rows, int cols, float p, uint64_t seed,
                        uint64_t offset, int dtype, cudaStream_t st);
// dx = dropout_bwd(dy) and bias_grad (+)= column sums of dx, in one pass over dy. Workspace:
// dropout_bwd_colsum_parts(rows, cols, dtype) * cols floats; 0 parts means "shape not supported,
// call dropout_bwd and colsum separately".
int dropout_bwd_colsum_parts(int64_t rows, int cols, int dtype);
cudaError_t dropout_bwd_colsum(const void* dy, void* dx, void* bias_grad, float* ws, int64_t rows,
                               int cols, float p, uint64_t seed, uint64_t offset, int dtype,
                               int grad_dtype, int accumulate, cudaStream_t st, int ws_mode = kWsImmediate);

// ---- column sums: out[c] (+)= sum_r x[r, c]  (bias gradients) -----------------------------
// Workspace: colsum_parts(rows) * cols floats.
int colsum_parts(int64_t rows);
cudaError_t colsum(const void* x, void* out, float* ws, int64_t rows, int cols, int dtype,
                   int out_dtype, int accumulate, cudaStream_t st);

// ---- softmax family (legacy 13-op attention path) ---------------------------------------------
// mode 0: plain, 1: causal (upper-triangular masked, x is [batch, sq, sk] with sq == sk),
// mode 2: explicit uint8 mask [mask_batch, sq, sk] (1 == masked -> -10000).
cudaError_t softmax_fwd(const void* x, const uint8_t* mask, void* y, int64_t batches, int heads,
                        int sq, int sk, float scale, int mode, int mask_batch, int dtype,
                        cudaStream_t st);
cudaError_t softmax_bwd(const void* dy, const void* y, void* dx, int64_t rows, int sq, int sk,
                        float scale, int mode, int dtype, cudaStream_t st);

// ---- embedding ----------------------------------------------------------------------------------
// out[t, :] = (vocab_start <= tok[t] < vocab_end ? word[tok[t]-vocab_start] : 0) + (add_pos ? pos[t % seq] : 0)
cudaError_t embedding_fwd(const int64_t* tokens, const void* word, const void* pos, void* out,
                          int64_t ntok, int seq, int hidden, int vocab_start, int vocab_end,
                          int add_pos, int dtype, cudaStream_t st);
// Scatter-add of dout rows into the word/position gradient buffers (grad dtype fp32 or 16-bit).
cudaError_t embedding_bwd(const int64_t* tokens, const void* dout, void* dword, void* dpos,
                          int64_t ntok, int seq, int hidden, int vocab_start, int vocab_end,
                          int add_pos, int dtype, int grad_dtype, cudaStream_t st);

// ---- vocab-parallel cross entropy -----------------------------------------------------------
// stats[row] = {local max, sum exp(x - local max), target logit or 0 when the target lives on another shard}
cudaError_t ce_local_stats(const void* logits, const int64_t* targets, float* stats, int64_t rows,
                           int vocab_local, int64_t ld, int vocab_start, int dtype,
                           cudaStream_t st);
// Combine `world` stats blocks ([world, rows, 3]) into loss[row], and keep gmax/gsum for backward.
cudaError_t ce_combine(const float* stats_all, float* loss, float* gmax, float* gsum, int64_t rows,
                       int world, cudaStream_t st);
// logits <- (softmax - onehot) * dloss[row]   (in place, 16-bit or fp32)
cudaError_t ce_bwd(void* logits, const int64_t* targets, const float* gmax, const float* gsum,
                   const float* dloss, int64_t rows, int vocab_local, int64_t ld, int vocab_start,
                   int dtype, cudaStream_t st);

// ---- optimizer -----------------------------------------------------------------------------------
// acc[0] += sum((g * inv_scale)^2), acc[1] = 1 if any non-finite value was seen.
cudaError_t grad_norm_sq(const void* grad, int64_t n, int grad_dtype, float inv_scale, float* acc,
                         cudaStream_t st);
struct AdamArgs {
  void* param;          // 16-bit or fp32 model parameter (written)
  float* master;        // fp32 master copy (may alias param when param is fp32)
  const void* grad;     // main_grad, grad_dtype
  float* exp_avg;
  float* exp_avg_sq;
  int64_t n;
  int param_dtype, grad_dtype;
  float lr, beta1, beta2, eps, weight_decay;
  float bias_correction1, bias_correction2;
  // Device scalars so no host synchronisation is needed:
  //   ctrl[0] = sum of squares of the (still loss-scaled) gradients over the whole model,
  //   ctrl[1] = found-inf flag, ctrl[2] = raw-to-true gradient factor (read when scale_from_ctrl != 0)
  const float* ctrl;
  int scale_from_ctrl;
  float inv_scale;      // raw-to-true gradient factor from the host (used when scale_from_ctrl == 0)
  float max_norm;       // <= 0 disables clipping
  int adamw;            // decoupled weight decay
};
cudaError_t fused_adam(const AdamArgs& a, cudaStream_t st);

// ---- gradient bucket pack / unpack -----------------------------------------------------------
// A segment copies `rows` runs of `run` elements: src + r*src_stride -> dst + r*dst_stride,
// multiplying by `scale`. The table lives in device memory.
struct CopySegment {
  const void* src;
  void* dst;
  int64_t rows, run, src_stride, dst_stride;
};
cudaError_t strided_copy_scale(const CopySegment* segs_dev, int nsegs, int64_t max_elems,
                               float scale, int src_dtype, int dst_dtype, cudaStream_t st);
cudaError_t scale_inplace(void* x, int64_t n, float scale, int dtype, cudaStream_t st);

// ---- synthetic batch (tokens, loss mask) ------------------------------------------------------
cudaError_t synthetic_batch(int64_t* tokens, int64_t* labels, float* loss_mask,
                            const int64_t* sample_ids, int nsamples, int seq, int vocab,
                            cudaStream_t st);

}  // namespace ethb
