// pybind11 / ATen bindings of the native library. Every function takes pre-allocated tensors and
// launches on the current CUDA stream; nothing here allocates device memory except where a
// function says so (peer-memory set-up).
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "attention_sm100.cuh"
#include "comm.cuh"
#include "elementwise.cuh"
#include "gemm_sm100.cuh"

namespace {

using torch::Tensor;
using OptTensor = c10::optional<Tensor>;

int dtype_code(const Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return 0;
    case at::kHalf: return 1;
    case at::kBFloat16: return 2;
    default: TORCH_CHECK(false, "unsupported dtype ", t.scalar_type());
  }
}
cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
void check(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e), " [", ethb::last_error_detail(), "]");
}
const void* optptr(const OptTensor& t) { return t.has_value() ? t->data_ptr() : nullptr; }
void need_cuda(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
}

// D[M,N] = alpha * A x B^T (+bias)(aux op)(+D).  A: [M,K] (a_mn=0) or [K,M] (a_mn=1);
// B: [N,K] (b_mn=0) or [K,N] (b_mn=1). Row strides are taken from the tensors.
void gemm(const Tensor& a, bool a_mn, const Tensor& b, bool b_mn, Tensor& d, const OptTensor& bias,
          const OptTensor& aux, int64_t aux_mode, const OptTensor& d2, bool accumulate,
          double alpha, const OptTensor& status, int64_t sm_count, double drop_p, int64_t drop_seed,
          int64_t drop_offset) {
  need_cuda(a, "a"); need_cuda(b, "b"); need_cuda(d, "d");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && d.dim() == 2, "gemm expects 2-D tensors");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && d.stride(1) == 1, "inner stride must be 1");
  TORCH_CHECK(a.scalar_type() == b.scalar_type(), "a/b dtype mismatch");
  c10::cuda::CUDAGuard guard(a.device());
  ethb::GemmArgs g{};
  g.M = static_cast<int>(a_mn ? a.size(1) : a.size(0));
  g.K = static_cast<int>(a_mn ? a.size(0) : a.size(1));
  g.N = static_cast<int>(b_mn ? b.size(1) : b.size(0));
  const int64_t kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(kb == g.K, "reduction dims differ: ", g.K, " vs ", kb);
  TORCH_CHECK(d.size(0) == g.M && d.size(1) == g.N, "bad output shape");
  g.A = a.data_ptr(); g.lda = a.stride(0); g.a_mn = a_mn;
  g.B = b.data_ptr(); g.ldb = b.stride(0); g.b_mn = b_mn;
  g.ab_dtype = dtype_code(a);
  TORCH_CHECK(g.ab_dtype != 0, "gemm operands must be fp16/bf16");
  g.D = d.data_ptr(); g.ldd = d.stride(0); g.d_dtype = dtype_code(d);
  g.D2 = nullptr;
  if (d2.has_value()) {
    TORCH_CHECK(d2->scalar_type() == a.scalar_type() && d2->stride(0) == d.stride(0) &&
                    d.scalar_type() == a.scalar_type(), "d2 must match d");
    g.D2 = d2->data_ptr();
  }
  g.bias = optptr(bias);
  if (bias.has_value()) TORCH_CHECK(bias->scalar_type() == a.scalar_type() && bias->numel() == g.N);
  g.aux = optptr(aux);
  g.ldaux = aux.has_value() ? aux->stride(0) : 0;
  g.aux_mode = aux.has_value() ? static_cast<int>(aux_mode) : 0;
  if (aux.has_value()) TORCH_CHECK(aux->scalar_type() == a.scalar_type() && aux->stride(1) == 1);
  g.accumulate = accumulate;
  g.alpha = static_cast<float>(alpha);
  g.status = status.has_value() ? status->data_ptr<int>() : nullptr;
  g.sm_count = static_cast<int>(sm_count);
  g.drop_p = static_cast<float>(drop_p);
  g.drop_seed = static_cast<unsigned long long>(drop_seed);
  g.drop_offset = static_cast<unsigned long long>(drop_offset);
  if (drop_p != 0.0) TORCH_CHECK(d.is_contiguous(), "epilogue dropout draws the mask of a contiguous output");
  check(ethb::gemm_tcgen05(g, cur_stream()), "gemm_tcgen05");
}

// Batched GEMM over two leading batch dimensions: d[i, j] = alpha * a[i, j] x b[i, j]^T (+ d[i, j]).
// a, b, d are 4-D views [B1, B2, rows, cols] with unit inner stride and arbitrary other strides, so
// the per-head q / k / v slices of a packed QKV activation are used in place. One launch of the
// tcgen05 GEMM per (i, j): the score (Q K^T) and context (P V) products of the unfused attention ops.
void gemm_batched(const Tensor& a, bool a_mn, const Tensor& b, bool b_mn, Tensor& d, double alpha,
                  bool accumulate, const OptTensor& status) {
  need_cuda(a, "a"); need_cuda(b, "b"); need_cuda(d, "d");
  TORCH_CHECK(a.dim() == 4 && b.dim() == 4 && d.dim() == 4, "gemm_batched expects 4-D views");
  TORCH_CHECK(a.stride(3) == 1 && b.stride(3) == 1 && d.stride(3) == 1, "inner stride must be 1");
  TORCH_CHECK(a.scalar_type() == b.scalar_type(), "a/b dtype mismatch");
  TORCH_CHECK(a.size(0) == b.size(0) && a.size(0) == d.size(0) && a.size(1) == b.size(1) && a.size(1) == d.size(1),
              "batch dimensions differ");
  c10::cuda::CUDAGuard guard(a.device());
  ethb::GemmArgs g{};
  g.M = static_cast<int>(a_mn ? a.size(3) : a.size(2));
  g.K = static_cast<int>(a_mn ? a.size(2) : a.size(3));
  g.N = static_cast<int>(b_mn ? b.size(3) : b.size(2));
  TORCH_CHECK((b_mn ? b.size(2) : b.size(3)) == g.K, "reduction dims differ");
  TORCH_CHECK(d.size(2) == g.M && d.size(3) == g.N, "bad output shape");
  g.lda = a.stride(2); g.a_mn = a_mn;
  g.ldb = b.stride(2); g.b_mn = b_mn;
  g.ldd = d.stride(2);
  g.ab_dtype = dtype_code(a);
  TORCH_CHECK(g.ab_dtype != 0, "gemm operands must be fp16/bf16");
  g.d_dtype = dtype_code(d);
  g.accumulate = accumulate;
  g.alpha = static_cast<float>(alpha);
  g.status = status.has_value() ? status->data_ptr<int>() : nullptr;
  const int64_t ea = a.element_size(), ed = d.element_size();
  auto stream = cur_stream();
  for (int64_t i = 0; i < a.size(0); ++i)
    for (int64_t j = 0; j < a.size(1); ++j) {
      g.A = static_cast<const char*>(a.data_ptr()) + (i * a.stride(0) + j * a.stride(1)) * ea;
      g.B = static_cast<const char*>(b.data_ptr()) + (i * b.stride(0) + j * b.stride(1)) * ea;
      g.D = static_cast<char*>(d.data_ptr()) + (i * d.stride(0) + j * d.stride(1)) * ed;
      check(ethb::gemm_tcgen05(g, stream), "gemm_batched");
    }
}

// GEMM fused with the tensor-parallel all-reduce. The result lands in every rank's `out` buffer
// (`out_ptrs[rank]` is this rank's, M x N with row stride ldd).
void gemm_allreduce(const Tensor& a, bool a_mn, const Tensor& b, bool b_mn, const OptTensor& bias,
                    const OptTensor& aux, double alpha, const OptTensor& status,
                    const std::vector<int64_t>& stage_ptrs, const std::vector<int64_t>& out_ptrs,
                    const std::vector<int64_t>& flag_ptrs, int64_t rank, int64_t epoch, int64_t max_tiles,
                    int64_t stage_elems, int64_t ldd, int64_t mode, double drop_p, int64_t drop_seed,
                    int64_t drop_offset) {
  need_cuda(a, "a"); need_cuda(b, "b");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1);
  TORCH_CHECK(a.scalar_type() == b.scalar_type(), "a/b dtype mismatch");
  c10::cuda::CUDAGuard guard(a.device());
  ethb::GemmArgs g{};
  g.M = static_cast<int>(a_mn ? a.size(1) : a.size(0));
  g.K = static_cast<int>(a_mn ? a.size(0) : a.size(1));
  g.N = static_cast<int>(b_mn ? b.size(1) : b.size(0));
  TORCH_CHECK((b_mn ? b.size(0) : b.size(1)) == g.K, "reduction dims differ");
  g.A = a.data_ptr(); g.lda = a.stride(0); g.a_mn = a_mn;
  g.B = b.data_ptr(); g.ldb = b.stride(0); g.b_mn = b_mn;
  g.ab_dtype = dtype_code(a);
  g.d_dtype = g.ab_dtype;
  const size_t w = stage_ptrs.size();
  TORCH_CHECK(w >= 2 && w <= ethb::kGemmMaxPeers && out_ptrs.size() == w && flag_ptrs.size() == w);
  g.D = reinterpret_cast<void*>(out_ptrs[rank]);
  g.ldd = ldd;
  g.bias = optptr(bias);
  if (bias.has_value()) TORCH_CHECK(bias->scalar_type() == a.scalar_type() && bias->numel() == g.N);
  g.aux = optptr(aux);
  g.ldaux = aux.has_value() ? aux->stride(0) : 0;
  g.aux_mode = aux.has_value() ? 1 : 0;
  g.alpha = static_cast<float>(alpha);
  g.status = status.has_value() ? status->data_ptr<int>() : nullptr;
  g.comm.world = static_cast<int>(w);
  g.comm.rank = static_cast<int>(rank);
  g.comm.epoch = static_cast<int>(epoch);
  g.comm.max_tiles = static_cast<int>(max_tiles);
  g.comm.stage_elems = stage_elems;
  g.comm.mode = static_cast<int>(mode);
  g.drop_p = static_cast<float>(drop_p);
  g.drop_seed = static_cast<unsigned long long>(drop_seed);
  g.drop_offset = static_cast<unsigned long long>(drop_offset);
  if (drop_p != 0.0) TORCH_CHECK(ldd == g.N, "epilogue dropout draws the mask of a contiguous output");
  for (size_t i = 0; i < w; ++i) {
    g.comm.stage[i] = reinterpret_cast<void*>(stage_ptrs[i]);
    g.comm.out[i] = reinterpret_cast<void*>(out_ptrs[i]);
    g.comm.flags[i] = reinterpret_cast<int*>(flag_ptrs[i]);
  }
  check(ethb::gemm_tcgen05(g, cur_stream()), "gemm_allreduce");
}

// All-gather of the row-sharded operand fused into the GEMM that consumes it (GemmComm mode 2).
// `a_full` is this rank's [M, K] operand buffer inside a symmetric allocation; a_ptrs are the base
// addresses of that buffer on every rank of the group.
void gemm_allgather(const Tensor& a_full, const Tensor& b, bool b_mn, Tensor& d, const OptTensor& bias,
                    const OptTensor& d2, const OptTensor& status, const std::vector<int64_t>& a_ptrs,
                    const std::vector<int64_t>& flag_ptrs, int64_t rank, int64_t epoch) {
  need_cuda(a_full, "a_full"); need_cuda(b, "b"); need_cuda(d, "d");
  TORCH_CHECK(a_full.dim() == 2 && b.dim() == 2 && d.dim() == 2 && a_full.stride(1) == 1 && b.stride(1) == 1 &&
              d.stride(1) == 1);
  TORCH_CHECK(a_full.scalar_type() == b.scalar_type(), "a/b dtype mismatch");
  c10::cuda::CUDAGuard guard(a_full.device());
  ethb::GemmArgs g{};
  g.M = static_cast<int>(a_full.size(0));
  g.K = static_cast<int>(a_full.size(1));
  g.N = static_cast<int>(b_mn ? b.size(1) : b.size(0));
  TORCH_CHECK((b_mn ? b.size(0) : b.size(1)) == g.K, "reduction dims differ");
  TORCH_CHECK(d.size(0) == g.M && d.size(1) == g.N, "bad output shape");
  TORCH_CHECK(g.K % 8 == 0, "K must be a multiple of 8");
  g.A = a_full.data_ptr(); g.lda = a_full.stride(0); g.a_mn = 0;
  g.B = b.data_ptr(); g.ldb = b.stride(0); g.b_mn = b_mn;
  g.ab_dtype = dtype_code(a_full);
  g.D = d.data_ptr(); g.ldd = d.stride(0); g.d_dtype = dtype_code(d);
  if (d2.has_value()) {
    TORCH_CHECK(d2->scalar_type() == a_full.scalar_type() && d2->stride(0) == d.stride(0) &&
                    d.scalar_type() == a_full.scalar_type(), "d2 must match d");
    g.D2 = d2->data_ptr();
  }
  g.bias = optptr(bias);
  if (bias.has_value()) TORCH_CHECK(bias->scalar_type() == a_full.scalar_type() && bias->numel() == g.N);
  g.alpha = 1.0f;
  g.status = status.has_value() ? status->data_ptr<int>() : nullptr;
  const size_t w = a_ptrs.size();
  TORCH_CHECK(w >= 2 && w <= ethb::kGemmMaxPeers && flag_ptrs.size() == w);
  TORCH_CHECK(reinterpret_cast<int64_t>(a_full.data_ptr()) == a_ptrs[rank], "a_full must be this rank's buffer");
  g.comm.world = static_cast<int>(w);
  g.comm.rank = static_cast<int>(rank);
  g.comm.epoch = static_cast<int>(epoch);
  g.comm.mode = 2;
  for (size_t i = 0; i < w; ++i) {
    g.comm.stage[i] = reinterpret_cast<void*>(a_ptrs[i]);
    g.comm.flags[i] = reinterpret_cast<int*>(flag_ptrs[i]);
  }
  check(ethb::gemm_tcgen05(g, cur_stream()), "gemm_allgather");
}

void layernorm_fwd(const Tensor& x, const Tensor& gamma, const Tensor& beta, Tensor& y,
                   Tensor& mean, Tensor& rstd, double eps) {
  need_cuda(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int hidden = static_cast<int>(x.size(-1));
  const int rows = static_cast<int>(x.numel() / hidden);
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous());
  check(ethb::layernorm_fwd(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), y.data_ptr(),
                            mean.data_ptr<float>(), rstd.data_ptr<float>(), rows, hidden,
                            static_cast<float>(eps), dtype_code(x), cur_stream()),
        "layernorm_fwd");
}
int64_t ln_bwd_parts(int64_t rows, int64_t hidden, bool fp32) {
  return ethb::ln_bwd_parts(static_cast<int>(rows), static_cast<int>(hidden), fp32 ? 0 : 2);
}
void layernorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& gamma, const Tensor& mean,
                   const Tensor& rstd, Tensor& dx, Tensor& dgamma, Tensor& dbeta, Tensor& ws,
                   bool accumulate, const c10::optional<Tensor>& dres, int64_t ws_mode) {
  c10::cuda::CUDAGuard guard(x.device());
  const int hidden = static_cast<int>(x.size(-1));
  const int rows = static_cast<int>(x.numel() / hidden);
  TORCH_CHECK(ws.numel() >= 2LL * ethb::ln_bwd_parts(rows, hidden, dtype_code(x)) * hidden, "ln workspace too small");
  TORCH_CHECK(dy.is_contiguous() && x.is_contiguous() && dx.is_contiguous());
  const void* res = nullptr;
  if (dres.has_value()) {
    TORCH_CHECK(dres->is_contiguous() && dres->numel() == x.numel() && dres->scalar_type() == x.scalar_type());
    res = dres->data_ptr();
  }
  check(ethb::layernorm_bwd(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr<float>(),
                            rstd.data_ptr<float>(), res, dx.data_ptr(), dgamma.data_ptr(),
                            dbeta.data_ptr(), ws.data_ptr<float>(), rows, hidden, dtype_code(x),
                            dtype_code(dgamma), accumulate, cur_stream(), static_cast<int>(ws_mode)),
        "layernorm_bwd");
}

void bias_gelu_fwd(const Tensor& x, const OptTensor& bias, Tensor& y) {
  c10::cuda::CUDAGuard guard(x.device());
  const int cols = static_cast<int>(x.size(-1));
  check(ethb::bias_gelu_fwd(x.data_ptr(), optptr(bias), y.data_ptr(), x.numel() / cols, cols,
                            dtype_code(x), cur_stream()), "bias_gelu_fwd");
}
void bias_gelu_bwd(const Tensor& dy, const Tensor& x, const OptTensor& bias, Tensor& dx) {
  c10::cuda::CUDAGuard guard(x.device());
  const int cols = static_cast<int>(x.size(-1));
  check(ethb::bias_gelu_bwd(dy.data_ptr(), x.data_ptr(), optptr(bias), dx.data_ptr(),
                            x.numel() / cols, cols, dtype_code(x), cur_stream()), "bias_gelu_bwd");
}
void bias_dropout_add_fwd(const Tensor& x, const OptTensor& bias, const OptTensor& residual,
                          Tensor& out, double p, int64_t seed, int64_t offset) {
  c10::cuda::CUDAGuard guard(x.device());
  const int cols = static_cast<int>(x.size(-1));
  check(ethb::bias_dropout_add_fwd(x.data_ptr(), optptr(bias), optptr(residual), out.data_ptr(),
                                   x.numel() / cols, cols, static_cast<float>(p),
                                   static_cast<uint64_t>(seed), static_cast<uint64_t>(offset),
                                   dtype_code(x), cur_stream()), "bias_dropout_add_fwd");
}
void dropout_bwd(const Tensor& dy, Tensor& dx, double p, int64_t seed, int64_t offset) {
  c10::cuda::CUDAGuard guard(dy.device());
  const int cols = static_cast<int>(dy.size(-1));
  check(ethb::dropout_bwd(dy.data_ptr(), dx.data_ptr(), dy.numel() / cols, cols,
                          static_cast<float>(p), static_cast<uint64_t>(seed),
                          static_cast<uint64_t>(offset), dtype_code(dy), cur_stream()),
        "dropout_bwd");
}
int64_t dropout_bwd_colsum_parts(int64_t rows, int64_t cols, bool fp32) {
  return ethb::dropout_bwd_colsum_parts(rows, static_cast<int>(cols), fp32 ? 0 : 2);
}
void dropout_bwd_colsum(const Tensor& dy, Tensor& dx, Tensor& bias_grad, Tensor& ws, double p, int64_t seed,
                        int64_t offset, bool accumulate, int64_t ws_mode) {
  c10::cuda::CUDAGuard guard(dy.device());
  const int cols = static_cast<int>(dy.size(-1));
  const int64_t rows = dy.numel() / cols;
  TORCH_CHECK(dy.is_contiguous() && dx.is_contiguous() && bias_grad.numel() == cols);
  const int parts = ethb::dropout_bwd_colsum_parts(rows, cols, dtype_code(dy));
  TORCH_CHECK(parts > 0, "dropout_bwd_colsum: unsupported shape");
  TORCH_CHECK(ws.numel() >= static_cast<int64_t>(parts) * cols, "dropout_bwd_colsum workspace too small");
  check(ethb::dropout_bwd_colsum(dy.data_ptr(), dx.data_ptr(), bias_grad.data_ptr(), ws.data_ptr<float>(), rows,
                                 cols, static_cast<float>(p), static_cast<uint64_t>(seed),
                                 static_cast<uint64_t>(offset), dtype_code(dy), dtype_code(bias_grad),
                                 accumulate, cur_stream(), static_cast<int>(ws_mode)),
        "dropout_bwd_colsum");
}
int64_t colsum_parts(int64_t rows) { return ethb::colsum_parts(rows); }
void colsum(const Tensor& x, Tensor& out, Tensor& ws, bool accumulate) {
  c10::cuda::CUDAGuard guard(x.device());
  const int cols = static_cast<int>(x.size(-1));
  const int64_t rows = x.numel() / cols;
  TORCH_CHECK(x.is_contiguous());
  TORCH_CHECK(ws.numel() >= ethb::colsum_parts(rows) * static_cast<int64_t>(cols));
  check(ethb::colsum(x.data_ptr(), out.data_ptr(), ws.data_ptr<float>(), rows, cols, dtype_code(x),
                     dtype_code(out), accumulate, cur_stream()), "colsum");
}

void softmax_fwd(const Tensor& x, const OptTensor& mask, Tensor& y, double scale, int64_t mode) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && x.dim() >= 3);
  const int sk = static_cast<int>(x.size(-1)), sq = static_cast<int>(x.size(-2));
  int heads = 1;
  int64_t batches = x.numel() / (static_cast<int64_t>(sq) * sk);
  int mask_batch = 1;
  if (x.dim() == 4) { heads = static_cast<int>(x.size(1)); batches = x.size(0); }
  if (mask.has_value()) mask_batch = static_cast<int>(mask->size(0));
  check(ethb::softmax_fwd(x.data_ptr(), mask.has_value() ? mask->data_ptr<uint8_t>() : nullptr,
                          y.data_ptr(), batches, heads, sq, sk, static_cast<float>(scale),
                          static_cast<int>(mode), mask_batch, dtype_code(x), cur_stream()),
        "softmax_fwd");
}
void softmax_bwd(const Tensor& dy, const Tensor& y, Tensor& dx, double scale, int64_t mode) {
  c10::cuda::CUDAGuard guard(y.device());
  const int sk = static_cast<int>(y.size(-1)), sq = static_cast<int>(y.size(-2));
  check(ethb::softmax_bwd(dy.data_ptr(), y.data_ptr(), dx.data_ptr(), y.numel() / sk, sq, sk,
                          static_cast<float>(scale), static_cast<int>(mode), dtype_code(y),
                          cur_stream()), "softmax_bwd");
}

void embedding_fwd(const Tensor& tokens, const Tensor& word, const Tensor& pos, Tensor& out,
                   int64_t seq, int64_t vocab_start, bool add_pos) {
  c10::cuda::CUDAGuard guard(word.device());
  TORCH_CHECK(tokens.scalar_type() == at::kLong && tokens.is_contiguous());
  const int hidden = static_cast<int>(word.size(1));
  check(ethb::embedding_fwd(tokens.data_ptr<int64_t>(), word.data_ptr(), pos.data_ptr(),
                            out.data_ptr(), tokens.numel(), static_cast<int>(seq), hidden,
                            static_cast<int>(vocab_start),
                            static_cast<int>(vocab_start + word.size(0)), add_pos,
                            dtype_code(word), cur_stream()), "embedding_fwd");
}
void embedding_bwd(const Tensor& tokens, const Tensor& dout, Tensor& dword, const OptTensor& dpos,
                   int64_t seq, int64_t vocab_start, bool add_pos) {
  c10::cuda::CUDAGuard guard(dout.device());
  const int hidden = static_cast<int>(dword.size(1));
  check(ethb::embedding_bwd(tokens.data_ptr<int64_t>(), dout.data_ptr(), dword.data_ptr(),
                            dpos.has_value() ? dpos->data_ptr() : nullptr, tokens.numel(),
                            static_cast<int>(seq), hidden, static_cast<int>(vocab_start),
                            static_cast<int>(vocab_start + dword.size(0)), add_pos,
                            dtype_code(dout), dtype_code(dword), cur_stream()), "embedding_bwd");
}

void ce_local_stats(const Tensor& logits, const Tensor& targets, Tensor& stats,
                    int64_t vocab_start) {
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1);
  check(ethb::ce_local_stats(logits.data_ptr(), targets.data_ptr<int64_t>(),
                             stats.data_ptr<float>(), logits.size(0),
                             static_cast<int>(logits.size(1)), logits.stride(0),
                             static_cast<int>(vocab_start), dtype_code(logits), cur_stream()),
        "ce_local_stats");
}
void ce_combine(const Tensor& stats_all, Tensor& loss, Tensor& gmax, Tensor& gsum, int64_t world) {
  c10::cuda::CUDAGuard guard(loss.device());
  check(ethb::ce_combine(stats_all.data_ptr<float>(), loss.data_ptr<float>(),
                         gmax.data_ptr<float>(), gsum.data_ptr<float>(), loss.numel(),
                         static_cast<int>(world), cur_stream()), "ce_combine");
}
void ce_bwd(Tensor& logits, const Tensor& targets, const Tensor& gmax, const Tensor& gsum,
            const Tensor& dloss, int64_t vocab_start) {
  c10::cuda::CUDAGuard guard(logits.device());
  check(ethb::ce_bwd(logits.data_ptr(), targets.data_ptr<int64_t>(), gmax.data_ptr<float>(),
                     gsum.data_ptr<float>(), dloss.data_ptr<float>(), logits.size(0),
                     static_cast<int>(logits.size(1)), logits.stride(0),
                     static_cast<int>(vocab_start), dtype_code(logits), cur_stream()), "ce_bwd");
}

void grad_norm_sq(const Tensor& grad, double inv_scale, Tensor& acc) {
  c10::cuda::CUDAGuard guard(grad.device());
  check(ethb::grad_norm_sq(grad.data_ptr(), grad.numel(), dtype_code(grad),
                           static_cast<float>(inv_scale), acc.data_ptr<float>(), cur_stream()),
        "grad_norm_sq");
}
void fused_adam(Tensor& param, Tensor& master, const Tensor& grad, Tensor& exp_avg,
                Tensor& exp_avg_sq, const OptTensor& ctrl, double lr, double beta1, double beta2,
                double eps, double weight_decay, int64_t step, double inv_scale, double max_norm,
                bool adamw, bool scale_from_ctrl) {
  c10::cuda::CUDAGuard guard(param.device());
  ethb::AdamArgs a{};
  a.param = param.data_ptr();
  a.master = master.data_ptr<float>();
  a.grad = grad.data_ptr();
  a.exp_avg = exp_avg.data_ptr<float>();
  a.exp_avg_sq = exp_avg_sq.data_ptr<float>();
  a.n = param.numel();
  TORCH_CHECK(master.numel() == a.n && grad.numel() == a.n && exp_avg.numel() == a.n);
  a.param_dtype = dtype_code(param);
  a.grad_dtype = dtype_code(grad);
  a.lr = static_cast<float>(lr); a.beta1 = static_cast<float>(beta1);
  a.beta2 = static_cast<float>(beta2); a.eps = static_cast<float>(eps);
  a.weight_decay = static_cast<float>(weight_decay);
  a.bias_correction1 = static_cast<float>(1.0 - std::pow(beta1, static_cast<double>(step)));
  a.bias_correction2 = static_cast<float>(1.0 - std::pow(beta2, static_cast<double>(step)));
  a.ctrl = ctrl.has_value() ? ctrl->data_ptr<float>() : nullptr;
  a.inv_scale = static_cast<float>(inv_scale);
  a.scale_from_ctrl = scale_from_ctrl;
  a.max_norm = static_cast<float>(max_norm);
  a.adamw = adamw;
  check(ethb::fused_adam(a, cur_stream()), "fused_adam");
}

// segs: int64 CUDA tensor [n, 6] = (src ptr, dst ptr, rows, run, src_stride, dst_stride)
void strided_copy_scale(const Tensor& segs, int64_t max_elems, double scale, int64_t src_dtype,
                        int64_t dst_dtype) {
  c10::cuda::CUDAGuard guard(segs.device());
  static_assert(sizeof(ethb::CopySegment) == 6 * sizeof(int64_t), "segment layout");
  check(ethb::strided_copy_scale(reinterpret_cast<const ethb::CopySegment*>(segs.data_ptr<int64_t>()),
                                 static_cast<int>(segs.size(0)), max_elems,
                                 static_cast<float>(scale), static_cast<int>(src_dtype),
                                 static_cast<int>(dst_dtype), cur_stream()), "strided_copy_scale");
}
void scale_inplace(Tensor& x, double scale) {
  c10::cuda::CUDAGuard guard(x.device());
  check(ethb::scale_inplace(x.data_ptr(), x.numel(), static_cast<float>(scale), dtype_code(x),
                            cur_stream()), "scale_inplace");
}
void synthetic_batch(Tensor& tokens, const OptTensor& labels, Tensor& loss_mask,
                     const Tensor& sample_ids, int64_t seq, int64_t vocab) {
  c10::cuda::CUDAGuard guard(tokens.device());
  check(ethb::synthetic_batch(tokens.data_ptr<int64_t>(),
                              labels.has_value() ? labels->data_ptr<int64_t>() : nullptr,
                              loss_mask.data_ptr<float>(), sample_ids.data_ptr<int64_t>(),
                              static_cast<int>(sample_ids.numel()), static_cast<int>(seq),
                              static_cast<int>(vocab), cur_stream()), "synthetic_batch");
}

// ---- attention -------------------------------------------------------------------------------
void attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, Tensor& o, Tensor& lse,
              double scale, bool causal, const OptTensor& status) {
  c10::cuda::CUDAGuard guard(q.device());
  // q/k/v/o: [batch, seq, heads, head_dim] views (any batch/seq/head strides, head_dim contiguous)
  TORCH_CHECK(q.dim() == 4 && q.stride(3) == 1 && k.stride(3) == 1 && v.stride(3) == 1 &&
              o.stride(3) == 1);
  ethb::AttnArgs a{};
  a.batch = static_cast<int>(q.size(0)); a.seq_q = static_cast<int>(q.size(1));
  a.heads = static_cast<int>(q.size(2)); a.head_dim = static_cast<int>(q.size(3));
  a.seq_k = static_cast<int>(k.size(1));
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.o = o.data_ptr();
  for (int i = 0; i < 3; ++i) {
    a.q_strides[i] = q.stride(i); a.k_strides[i] = k.stride(i); a.v_strides[i] = v.stride(i);
    a.o_strides[i] = o.stride(i);
  }
  a.lse = lse.data_ptr<float>();
  a.scale = static_cast<float>(scale);
  a.causal = causal;
  a.dtype = dtype_code(q);
  a.status = status.has_value() ? status->data_ptr<int>() : nullptr;
  check(ethb::attention_fwd(a, cur_stream()), "attention_fwd");
}
void attn_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o,
              const Tensor& d_o, const Tensor& lse, Tensor& dq, Tensor& dk, Tensor& dv,
              Tensor& delta, Tensor& dq_accum, double scale, bool causal, const OptTensor& status) {
  c10::cuda::CUDAGuard guard(q.device());
  ethb::AttnArgs a{};
  a.batch = static_cast<int>(q.size(0)); a.seq_q = static_cast<int>(q.size(1));
  a.heads = static_cast<int>(q.size(2)); a.head_dim = static_cast<int>(q.size(3));
  a.seq_k = static_cast<int>(k.size(1));
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.o = const_cast<void*>(o.data_ptr());
  a.d_o = d_o.data_ptr(); a.dq = dq.data_ptr(); a.dk = dk.data_ptr(); a.dv = dv.data_ptr();
  for (int i = 0; i < 3; ++i) {
    a.q_strides[i] = q.stride(i); a.k_strides[i] = k.stride(i); a.v_strides[i] = v.stride(i);
    a.o_strides[i] = o.stride(i); a.do_strides[i] = d_o.stride(i);
    a.dq_strides[i] = dq.stride(i); a.dk_strides[i] = dk.stride(i); a.dv_strides[i] = dv.stride(i);
  }
  a.lse = const_cast<float*>(lse.data_ptr<float>());
  a.delta = delta.data_ptr<float>();
  a.dq_accum = dq_accum.data_ptr<float>();
  a.scale = static_cast<float>(scale);
  a.causal = causal;
  a.dtype = dtype_code(q);
  a.status = status.has_value() ? status->data_ptr<int>() : nullptr;
  check(ethb::attention_bwd(a, cur_stream()), "attention_bwd");
}

// ---- peer memory -------------------------------------------------------------------------------
ethb::PeerPtrs to_peers(const std::vector<int64_t>& ptrs) {
  TORCH_CHECK(ptrs.size() <= ethb::kMaxPeers, "too many peers");
  ethb::PeerPtrs p{};
  for (size_t i = 0; i < ptrs.size(); ++i) p.ptrs[i] = reinterpret_cast<void*>(ptrs[i]);
  return p;
}
// Returns (device pointer, 64-byte IPC handle).
std::pair<int64_t, py::bytes> peer_alloc(int64_t bytes) {
  void* ptr = nullptr;
  unsigned char h[64];
  check(ethb::peer_alloc(static_cast<size_t>(bytes), &ptr, h), "peer_alloc");
  return {reinterpret_cast<int64_t>(ptr), py::bytes(reinterpret_cast<const char*>(h), 64)};
}
int64_t peer_open(const std::string& handle) {
  TORCH_CHECK(handle.size() == 64, "IPC handle must be 64 bytes");
  void* ptr = nullptr;
  check(ethb::peer_open(reinterpret_cast<const unsigned char*>(handle.data()), &ptr), "peer_open");
  return reinterpret_cast<int64_t>(ptr);
}
void peer_close(int64_t ptr) { check(ethb::peer_close(reinterpret_cast<void*>(ptr)), "peer_close"); }
void peer_free(int64_t ptr) { check(ethb::peer_free(reinterpret_cast<void*>(ptr)), "peer_free"); }
// Wrap raw device memory (owned elsewhere) as a tensor.
Tensor tensor_from_ptr(int64_t ptr, std::vector<int64_t> shape, py::object dtype, int64_t device) {
  auto st = torch::python::detail::py_object_to_dtype(dtype);
  auto opts = torch::TensorOptions().dtype(st).device(torch::kCUDA, static_cast<int>(device));
  return torch::from_blob(reinterpret_cast<void*>(ptr), shape, opts);
}
void peer_barrier(const std::vector<int64_t>& flags, int64_t rank, int64_t epoch,
                  const OptTensor& status) {
  check(ethb::peer_barrier(to_peers(flags), static_cast<int>(rank), static_cast<int>(flags.size()),
                           static_cast<int>(epoch),
                           status.has_value() ? status->data_ptr<int>() : nullptr, cur_stream()),
        "peer_barrier");
}
void peer_allreduce(const std::vector<int64_t>& bufs, const std::vector<int64_t>& flags,
                    int64_t rank, int64_t epoch, int64_t n, int64_t dtype, double scale,
                    Tensor& out, const OptTensor& norm_acc, double norm_weight,
                    const OptTensor& status) {
  c10::cuda::CUDAGuard guard(out.device());
  ethb::ReduceArgs a{};
  a.bufs = to_peers(bufs);
  a.flags = to_peers(flags);
  a.rank = static_cast<int>(rank);
  a.world = static_cast<int>(bufs.size());
  a.epoch = static_cast<int>(epoch);
  a.n = n;
  a.dtype = static_cast<int>(dtype);
  a.scale = static_cast<float>(scale);
  a.out = out.data_ptr();
  a.out_dtype = dtype_code(out);
  a.norm_acc = norm_acc.has_value() ? norm_acc->data_ptr<float>() : nullptr;
  a.norm_weight = static_cast<float>(norm_weight);
  a.status = status.has_value() ? status->data_ptr<int>() : nullptr;
  check(ethb::peer_allreduce(a, cur_stream()), "peer_allreduce");
}

// pieces: int64 CUDA tensor [P, 4] = (element offset, rows, run, stride); bases / flags: per-rank addresses
void peer_reduce_pieces(const std::vector<int64_t>& bases, const std::vector<int64_t>& flags, int64_t rank,
                        int64_t epoch, const Tensor& pieces, int64_t dtype, double scale) {
  c10::cuda::CUDAGuard guard(pieces.device());
  TORCH_CHECK(pieces.is_cuda() && pieces.dim() == 2 && pieces.size(1) == 4 && pieces.is_contiguous() &&
              pieces.scalar_type() == at::kLong, "pieces must be a contiguous int64 CUDA tensor [P, 4]");
  TORCH_CHECK(bases.size() == flags.size() && bases.size() >= 1 && bases.size() <= ethb::kMaxPeers);
  ethb::PieceReduceArgs a{};
  a.bases = to_peers(bases);
  a.flags = to_peers(flags);
  a.pieces = pieces.data_ptr<int64_t>();
  a.num_pieces = static_cast<int>(pieces.size(0));
  a.rank = static_cast<int>(rank);
  a.world = static_cast<int>(bases.size());
  a.epoch = static_cast<int>(epoch);
  a.dtype = static_cast<int>(dtype);
  a.scale = static_cast<float>(scale);
  check(ethb::peer_reduce_pieces(a, cur_stream()), "peer_reduce_pieces");
}
void peer_flags(const std::vector<int64_t>& flags, int64_t rank, int64_t epoch, int64_t signal_base,
                int64_t wait_base, const Tensor& status) {
  c10::cuda::CUDAGuard guard(status.device());
  check(ethb::peer_flags(to_peers(flags), static_cast<int>(rank), static_cast<int>(flags.size()),
                         static_cast<int>(epoch), static_cast<int>(signal_base), static_cast<int>(wait_base),
                         status.data_ptr<int>(), cur_stream()), "peer_flags");
}

ethb::FlagList to_flag_list(const std::vector<int64_t>& ptrs) {
  TORCH_CHECK(!ptrs.empty() && ptrs.size() <= 2 * ethb::kMaxPeers, "between 1 and 16 flag addresses");
  ethb::FlagList f{};
  f.count = static_cast<int>(ptrs.size());
  for (size_t i = 0; i < ptrs.size(); ++i) {
    TORCH_CHECK(ptrs[i] != 0 && ptrs[i] % 4 == 0, "flag addresses must be non-null and 4-byte aligned");
    f.ptrs[i] = reinterpret_cast<int*>(ptrs[i]);
  }
  return f;
}
// Raw-address 2-D copy on the current stream of `device` (addresses may be peer-mapped).
void peer_copy_2d(int64_t dst, int64_t dst_pitch, int64_t src, int64_t src_pitch, int64_t width_bytes, int64_t rows,
                  int64_t device) {
  TORCH_CHECK(dst != 0 && src != 0 && width_bytes >= 0 && rows >= 0, "bad copy arguments");
  c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
  check(ethb::peer_copy_2d(reinterpret_cast<void*>(dst), static_cast<size_t>(dst_pitch),
                           reinterpret_cast<const void*>(src), static_cast<size_t>(src_pitch),
                           static_cast<size_t>(width_bytes), static_cast<size_t>(rows), cur_stream()),
        "peer_copy_2d");
}
void flags_post(const std::vector<int64_t>& ptrs, int64_t value, int64_t device) {
  c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
  check(ethb::flags_post(to_flag_list(ptrs), static_cast<int>(value), cur_stream()), "flags_post");
}
void flags_wait(const std::vector<int64_t>& ptrs, int64_t value, int64_t limit_scale, const Tensor& status) {
  c10::cuda::CUDAGuard guard(status.device());
  check(ethb::flags_wait(to_flag_list(ptrs), static_cast<int>(value), static_cast<int>(limit_scale),
                         status.data_ptr<int>(), cur_stream()), "flags_wait");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm, py::arg("a"), py::arg("a_mn"), py::arg("b"), py::arg("b_mn"), py::arg("d"), py::arg("bias"),
        py::arg("aux"), py::arg("aux_mode"), py::arg("d2"), py::arg("accumulate"), py::arg("alpha"), py::arg("status"),
        py::arg("sm_count"), py::arg("drop_p") = 0.0, py::arg("drop_seed") = 0, py::arg("drop_offset") = 0);
  m.def("gemm_batched", &gemm_batched);
  m.def("gemm_allreduce", &gemm_allreduce, py::arg("a"), py::arg("a_mn"), py::arg("b"), py::arg("b_mn"),
        py::arg("bias"), py::arg("aux"), py::arg("alpha"), py::arg("status"), py::arg("stage_ptrs"), py::arg("out_ptrs"),
        py::arg("flag_ptrs"), py::arg("rank"), py::arg("epoch"), py::arg("max_tiles"), py::arg("stage_elems"),
        py::arg("ldd"), py::arg("mode"), py::arg("drop_p") = 0.0, py::arg("drop_seed") = 0, py::arg("drop_offset") = 0);
  m.def("gemm_allgather", &gemm_allgather);
  m.def("layernorm_fwd", &layernorm_fwd);
  m.def("ln_bwd_parts", &ln_bwd_parts);
  m.def("ln_bwd_fused_ok", [](int64_t hidden, bool fp32) {
    return ethb::ln_bwd_fused_ok(static_cast<int>(hidden), fp32 ? 0 : 2);
  });
  m.def("layernorm_bwd", &layernorm_bwd, py::arg("dy"), py::arg("x"), py::arg("gamma"), py::arg("mean"),
        py::arg("rstd"), py::arg("dx"), py::arg("dgamma"), py::arg("dbeta"), py::arg("ws"), py::arg("accumulate"),
        py::arg("dres") = py::none(), py::arg("ws_mode") = 0);
  m.def("bias_gelu_fwd", &bias_gelu_fwd);
  m.def("bias_gelu_bwd", &bias_gelu_bwd);
  m.def("bias_dropout_add_fwd", &bias_dropout_add_fwd);
  m.def("dropout_bwd", &dropout_bwd);
  m.def("colsum_parts", &colsum_parts);
  m.def("dropout_bwd_colsum_parts", &dropout_bwd_colsum_parts);
  m.def("dropout_bwd_colsum", &dropout_bwd_colsum, py::arg("dy"), py::arg("dx"), py::arg("bias_grad"), py::arg("ws"),
        py::arg("p"), py::arg("seed"), py::arg("offset"), py::arg("accumulate"), py::arg("ws_mode") = 0);
  m.def("colsum", &colsum);
  m.def("softmax_fwd", &softmax_fwd);
  m.def("softmax_bwd", &softmax_bwd);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("ce_local_stats", &ce_local_stats);
  m.def("ce_combine", &ce_combine);
  m.def("ce_bwd", &ce_bwd);
  m.def("grad_norm_sq", &grad_norm_sq);
  m.def("fused_adam", &fused_adam);
  m.def("strided_copy_scale", &strided_copy_scale);
  m.def("scale_inplace", &scale_inplace);
  m.def("synthetic_batch", &synthetic_batch);
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_bwd", &attn_bwd);
  m.def("launch_count", [] { return ethb::launch_count(); });
  m.def("set_gemm_variant", [](int v) { ethb::set_gemm_variant(v); });
  m.def("set_gemm_tail_split", [](int on) { ethb::set_gemm_tail_split(on); });
  m.def("peer_alloc", &peer_alloc);
  m.def("peer_open", &peer_open);
  m.def("peer_close", &peer_close);
  m.def("peer_free", &peer_free);
  m.def("tensor_from_ptr", &tensor_from_ptr);
  m.def("peer_barrier", &peer_barrier);
  m.def("peer_allreduce", &peer_allreduce);
  m.def("peer_reduce_pieces", &peer_reduce_pieces);
  m.def("peer_flags", &peer_flags);
  m.def("peer_copy_2d", &peer_copy_2d);
  m.def("flags_post", &flags_post);
  m.def("flags_wait", &flags_wait);
}
