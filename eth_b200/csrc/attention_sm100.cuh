// C++ launchers of the tcgen05 flash-attention kernels (see attention_sm100.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ethb {

// q/k/v/o (and their gradients) are 4-D views [batch, seq, heads, head_dim] with head_dim
// contiguous; strides[] = element strides of (batch, seq, heads). head_dim is 64 or 128.
struct AttnArgs {
  int batch, heads, seq_q, seq_k, head_dim;
  const void *q, *k, *v;
  void* o;
  const void* d_o;
  void *dq, *dk, *dv;
  int64_t q_strides[3], k_strides[3], v_strides[3], o_strides[3];
  int64_t do_strides[3], dq_strides[3], dk_strides[3], dv_strides[3];
  float* lse;       // [batch, heads, seq_q]  log-sum-exp of the scaled scores (natural log)
  float* delta;     // [batch, heads, seq_q]  rowsum(dO * O), written by attention_bwd
  float* dq_accum;  // unused by the current backward (dQ has its own pass); may be null
  float scale;
  int causal;
  int dtype;        // kF16 / kBF16
  int* status;
};

cudaError_t attention_fwd(const AttnArgs& a, cudaStream_t st);
cudaError_t attention_bwd(const AttnArgs& a, cudaStream_t st);

}  // namespace ethb
