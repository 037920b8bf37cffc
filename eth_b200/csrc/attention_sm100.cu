#include "attention_sm100.cuh"
namespace ethb {
cudaError_t attention_fwd(const AttnArgs&, cudaStream_t) { return cudaErrorNotSupported; }
cudaError_t attention_bwd(const AttnArgs&, cudaStream_t) { return cudaErrorNotSupported; }
}  // namespace ethb
