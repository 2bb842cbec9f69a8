// Host-side launch interface of the token-serial (fused recurrent) GLA kernels.
#pragma once
#include "common.cuh"

namespace tops {
namespace recurrent {
int fwd(const tops_recurrent_fwd_params& p, cudaStream_t st);
size_t bwd_workspace_bytes(const tops_recurrent_bwd_params& p);
int bwd(const tops_recurrent_bwd_params& p, void* workspace, cudaStream_t st);
}  // namespace recurrent
}  // namespace tops
