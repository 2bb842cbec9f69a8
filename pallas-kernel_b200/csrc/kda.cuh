// Host-side launch interface of the KDA (gated delta rule) kernels.
#pragma once
#include "common.cuh"

namespace tops {
namespace kda {
int fwd(const tops_kda_fwd_params& p, cudaStream_t st);
size_t bwd_workspace_bytes(const tops_kda_bwd_params& p);
int bwd(const tops_kda_bwd_params& p, void* workspace, cudaStream_t st);
}  // namespace kda
}  // namespace tops
