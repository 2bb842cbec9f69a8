// Host-side interface of the elementwise / row kernels next to the attention path: gate activations,
// L2 normalisation of q and k, gated RMS norm of the output.
#pragma once
#include <type_traits>

#include "common.cuh"

namespace tops {
namespace elementwise {
int gate_check(const tops_gate_act_params& p);
int gate_fwd(const tops_gate_act_params& p, cudaStream_t st);
size_t gate_bwd_workspace_bytes(const tops_gate_act_bwd_params& p);
int gate_bwd(const tops_gate_act_bwd_params& p, void* ws, cudaStream_t st);
int norm_check(const tops_norm_params& p);
int l2norm_fwd(const tops_norm_params& p, cudaStream_t st);
int l2norm_bwd(const tops_norm_params& p, cudaStream_t st);
int rmsnorm_gated_fwd(const tops_norm_params& p, cudaStream_t st);
size_t rmsnorm_gated_bwd_workspace_bytes(const tops_norm_params& p);
int rmsnorm_gated_bwd(const tops_norm_params& p, void* ws, cudaStream_t st);
}  // namespace elementwise
}  // namespace tops
