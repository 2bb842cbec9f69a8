#include "gla_sm100.cuh"
namespace tops { namespace sm100 {
bool supported(const tops_chunk_problem&) { return false; }
size_t fwd_workspace_bytes(const tops_chunk_fwd_params&) { return 0; }
int chunk_fwd(const tops_chunk_fwd_params&, void*, size_t, cudaStream_t) { return TOPS_E_UNSUPPORTED; }
size_t bwd_workspace_bytes(const tops_chunk_bwd_params&) { return 0; }
int chunk_bwd(const tops_chunk_bwd_params&, void*, size_t, cudaStream_t) { return TOPS_E_UNSUPPORTED; }
}}
