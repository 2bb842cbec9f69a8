// Host-side interface of the chunked KDA kernels on tcgen05 / TMA (sm_100a).
#pragma once
#include "common.cuh"

namespace tops {
namespace sm100 {
// True when the chunked tensor-core kernels take this problem (bf16 q/k/v/g/beta, K = V = 128,
// chunk 64, whole chunks, dense batch).
bool kda_supported(const tops_chunk_kda_fwd_params& p);
int kda_chunk_fwd(const tops_chunk_kda_fwd_params& p, cudaStream_t st);
bool kda_bwd_supported(const tops_chunk_kda_bwd_params& p);
size_t kda_chunk_bwd_workspace_bytes(const tops_chunk_kda_bwd_params& p);
int kda_chunk_bwd(const tops_chunk_kda_bwd_params& p, void* ws, cudaStream_t st);
// The error word of the bounded waits in the KDA kernels (same convention as device_error()).
int kda_device_error(int* out);
int kda_device_error_set(int code);
}  // namespace sm100
}  // namespace tops
