// Host-side interface of the tcgen05 / TMA (sm_100a) chunked GLA kernels.
#pragma once
#include "common.cuh"

namespace tops {
namespace sm100 {
// True when the tcgen05 kernels take this problem (bf16, K = V = 128, chunk 64,
// whole chunks, dense batch, per-channel gates).
bool supported(const tops_chunk_problem& pb);
size_t fwd_workspace_bytes(const tops_chunk_fwd_params& p);
int chunk_fwd(const tops_chunk_fwd_params& p, void* ws, size_t ws_bytes, cudaStream_t st);
// output dtype combinations the backward kernel writes: (dq/dk, dg) = (fp32, fp32), (bf16, fp32), (bf16, bf16)
bool bwd_dtypes_ok(const tops_chunk_bwd_params& p);
size_t bwd_workspace_bytes(const tops_chunk_bwd_params& p);
int chunk_bwd(const tops_chunk_bwd_params& p, void* ws, size_t ws_bytes, cudaStream_t st);
// Shard summary for the state exchange of a time-sharded sequence (see tops_b200_chunk_state_exchange_pack).
size_t summary_workspace_bytes(const tops_chunk_problem& pb);
int state_summary(const tops_chunk_problem& pb, bool reverse, const void* x, const void* g, const void* y,
                  float* state_out, void* ws, cudaStream_t st);
// Reads the device error word (0 = no bounded wait has ever given up).
int device_error(int* out);
// Test hook: the next state-scan launch never issues the x/y tile load of chunk `chunk` of each block.
void test_skip_load(int chunk);
// Overwrites the device error word (0 clears it).
int device_error_set(int code);
}  // namespace sm100
}  // namespace tops
