// Shared device/host helpers for the tops_b200 kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tops_b200.h"

namespace tops {

// ---- launch accounting (read back through tops_b200_launch_count) ----------
void count_launch(int n = 1);

#define TOPS_CUDA_OK(expr)                         \
  do {                                             \
    cudaError_t _e = (expr);                       \
    if (_e != cudaSuccess) return TOPS_E_CUDA;     \
  } while (0)

// Optional per-kernel timing: when enabled through tops_b200_profile_enable, a
// KernelScope records a CUDA event pair around the launches made inside it, on
// the stream they go to.  Disabled, it costs one relaxed atomic load.
struct KernelScope {
  KernelScope(const char* label, cudaStream_t st);
  ~KernelScope();
  int slot;
  cudaStream_t st;
};

// The CUDA runtime error behind the most recent TOPS_E_CUDA (read back through tops_b200_last_cuda_error).
void record_cuda_error(int code, const char* where);

inline int post_launch(const char* where = "kernel launch") {
  count_launch();
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return TOPS_OK;
  record_cuda_error((int)e, where);
  return TOPS_E_CUDA;
}

inline size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }
inline int cdiv(int a, int b) { return (a + b - 1) / b; }
inline size_t dtype_size(int dt) { return dt == TOPS_F32 ? 4 : 2; }

// ---- element conversion -----------------------------------------------------
template <class T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }

template <class T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }

// Round an fp32 value to the precision of T and widen it again: the oracle's
// ".astype(input dtype)" cast points.
template <class T> __device__ __forceinline__ float round_to(float x) { return to_f<T>(from_f<T>(x)); }

// Load a gate value that may be stored in fp32, bf16 or fp16.
__device__ __forceinline__ float load_any(const void* p, int dtype, size_t i) {
  if (dtype == TOPS_F32) return reinterpret_cast<const float*>(p)[i];
  if (dtype == TOPS_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}
__device__ __forceinline__ void store_any(void* p, int dtype, size_t i, float x) {
  if (dtype == TOPS_F32) reinterpret_cast<float*>(p)[i] = x;
  else if (dtype == TOPS_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(x);
  else reinterpret_cast<__half*>(p)[i] = __float2half_rn(x);
}

// ---- where the chunks of a (possibly packed) batch live ---------------------
// Dense batch: sequence n == batch row n, T tokens each, NT chunks each.
// Packed batch (cu != nullptr): one batch row; sequence n owns tokens
// [cu[n], cu[n+1]) and chunks [cs[n], cs[n+1]) of the global chunk list.
struct SeqMap {
  const int32_t* cu;         // device [N+1] or nullptr
  const int32_t* cs;         // device [N+1] chunk prefix counts (packed only)
  const int32_t* chunk_seq;  // device [NT_total] sequence of each chunk (packed only)
  int N, T, C, NT;           // NT: chunks per sequence (dense) / total (packed)
};

struct ChunkPos {
  int batch;   // row of the [B,T,...] tensors
  int t0;      // first token
  int len;     // valid tokens (<= C)
  int slot;    // index along the NT axis of [B,NT,H,K,V] tensors
};

// chunk `ci` (0-based inside the sequence) of sequence `n`
__device__ __forceinline__ ChunkPos chunk_in_seq(const SeqMap& m, int n, int ci) {
  ChunkPos p;
  if (m.cu == nullptr) {
    p.batch = n; p.t0 = ci * m.C; p.len = min(m.C, m.T - p.t0); p.slot = ci;
  } else {
    int bos = m.cu[n], eos = m.cu[n + 1];
    p.batch = 0; p.t0 = bos + ci * m.C; p.len = min(m.C, eos - p.t0); p.slot = m.cs[n] + ci;
  }
  return p;
}
__device__ __forceinline__ int chunks_in_seq(const SeqMap& m, int n) {
  return m.cu == nullptr ? m.NT : m.cs[n + 1] - m.cs[n];
}
// global chunk id -> (sequence, position); dense ids are n*NT + ci
__device__ __forceinline__ ChunkPos chunk_global(const SeqMap& m, int gid, int* seq = nullptr) {
  int n, ci;
  if (m.cu == nullptr) { n = gid / m.NT; ci = gid - n * m.NT; }
  else { n = m.chunk_seq[gid]; ci = gid - m.cs[n]; }
  if (seq) *seq = n;
  return chunk_in_seq(m, n, ci);
}

}  // namespace tops
