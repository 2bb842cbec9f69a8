// Host-side launch interface of the shape-generic chunked kernels.
#pragma once
#include "common.cuh"

namespace tops {

// A chunked problem after validation: where chunks live plus the gate source.
struct Problem {
  SeqMap m;
  int H, K, V;
  int dtype;
  int gate_kind;
  const float* gcum;  // chunk-local cumsum (fp32) or g_gamma[H]
  float scale;
  int total_chunks;   // B*NT (dense) or the packed chunk count
};

struct BwdBuffers {
  const void *q, *k, *v, *do_;
  float *A, *dA;          // [total_chunks*H][C][C]
  const float *h, *dh;    // [B,NT,H,K,V] fp32
  void *dq, *dk, *dv;
  int grad_dtype;
  float* dg_stage;        // per-channel: final dg; scalar: per-K-tile partials; or null
  size_t dg_tile_stride;
};

namespace generic {
int launch_cumsum(const SeqMap& m, int H, int D, int dtype, int reverse, const void* g, float* out,
                  int total_chunks, cudaStream_t st);
int launch_prepare_chunks(const int32_t* cu, int N, int C, int32_t* cs, int32_t* chunk_seq, cudaStream_t st);
// forward (bwd=false): x=k, y=v, s0=h0, states=h, s_final=ht
// reverse (bwd=true):  x=q, y=do, s0=dht, states=dh, s_final=dh0
int launch_scan(const Problem& pb, bool bwd, const void* x, const void* y, const float* s0, void* states,
                int states_f32, float* s_final, cudaStream_t st);
int launch_fwd_o(const Problem& pb, const void* q, const void* k, const void* v, const void* h, int h_f32,
                 void* o, float* A_out, int round_A, cudaStream_t st);
int launch_bwd(const Problem& pb, const BwdBuffers& b, cudaStream_t st);
int launch_fold_shards(const float* first, const float* P, const float* S, float* out_in, float* out_all, int R, int rank,
                       int reverse, size_t BH, int K, int V, cudaStream_t st);
int launch_sum_partials(const float* part, size_t stride, int n, float* out, size_t count, cudaStream_t st);
}  // namespace generic
}  // namespace tops
