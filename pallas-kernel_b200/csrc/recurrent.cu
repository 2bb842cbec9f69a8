// Token-serial GLA recurrence: h *= exp(gk)[:,None]; h *= exp(gv)[None,:];
// h += k (x) v; o = scale * q^T h   (reference: tops/cpu/ops/gla/fused_recurrent.py).
//
// Forward: one block per (sequence, head, 32-column slice of V).  The state
// slice lives in registers, is read once and written once, so a one-token call
// (decode) moves exactly the state bytes plus the token vectors; state rows
// are accessed as float4 along V.  Backward: one block per (sequence, head)
// holding the whole K x V state in registers, two passes over time.
#include "recurrent.cuh"

namespace tops {
namespace recurrent {

struct SeqRange { int b, bos, eos; };
__device__ __forceinline__ SeqRange seq_range(const int32_t* cu, int n, int T) {
  if (cu == nullptr) return {n, 0, T};
  return {0, cu[n], cu[n + 1]};
}

constexpr int FW_THREADS = 128;
constexpr int FW_BV = 32;

template <int RK>
__global__ void __launch_bounds__(FW_THREADS) k_rec_fwd(tops_recurrent_fwd_params a) {
  __shared__ float qs[16 * RK], ks[16 * RK], eks[16 * RK];
  __shared__ float vs[FW_BV], evs[FW_BV];
  __shared__ float red[16][FW_BV + 1];
  const int tid = threadIdx.x, vq = tid & 7, kr = tid >> 3;
  const int n = blockIdx.y / a.H, h = blockIdx.y % a.H;
  const int v0 = blockIdx.x * FW_BV;
  const int K = a.K, V = a.V;
  const SeqRange sr = seq_range(a.cu_seqlens, n, a.T);
  const bool vec = (V % 4) == 0;
  const size_t sbase = ((size_t)n * a.H + h) * K * (size_t)V;
  const int col = v0 + 4 * vq;

  float S[RK][4];
#pragma unroll
  for (int r = 0; r < RK; ++r) {
    int k = kr + 16 * r;
#pragma unroll
    for (int c = 0; c < 4; ++c) S[r][c] = 0.f;
    if (a.state_in && k < K) {
      if (vec && col < V) {
        // the state is touched once per call: streaming loads and stores keep it from displacing the rest of L2
        float4 x = __ldcs(reinterpret_cast<const float4*>(a.state_in + sbase + (size_t)k * V + col));
        S[r][0] = x.x; S[r][1] = x.y; S[r][2] = x.z; S[r][3] = x.w;
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c)
          if (col + c < V) S[r][c] = a.state_in[sbase + (size_t)k * V + col + c];
      }
    }
  }

  const int len = sr.eos - sr.bos;
  for (int step = 0; step < len; ++step) {
    const int t = a.reverse ? sr.eos - 1 - step : sr.bos + step;
    const size_t tok = ((size_t)sr.b * a.T + t) * a.H + h;
    for (int i = tid; i < K; i += FW_THREADS) {
      qs[i] = load_any(a.q, a.dtype, tok * K + i) * a.scale;
      ks[i] = load_any(a.k, a.dtype, tok * K + i);
      eks[i] = a.gk ? expf(load_any(a.gk, a.gate_dtype, tok * K + i)) : 1.f;
    }
    if (tid < FW_BV) {
      bool ok = v0 + tid < V;
      vs[tid] = ok ? load_any(a.v, a.dtype, tok * V + v0 + tid) : 0.f;
      evs[tid] = (ok && a.gv) ? expf(load_any(a.gv, a.gate_dtype, tok * V + v0 + tid)) : 1.f;
    }
    __syncthreads();
    float po[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < RK; ++r) {
      int k = kr + 16 * r;
      if (k < K) {
        float ek = eks[k], kk = ks[k], qq = qs[k];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float x = S[r][c] * ek;
          x = x * evs[4 * vq + c];
          x = fmaf(kk, vs[4 * vq + c], x);
          S[r][c] = x;
          po[c] = fmaf(x, qq, po[c]);
        }
      }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) red[kr][4 * vq + c] = po[c];
    __syncthreads();
    if (tid < FW_BV && v0 + tid < V) {
      float s = 0.f;
#pragma unroll
      for (int g = 0; g < 16; ++g) s += red[g][tid];
      store_any(a.o, a.o_dtype, tok * V + v0 + tid, s);
    }
    __syncthreads();
  }

  if (a.state_out) {
#pragma unroll
    for (int r = 0; r < RK; ++r) {
      int k = kr + 16 * r;
      if (k >= K) continue;
      if (vec && col < V) {
        __stcs(reinterpret_cast<float4*>(a.state_out + sbase + (size_t)k * V + col),
               make_float4(S[r][0], S[r][1], S[r][2], S[r][3]));
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c)
          if (col + c < V) a.state_out[sbase + (size_t)k * V + col + c] = S[r][c];
      }
    }
  }
}

int fwd(const tops_recurrent_fwd_params& p, cudaStream_t st) {
  const int N = p.cu_seqlens ? p.N : p.B;
  dim3 grid(cdiv(p.V, FW_BV), N * p.H);
  KernelScope ks("recurrent_fwd", st);
  if (p.K <= 64) k_rec_fwd<4><<<grid, FW_THREADS, 0, st>>>(p);
  else if (p.K <= 128) k_rec_fwd<8><<<grid, FW_THREADS, 0, st>>>(p);
  else if (p.K <= 256) k_rec_fwd<16><<<grid, FW_THREADS, 0, st>>>(p);
  else return TOPS_E_BAD_SHAPE;
  return post_launch();
}

// ---------------------------------------------------------------------------
// backward: 256 threads = 16 row groups x 16 column groups; thread (kg, vg)
// owns rows kg + 16 r and columns vg + 16 j.
// ---------------------------------------------------------------------------
constexpr int BW_THREADS = 256;

template <int R>  // K, V <= 16 R
__global__ void __launch_bounds__(BW_THREADS) k_rec_bwd(tops_recurrent_bwd_params a, float* dq32) {
  __shared__ float qs[16 * R], ks[16 * R], eks[16 * R], dqs[16 * R], dks[16 * R];
  __shared__ float vs[16 * R], evs[16 * R], dos[16 * R], os[16 * R];
  __shared__ float red[16][16 * R + 1];
  const int tid = threadIdx.x, vg = tid & 15, kg = tid >> 4;
  const int n = blockIdx.x / a.H, h = blockIdx.x % a.H;
  const int K = a.K, V = a.V;
  const SeqRange sr = seq_range(a.cu_seqlens, n, a.T);
  const size_t sbase = ((size_t)n * a.H + h) * K * (size_t)V;
  const int len = sr.eos - sr.bos;

  float S[R][R];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int j = 0; j < R; ++j) {
      int k = kg + 16 * r, v = vg + 16 * j;
      S[r][j] = (a.h0 && k < K && v < V) ? a.h0[sbase + (size_t)k * V + v] : 0.f;
    }

  // ---- pass 1: replay the recurrence, dq_t = scale * sum_v h_t[k,v] do_t[v]
  for (int step = 0; step < len; ++step) {
    const int t = a.reverse ? sr.eos - 1 - step : sr.bos + step;
    const size_t tok = ((size_t)sr.b * a.T + t) * a.H + h;
    for (int i = tid; i < 16 * R; i += BW_THREADS) {
      bool okk = i < K, okv = i < V;
      ks[i] = okk ? load_any(a.k, a.dtype, tok * K + i) : 0.f;
      eks[i] = (okk && a.gk) ? expf(load_any(a.gk, a.gate_dtype, tok * K + i)) : 1.f;
      vs[i] = okv ? load_any(a.v, a.dtype, tok * V + i) : 0.f;
      evs[i] = (okv && a.gv) ? expf(load_any(a.gv, a.gate_dtype, tok * V + i)) : 1.f;
      dos[i] = okv ? load_any(a.do_, a.dtype, tok * V + i) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) {
      int k = kg + 16 * r;
      float part = 0.f;
#pragma unroll
      for (int j = 0; j < R; ++j) {
        int v = vg + 16 * j;
        float x = S[r][j] * eks[k];
        x = x * evs[v];
        x = fmaf(ks[k], vs[v], x);
        S[r][j] = x;
        part = fmaf(x, dos[v], part);
      }
      part += __shfl_xor_sync(0xffffffffu, part, 8);
      part += __shfl_xor_sync(0xffffffffu, part, 4);
      part += __shfl_xor_sync(0xffffffffu, part, 2);
      part += __shfl_xor_sync(0xffffffffu, part, 1);
      if (vg == 0 && k < K) dq32[tok * K + k] = a.scale * part;
    }
    __syncthreads();
  }

  // ---- seed of the running gate gradients: sum(h_final * dht)
  float runk[R], runv[R];
#pragma unroll
  for (int r = 0; r < R; ++r) { runk[r] = 0.f; runv[r] = 0.f; }
  {
    float D[R][R];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int j = 0; j < R; ++j) {
        int k = kg + 16 * r, v = vg + 16 * j;
        D[r][j] = (a.dht && k < K && v < V) ? a.dht[sbase + (size_t)k * V + v] : 0.f;
      }
    // runk[k] = sum_v h dh  (reduce over the 16 column groups = 16 adjacent lanes)
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float part = 0.f;
#pragma unroll
      for (int j = 0; j < R; ++j) part = fmaf(S[r][j], D[r][j], part);
      part += __shfl_xor_sync(0xffffffffu, part, 8);
      part += __shfl_xor_sync(0xffffffffu, part, 4);
      part += __shfl_xor_sync(0xffffffffu, part, 2);
      part += __shfl_xor_sync(0xffffffffu, part, 1);
      runk[r] = part;  // identical in all 16 lanes of the row group
    }
    // runv[v] = sum_k h dh  (reduce over row groups through shared memory)
#pragma unroll
    for (int j = 0; j < R; ++j) {
      float part = 0.f;
#pragma unroll
      for (int r = 0; r < R; ++r) part = fmaf(S[r][j], D[r][j], part);
      red[kg][vg + 16 * j] = part;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < R; ++j) {
      float s = 0.f;
#pragma unroll
      for (int g = 0; g < 16; ++g) s += red[g][vg + 16 * j];
      runv[j] = s;  // identical in all 16 threads that share vg
    }
    __syncthreads();
    // the state registers now carry dh
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int j = 0; j < R; ++j) S[r][j] = D[r][j];
  }

  // ---- pass 2: walk time backwards
  for (int step = len - 1; step >= 0; --step) {
    const int t = a.reverse ? sr.eos - 1 - step : sr.bos + step;
    const size_t tok = ((size_t)sr.b * a.T + t) * a.H + h;
    for (int i = tid; i < 16 * R; i += BW_THREADS) {
      bool okk = i < K, okv = i < V;
      qs[i] = okk ? load_any(a.q, a.dtype, tok * K + i) : 0.f;
      ks[i] = okk ? load_any(a.k, a.dtype, tok * K + i) : 0.f;
      eks[i] = (okk && a.gk) ? expf(load_any(a.gk, a.gate_dtype, tok * K + i)) : 1.f;
      dqs[i] = okk ? dq32[tok * K + i] : 0.f;
      vs[i] = okv ? load_any(a.v, a.dtype, tok * V + i) : 0.f;
      evs[i] = (okv && a.gv) ? expf(load_any(a.gv, a.gate_dtype, tok * V + i)) : 1.f;
      dos[i] = okv ? load_any(a.do_, a.dtype, tok * V + i) : 0.f;
      os[i] = (okv && a.gv) ? a.o[tok * V + i] : 0.f;
    }
    __syncthreads();
    // dh += (q*scale) (x) do ; dk[k] = sum_v dh v ; dv[v] = sum_k dh k
    float dvp[R];
#pragma unroll
    for (int j = 0; j < R; ++j) dvp[j] = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      int k = kg + 16 * r;
      float qk = qs[k] * a.scale, part = 0.f;
#pragma unroll
      for (int j = 0; j < R; ++j) {
        int v = vg + 16 * j;
        float x = fmaf(qk, dos[v], S[r][j]);
        S[r][j] = x;
        part = fmaf(x, vs[v], part);
        dvp[j] = fmaf(x, ks[k], dvp[j]);
      }
      part += __shfl_xor_sync(0xffffffffu, part, 8);
      part += __shfl_xor_sync(0xffffffffu, part, 4);
      part += __shfl_xor_sync(0xffffffffu, part, 2);
      part += __shfl_xor_sync(0xffffffffu, part, 1);
      if (vg == 0) dks[k] = part;
      // running per-key gate gradient (same value in the 16 lanes of the row group)
      runk[r] += qs[k] * dqs[k] - ks[k] * part;
      if (vg == 0 && k < K) {
        store_any(a.dk, a.dtype, tok * K + k, part);
        store_any(a.dq, a.dtype, tok * K + k, dqs[k]);
        if (a.gk) store_any(a.dgk, a.gate_dtype, tok * K + k, runk[r]);
      }
    }
#pragma unroll
    for (int j = 0; j < R; ++j) red[kg][vg + 16 * j] = dvp[j];
    __syncthreads();
#pragma unroll
    for (int j = 0; j < R; ++j) {
      int v = vg + 16 * j;
      float s = 0.f;
#pragma unroll
      for (int g = 0; g < 16; ++g) s += red[g][v];
      runv[j] += os[v] * dos[v] - vs[v] * s;
      if (kg == 0 && v < V) {
        store_any(a.dv, a.dtype, tok * V + v, s);
        if (a.gv) store_any(a.dgv, a.gate_dtype, tok * V + v, runv[j]);
      }
    }
    // dh *= exp(gk)[:,None] * exp(gv)[None,:]
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int j = 0; j < R; ++j) S[r][j] = S[r][j] * eks[kg + 16 * r] * evs[vg + 16 * j];
    __syncthreads();
  }
  if (a.dh0) {
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int j = 0; j < R; ++j) {
        int k = kg + 16 * r, v = vg + 16 * j;
        if (k < K && v < V) a.dh0[sbase + (size_t)k * V + v] = S[r][j];
      }
  }
}

size_t bwd_workspace_bytes(const tops_recurrent_bwd_params& p) {
  return align_up((size_t)p.B * p.T * p.H * p.K * sizeof(float)) + 256;
}

int bwd(const tops_recurrent_bwd_params& p, void* workspace, cudaStream_t st) {
  const int N = p.cu_seqlens ? p.N : p.B;
  const int D = p.K > p.V ? p.K : p.V;
  float* dq32 = reinterpret_cast<float*>(workspace);
  dim3 grid(N * p.H);
  KernelScope ks("recurrent_bwd", st);
  if (D <= 32) k_rec_bwd<2><<<grid, BW_THREADS, 0, st>>>(p, dq32);
  else if (D <= 64) k_rec_bwd<4><<<grid, BW_THREADS, 0, st>>>(p, dq32);
  else if (D <= 128) k_rec_bwd<8><<<grid, BW_THREADS, 0, st>>>(p, dq32);
  else return TOPS_E_BAD_SHAPE;
  return post_launch();
}

}  // namespace recurrent
}  // namespace tops
