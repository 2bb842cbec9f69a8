// KDA (gated delta rule) as a token-serial recurrence
//   S' = S exp(g_t)[:,None];  e = v_t - k_t^T S';  S = S' + (beta_t k_t) (x) e;  o_t = (q_t scale)^T S
// (reference: tops/cpu/ops/kda/naive.py:10-118, tops/ops/kda/fused_recurrent.py:19-105) and its
// explicit backward (tops/cpu/ops/kda/fused_recurrent.py:212-418).
//
// Forward: one block per (batch, head, 32-column slice of V), state slice in
// registers.  Backward: the forward kernel also records the state at every
// 64-token boundary; one block per (batch, head) then walks the boundaries
// backwards, replays the 64 tokens of a segment (storing the decayed states
// h'_t and the prediction errors e_t of that segment in scratch), and runs the
// reverse recurrence over the segment with the state gradient in registers.
// These kernels are the correctness path for KDA; the chunked WY / UT-transform
// formulation on the tensor cores is not built.
#include "kda.cuh"

namespace tops {
namespace kda {

constexpr int SEGMENT = 64;   // tokens between recorded states
constexpr int FW_THREADS = 128;
constexpr int FW_BV = 32;

template <int RK>
__global__ void __launch_bounds__(FW_THREADS) k_kda_fwd(tops_kda_fwd_params a, float* seg_states) {
  __shared__ float qs[16 * RK], ks[16 * RK], egs[16 * RK];
  __shared__ float vs[FW_BV];
  __shared__ float red[16][FW_BV + 1];
  __shared__ float beta_s;
  const int tid = threadIdx.x, vq = tid & 7, kr = tid >> 3;
  const int b = blockIdx.y / a.H, h = blockIdx.y % a.H;
  const int v0 = blockIdx.x * FW_BV;
  const int K = a.K, V = a.V;
  const size_t sbase = ((size_t)blockIdx.y) * K * (size_t)V;
  const int col = v0 + 4 * vq;
  const int nseg = (a.T + SEGMENT - 1) / SEGMENT;

  float S[RK][4];
#pragma unroll
  for (int r = 0; r < RK; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      int k = kr + 16 * r;
      S[r][c] = (a.h0 && k < K && col + c < V) ? a.h0[sbase + (size_t)k * V + col + c] : 0.f;
    }

  // The vectors of token t+1 are fetched into registers while token t is processed, so that the
  // HBM latency of one token hides behind the arithmetic and barriers of the previous one.
  constexpr int NL = (16 * RK + FW_THREADS - 1) / FW_THREADS;
  float rq[NL], rk[NL], rg[NL], rv = 0.f, rb = 0.f;
  auto fetch = [&](int t) {
    const size_t tok = ((size_t)b * a.T + t) * a.H + h;
#pragma unroll
    for (int n = 0; n < NL; ++n) {
      const int i = tid + n * FW_THREADS;
      if (i < K) {
        rq[n] = load_any(a.q, a.dtype, tok * K + i) * a.scale;
        rk[n] = load_any(a.k, a.dtype, tok * K + i);
        rg[n] = load_any(a.g, a.gate_dtype, tok * K + i);
      }
    }
    if (tid < FW_BV) rv = (v0 + tid < V) ? load_any(a.v, a.dtype, tok * V + v0 + tid) : 0.f;
    if (tid == 0) rb = load_any(a.beta, a.dtype, tok);
  };
  if (a.T > 0) fetch(0);
  for (int t = 0; t < a.T; ++t) {
    if (seg_states && (t % SEGMENT) == 0) {
      float* dst = seg_states + ((size_t)blockIdx.y * nseg + t / SEGMENT) * K * (size_t)V;
#pragma unroll
      for (int r = 0; r < RK; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          int k = kr + 16 * r;
          if (k < K && col + c < V) dst[(size_t)k * V + col + c] = S[r][c];
        }
    }
    const size_t tok = ((size_t)b * a.T + t) * a.H + h;
#pragma unroll
    for (int n = 0; n < NL; ++n) {
      const int i = tid + n * FW_THREADS;
      if (i < K) {
        qs[i] = rq[n];
        ks[i] = rk[n];
        egs[i] = expf(rg[n]);
      }
    }
    if (tid < FW_BV) vs[tid] = rv;
    if (tid == 0) beta_s = rb;
    __syncthreads();
    if (t + 1 < a.T) fetch(t + 1);
    // decay, and this thread's share of k^T S'
    float pp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < RK; ++r) {
      int k = kr + 16 * r;
      if (k < K) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          S[r][c] *= egs[k];
          pp[c] = fmaf(ks[k], S[r][c], pp[c]);
        }
      }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) red[kr][4 * vq + c] = pp[c];
    __syncthreads();
    float e[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      float s = 0.f;
#pragma unroll
      for (int gq = 0; gq < 16; ++gq) s += red[gq][4 * vq + c];
      e[c] = (vs[4 * vq + c] - s) * beta_s;
    }
    __syncthreads();
    // delta update and this thread's share of q^T S
    float po[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < RK; ++r) {
      int k = kr + 16 * r;
      if (k < K) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          S[r][c] = fmaf(ks[k], e[c], S[r][c]);
          po[c] = fmaf(qs[k], S[r][c], po[c]);
        }
      }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) red[kr][4 * vq + c] = po[c];
    __syncthreads();
    if (tid < FW_BV && v0 + tid < V) {
      float s = 0.f;
#pragma unroll
      for (int gq = 0; gq < 16; ++gq) s += red[gq][tid];
      store_any(a.o, a.dtype, tok * V + v0 + tid, s);
    }
    __syncthreads();
  }
  if (a.ht) {
#pragma unroll
    for (int r = 0; r < RK; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        int k = kr + 16 * r;
        if (k < K && col + c < V) a.ht[sbase + (size_t)k * V + col + c] = S[r][c];
      }
  }
}

static int launch_fwd(const tops_kda_fwd_params& p, float* seg_states, cudaStream_t st) {
  dim3 grid(cdiv(p.V, FW_BV), p.B * p.H);
  KernelScope ks("kda_recurrent_fwd", st);
  if (p.K <= 64) k_kda_fwd<4><<<grid, FW_THREADS, 0, st>>>(p, seg_states);
  else if (p.K <= 128) k_kda_fwd<8><<<grid, FW_THREADS, 0, st>>>(p, seg_states);
  else if (p.K <= 256) k_kda_fwd<16><<<grid, FW_THREADS, 0, st>>>(p, seg_states);
  else return TOPS_E_BAD_SHAPE;
  return post_launch();
}

int fwd(const tops_kda_fwd_params& p, cudaStream_t st) { return launch_fwd(p, nullptr, st); }

// ---------------------------------------------------------------------------
// backward: 256 threads = 16 key groups x 16 value groups; thread (kg, vg)
// owns rows kg + 16 r and columns vg + 16 j of the K x V matrices.
// ---------------------------------------------------------------------------
constexpr int BW_THREADS = 256;

__device__ __forceinline__ float reduce16(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 8);
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  return x;
}

template <int R>  // K, V <= 16 R
__global__ void __launch_bounds__(BW_THREADS) k_kda_bwd(tops_kda_bwd_params a, const float* seg_states,
                                                         float* hp_scratch, float* e_scratch) {
  constexpr int DM = 16 * R;
  __shared__ float qs[DM], ks[DM], egs[DM], vs[DM], dos[DM], es[DM], des[DM];
  __shared__ float red[16][DM + 1];
  __shared__ float beta_s, dbeta_s[8];
  const int tid = threadIdx.x, vg = tid & 15, kg = tid >> 4, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.x / a.H, h = blockIdx.x % a.H;
  const int K = a.K, V = a.V;
  const size_t sbase = (size_t)blockIdx.x * K * (size_t)V;
  const int nseg = (a.T + SEGMENT - 1) / SEGMENT;
  float* hp_blk = hp_scratch + (size_t)blockIdx.x * SEGMENT * K * (size_t)V;
  float* e_blk = e_scratch + (size_t)blockIdx.x * SEGMENT * V;

  float dh[R][R];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int j = 0; j < R; ++j) {
      int k = kg + 16 * r, v = vg + 16 * j;
      dh[r][j] = (a.dht && k < K && v < V) ? a.dht[sbase + (size_t)k * V + v] : 0.f;
    }

  for (int sg = nseg - 1; sg >= 0; --sg) {
    const int t0 = sg * SEGMENT, t1 = min(a.T, t0 + SEGMENT);
    // ---- replay the segment from its recorded start state: h'_t, e_t, dq_t
    {
      float S[R][R];
      const float* src = seg_states + ((size_t)blockIdx.x * nseg + sg) * K * (size_t)V;
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int j = 0; j < R; ++j) {
          int k = kg + 16 * r, v = vg + 16 * j;
          S[r][j] = (k < K && v < V) ? src[(size_t)k * V + v] : 0.f;
        }
      // (token t+1 is fetched into registers while token t is processed; DM <= BW_THREADS)
      float rk = 0.f, rg = 0.f, rv = 0.f, rdo = 0.f, rb = 0.f;
      auto fetch = [&](int t) {
        const size_t tok = ((size_t)b * a.T + t) * a.H + h;
        if (tid < DM) {
          const bool okk = tid < K, okv = tid < V;
          rk = okk ? load_any(a.k, a.dtype, tok * K + tid) : 0.f;
          rg = okk ? load_any(a.g, a.gate_dtype, tok * K + tid) : 0.f;
          rv = okv ? load_any(a.v, a.dtype, tok * V + tid) : 0.f;
          rdo = okv ? load_any(a.do_, a.dtype, tok * V + tid) : 0.f;
        }
        if (tid == 0) rb = load_any(a.beta, a.dtype, tok);
      };
      fetch(t0);
      for (int t = t0; t < t1; ++t) {
        const size_t tok = ((size_t)b * a.T + t) * a.H + h;
        if (tid < DM) {
          ks[tid] = rk;
          egs[tid] = expf(rg);
          vs[tid] = rv;
          dos[tid] = rdo;
        }
        if (tid == 0) beta_s = rb;
        __syncthreads();
        if (t + 1 < t1) fetch(t + 1);
        float* hp_t = hp_blk + (size_t)(t - t0) * K * V;
        float pp[R];
#pragma unroll
        for (int j = 0; j < R; ++j) pp[j] = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          int k = kg + 16 * r;
#pragma unroll
          for (int j = 0; j < R; ++j) {
            int v = vg + 16 * j;
            float x = S[r][j] * egs[k];
            S[r][j] = x;
            if (k < K && v < V) hp_t[(size_t)k * V + v] = x;
            pp[j] = fmaf(ks[k], x, pp[j]);
          }
        }
#pragma unroll
        for (int j = 0; j < R; ++j) red[kg][vg + 16 * j] = pp[j];
        __syncthreads();
        if (tid < DM) {
          float s = 0.f;
#pragma unroll
          for (int gq = 0; gq < 16; ++gq) s += red[gq][tid];
          float e = vs[tid] - s;
          es[tid] = e;
          if (tid < V) e_blk[(size_t)(t - t0) * V + tid] = e;
        }
        __syncthreads();
        const float bt = beta_s;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          int k = kg + 16 * r;
          float part = 0.f;
#pragma unroll
          for (int j = 0; j < R; ++j) {
            int v = vg + 16 * j;
            float x = fmaf(bt * ks[k], es[v], S[r][j]);
            S[r][j] = x;
            part = fmaf(x, dos[v], part);
          }
          part = reduce16(part);
          if (vg == 0 && k < K) store_any(a.dq, a.dtype, tok * K + k, part * a.scale);
        }
        __syncthreads();
      }
    }
    // ---- reverse recurrence over the segment
    float xq = 0.f, xk = 0.f, xg = 0.f, xdo = 0.f, xe = 0.f, xb = 0.f;
    auto fetch_rev = [&](int t) {
      const size_t tok = ((size_t)b * a.T + t) * a.H + h;
      if (tid < DM) {
        const bool okk = tid < K, okv = tid < V;
        xq = okk ? load_any(a.q, a.dtype, tok * K + tid) * a.scale : 0.f;
        xk = okk ? load_any(a.k, a.dtype, tok * K + tid) : 0.f;
        xg = okk ? load_any(a.g, a.gate_dtype, tok * K + tid) : 0.f;
        xdo = okv ? load_any(a.do_, a.dtype, tok * V + tid) : 0.f;
        xe = okv ? e_blk[(size_t)(t - t0) * V + tid] : 0.f;
      }
      if (tid == 0) xb = load_any(a.beta, a.dtype, tok);
    };
    fetch_rev(t1 - 1);
    for (int t = t1 - 1; t >= t0; --t) {
      const size_t tok = ((size_t)b * a.T + t) * a.H + h;
      if (tid < DM) {
        qs[tid] = xq;
        ks[tid] = xk;
        egs[tid] = expf(xg);
        dos[tid] = xdo;
        es[tid] = xe;
      }
      if (tid == 0) beta_s = xb;
      __syncthreads();
      if (t > t0) fetch_rev(t - 1);
      const float bt = beta_s;
      const float* hp_t = hp_blk + (size_t)(t - t0) * K * V;
      // dh += (q scale) (x) do ;  k^T dh
      float pk[R];
#pragma unroll
      for (int j = 0; j < R; ++j) pk[j] = 0.f;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        int k = kg + 16 * r;
#pragma unroll
        for (int j = 0; j < R; ++j) {
          int v = vg + 16 * j;
          float x = fmaf(qs[k], dos[v], dh[r][j]);
          dh[r][j] = x;
          pk[j] = fmaf(x, ks[k], pk[j]);
        }
      }
#pragma unroll
      for (int j = 0; j < R; ++j) red[kg][vg + 16 * j] = pk[j];
      __syncthreads();
      if (tid < DM) {
        float s = 0.f;
#pragma unroll
        for (int gq = 0; gq < 16; ++gq) s += red[gq][tid];
        float de = bt * s;
        des[tid] = de;
        if (tid < V) store_any(a.dv, a.dtype, tok * V + tid, de);
        // dbeta = sum_v (k^T dh) e
        float x = (tid < V) ? s * es[tid] : 0.f;
        x += __shfl_xor_sync(0xffffffffu, x, 16);
        x = reduce16(x);
        if (lane == 0) dbeta_s[warp] = x;
      }
      __syncthreads();
      if (tid == 0) {
        float s = 0.f;
        for (int w = 0; w < DM / 32; ++w) s += dbeta_s[w];
        store_any(a.dbeta, a.dtype, tok, s);
      }
      // dk, dg, and the step back through the delta update and the decay
#pragma unroll
      for (int r = 0; r < R; ++r) {
        int k = kg + 16 * r;
        float pdk = 0.f, pdg = 0.f;
#pragma unroll
        for (int j = 0; j < R; ++j) {
          int v = vg + 16 * j;
          float hp = (k < K && v < V) ? hp_t[(size_t)k * V + v] : 0.f;
          float x = dh[r][j];
          pdk += bt * x * es[v] - des[v] * hp;
          float dhp = x - ks[k] * des[v];
          pdg = fmaf(dhp, hp, pdg);
          dh[r][j] = dhp * egs[k];
        }
        pdk = reduce16(pdk);
        pdg = reduce16(pdg);
        if (vg == 0 && k < K) {
          store_any(a.dk, a.dtype, tok * K + k, pdk);
          store_any(a.dg, a.gate_dtype, tok * K + k, pdg);
        }
      }
      __syncthreads();
    }
  }
  if (a.dh0) {
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int j = 0; j < R; ++j) {
        int k = kg + 16 * r, v = vg + 16 * j;
        if (k < K && v < V) a.dh0[sbase + (size_t)k * V + v] = dh[r][j];
      }
  }
}

static size_t seg_elems(const tops_kda_bwd_params& p) {
  return (size_t)p.B * p.H * cdiv(p.T, SEGMENT) * p.K * p.V;
}
static size_t hp_elems(const tops_kda_bwd_params& p) { return (size_t)p.B * p.H * SEGMENT * p.K * p.V; }
static size_t e_elems(const tops_kda_bwd_params& p) { return (size_t)p.B * p.H * SEGMENT * p.V; }

size_t bwd_workspace_bytes(const tops_kda_bwd_params& p) {
  return align_up(seg_elems(p) * 4) + align_up(hp_elems(p) * 4) + align_up(e_elems(p) * 4) +
         align_up((size_t)p.B * p.T * p.H * p.V * dtype_size(p.dtype)) + 256;
}

int bwd(const tops_kda_bwd_params& p, void* workspace, cudaStream_t st) {
  if (p.K > 128 || p.V > 128) return TOPS_E_BAD_SHAPE;
  char* w = reinterpret_cast<char*>(workspace);
  float* seg = reinterpret_cast<float*>(w); w += align_up(seg_elems(p) * 4);
  float* hp = reinterpret_cast<float*>(w); w += align_up(hp_elems(p) * 4);
  float* es = reinterpret_cast<float*>(w); w += align_up(e_elems(p) * 4);
  void* o_tmp = w;
  // forward replay that records the state at every segment boundary
  tops_kda_fwd_params f{};
  f.B = p.B; f.T = p.T; f.H = p.H; f.K = p.K; f.V = p.V; f.dtype = p.dtype; f.gate_dtype = p.gate_dtype; f.scale = p.scale;
  f.q = p.q; f.k = p.k; f.v = p.v; f.g = p.g; f.beta = p.beta; f.h0 = p.h0; f.o = o_tmp; f.ht = nullptr;
  int rc = launch_fwd(f, seg, st);
  if (rc) return rc;
  const int Dm = p.K > p.V ? p.K : p.V;
  KernelScope ks("kda_recurrent_bwd", st);
  if (Dm <= 32) k_kda_bwd<2><<<p.B * p.H, BW_THREADS, 0, st>>>(p, seg, hp, es);
  else if (Dm <= 64) k_kda_bwd<4><<<p.B * p.H, BW_THREADS, 0, st>>>(p, seg, hp, es);
  else k_kda_bwd<8><<<p.B * p.H, BW_THREADS, 0, st>>>(p, seg, hp, es);
  return post_launch();
}

}  // namespace kda
}  // namespace tops
