// KDA (gated delta rule) as a token-serial recurrence
//   S' = S exp(g_t)[:,None];  e = v_t - k_t^T S';  S = S' + (beta_t k_t) (x) e;  o_t = (q_t scale)^T S
// (reference: tops/cpu/ops/kda/naive.py:10-118, tops/ops/kda/fused_recurrent.py:19-105) and its
// explicit backward (tops/cpu/ops/kda/fused_recurrent.py:212-418).
//
// Forward and backward run one block per (batch, head, 32-column slice of V) with a warp per 8
// columns (k_kda_fwd_w, k_kda_bwd_w below).  The backward first re-runs the forward, which then
// records the state at every 64-token boundary; it walks the boundaries backwards, replays the
// 64 tokens of a segment (storing the decayed states h'_t of that segment in scratch), and runs
// the reverse recurrence over the segment with the state gradient in registers.
// k_kda_fwd<RK> is the older block-wide forward, kept for 128 < K <= 256.
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


// ---------------------------------------------------------------------------
// Warp-per-column-group kernels (K <= 128).  A warp owns 8 value columns of one
// (batch, head): lane l holds rows l, l + 32, l + 64, l + 96 of those columns,
// so every sum over the key dimension is a warp reduction and every sum over
// the value columns is a sum inside a thread.  The recurrences of different
// columns are independent, so the warps of a block never wait for each other
// in the forward pass; in the backward pass they meet once per token and loop
// to add up their shares of dq, dk, dg and dbeta.  The vectors of 16 tokens at a
// time are staged in shared memory as fp32.
// ---------------------------------------------------------------------------
constexpr int W_THREADS = 128;   // 4 warps = 32 value columns per block
constexpr int W_CW = 8;          // columns per warp
constexpr int W_RJ = 4;          // rows per lane

constexpr int W_TT = 16;         // tokens staged in shared memory at a time

// Sums eight per-lane values over the warp with 9 shuffles instead of 40: each exchange halves the
// number of values a lane is responsible for.  Every lane gets the total of column (lane >> 2) & 7
// (so lane 4 c holds column c).
__device__ __forceinline__ float warp_sum8(const float (&v)[W_CW], int lane) {
  const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
  float k4[4], k2[2];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    k4[i] = (b4 ? v[i + 4] : v[i]) + __shfl_xor_sync(0xffffffffu, b4 ? v[i] : v[i + 4], 16);
#pragma unroll
  for (int i = 0; i < 2; ++i)
    k2[i] = (b3 ? k4[i + 2] : k4[i]) + __shfl_xor_sync(0xffffffffu, b3 ? k4[i] : k4[i + 2], 8);
  float x = (b2 ? k2[1] : k2[0]) + __shfl_xor_sync(0xffffffffu, b2 ? k2[0] : k2[1], 4);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  return x;
}

// The vectors of W_TT consecutive tokens (time order t0 .. t0 + n - 1) of one (batch, head) as fp32 in
// shared memory: one exposed HBM latency per tile instead of one per token.
struct TokenTile {
  float q[W_TT][128], k[W_TT][128], eg[W_TT][128];   // q scaled; eg = exp(g)
  float v[W_TT][32], d[W_TT][32], beta[W_TT];        // v, do: this block's 32 columns
};
template <bool WITH_Q, bool WITH_V, bool WITH_DO>
__device__ __forceinline__ void load_tile(TokenTile& tl, const void* q, const void* k, const void* g, const void* v,
                                          const void* d, const void* beta, int dtype, int gate_dtype, int b, int h,
                                          int T, int H, int K, int V, int v0, int t0, int n, float scale) {
  for (int i = threadIdx.x; i < n * 128; i += blockDim.x) {
    const int tt = i >> 7, kk = i & 127;
    const size_t tok = ((size_t)b * T + t0 + tt) * H + h;
    const bool ok = kk < K;
    if (WITH_Q) tl.q[tt][kk] = ok ? load_any(q, dtype, tok * K + kk) * scale : 0.f;
    tl.k[tt][kk] = ok ? load_any(k, dtype, tok * K + kk) : 0.f;
    tl.eg[tt][kk] = ok ? __expf(load_any(g, gate_dtype, tok * K + kk)) : 1.f;
  }
  for (int i = threadIdx.x; i < n * 32; i += blockDim.x) {
    const int tt = i >> 5, c = i & 31;
    const size_t tok = ((size_t)b * T + t0 + tt) * H + h;
    const bool ok = v0 + c < V;
    if (WITH_V) tl.v[tt][c] = ok ? load_any(v, dtype, tok * V + v0 + c) : 0.f;
    if (WITH_DO) tl.d[tt][c] = ok ? load_any(d, dtype, tok * V + v0 + c) : 0.f;
  }
  if (threadIdx.x < n) tl.beta[threadIdx.x] = load_any(beta, dtype, ((size_t)b * T + t0 + threadIdx.x) * H + h);
}

__global__ void __launch_bounds__(W_THREADS) k_kda_fwd_w(tops_kda_fwd_params a, float* seg_states) {
  __shared__ TokenTile tl;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int b = blockIdx.y / a.H, h = blockIdx.y % a.H;
  const int v0 = blockIdx.x * 32, c0 = v0 + warp * W_CW, cw = warp * W_CW;
  const int K = a.K, V = a.V;
  const size_t sbase = (size_t)blockIdx.y * K * (size_t)V;
  const int nseg = (a.T + SEGMENT - 1) / SEGMENT;

  float S[W_RJ][W_CW];
#pragma unroll
  for (int j = 0; j < W_RJ; ++j)
#pragma unroll
    for (int c = 0; c < W_CW; ++c) {
      const int kk = lane + 32 * j;
      S[j][c] = (a.h0 && kk < K && c0 + c < V) ? a.h0[sbase + (size_t)kk * V + c0 + c] : 0.f;
    }
  auto store_state = [&](float* dst) {
#pragma unroll
    for (int j = 0; j < W_RJ; ++j)
#pragma unroll
      for (int c = 0; c < W_CW; ++c) {
        const int kk = lane + 32 * j;
        if (kk < K && c0 + c < V) dst[(size_t)kk * V + c0 + c] = S[j][c];
      }
  };
  for (int t0 = 0; t0 < a.T; t0 += W_TT) {
    const int n = min(W_TT, a.T - t0);
    __syncthreads();   // every warp is done with the previous tile
    load_tile<true, true, false>(tl, a.q, a.k, a.g, a.v, nullptr, a.beta, a.dtype, a.gate_dtype, b, h, a.T, a.H, K, V,
                                 v0, t0, n, a.scale);
    __syncthreads();
    for (int tt = 0; tt < n; ++tt) {
      const int t = t0 + tt;
      if (seg_states && (t % SEGMENT) == 0)
        store_state(seg_states + ((size_t)blockIdx.y * nseg + t / SEGMENT) * K * (size_t)V);
      const size_t tok = ((size_t)b * a.T + t) * a.H + h;
      float kq[W_RJ], kk_[W_RJ];
      float pp[W_CW];
#pragma unroll
      for (int c = 0; c < W_CW; ++c) pp[c] = 0.f;
#pragma unroll
      for (int j = 0; j < W_RJ; ++j) {
        const float eg = tl.eg[tt][lane + 32 * j];
        kk_[j] = tl.k[tt][lane + 32 * j];
        kq[j] = tl.q[tt][lane + 32 * j];
#pragma unroll
        for (int c = 0; c < W_CW; ++c) {
          S[j][c] *= eg;
          pp[c] = fmaf(kk_[j], S[j][c], pp[c]);
        }
      }
      const int myc = (lane >> 2) & 7;   // the column whose sums this lane ends up with
      const float e_mine = (tl.v[tt][cw + myc] - warp_sum8(pp, lane)) * tl.beta[tt];
      float acc[W_CW];
#pragma unroll
      for (int c = 0; c < W_CW; ++c) {
        const float e = __shfl_sync(0xffffffffu, e_mine, 4 * c);
        acc[c] = 0.f;
#pragma unroll
        for (int j = 0; j < W_RJ; ++j) {
          S[j][c] = fmaf(kk_[j], e, S[j][c]);
          acc[c] = fmaf(kq[j], S[j][c], acc[c]);
        }
      }
      const float o_mine = warp_sum8(acc, lane);
      if ((lane & 3) == 0 && c0 + myc < V) store_any(a.o, a.dtype, tok * V + c0 + myc, o_mine);
    }
  }
  if (a.ht) store_state(a.ht + sbase);
}

// Backward.  Scratch per warp: the decayed states h'_t ([t][k][8]) of the current 64-token segment.
// Partial sums over this block's 32 columns go to dq_part / dk_part / dg_part [slice][B,T,H,K] and
// db_part [slice][B,T,H].
__global__ void __launch_bounds__(W_THREADS) k_kda_bwd_w(tops_kda_bwd_params a, const float* seg_states, float* hp_scratch,
                                                         float* dq_part, float* dk_part, float* dg_part, float* db_part) {
  extern __shared__ float bw_smem[];
  TokenTile& tl = *reinterpret_cast<TokenTile*>(bw_smem);
  float (*es)[32] = reinterpret_cast<float (*)[32]>(bw_smem + sizeof(TokenTile) / 4);              // [SEGMENT][32]
  float (*red_a)[4][128] = reinterpret_cast<float (*)[4][128]>(&es[SEGMENT][0]);                   // [2][4][128]
  float (*red_b)[4][128] = reinterpret_cast<float (*)[4][128]>(&red_a[2][0][0]);                   // [2][4][128]
  float (*red_s)[4] = reinterpret_cast<float (*)[4]>(&red_b[2][0][0]);                             // [2][4]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b = blockIdx.y / a.H, h = blockIdx.y % a.H;
  const int slice = blockIdx.x, v0 = slice * 32, c0 = v0 + warp * W_CW, cw = warp * W_CW;
  const int K = a.K, V = a.V;
  const int nseg = (a.T + SEGMENT - 1) / SEGMENT;
  const size_t bh = blockIdx.y;
  const size_t sbase = bh * K * (size_t)V;
  const size_t wid = (bh * gridDim.x + slice) * 4 + warp;
  float* hp_w = hp_scratch + wid * SEGMENT * (size_t)K * W_CW;
  const size_t ntk = (size_t)a.B * a.T * a.H * K, nt = (size_t)a.B * a.T * a.H;
  float* dq_p = dq_part + slice * ntk;
  float* dk_p = dk_part + slice * ntk;
  float* dg_p = dg_part + slice * ntk;
  float* db_p = db_part + slice * nt;

  float dh[W_RJ][W_CW];
#pragma unroll
  for (int j = 0; j < W_RJ; ++j)
#pragma unroll
    for (int c = 0; c < W_CW; ++c) {
      const int kk = lane + 32 * j;
      dh[j][c] = (a.dht && kk < K && c0 + c < V) ? a.dht[sbase + (size_t)kk * V + c0 + c] : 0.f;
    }
  int step = 0;   // parity of the shared partial-sum buffers

  for (int sg = nseg - 1; sg >= 0; --sg) {
    const int s0 = sg * SEGMENT, s1 = min(a.T, s0 + SEGMENT);
    // ---- replay the segment from its recorded start state: h'_t, e_t, dq_t
    {
      float S[W_RJ][W_CW];
      const float* src = seg_states + (bh * nseg + sg) * K * (size_t)V;
#pragma unroll
      for (int j = 0; j < W_RJ; ++j)
#pragma unroll
        for (int c = 0; c < W_CW; ++c) {
          const int kk = lane + 32 * j;
          S[j][c] = (kk < K && c0 + c < V) ? src[(size_t)kk * V + c0 + c] : 0.f;
        }
      for (int t0 = s0; t0 < s1; t0 += W_TT) {
        const int n = min(W_TT, s1 - t0);
        __syncthreads();
        load_tile<false, true, true>(tl, nullptr, a.k, a.g, a.v, a.do_, a.beta, a.dtype, a.gate_dtype, b, h, a.T, a.H, K,
                                     V, v0, t0, n, 1.f);
        __syncthreads();
        for (int tt = 0; tt < n; ++tt, ++step) {
          const int t = t0 + tt;
          const size_t tok = ((size_t)b * a.T + t) * a.H + h;
          float* hp_t = hp_w + (size_t)(t - s0) * K * W_CW;
          float kk_[W_RJ];
          float pp[W_CW];
#pragma unroll
          for (int c = 0; c < W_CW; ++c) pp[c] = 0.f;
#pragma unroll
          for (int j = 0; j < W_RJ; ++j) {
            const int kr = lane + 32 * j;
            const float eg = tl.eg[tt][kr];
            kk_[j] = tl.k[tt][kr];
#pragma unroll
            for (int c = 0; c < W_CW; ++c) {
              S[j][c] *= eg;
              pp[c] = fmaf(kk_[j], S[j][c], pp[c]);
            }
            if (kr < K) {
              float4* dst = reinterpret_cast<float4*>(hp_t + (size_t)kr * W_CW);
              dst[0] = make_float4(S[j][0], S[j][1], S[j][2], S[j][3]);
              dst[1] = make_float4(S[j][4], S[j][5], S[j][6], S[j][7]);
            }
          }
          const float beta = tl.beta[tt];
          float dqv[W_RJ] = {0.f, 0.f, 0.f, 0.f};
          const int myc = (lane >> 2) & 7;   // the column whose sums this lane ends up with
          const float e_mine = tl.v[tt][cw + myc] - warp_sum8(pp, lane);
#pragma unroll
          for (int c = 0; c < W_CW; ++c) {
            const float be = beta * __shfl_sync(0xffffffffu, e_mine, 4 * c), dc = tl.d[tt][cw + c];
#pragma unroll
            for (int j = 0; j < W_RJ; ++j) {
              S[j][c] = fmaf(kk_[j], be, S[j][c]);
              dqv[j] = fmaf(S[j][c], dc, dqv[j]);
            }
          }
          if ((lane & 3) == 0) es[t - s0][cw + myc] = e_mine;
          // this block's share of dq_t = scale sum_v h_t[k, v] do_t[v]
          const int par = step & 1;
#pragma unroll
          for (int j = 0; j < W_RJ; ++j) red_a[par][warp][lane + 32 * j] = dqv[j];
          __syncthreads();
          if (tid < K)
            dq_p[tok * K + tid] =
                (red_a[par][0][tid] + red_a[par][1][tid] + red_a[par][2][tid] + red_a[par][3][tid]) * a.scale;
        }
      }
    }
    // ---- reverse recurrence over the segment, tile by tile from its end
    for (int t1 = s1; t1 > s0; t1 -= W_TT) {
      const int t0 = max(s0, t1 - W_TT), n = t1 - t0;
      __syncthreads();
      load_tile<true, false, true>(tl, a.q, a.k, a.g, nullptr, a.do_, a.beta, a.dtype, a.gate_dtype, b, h, a.T, a.H, K, V,
                                   v0, t0, n, a.scale);
      __syncthreads();
      for (int tt = n - 1; tt >= 0; --tt, ++step) {
        const int t = t0 + tt;
        const size_t tok = ((size_t)b * a.T + t) * a.H + h;
        // h'_t of this lane's rows (written by this lane during the replay)
        float hp[W_RJ][W_CW];
        const float* hp_t = hp_w + (size_t)(t - s0) * K * W_CW;
        float kq[W_RJ], kk_[W_RJ], keg[W_RJ];
#pragma unroll
        for (int j = 0; j < W_RJ; ++j) {
          const int kr = lane + 32 * j;
          float4 x = make_float4(0.f, 0.f, 0.f, 0.f), y = x;
          if (kr < K) {
            const float4* src = reinterpret_cast<const float4*>(hp_t + (size_t)kr * W_CW);
            x = src[0];
            y = src[1];
          }
          hp[j][0] = x.x; hp[j][1] = x.y; hp[j][2] = x.z; hp[j][3] = x.w;
          hp[j][4] = y.x; hp[j][5] = y.y; hp[j][6] = y.z; hp[j][7] = y.w;
          kq[j] = tl.q[tt][kr];
          kk_[j] = tl.k[tt][kr];
          keg[j] = tl.eg[tt][kr];
        }
        const float beta = tl.beta[tt];
        // dh += (q scale) (x) do ;  k^T dh ;  de = beta k^T dh
        float de[W_CW], ec[W_CW], pk[W_CW], dbeta = 0.f;
#pragma unroll
        for (int c = 0; c < W_CW; ++c) {
          const float dc = tl.d[tt][cw + c];
          ec[c] = es[t - s0][cw + c];
          pk[c] = 0.f;
#pragma unroll
          for (int j = 0; j < W_RJ; ++j) {
            dh[j][c] = fmaf(kq[j], dc, dh[j][c]);
            pk[c] = fmaf(dh[j][c], kk_[j], pk[c]);
          }
        }
        const int myc = (lane >> 2) & 7;   // the column whose sums this lane ends up with
        const float pk_mine = warp_sum8(pk, lane);
#pragma unroll
        for (int c = 0; c < W_CW; ++c) {
          const float s = __shfl_sync(0xffffffffu, pk_mine, 4 * c);
          de[c] = beta * s;
          dbeta = fmaf(s, ec[c], dbeta);   // columns beyond V have e = 0
        }
        if ((lane & 3) == 0 && c0 + myc < V) store_any(a.dv, a.dtype, tok * V + c0 + myc, beta * pk_mine);
        // dk, dg, and the step back through the delta update and the decay
        const int par = step & 1;
#pragma unroll
        for (int j = 0; j < W_RJ; ++j) {
          float pdk = 0.f, pdg = 0.f;
#pragma unroll
          for (int c = 0; c < W_CW; ++c) {
            const float x = dh[j][c];
            pdk += beta * x * ec[c] - de[c] * hp[j][c];
            const float dhp = x - kk_[j] * de[c];
            pdg = fmaf(dhp, hp[j][c], pdg);
            dh[j][c] = dhp * keg[j];
          }
          red_a[par][warp][lane + 32 * j] = pdk;
          red_b[par][warp][lane + 32 * j] = pdg;
        }
        if (lane == 0) red_s[par][warp] = dbeta;
        __syncthreads();
        if (tid < K) {
          dk_p[tok * K + tid] = red_a[par][0][tid] + red_a[par][1][tid] + red_a[par][2][tid] + red_a[par][3][tid];
          dg_p[tok * K + tid] = red_b[par][0][tid] + red_b[par][1][tid] + red_b[par][2][tid] + red_b[par][3][tid];
        }
        if (tid == 0) db_p[tok] = red_s[par][0] + red_s[par][1] + red_s[par][2] + red_s[par][3];
      }
    }
  }
  if (a.dh0) {
#pragma unroll
    for (int j = 0; j < W_RJ; ++j)
#pragma unroll
      for (int c = 0; c < W_CW; ++c) {
        const int kk = lane + 32 * j;
        if (kk < K && c0 + c < V) a.dh0[sbase + (size_t)kk * V + c0 + c] = dh[j][c];
      }
  }
}
constexpr size_t BW_SMEM = sizeof(TokenTile) + (SEGMENT * 32 + 2 * 2 * 4 * 128 + 2 * 4) * sizeof(float);

static int launch_fwd(const tops_kda_fwd_params& p, float* seg_states, cudaStream_t st) {
  dim3 grid(cdiv(p.V, FW_BV), p.B * p.H);
  KernelScope ks("kda_recurrent_fwd", st);
  if (p.K <= 128) k_kda_fwd_w<<<grid, W_THREADS, 0, st>>>(p, seg_states);
  else if (p.K <= 256) k_kda_fwd<16><<<grid, FW_THREADS, 0, st>>>(p, seg_states);
  else return TOPS_E_BAD_SHAPE;
  return post_launch();
}

int fwd(const tops_kda_fwd_params& p, cudaStream_t st) { return launch_fwd(p, nullptr, st); }

// adds the slices' partial sums in slice order and writes dq, dk, dg, dbeta in their output dtypes
__global__ void k_kda_bwd_finish(tops_kda_bwd_params a, const float* dq_part, const float* dk_part, const float* dg_part,
                                 const float* db_part, int nslice) {
  const size_t ntk = (size_t)a.B * a.T * a.H * a.K, nt = (size_t)a.B * a.T * a.H;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < ntk; i += (size_t)gridDim.x * blockDim.x) {
    float q = 0.f, k = 0.f, g = 0.f;
    for (int s = 0; s < nslice; ++s) {
      q += dq_part[s * ntk + i];
      k += dk_part[s * ntk + i];
      g += dg_part[s * ntk + i];
    }
    store_any(a.dq, a.dtype, i, q);
    store_any(a.dk, a.dtype, i, k);
    store_any(a.dg, a.gate_dtype, i, g);
    if (i < nt) {
      float bsum = 0.f;
      for (int s = 0; s < nslice; ++s) bsum += db_part[s * nt + i];
      store_any(a.dbeta, a.dtype, i, bsum);
    }
  }
}

static int n_slices(const tops_kda_bwd_params& p) { return cdiv(p.V, 32); }
static size_t seg_elems(const tops_kda_bwd_params& p) {
  return (size_t)p.B * p.H * cdiv(p.T, SEGMENT) * p.K * p.V;
}
static size_t hp_elems(const tops_kda_bwd_params& p) { return (size_t)p.B * p.H * n_slices(p) * SEGMENT * p.K * 32; }
static size_t e_elems(const tops_kda_bwd_params& p) { return (size_t)p.B * p.H * n_slices(p) * SEGMENT * 32; }
static size_t part_elems(const tops_kda_bwd_params& p) {
  return (size_t)n_slices(p) * ((size_t)p.B * p.T * p.H * (3 * (size_t)p.K + 1));
}

size_t bwd_workspace_bytes(const tops_kda_bwd_params& p) {
  return align_up(seg_elems(p) * 4) + align_up(hp_elems(p) * 4) + align_up(e_elems(p) * 4) +
         align_up(part_elems(p) * 4) + align_up((size_t)p.B * p.T * p.H * p.V * dtype_size(p.dtype)) + 256;
}

int bwd(const tops_kda_bwd_params& p, void* workspace, cudaStream_t st) {
  if (p.K > 128 || p.V > 128) return TOPS_E_BAD_SHAPE;
  const int ns = n_slices(p);
  const size_t ntk = (size_t)p.B * p.T * p.H * p.K;
  char* w = reinterpret_cast<char*>(workspace);
  float* seg = reinterpret_cast<float*>(w); w += align_up(seg_elems(p) * 4);
  float* hp = reinterpret_cast<float*>(w); w += align_up(hp_elems(p) * 4);
  w += align_up(e_elems(p) * 4);
  float* part = reinterpret_cast<float*>(w); w += align_up(part_elems(p) * 4);
  float *dq_p = part, *dk_p = dq_p + ns * ntk, *dg_p = dk_p + ns * ntk, *db_p = dg_p + ns * ntk;
  void* o_tmp = w;
  // forward replay that records the state at every segment boundary
  tops_kda_fwd_params f{};
  f.B = p.B; f.T = p.T; f.H = p.H; f.K = p.K; f.V = p.V; f.dtype = p.dtype; f.gate_dtype = p.gate_dtype; f.scale = p.scale;
  f.q = p.q; f.k = p.k; f.v = p.v; f.g = p.g; f.beta = p.beta; f.h0 = p.h0; f.o = o_tmp; f.ht = nullptr;
  int rc = launch_fwd(f, seg, st);
  if (rc) return rc;
  {
    dim3 grid(ns, p.B * p.H);
    if (cudaFuncSetAttribute(k_kda_bwd_w, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)BW_SMEM) != cudaSuccess)
      return TOPS_E_CUDA;
    KernelScope ks("kda_recurrent_bwd", st);
    k_kda_bwd_w<<<grid, W_THREADS, BW_SMEM, st>>>(p, seg, hp, dq_p, dk_p, dg_p, db_p);
    if ((rc = post_launch())) return rc;
  }
  KernelScope ks("kda_bwd_finish", st);
  k_kda_bwd_finish<<<1184, 256, 0, st>>>(p, dq_p, dk_p, dg_p, db_p, ns);
  return post_launch();
}

}  // namespace kda
}  // namespace tops
