// Shape-generic chunked GLA / simple_gla kernels (fp32 FMA on CUDA cores).
//
// These cover every dtype (fp32 / bf16 / fp16), any K and V, chunk sizes 16,
// 32 and 64, ragged T and packed batches.  They are the path for fp32 inputs
// (which must match an fp32 CPU computation to 1e-4) and for shapes the
// tcgen05 kernels do not take.  Arithmetic follows the reference's chunked
// algorithm (tops/cpu/ops/gla/chunk.py, tops/cpu/ops/common/chunk_h.py):
// operands that the reference rounds to the input dtype before a contraction
// are rounded here too; every contraction accumulates in fp32.
//
// Scalar (simple_gla) gates are treated as a per-channel gate that has the
// same value on every channel; the math is identical and only the rounding
// points differ from the reference's scalar-gate formulation.
#include "common.cuh"
#include "gla_generic.cuh"

namespace tops {
namespace generic {

constexpr int NTH = 256;  // threads per block, arranged 16 x 16
constexpr int BT = 64;    // tile extent along K and along V
constexpr int LD = 65;    // padded row length of a shared tile (bank-conflict free)

// ---------------------------------------------------------------------------
// acc[i][j] += sum_kk a(ty+16i, kk) * b(kk, tx+16j)
// ---------------------------------------------------------------------------
template <int TM, int TN, class FA, class FB>
__device__ __forceinline__ void tile_mma(float (&acc)[TM][TN], int kd, FA a, FB b) {
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll 4
  for (int kk = 0; kk < kd; ++kk) {
    float av[TM], bv[TN];
#pragma unroll
    for (int i = 0; i < TM; ++i) av[i] = a(ty + 16 * i, kk);
#pragma unroll
    for (int j = 0; j < TN; ++j) bv[j] = b(kk, tx + 16 * j);
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
  }
}

template <int TM, int TN>
__device__ __forceinline__ void zero(float (&acc)[TM][TN]) {
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
}

// ---------------------------------------------------------------------------
// Cumulative gate accessor.  Row i of a chunk that has `len` valid rows reads
// row min(i, len-1): padded rows repeat the last valid value, like the
// reference's zero-padded gates do after the cumulative sum.
// ---------------------------------------------------------------------------
struct Gate {
  const float* gc;  // cumsum [B,T,H,K] / [B,T,H], or gamma[H]
  int kind;         // TOPS_GATE_*
  int H, K;
  __device__ __forceinline__ float at(const ChunkPos& p, int T, int h, int i, int k) const {
    if (kind == TOPS_GATE_NONE) return 0.f;
    int r = min(i, p.len - 1);
    if (kind == TOPS_GATE_GAMMA) return gc[h] * float(r + 1);
    size_t tok = (size_t)p.batch * T + p.t0 + r;
    if (kind == TOPS_GATE_SCALAR) return gc[tok * H + h];
    return gc[(tok * H + h) * K + k];
  }
};

// ===========================================================================
// chunk-local cumulative sum
// ===========================================================================
__global__ void k_cumsum(SeqMap m, int H, int D, int dtype, int reverse, const void* g, float* out,
                         int total_chunks) {
  // one thread per (chunk, h, d); d fastest so loads coalesce
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t per_chunk = (size_t)H * D;
  if (idx >= per_chunk * total_chunks) return;
  int gid = idx / per_chunk;
  int hd = idx - (size_t)gid * per_chunk;
  ChunkPos p = chunk_global(m, gid);
  size_t base = ((size_t)p.batch * m.T + p.t0) * per_chunk + hd;
  float s = 0.f;
  if (!reverse) {
    for (int i = 0; i < p.len; ++i) {
      s += load_any(g, dtype, base + i * per_chunk);
      out[base + i * per_chunk] = s;
    }
  } else {
    for (int i = p.len - 1; i >= 0; --i) {
      s += load_any(g, dtype, base + i * per_chunk);
      out[base + i * per_chunk] = s;
    }
  }
}

// ===========================================================================
// State scans: forward (chunk-start states h_c) and reverse (dh_c)
// ===========================================================================
template <class T>
struct ScanArgs {
  SeqMap m;
  Gate gate;
  int H, K, V;
  const T* x;        // k (forward) or q (reverse)        [B,T,H,K]
  const T* y;        // v (forward) or do (reverse)       [B,T,H,V]
  const float* s0;   // h0 / dht                          [N,H,K,V] or null
  void* states;      // h / dh                            [B,NT,H,K,V] or null
  int states_f32;    // 1: fp32, 0: T
  float* s_final;    // ht / dh0                          [N,H,K,V] or null
  float scale;
};

template <class T, int C, bool BWD>
__global__ void __launch_bounds__(NTH) k_state_scan(ScanArgs<T> a) {
  __shared__ float xs[C * LD];
  __shared__ float ys[C * LD];
  __shared__ float decay[BT];
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int tilesV = (a.V + BT - 1) / BT;
  const int k0 = (blockIdx.x / tilesV) * BT, v0 = (blockIdx.x % tilesV) * BT;
  const int n = blockIdx.y / a.H, h = blockIdx.y % a.H;
  const int nch = chunks_in_seq(a.m, n);

  float S[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int kk = k0 + ty + 16 * i, vv = v0 + tx + 16 * j;
      S[i][j] = (a.s0 && kk < a.K && vv < a.V) ? a.s0[(((size_t)n * a.H + h) * a.K + kk) * a.V + vv] : 0.f;
    }

  for (int step = 0; step < nch; ++step) {
    const int ci = BWD ? nch - 1 - step : step;
    const ChunkPos p = chunk_in_seq(a.m, n, ci);
    // 1. record the state seen by this chunk
    if (a.states) {
      size_t base = (((size_t)p.batch * a.m.NT + p.slot) * a.H + h) * a.K * (size_t)a.V;
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          int kk = k0 + ty + 16 * i, vv = v0 + tx + 16 * j;
          if (kk < a.K && vv < a.V) {
            size_t o = base + (size_t)kk * a.V + vv;
            if (a.states_f32) reinterpret_cast<float*>(a.states)[o] = S[i][j];
            else reinterpret_cast<T*>(a.states)[o] = from_f<T>(S[i][j]);
          }
        }
    }
    // 2. stage the gated operands
    const bool per_ch = a.gate.kind == TOPS_GATE_PER_CHANNEL;
    for (int idx = tid; idx < C * BT; idx += NTH) {
      int i = idx / BT, c = idx % BT;
      float xv = 0.f, yv = 0.f;
      size_t tok = (size_t)p.batch * a.m.T + p.t0 + i;
      if (i < p.len) {
        if (k0 + c < a.K) {
          float raw = to_f(a.x[(tok * a.H + h) * a.K + k0 + c]);
          float gi = a.gate.at(p, a.m.T, h, i, k0 + c);
          if (!BWD) {
            // forward: per-channel gates act on k, scalar gates act on v
            xv = per_ch ? round_to<T>(raw * expf(a.gate.at(p, a.m.T, h, C - 1, k0 + c) - gi)) : raw;
          } else {
            xv = per_ch ? round_to<T>(raw * a.scale * expf(gi))
                        : round_to<T>(round_to<T>(raw * a.scale) * expf(gi));
          }
        }
        if (v0 + c < a.V) {
          float raw = to_f(a.y[(tok * a.H + h) * a.V + v0 + c]);
          if (!BWD && !per_ch && a.gate.kind != TOPS_GATE_NONE) {
            float gi = a.gate.at(p, a.m.T, h, i, 0);
            raw = round_to<T>(raw * expf(a.gate.at(p, a.m.T, h, C - 1, 0) - gi));
          }
          yv = raw;
        }
      }
      xs[i * LD + c] = xv;
      ys[i * LD + c] = yv;
    }
    if (tid < BT) decay[tid] = (k0 + tid < a.K) ? expf(a.gate.at(p, a.m.T, h, C - 1, k0 + tid)) : 1.f;
    __syncthreads();
    // 3. S = S * decay + x^T y
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float d = decay[ty + 16 * i];
#pragma unroll
      for (int j = 0; j < 4; ++j) S[i][j] *= d;
    }
    tile_mma<4, 4>(S, C, [&](int r, int i) { return xs[i * LD + r]; }, [&](int i, int c) { return ys[i * LD + c]; });
    __syncthreads();
  }
  if (a.s_final) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int kk = k0 + ty + 16 * i, vv = v0 + tx + 16 * j;
        if (kk < a.K && vv < a.V) a.s_final[(((size_t)n * a.H + h) * a.K + kk) * a.V + vv] = S[i][j];
      }
  }
}

// ===========================================================================
// Forward output: A = tril(q~ k~^T) * scale, o = scale * qg h + A v
// ===========================================================================
template <class T>
struct FwdOArgs {
  SeqMap m;
  Gate gate;
  int H, K, V;
  const T *q, *k, *v;
  const void* h;  // [B,NT,H,K,V]
  int h_f32;
  T* o;
  float* A_out;   // [B,T,H,C] or null
  float scale;
  int round_A;    // 1: round A to T before A v (GLA); 0: keep fp32 (simple_gla)
};

template <class T, int C>
__global__ void __launch_bounds__(NTH) k_fwd_o(FwdOArgs<T> a) {
  extern __shared__ float sm[];
  float* qa = sm;               // [C][LD] q * exp(G - mid)
  float* ka = qa + C * LD;      // [C][LD] k * exp(mid - G)
  float* qg = ka + C * LD;      // [C][LD] round(q * exp(G))
  float* gs = qg + C * LD;      // [C][LD] G
  float* hs = gs + C * LD;      // [BT][LD] state tile; later v tile
  float* As = hs + BT * LD;     // [C][C+1]
  constexpr int TC = C / 16;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int h = blockIdx.z, v0 = blockIdx.y * BT;
  const ChunkPos p = chunk_global(a.m, blockIdx.x);
  const size_t tok0 = (size_t)p.batch * a.m.T + p.t0;
  const size_t hbase = (((size_t)p.batch * a.m.NT + p.slot) * a.H + h) * a.K * (size_t)a.V;

  float accA[TC][TC], accO[TC][4];
  zero(accA);
  zero(accO);
  for (int k0 = 0; k0 < a.K; k0 += BT) {
    for (int idx = tid; idx < C * BT; idx += NTH) {
      int i = idx / BT, c = idx % BT;
      gs[i * LD + c] = (k0 + c < a.K) ? a.gate.at(p, a.m.T, h, i, k0 + c) : 0.f;
    }
    for (int idx = tid; idx < BT * BT; idx += NTH) {
      int r = idx / BT, c = idx % BT;
      float x = 0.f;
      if (k0 + r < a.K && v0 + c < a.V) {
        size_t o = hbase + (size_t)(k0 + r) * a.V + v0 + c;
        x = a.h_f32 ? round_to<T>(reinterpret_cast<const float*>(a.h)[o]) : to_f(reinterpret_cast<const T*>(a.h)[o]);
      }
      hs[r * LD + c] = x;
    }
    __syncthreads();
    for (int idx = tid; idx < C * BT; idx += NTH) {
      int i = idx / BT, c = idx % BT;
      float qv = 0.f, kv = 0.f;
      if (i < p.len && k0 + c < a.K) {
        qv = to_f(a.q[((tok0 + i) * a.H + h) * a.K + k0 + c]);
        kv = to_f(a.k[((tok0 + i) * a.H + h) * a.K + k0 + c]);
      }
      float g = gs[i * LD + c];
      float mid = 0.5f * (gs[c] + gs[(C - 1) * LD + c]);
      qa[i * LD + c] = qv * expf(g - mid);
      ka[i * LD + c] = kv * expf(mid - g);
      qg[i * LD + c] = round_to<T>(qv * expf(g));
    }
    __syncthreads();
    tile_mma<TC, TC>(accA, BT, [&](int i, int kk) { return qa[i * LD + kk]; }, [&](int kk, int j) { return ka[j * LD + kk]; });
    tile_mma<TC, 4>(accO, BT, [&](int i, int kk) { return qg[i * LD + kk]; }, [&](int kk, int c) { return hs[kk * LD + c]; });
    __syncthreads();
  }
  // masked, scaled intra matrix
#pragma unroll
  for (int i = 0; i < TC; ++i)
#pragma unroll
    for (int j = 0; j < TC; ++j) {
      int r = ty + 16 * i, c = tx + 16 * j;
      float x = (r >= c) ? accA[i][j] * a.scale : 0.f;
      if (a.A_out && blockIdx.y == 0 && r < p.len) a.A_out[((tok0 + r) * a.H + h) * C + c] = x;
      As[r * (C + 1) + c] = a.round_A ? round_to<T>(x) : x;
    }
  for (int idx = tid; idx < C * BT; idx += NTH) {
    int i = idx / BT, c = idx % BT;
    hs[i * LD + c] = (i < p.len && v0 + c < a.V) ? to_f(a.v[((tok0 + i) * a.H + h) * a.V + v0 + c]) : 0.f;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < TC; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) accO[i][j] *= a.scale;
  tile_mma<TC, 4>(accO, C, [&](int i, int jj) { return As[i * (C + 1) + jj]; }, [&](int jj, int c) { return hs[jj * LD + c]; });
#pragma unroll
  for (int i = 0; i < TC; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int r = ty + 16 * i, c = v0 + tx + 16 * j;
      if (r < p.len && c < a.V) a.o[((tok0 + r) * a.H + h) * a.V + c] = from_f<T>(accO[i][j]);
    }
}

// ===========================================================================
// Backward, step 1: A (recomputed) and dA = tril(do v^T) * scale  -> workspace
// ===========================================================================
template <class T>
struct BwdAArgs {
  SeqMap m;
  Gate gate;
  int H, K, V;
  const T *q, *k, *v, *do_;
  float* A;   // [chunks*H][C][C]
  float* dA;  // [chunks*H][C][C]
  float scale;
};

template <class T, int C>
__global__ void __launch_bounds__(NTH) k_bwd_A(BwdAArgs<T> a) {
  extern __shared__ float sm[];
  float* xa = sm;            // [C][LD]
  float* xb = xa + C * LD;   // [C][LD]
  float* gs = xb + C * LD;   // [C][LD]
  constexpr int TC = C / 16;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int h = blockIdx.y;
  const ChunkPos p = chunk_global(a.m, blockIdx.x);
  const size_t tok0 = (size_t)p.batch * a.m.T + p.t0;
  const size_t obase = ((size_t)blockIdx.x * a.H + h) * C * C;
  float acc[TC][TC];
  zero(acc);
  for (int k0 = 0; k0 < a.K; k0 += BT) {
    for (int idx = tid; idx < C * BT; idx += NTH) {
      int i = idx / BT, c = idx % BT;
      gs[i * LD + c] = (k0 + c < a.K) ? a.gate.at(p, a.m.T, h, i, k0 + c) : 0.f;
    }
    __syncthreads();
    for (int idx = tid; idx < C * BT; idx += NTH) {
      int i = idx / BT, c = idx % BT;
      float qv = 0.f, kv = 0.f;
      if (i < p.len && k0 + c < a.K) {
        qv = to_f(a.q[((tok0 + i) * a.H + h) * a.K + k0 + c]);
        kv = to_f(a.k[((tok0 + i) * a.H + h) * a.K + k0 + c]);
      }
      float g = gs[i * LD + c];
      float mid = 0.5f * (gs[c] + gs[(C - 1) * LD + c]);
      xa[i * LD + c] = qv * expf(g - mid);
      xb[i * LD + c] = kv * expf(mid - g);
    }
    __syncthreads();
    tile_mma<TC, TC>(acc, BT, [&](int i, int kk) { return xa[i * LD + kk]; }, [&](int kk, int j) { return xb[j * LD + kk]; });
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TC; ++i)
#pragma unroll
    for (int j = 0; j < TC; ++j) {
      int r = ty + 16 * i, c = tx + 16 * j;
      a.A[obase + r * C + c] = (r >= c) ? acc[i][j] * a.scale : 0.f;
    }
  zero(acc);
  for (int v0 = 0; v0 < a.V; v0 += BT) {
    for (int idx = tid; idx < C * BT; idx += NTH) {
      int i = idx / BT, c = idx % BT;
      float dv = 0.f, vv = 0.f;
      if (i < p.len && v0 + c < a.V) {
        dv = to_f(a.do_[((tok0 + i) * a.H + h) * a.V + v0 + c]);
        vv = to_f(a.v[((tok0 + i) * a.H + h) * a.V + v0 + c]);
      }
      xa[i * LD + c] = dv;
      xb[i * LD + c] = vv;
    }
    __syncthreads();
    tile_mma<TC, TC>(acc, BT, [&](int i, int kk) { return xa[i * LD + kk]; }, [&](int kk, int j) { return xb[j * LD + kk]; });
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TC; ++i)
#pragma unroll
    for (int j = 0; j < TC; ++j) {
      int r = ty + 16 * i, c = tx + 16 * j;
      a.dA[obase + r * C + c] = (r >= c) ? acc[i][j] * a.scale : 0.f;
    }
}

// ===========================================================================
// Backward, step 2: dv = A^T do + round(k exp(G_n - G)) round(dh)
// ===========================================================================
template <class T>
struct BwdDvArgs {
  SeqMap m;
  Gate gate;
  int H, K, V;
  const T *k, *do_;
  const float* A;   // workspace
  const float* dh;  // [B,NT,H,K,V] fp32
  T* dv;
};

template <class T, int C>
__global__ void __launch_bounds__(NTH) k_bwd_dv(BwdDvArgs<T> a) {
  extern __shared__ float sm[];
  float* As = sm;                  // [C][C+1]
  float* dos = As + C * (C + 1);   // [C][LD]
  float* kg = dos + C * LD;        // [C][LD]
  float* dhs = kg + C * LD;        // [BT][LD]
  constexpr int TC = C / 16;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int h = blockIdx.z, v0 = blockIdx.y * BT;
  const ChunkPos p = chunk_global(a.m, blockIdx.x);
  const size_t tok0 = (size_t)p.batch * a.m.T + p.t0;
  const size_t abase = ((size_t)blockIdx.x * a.H + h) * C * C;
  const size_t hbase = (((size_t)p.batch * a.m.NT + p.slot) * a.H + h) * a.K * (size_t)a.V;
  for (int idx = tid; idx < C * C; idx += NTH) As[(idx / C) * (C + 1) + idx % C] = a.A[abase + idx];
  for (int idx = tid; idx < C * BT; idx += NTH) {
    int i = idx / BT, c = idx % BT;
    dos[i * LD + c] = (i < p.len && v0 + c < a.V) ? to_f(a.do_[((tok0 + i) * a.H + h) * a.V + v0 + c]) : 0.f;
  }
  __syncthreads();
  float acc[TC][4];
  zero(acc);
  tile_mma<TC, 4>(acc, C, [&](int j, int i) { return As[i * (C + 1) + j]; }, [&](int i, int c) { return dos[i * LD + c]; });
  for (int k0 = 0; k0 < a.K; k0 += BT) {
    for (int idx = tid; idx < C * BT; idx += NTH) {
      int i = idx / BT, c = idx % BT;
      float x = 0.f;
      if (i < p.len && k0 + c < a.K) {
        float kv = to_f(a.k[((tok0 + i) * a.H + h) * a.K + k0 + c]);
        x = round_to<T>(kv * expf(a.gate.at(p, a.m.T, h, C - 1, k0 + c) - a.gate.at(p, a.m.T, h, i, k0 + c)));
      }
      kg[i * LD + c] = x;
    }
    for (int idx = tid; idx < BT * BT; idx += NTH) {
      int r = idx / BT, c = idx % BT;
      dhs[r * LD + c] = (k0 + r < a.K && v0 + c < a.V) ? round_to<T>(a.dh[hbase + (size_t)(k0 + r) * a.V + v0 + c]) : 0.f;
    }
    __syncthreads();
    tile_mma<TC, 4>(acc, BT, [&](int i, int kk) { return kg[i * LD + kk]; }, [&](int kk, int c) { return dhs[kk * LD + c]; });
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TC; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int r = ty + 16 * i, c = v0 + tx + 16 * j;
      if (r < p.len && c < a.V) a.dv[((tok0 + r) * a.H + h) * a.V + c] = from_f<T>(acc[i][j]);
    }
}

// ===========================================================================
// Backward, step 3: dq, dk (intra + inter) and the gate gradient
// ===========================================================================
template <class T>
struct BwdQkgArgs {
  SeqMap m;
  Gate gate;
  int H, K, V;
  const T *q, *k, *v, *do_;
  const float* dA;  // workspace
  const float* h;   // [B,NT,H,K,V] fp32
  const float* dh;  // [B,NT,H,K,V] fp32
  void *dq, *dk;
  int grad_dtype;
  float* dg;        // per-channel: [B,T,H,K]; scalar: partials [tilesK][B*T*H]; or null
  size_t dg_tile_stride;  // scalar gates: elements between K-tile partials
  float scale;
};

template <class T, int C>
__global__ void __launch_bounds__(NTH) k_bwd_dqkg(BwdQkgArgs<T> a) {
  extern __shared__ float sm[];
  float* qs = sm;                  // [C][LD] q
  float* ks = qs + C * LD;         // [C][LD] k
  float* gs = ks + C * LD;         // [C][LD] G
  float* t0s = gs + C * LD;        // [C][LD] scratch: k exp(mid-G) / do / dg_raw
  float* t1s = t0s + C * LD;       // [C][LD] scratch: q exp(G-mid) / v  / dk_inter*k
  float* hs = t1s + C * LD;        // [BT][LD]
  float* dhs = hs + BT * LD;       // [BT][LD]
  float* dAs = dhs + BT * LD;      // [C][C+1]
  float* hdh = dAs + C * (C + 1);  // [BT]
  constexpr int TC = C / 16;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int h = blockIdx.z, k0 = blockIdx.y * BT;
  const ChunkPos p = chunk_global(a.m, blockIdx.x);
  const size_t tok0 = (size_t)p.batch * a.m.T + p.t0;
  const size_t abase = ((size_t)blockIdx.x * a.H + h) * C * C;
  const size_t hbase = (((size_t)p.batch * a.m.NT + p.slot) * a.H + h) * a.K * (size_t)a.V;

  for (int idx = tid; idx < C * C; idx += NTH) dAs[(idx / C) * (C + 1) + idx % C] = a.dA[abase + idx];
  for (int idx = tid; idx < C * BT; idx += NTH) {
    int i = idx / BT, c = idx % BT;
    float qv = 0.f, kv = 0.f;
    if (i < p.len && k0 + c < a.K) {
      qv = to_f(a.q[((tok0 + i) * a.H + h) * a.K + k0 + c]);
      kv = to_f(a.k[((tok0 + i) * a.H + h) * a.K + k0 + c]);
    }
    qs[i * LD + c] = qv;
    ks[i * LD + c] = kv;
    gs[i * LD + c] = (k0 + c < a.K) ? a.gate.at(p, a.m.T, h, i, k0 + c) : 0.f;
  }
  if (tid < BT) hdh[tid] = 0.f;
  __syncthreads();
  for (int idx = tid; idx < C * BT; idx += NTH) {
    int i = idx / BT, c = idx % BT;
    float g = gs[i * LD + c];
    float mid = 0.5f * (gs[c] + gs[(C - 1) * LD + c]);
    t0s[i * LD + c] = ks[i * LD + c] * expf(mid - g);
    t1s[i * LD + c] = qs[i * LD + c] * expf(g - mid);
  }
  __syncthreads();
  float dq[TC][4], dk[TC][4];
  zero(dq);
  zero(dk);
  // intra-chunk: dq_i = sum_j dA_ij k~_j ; dk_j = sum_i dA_ij q~_i
  tile_mma<TC, 4>(dq, C, [&](int i, int j) { return dAs[i * (C + 1) + j]; }, [&](int j, int c) { return t0s[j * LD + c]; });
  tile_mma<TC, 4>(dk, C, [&](int j, int i) { return dAs[i * (C + 1) + j]; }, [&](int i, int c) { return t1s[i * LD + c]; });
#pragma unroll
  for (int i = 0; i < TC; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int r = ty + 16 * i, c = tx + 16 * j;
      float g = gs[r * LD + c];
      float mid = 0.5f * (gs[c] + gs[(C - 1) * LD + c]);
      dq[i][j] *= expf(g - mid);
      dk[i][j] *= expf(mid - g);
    }
  __syncthreads();
  // inter-chunk: dq += scale exp(G) (do round(h)^T) ; dk += exp(G_n - G) (v round(dh)^T)
  float dqi[TC][4], dki[TC][4];
  zero(dqi);
  zero(dki);
  float hd = 0.f;
  for (int v0 = 0; v0 < a.V; v0 += BT) {
    for (int idx = tid; idx < C * BT; idx += NTH) {
      int i = idx / BT, c = idx % BT;
      float dv = 0.f, vv = 0.f;
      if (i < p.len && v0 + c < a.V) {
        dv = to_f(a.do_[((tok0 + i) * a.H + h) * a.V + v0 + c]);
        vv = to_f(a.v[((tok0 + i) * a.H + h) * a.V + v0 + c]);
      }
      t0s[i * LD + c] = dv;
      t1s[i * LD + c] = vv;
    }
    for (int idx = tid; idx < BT * BT; idx += NTH) {
      int r = idx / BT, c = idx % BT;
      bool ok = k0 + r < a.K && v0 + c < a.V;
      size_t o = hbase + (size_t)(k0 + r) * a.V + v0 + c;
      hs[r * LD + c] = ok ? a.h[o] : 0.f;
      dhs[r * LD + c] = ok ? a.dh[o] : 0.f;
    }
    __syncthreads();
    tile_mma<TC, 4>(dqi, BT, [&](int i, int vv) { return t0s[i * LD + vv]; }, [&](int vv, int c) { return round_to<T>(hs[c * LD + vv]); });
    tile_mma<TC, 4>(dki, BT, [&](int i, int vv) { return t1s[i * LD + vv]; }, [&](int vv, int c) { return round_to<T>(dhs[c * LD + vv]); });
    {  // sum_v h * dh per channel: 4 threads per channel
      int r = tid >> 2, part = tid & 3;
      for (int c = part * 16; c < part * 16 + 16; ++c) hd = fmaf(hs[r * LD + c], dhs[r * LD + c], hd);
    }
    __syncthreads();
  }
  hd += __shfl_xor_sync(0xffffffffu, hd, 1);
  hd += __shfl_xor_sync(0xffffffffu, hd, 2);
  if ((tid & 3) == 0) hdh[tid >> 2] = hd;
  // combine, write dq / dk, stage the gate-gradient terms
#pragma unroll
  for (int i = 0; i < TC; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int r = ty + 16 * i, c = tx + 16 * j;
      float g = gs[r * LD + c], gn = gs[(C - 1) * LD + c];
      float dqt = dq[i][j] + a.scale * expf(g) * dqi[i][j];
      float dkin = expf(gn - g) * dki[i][j];
      float dkt = dk[i][j] + dkin;
      if (r < p.len && k0 + c < a.K) {
        size_t o = ((tok0 + r) * a.H + h) * a.K + k0 + c;
        store_any(a.dq, a.grad_dtype, o, dqt);
        store_any(a.dk, a.grad_dtype, o, dkt);
      }
      t0s[r * LD + c] = qs[r * LD + c] * dqt - ks[r * LD + c] * dkt;
      t1s[r * LD + c] = dkin * ks[r * LD + c];
    }
  __syncthreads();
  if (a.dg == nullptr) return;
  // dg = suffix-sum over rows of dg_raw + [exp(G_n) sum_v h dh + sum_i dk_inter k]
  if (tid < BT) {
    int c = tid;
    float tail = 0.f;
    for (int i = 0; i < C; ++i) tail += t1s[i * LD + c];
    tail += expf(gs[(C - 1) * LD + c]) * hdh[c];
    float run = 0.f;
    for (int i = C - 1; i >= 0; --i) {
      run += t0s[i * LD + c];
      t0s[i * LD + c] = run + tail;
    }
  }
  __syncthreads();
  if (a.gate.kind == TOPS_GATE_PER_CHANNEL) {
    for (int idx = tid; idx < C * BT; idx += NTH) {
      int i = idx / BT, c = idx % BT;
      if (i < p.len && k0 + c < a.K) a.dg[((tok0 + i) * a.H + h) * a.K + k0 + c] = t0s[i * LD + c];
    }
  } else if (tid < C && tid < p.len) {
    float s = 0.f;
    int kmax = min(BT, a.K - k0);
    for (int c = 0; c < kmax; ++c) s += t0s[tid * LD + c];
    a.dg[blockIdx.y * a.dg_tile_stride + (tok0 + tid) * a.H + h] = s;
  }
}

__global__ void k_sum_partials(const float* part, size_t stride, int n, float* out, size_t count) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  float s = 0.f;
  for (int t = 0; t < n; ++t) s += part[t * stride + i];
  out[i] = s;
}

// packed batches: chunk prefix counts and the sequence of each chunk
__global__ void k_prepare_chunks(const int32_t* cu, int N, int C, int32_t* cs, int32_t* chunk_seq) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int tot = 0;
  for (int n = 0; n < N; ++n) {
    cs[n] = tot;
    int nc = (cu[n + 1] - cu[n] + C - 1) / C;
    for (int c = 0; c < nc; ++c) chunk_seq[tot + c] = n;
    tot += nc;
  }
  cs[N] = tot;
}

// ---------------------------------------------------------------------------
// host launchers
// ---------------------------------------------------------------------------
template <class F>
static int set_smem(F f, size_t bytes) {
  if (bytes > 48 * 1024) TOPS_CUDA_OK(cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return TOPS_OK;
}

int launch_cumsum(const SeqMap& m, int H, int D, int dtype, int reverse, const void* g, float* out,
                  int total_chunks, cudaStream_t st) {
  size_t n = (size_t)total_chunks * H * D;
  if (n == 0) return TOPS_OK;
  KernelScope ks("generic_cumsum", st);
  k_cumsum<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(m, H, D, dtype, reverse, g, out, total_chunks);
  return post_launch();
}

int launch_prepare_chunks(const int32_t* cu, int N, int C, int32_t* cs, int32_t* chunk_seq, cudaStream_t st) {
  KernelScope ks("generic_prepare_chunks", st);
  k_prepare_chunks<<<1, 32, 0, st>>>(cu, N, C, cs, chunk_seq);
  return post_launch();
}

template <class T, int C>
static int scan_T(const Problem& pb, bool bwd, const void* x, const void* y, const float* s0, void* states,
                  int states_f32, float* s_final, cudaStream_t st) {
  ScanArgs<T> a;
  a.m = pb.m; a.gate = Gate{pb.gcum, pb.gate_kind, pb.H, pb.K}; a.H = pb.H; a.K = pb.K; a.V = pb.V;
  a.x = (const T*)x; a.y = (const T*)y; a.s0 = s0; a.states = states; a.states_f32 = states_f32;
  a.s_final = s_final; a.scale = pb.scale;
  dim3 grid(cdiv(pb.K, BT) * cdiv(pb.V, BT), pb.m.N * pb.H);
  KernelScope ks(bwd ? "generic_scan_dh" : "generic_scan_h", st);
  if (bwd) k_state_scan<T, C, true><<<grid, NTH, 0, st>>>(a);
  else k_state_scan<T, C, false><<<grid, NTH, 0, st>>>(a);
  return post_launch();
}

template <class T, int C>
static int fwd_o_T(const Problem& pb, const void* q, const void* k, const void* v, const void* h, int h_f32,
                   void* o, float* A_out, int round_A, cudaStream_t st) {
  FwdOArgs<T> a;
  a.m = pb.m; a.gate = Gate{pb.gcum, pb.gate_kind, pb.H, pb.K}; a.H = pb.H; a.K = pb.K; a.V = pb.V;
  a.q = (const T*)q; a.k = (const T*)k; a.v = (const T*)v; a.h = h; a.h_f32 = h_f32; a.o = (T*)o;
  a.A_out = A_out; a.scale = pb.scale; a.round_A = round_A;
  size_t smem = sizeof(float) * (4 * C * LD + BT * LD + C * (C + 1));
  int rc = set_smem(k_fwd_o<T, C>, smem);
  if (rc) return rc;
  dim3 grid(pb.total_chunks, cdiv(pb.V, BT), pb.H);
  KernelScope ks("generic_fwd_o", st);
  k_fwd_o<T, C><<<grid, NTH, smem, st>>>(a);
  return post_launch();
}

template <class T, int C>
static int bwd_T(const Problem& pb, const BwdBuffers& b, cudaStream_t st) {
  Gate gate{pb.gcum, pb.gate_kind, pb.H, pb.K};
  {
    BwdAArgs<T> a;
    a.m = pb.m; a.gate = gate; a.H = pb.H; a.K = pb.K; a.V = pb.V;
    a.q = (const T*)b.q; a.k = (const T*)b.k; a.v = (const T*)b.v; a.do_ = (const T*)b.do_;
    a.A = b.A; a.dA = b.dA; a.scale = pb.scale;
    size_t smem = sizeof(float) * 3 * C * LD;
    int rc = set_smem(k_bwd_A<T, C>, smem);
    if (rc) return rc;
    KernelScope ks("generic_bwd_A", st);
    k_bwd_A<T, C><<<dim3(pb.total_chunks, pb.H), NTH, smem, st>>>(a);
    if ((rc = post_launch())) return rc;
  }
  {
    BwdDvArgs<T> a;
    a.m = pb.m; a.gate = gate; a.H = pb.H; a.K = pb.K; a.V = pb.V;
    a.k = (const T*)b.k; a.do_ = (const T*)b.do_; a.A = b.A; a.dh = b.dh; a.dv = (T*)b.dv;
    size_t smem = sizeof(float) * (C * (C + 1) + 2 * C * LD + BT * LD);
    int rc = set_smem(k_bwd_dv<T, C>, smem);
    if (rc) return rc;
    KernelScope ks("generic_bwd_dv", st);
    k_bwd_dv<T, C><<<dim3(pb.total_chunks, cdiv(pb.V, BT), pb.H), NTH, smem, st>>>(a);
    if ((rc = post_launch())) return rc;
  }
  {
    BwdQkgArgs<T> a;
    a.m = pb.m; a.gate = gate; a.H = pb.H; a.K = pb.K; a.V = pb.V;
    a.q = (const T*)b.q; a.k = (const T*)b.k; a.v = (const T*)b.v; a.do_ = (const T*)b.do_;
    a.dA = b.dA; a.h = b.h; a.dh = b.dh; a.dq = b.dq; a.dk = b.dk; a.grad_dtype = b.grad_dtype;
    a.dg = b.dg_stage; a.dg_tile_stride = b.dg_tile_stride; a.scale = pb.scale;
    size_t smem = sizeof(float) * (5 * C * LD + 2 * BT * LD + C * (C + 1) + BT);
    int rc = set_smem(k_bwd_dqkg<T, C>, smem);
    if (rc) return rc;
    KernelScope ks("generic_bwd_dqkg", st);
    k_bwd_dqkg<T, C><<<dim3(pb.total_chunks, cdiv(pb.K, BT), pb.H), NTH, smem, st>>>(a);
    if ((rc = post_launch())) return rc;
  }
  return TOPS_OK;
}

#define DISPATCH_T_C(pb, CALL)                                                        \
  do {                                                                                \
    if ((pb).dtype == TOPS_F32) { DISPATCH_C(float, pb, CALL); }                      \
    else if ((pb).dtype == TOPS_BF16) { DISPATCH_C(__nv_bfloat16, pb, CALL); }        \
    else if ((pb).dtype == TOPS_F16) { DISPATCH_C(__half, pb, CALL); }                \
    return TOPS_E_BAD_DTYPE;                                                          \
  } while (0)
#define DISPATCH_C(TT, pb, CALL)                                  \
  do {                                                            \
    using T = TT;                                                 \
    if ((pb).m.C == 16) { constexpr int C = 16; return CALL; }    \
    if ((pb).m.C == 32) { constexpr int C = 32; return CALL; }    \
    if ((pb).m.C == 64) { constexpr int C = 64; return CALL; }    \
    return TOPS_E_BAD_SHAPE;                                      \
  } while (0)

int launch_scan(const Problem& pb, bool bwd, const void* x, const void* y, const float* s0, void* states,
                int states_f32, float* s_final, cudaStream_t st) {
  DISPATCH_T_C(pb, (scan_T<T, C>(pb, bwd, x, y, s0, states, states_f32, s_final, st)));
}

int launch_fwd_o(const Problem& pb, const void* q, const void* k, const void* v, const void* h, int h_f32,
                 void* o, float* A_out, int round_A, cudaStream_t st) {
  DISPATCH_T_C(pb, (fwd_o_T<T, C>(pb, q, k, v, h, h_f32, o, A_out, round_A, st)));
}

int launch_bwd(const Problem& pb, const BwdBuffers& b, cudaStream_t st) {
  DISPATCH_T_C(pb, (bwd_T<T, C>(pb, b, st)));
}

int launch_sum_partials(const float* part, size_t stride, int n, float* out, size_t count, cudaStream_t st) {
  if (count == 0) return TOPS_OK;
  KernelScope ks("generic_sum_partials", st);
  k_sum_partials<<<(unsigned)((count + 255) / 256), 256, 0, st>>>(part, stride, n, out, count);
  return post_launch();
}

// State entering (forward) or state gradient leaving (reverse) time shard `rank` of `R`: the value at the
// outer end pushed through the shards in between, h <- h * exp(P_s) + S_s, shard by shard in a fixed order.
//   first [BH,K,V] or null (zero);  P [R,BH,K];  S [R,BH,K,V];  out_in, out_all [BH,K,V] (out_all may be null:
//   the value pushed through every shard, i.e. the final state / the gradient of the initial state)
__global__ void k_fold_shards(const float* __restrict__ first, const float* __restrict__ P, const float* __restrict__ S,
                              float* __restrict__ out_in, float* __restrict__ out_all, int R, int rank, int reverse,
                              size_t BH, int K, int V) {
  const size_t n4 = BH * K * V / 4;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const size_t e = i * 4, bhk = e / V;
    float4 cur = first ? *reinterpret_cast<const float4*>(first + e) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int t = 0; t < R; ++t) {
      const int s = reverse ? R - 1 - t : t;
      if (s == rank) *reinterpret_cast<float4*>(out_in + e) = cur;
      const float w = __expf(P[(size_t)s * BH * K + bhk]);
      const float4 add = *reinterpret_cast<const float4*>(S + (size_t)s * BH * K * V + e);
      cur = make_float4(fmaf(cur.x, w, add.x), fmaf(cur.y, w, add.y), fmaf(cur.z, w, add.z), fmaf(cur.w, w, add.w));
    }
    if (out_all) *reinterpret_cast<float4*>(out_all + e) = cur;
  }
}

int launch_fold_shards(const float* first, const float* P, const float* S, float* out_in, float* out_all, int R, int rank,
                       int reverse, size_t BH, int K, int V, cudaStream_t st) {
  const size_t n4 = BH * K * V / 4;
  const int grid = (int)((n4 + 255) / 256 < 148 * 8 ? (n4 + 255) / 256 : 148 * 8);
  KernelScope ks("fold_shards", st);
  k_fold_shards<<<grid, 256, 0, st>>>(first, P, S, out_in, out_all, R, rank, reverse, BH, K, V);
  return post_launch();
}

}  // namespace generic
}  // namespace tops
