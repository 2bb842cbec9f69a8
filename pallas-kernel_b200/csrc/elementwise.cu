// The steps either side of the attention kernels: gate activations (and their backward with the
// parameter reductions), q/k L2 normalisation, and the gated RMS norm of the output.  All are one pass
// over HBM: every input is read once and every output written once, four elements per thread and access
// (8 or 16 bytes), rows reduced inside a warp with shuffles.  Column reductions (dA_log, d dt_bias, d weight)
// go through per-row-block partial sums that a second kernel adds in a fixed order.
#include "elementwise.cuh"

namespace tops {
namespace elementwise {
namespace {

template <class T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 x = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
  }
};
template <> struct Vec4<__half> {
  static __device__ __forceinline__ void load(const __half* p, float (&v)[4]) {
    const uint2 x = *reinterpret_cast<const uint2*>(p);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&x.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&x.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
  static __device__ __forceinline__ void store(__half* p, const float (&v)[4]) {
    const __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
  }
};

__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float softplusf(float x) { return x > 20.f ? x : log1pf(__expf(x)); }
__device__ __forceinline__ float log_sigmoidf(float x) { return fminf(x, 0.f) - log1pf(__expf(-fabsf(x))); }
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// ---------------------------------------------------------------------------
// gate activations
// ---------------------------------------------------------------------------
struct GateConst {
  const float* A_log;    // [H] (KDA kinds)
  const float* dt_bias;  // [H*K] or null
  float lower_bound, normalizer, clamp_min;
  int has_clamp;
};

// value and derivative with respect to the raw gate x (bias already added) of one element
__device__ __forceinline__ float gate_value(int kind, float x, float eA, const GateConst& c) {
  if (kind == TOPS_GATE_ACT_KDA) return -eA * softplusf(x);
  if (kind == TOPS_GATE_ACT_KDA_LOWER_BOUND) return c.lower_bound * sigmoidf(eA * x);
  float y = log_sigmoidf(x) / c.normalizer;
  return (c.has_clamp && y < c.clamp_min) ? c.clamp_min : y;
}

template <class TI, class TO>
__global__ void k_gate_fwd(const TI* __restrict__ g, TO* __restrict__ out, size_t n4, int H, int K, int kind, GateConst c) {
  const int HK = H * K;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const size_t e = i * 4;
    const int hk = (int)(e % HK);
    float x[4], y[4];
    Vec4<TI>::load(g + e, x);
    const float eA = kind == TOPS_GATE_ACT_LOG_SIGMOID ? 0.f : __expf(c.A_log[hk / K]);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float xb = x[t] + ((kind != TOPS_GATE_ACT_LOG_SIGMOID && c.dt_bias) ? c.dt_bias[hk + t] : 0.f);
      y[t] = gate_value(kind, xb, eA, c);
    }
    Vec4<TO>::store(out + e, y);
  }
}

// Backward: dg per element; per row block and column, the sums that become d dt_bias (sum of dg) and
// dA_log (sum of dy * y, or of dg * x for the lower-bound form).  Thread = 4 columns, block = 256 threads
// = 1024 columns, blockIdx.y = row block.
template <class TI, class TD>
__global__ void k_gate_bwd(const TI* __restrict__ g, const TD* __restrict__ dy, TI* __restrict__ dg, size_t rows, int H,
                           int K, int kind, GateConst c, int rows_per_block, float* __restrict__ part_bias,
                           float* __restrict__ part_A) {
  const int HK = H * K;
  const int col = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (col >= HK) return;
  const float eA = kind == TOPS_GATE_ACT_LOG_SIGMOID ? 0.f : __expf(c.A_log[col / K]);
  float bias[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f}, sa[4] = {0.f, 0.f, 0.f, 0.f};
  if (kind != TOPS_GATE_ACT_LOG_SIGMOID && c.dt_bias) Vec4<float>::load(c.dt_bias + col, bias);
  const size_t r0 = (size_t)blockIdx.y * rows_per_block;
  const size_t r1 = r0 + rows_per_block < rows ? r0 + rows_per_block : rows;
  for (size_t r = r0; r < r1; ++r) {
    float x[4], d[4], o[4];
    Vec4<TI>::load(g + r * HK + col, x);
    Vec4<TD>::load(dy + r * HK + col, d);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float xb = x[t] + bias[t];
      if (kind == TOPS_GATE_ACT_KDA) {
        o[t] = -eA * d[t] * sigmoidf(xb);
        sa[t] += d[t] * (-eA * softplusf(xb));
      } else if (kind == TOPS_GATE_ACT_KDA_LOWER_BOUND) {
        const float s = sigmoidf(eA * xb);
        o[t] = d[t] * c.lower_bound * s * (1.f - s) * eA;
        sa[t] += o[t] * xb;
      } else {
        const float y = log_sigmoidf(xb) / c.normalizer;
        o[t] = (c.has_clamp && y < c.clamp_min) ? 0.f : d[t] * (1.f - sigmoidf(xb)) / c.normalizer;
      }
      sb[t] += o[t];
    }
    Vec4<TI>::store(dg + r * HK + col, o);
  }
  if (part_bias) Vec4<float>::store(part_bias + (size_t)blockIdx.y * HK + col, sb);
  if (part_A) Vec4<float>::store(part_A + (size_t)blockIdx.y * HK + col, sa);
}

// out[col] = sum over row blocks of part[blk][col]: 32 columns x 32 row lanes per block, every lane walks its
// rows in order and the 32 lane sums are added in order, so the result does not depend on scheduling
__global__ void __launch_bounds__(1024) k_sum_blocks(const float* __restrict__ part, int nblk, int ncol,
                                                     float* __restrict__ out) {
  __shared__ float sm[32][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + cx;
  float s = 0.f;
  if (col < ncol)
    for (int b = ry; b < nblk; b += 32) s += part[(size_t)b * ncol + col];
  sm[ry][cx] = s;
  __syncthreads();
  if (ry == 0 && col < ncol) {
    float t = 0.f;
#pragma unroll
    for (int r = 0; r < 32; ++r) t += sm[r][cx];
    out[col] = t;
  }
}
// dA[h] = sum over row blocks and the K columns of head h; one block of 32 warps per head, warp w takes the
// row blocks w, w + 32, ...
__global__ void __launch_bounds__(1024) k_sum_heads(const float* __restrict__ part, int nblk, int H, int K,
                                                    float* __restrict__ out) {
  __shared__ float sm[32];
  const int h = blockIdx.x, lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  float s = 0.f;
  for (int b = w; b < nblk; b += 32)
    for (int k = lane; k < K; k += 32) s += part[((size_t)b * H + h) * K + k];
  s = warp_sum(s);
  if (lane == 0) sm[w] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) t += sm[i];
    out[h] = t;
  }
}


// ---------------------------------------------------------------------------
// L2 normalisation over the last dimension (D <= 1024, D % 4 == 0): one warp per row
// ---------------------------------------------------------------------------
template <class T>
__global__ void k_l2norm_fwd(const T* __restrict__ x, T* __restrict__ y, float* __restrict__ rstd, size_t rows, int D,
                             float eps) {
  const size_t row = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float v[8][4];
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int c = (u * 32 + lane) * 4;
    if (c < D) {
      Vec4<T>::load(x + row * D + c, v[u]);
#pragma unroll
      for (int t = 0; t < 4; ++t) ss = fmaf(v[u][t], v[u][t], ss);
    }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss + eps);
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int c = (u * 32 + lane) * 4;
    if (c < D) {
      float o[4] = {v[u][0] * r, v[u][1] * r, v[u][2] * r, v[u][3] * r};
      Vec4<T>::store(y + row * D + c, o);
    }
  }
  if (rstd && lane == 0) rstd[row] = r;
}

// dx = r (dy - y (dy . y)) with y = x r
template <class T>
__global__ void k_l2norm_bwd(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ dx, size_t rows, int D,
                             float eps) {
  const size_t row = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float v[8][4], d[8][4];
  float ss = 0.f, dot = 0.f;
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int c = (u * 32 + lane) * 4;
    if (c < D) {
      Vec4<T>::load(x + row * D + c, v[u]);
      Vec4<T>::load(dy + row * D + c, d[u]);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        ss = fmaf(v[u][t], v[u][t], ss);
        dot = fmaf(v[u][t], d[u][t], dot);
      }
    }
  }
  ss = warp_sum(ss);
  dot = warp_sum(dot);
  const float r = rsqrtf(ss + eps);
  const float k = dot * r * r;   // (dy . y) r = (dy . x) r^2
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int c = (u * 32 + lane) * 4;
    if (c < D) {
      float o[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) o[t] = r * (d[u][t] - v[u][t] * k);
      Vec4<T>::store(dx + row * D + c, o);
    }
  }
}

// ---------------------------------------------------------------------------
// gated RMS norm: y = x rsqrt(mean(x^2) + eps) w silu(g)      (D <= 1024, D % 4 == 0)
// ---------------------------------------------------------------------------
template <class T>
__global__ void k_rmsnorm_gated_fwd(const T* __restrict__ x, const T* __restrict__ g, const float* __restrict__ w,
                                    T* __restrict__ y, size_t rows, int D, float eps) {
  const size_t row = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float v[8][4];
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int c = (u * 32 + lane) * 4;
    if (c < D) {
      Vec4<T>::load(x + row * D + c, v[u]);
#pragma unroll
      for (int t = 0; t < 4; ++t) ss = fmaf(v[u][t], v[u][t], ss);
    }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)D + eps);
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int c = (u * 32 + lane) * 4;
    if (c < D) {
      float gv[4], wv[4] = {1.f, 1.f, 1.f, 1.f}, o[4];
      Vec4<T>::load(g + row * D + c, gv);
      if (w) Vec4<float>::load(w + c, wv);
#pragma unroll
      for (int t = 0; t < 4; ++t) o[t] = v[u][t] * r * wv[t] * (gv[t] * sigmoidf(gv[t]));
      Vec4<T>::store(y + row * D + c, o);
    }
  }
}

// One warp walks `rows_per_warp` rows and keeps the weight gradient of its columns in registers;
// partial sums per warp go to part_w[warp][D].
template <class T>
__global__ void k_rmsnorm_gated_bwd(const T* __restrict__ x, const T* __restrict__ g, const float* __restrict__ w,
                                    const T* __restrict__ dy, T* __restrict__ dx, T* __restrict__ dg,
                                    float* __restrict__ part_w, size_t rows, int D, float eps, int rows_per_warp) {
  const size_t wid = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const size_t r0 = wid * rows_per_warp;
  if (r0 >= rows) return;
  const size_t r1 = r0 + rows_per_warp < rows ? r0 + rows_per_warp : rows;
  float dw[8][4];
#pragma unroll
  for (int u = 0; u < 8; ++u)
#pragma unroll
    for (int t = 0; t < 4; ++t) dw[u][t] = 0.f;
  for (size_t row = r0; row < r1; ++row) {
    float v[8][4], a[8][4];   // x; then dy w silu(g) = d(normalised x)
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int c = (u * 32 + lane) * 4;
      if (c < D) {
        Vec4<T>::load(x + row * D + c, v[u]);
#pragma unroll
        for (int t = 0; t < 4; ++t) ss = fmaf(v[u][t], v[u][t], ss);
      }
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / (float)D + eps);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int c = (u * 32 + lane) * 4;
      if (c < D) {
        float gv[4], dv[4], wv[4] = {1.f, 1.f, 1.f, 1.f}, og[4];
        Vec4<T>::load(g + row * D + c, gv);
        Vec4<T>::load(dy + row * D + c, dv);
        if (w) Vec4<float>::load(w + c, wv);
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float s = sigmoidf(gv[t]), silu = gv[t] * s, xn = v[u][t] * r;
          og[t] = dv[t] * xn * wv[t] * (s * (1.f + gv[t] * (1.f - s)));   // d silu / dg = s (1 + g (1 - s))
          dw[u][t] += dv[t] * xn * silu;
          a[u][t] = dv[t] * wv[t] * silu;
          dot = fmaf(a[u][t], xn, dot);
        }
        Vec4<T>::store(dg + row * D + c, og);
      }
    }
    dot = warp_sum(dot) / (float)D;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int c = (u * 32 + lane) * 4;
      if (c < D) {
        float o[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) o[t] = r * (a[u][t] - v[u][t] * r * dot);
        Vec4<T>::store(dx + row * D + c, o);
      }
    }
  }
  if (part_w) {
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int c = (u * 32 + lane) * 4;
      if (c < D) Vec4<float>::store(part_w + wid * D + c, dw[u]);
    }
  }
}

template <class F>
int dispatch(int dtype, F f) {
  if (dtype == TOPS_F32) return f((float*)nullptr);
  if (dtype == TOPS_BF16) return f((__nv_bfloat16*)nullptr);
  if (dtype == TOPS_F16) return f((__half*)nullptr);
  return TOPS_E_BAD_DTYPE;
}

GateConst gate_const(const tops_gate_act_params& p) {
  GateConst c;
  c.A_log = p.A_log; c.dt_bias = p.dt_bias; c.lower_bound = p.lower_bound; c.normalizer = p.normalizer;
  c.clamp_min = p.clamp_min; c.has_clamp = p.has_clamp_min;
  return c;
}

constexpr int kGateRowsPerBlock = 64;
int gate_row_blocks(size_t rows) { return (int)((rows + kGateRowsPerBlock - 1) / kGateRowsPerBlock); }
constexpr int kNormRowsPerWarp = 32;
size_t norm_warps(size_t rows) { return (rows + kNormRowsPerWarp - 1) / kNormRowsPerWarp; }

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

int gate_check(const tops_gate_act_params& p) {
  if (p.rows < 1 || p.H < 1 || p.K < 1 || p.K % 4 != 0) return TOPS_E_BAD_SHAPE;
  if (p.kind < TOPS_GATE_ACT_KDA || p.kind > TOPS_GATE_ACT_LOG_SIGMOID) return TOPS_E_BAD_SHAPE;
  if (p.kind != TOPS_GATE_ACT_LOG_SIGMOID && !p.A_log) return TOPS_E_NULL;
  if (p.kind == TOPS_GATE_ACT_LOG_SIGMOID && !(p.normalizer != 0.f)) return TOPS_E_BAD_SHAPE;
  if (!aligned16(p.g) || !aligned16(p.out) || !aligned16(p.dt_bias)) return TOPS_E_ALIGN;
  return TOPS_OK;
}

int gate_fwd(const tops_gate_act_params& p, cudaStream_t st) {
  const size_t n4 = (size_t)p.rows * p.H * p.K / 4;
  const int grid = (int)((n4 + 255) / 256 < 148 * 16 ? (n4 + 255) / 256 : 148 * 16);
  const GateConst c = gate_const(p);
  KernelScope ks("gate_act_fwd", st);
  int rc = dispatch(p.dtype, [&](auto* ti) {
    using TI = std::remove_pointer_t<decltype(ti)>;
    return dispatch(p.out_dtype, [&](auto* to) {
      using TO = std::remove_pointer_t<decltype(to)>;
      k_gate_fwd<TI, TO><<<grid, 256, 0, st>>>(reinterpret_cast<const TI*>(p.g), reinterpret_cast<TO*>(p.out), n4, p.H,
                                               p.K, p.kind, c);
      return TOPS_OK;
    });
  });
  return rc ? rc : post_launch();
}

size_t gate_bwd_workspace_bytes(const tops_gate_act_bwd_params& p) {
  return align_up((size_t)gate_row_blocks(p.fwd.rows) * p.fwd.H * p.fwd.K * sizeof(float)) * 2 + 256;
}

int gate_bwd(const tops_gate_act_bwd_params& p, void* ws, cudaStream_t st) {
  const tops_gate_act_params& f = p.fwd;
  if (!aligned16(p.dy) || !aligned16(p.dg) || !aligned16(ws)) return TOPS_E_ALIGN;
  const int HK = f.H * f.K, nblk = gate_row_blocks(f.rows);
  const bool kda = f.kind != TOPS_GATE_ACT_LOG_SIGMOID;
  float* part_bias = (kda && p.dbias) ? reinterpret_cast<float*>(ws) : nullptr;
  float* part_A = (kda && p.dA_log) ? reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + align_up((size_t)nblk * HK * sizeof(float)))
                                    : nullptr;
  const GateConst c = gate_const(f);
  dim3 grid((HK / 4 + 255) / 256, nblk);
  {
    KernelScope ks("gate_act_bwd", st);
    int rc = dispatch(f.dtype, [&](auto* ti) {
      using TI = std::remove_pointer_t<decltype(ti)>;
      return dispatch(p.dy_dtype, [&](auto* td) {
        using TD = std::remove_pointer_t<decltype(td)>;
        k_gate_bwd<TI, TD><<<grid, 256, 0, st>>>(reinterpret_cast<const TI*>(f.g), reinterpret_cast<const TD*>(p.dy),
                                                 reinterpret_cast<TI*>(p.dg), (size_t)f.rows, f.H, f.K, f.kind, c,
                                                 kGateRowsPerBlock, part_bias, part_A);
        return TOPS_OK;
      });
    });
    if (rc) return rc;
    if ((rc = post_launch())) return rc;
  }
  if (part_bias) {
    KernelScope ks("gate_act_bwd_sum", st);
    k_sum_blocks<<<(HK + 31) / 32, 1024, 0, st>>>(part_bias, nblk, HK, p.dbias);
    int rc = post_launch();
    if (rc) return rc;
  }
  if (part_A) {
    KernelScope ks("gate_act_bwd_sum", st);
    k_sum_heads<<<f.H, 1024, 0, st>>>(part_A, nblk, f.H, f.K, p.dA_log);
    return post_launch();
  }
  return TOPS_OK;
}

int norm_check(const tops_norm_params& p) {
  if (p.rows < 1 || p.D < 4 || p.D > 1024 || p.D % 4 != 0) return TOPS_E_BAD_SHAPE;
  if (!p.x || !p.y) return TOPS_E_NULL;
  if (!aligned16(p.x) || !aligned16(p.y) || !aligned16(p.gate) || !aligned16(p.weight) || !aligned16(p.dy) ||
      !aligned16(p.dx) || !aligned16(p.dgate))
    return TOPS_E_ALIGN;
  return TOPS_OK;
}

int l2norm_fwd(const tops_norm_params& p, cudaStream_t st) {
  const int grid = (int)((p.rows + 7) / 8);
  KernelScope ks("l2norm_fwd", st);
  int rc = dispatch(p.dtype, [&](auto* t) {
    using T = std::remove_pointer_t<decltype(t)>;
    k_l2norm_fwd<T><<<grid, 256, 0, st>>>(reinterpret_cast<const T*>(p.x), reinterpret_cast<T*>(p.y), p.rstd, (size_t)p.rows,
                                          p.D, p.eps);
    return TOPS_OK;
  });
  return rc ? rc : post_launch();
}

int l2norm_bwd(const tops_norm_params& p, cudaStream_t st) {
  if (!p.dy || !p.dx) return TOPS_E_NULL;
  const int grid = (int)((p.rows + 7) / 8);
  KernelScope ks("l2norm_bwd", st);
  int rc = dispatch(p.dtype, [&](auto* t) {
    using T = std::remove_pointer_t<decltype(t)>;
    k_l2norm_bwd<T><<<grid, 256, 0, st>>>(reinterpret_cast<const T*>(p.x), reinterpret_cast<const T*>(p.dy),
                                          reinterpret_cast<T*>(p.dx), (size_t)p.rows, p.D, p.eps);
    return TOPS_OK;
  });
  return rc ? rc : post_launch();
}

int rmsnorm_gated_fwd(const tops_norm_params& p, cudaStream_t st) {
  if (!p.gate) return TOPS_E_NULL;
  const int grid = (int)((p.rows + 7) / 8);
  KernelScope ks("rmsnorm_gated_fwd", st);
  int rc = dispatch(p.dtype, [&](auto* t) {
    using T = std::remove_pointer_t<decltype(t)>;
    k_rmsnorm_gated_fwd<T><<<grid, 256, 0, st>>>(reinterpret_cast<const T*>(p.x), reinterpret_cast<const T*>(p.gate), p.weight,
                                                 reinterpret_cast<T*>(p.y), (size_t)p.rows, p.D, p.eps);
    return TOPS_OK;
  });
  return rc ? rc : post_launch();
}

size_t rmsnorm_gated_bwd_workspace_bytes(const tops_norm_params& p) {
  return align_up(norm_warps((size_t)p.rows) * p.D * sizeof(float)) + 256;
}

int rmsnorm_gated_bwd(const tops_norm_params& p, void* ws, cudaStream_t st) {
  if (!p.gate || !p.dy || !p.dx || !p.dgate) return TOPS_E_NULL;
  if (!aligned16(ws)) return TOPS_E_ALIGN;
  const size_t warps = norm_warps((size_t)p.rows);
  float* part = p.dweight ? reinterpret_cast<float*>(ws) : nullptr;
  {
    KernelScope ks("rmsnorm_gated_bwd", st);
    int rc = dispatch(p.dtype, [&](auto* t) {
      using T = std::remove_pointer_t<decltype(t)>;
      k_rmsnorm_gated_bwd<T><<<(int)((warps + 7) / 8), 256, 0, st>>>(
          reinterpret_cast<const T*>(p.x), reinterpret_cast<const T*>(p.gate), p.weight, reinterpret_cast<const T*>(p.dy),
          reinterpret_cast<T*>(p.dx), reinterpret_cast<T*>(p.dgate), part, (size_t)p.rows, p.D, p.eps, kNormRowsPerWarp);
      return TOPS_OK;
    });
    if (rc) return rc;
    if ((rc = post_launch())) return rc;
  }
  if (part) {
    KernelScope ks("rmsnorm_gated_bwd_sum", st);
    k_sum_blocks<<<(p.D + 31) / 32, 1024, 0, st>>>(part, (int)warps, p.D, p.dweight);
    return post_launch();
  }
  return TOPS_OK;
}

}  // namespace elementwise
}  // namespace tops
