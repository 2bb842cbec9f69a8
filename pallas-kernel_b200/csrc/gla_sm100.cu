// Chunked GLA on the 5th-generation tensor cores (sm_100a): bf16 operands staged
// in shared memory by TMA, contractions issued with tcgen05.mma into tensor
// memory, fp32 accumulation, gates and state kept in fp32.
//
// Shapes taken here: bf16 q/k/v/g, K = V = 128, chunk 64, T a multiple of 64,
// dense batch, per-channel gates.  Everything else runs on the generic kernels.
//
// Data layout.  Activations stay in the caller's [B,T,H,D] layout; a chunk of
// one head is a 64 x 128 tile whose rows are H*D elements apart, fetched as two
// 64 x 64 TMA boxes (SWIZZLE_128B) straight into the tile format UMMA
// descriptors read (sm100_prims.cuh).  Chunk-start states h_c and their
// gradients dh_c are kept as bf16 [B,NT,H,K,V] scratch in HBM: they are only
// ever used as bf16 tensor-core operands; the running state itself is fp32 in
// registers of the scan kernels.
//
// Kernels
//   k_scan<false>  h_c,  h <- h * exp(G_n) + (k exp(G_n - G))^T v       (forward scan)
//   k_scan<true>   dh_c, dh <- dh * exp(G_n) + (q scale exp(G))^T do    (reverse scan)
//   k_fwd_o        A = tril(q~ k~^T) scale;  o = q~ (h_c exp(mid) scale) + A v
//   k_bwd_main     dA, dv, dq, dk, dg of one chunk from q, k, v, g, do, h_c, dh_c
// with G the chunk-local cumulative gate and q~ = q exp(G - mid),
// k~ = k exp(mid - G), mid = (G_0 + G_n) / 2 per channel.
#include <mutex>

#include "gla_sm100.cuh"
#include "sm100_prims.cuh"

namespace tops {
namespace sm100 {

__device__ int g_error;  // first bounded wait that gave up (0 = none)

namespace {

constexpr int C = 64;    // chunk
constexpr int D = 128;   // K = V
constexpr int NTHREADS = 128;
constexpr uint32_t SLAB64 = 64 * 128;    // bytes of a 64-row slab
constexpr uint32_t TILE64 = 2 * SLAB64;  // 64 x 128 bf16 tile
constexpr uint32_t TILE128 = 2 * 128 * 128;  // 128 x 128 bf16 tile

__device__ __forceinline__ uint8_t* align1024(uint8_t* p) {
  return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~static_cast<uintptr_t>(1023));
}
__device__ __forceinline__ float ld_bf16(const uint8_t* tile, uint32_t off) {
  return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(tile + off));
}
__device__ __forceinline__ void st_bf16(uint8_t* tile, uint32_t off, float x) {
  *reinterpret_cast<__nv_bfloat16*>(tile + off) = __float2bfloat16_rn(x);
}
// offset of (row i, this thread's column) in a 64-row tile; colbase / cchunk from col_prep
struct ColAddr {
  uint32_t base, cchunk;
  __device__ __forceinline__ uint32_t at(int i) const { return base + (uint32_t)i * 128u + (((cchunk ^ (uint32_t)i) & 7u) << 4); }
};
__device__ __forceinline__ ColAddr col_prep(int rows, int col) {
  return ColAddr{(uint32_t)((col >> 6) * rows * 128 + (col & 7) * 2), (uint32_t)((col & 63) >> 3)};
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ void fail(int code) { atomicCAS(&g_error, 0, code); }

// ===========================================================================
// State scans
// ===========================================================================
struct ScanParams {
  CUtensorMap mx, mg, my;  // x: k (fwd) / q (bwd); y: v / do
  const float* s0;         // h0 / dht  [B,H,K,V] or null
  __nv_bfloat16* states;   // h / dh    [B,NT,H,K,V]
  float* s_final;          // ht / dh0  or null
  int T, H, NT;
  float scale;
};

template <bool BWD>
__global__ void __launch_bounds__(NTHREADS) k_scan(const __grid_constant__ ScanParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  constexpr uint32_t STAGE = 2 * TILE64 + SLAB64;  // x, g, y-half
  uint8_t* xg = smem + 2 * STAGE;                   // gated x, 64 x 128
  __shared__ uint64_t full[2], mma_bar;
  __shared__ uint32_t tmem_slot;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int vh = blockIdx.x, bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int NT = p.NT;

  if (tid == 0) {
    mbar_init(&full[0], 1); mbar_init(&full[1], 1); mbar_init(&mma_bar, 1);
    fence_barrier_init();
    tma_prefetch_desc(&p.mx); tma_prefetch_desc(&p.mg); tma_prefetch_desc(&p.my);
  }
  if (warp == 0) { tmem_alloc(&tmem_slot, 64); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_slot;

  auto issue = [&](int step) {
    const int ci = BWD ? NT - 1 - step : step;
    const int s = step & 1;
    uint8_t* st = smem + s * STAGE;
    const int row = b * p.T + ci * C;
    mbar_expect_tx(&full[s], STAGE);
    tma_load_3d(st, &p.mx, &full[s], 0, h, row);
    tma_load_3d(st + SLAB64, &p.mx, &full[s], 64, h, row);
    tma_load_3d(st + TILE64, &p.mg, &full[s], 0, h, row);
    tma_load_3d(st + TILE64 + SLAB64, &p.mg, &full[s], 64, h, row);
    tma_load_3d(st + 2 * TILE64, &p.my, &full[s], vh * 64, h, row);
  };
  if (tid == 0) { issue(0); if (NT > 1) issue(1); }

  // fp32 state: row k = tid, columns vh*64 .. vh*64+63
  float S[64];
  {
    const float* src = p.s0 ? p.s0 + ((size_t)bh * D + tid) * D + vh * 64 : nullptr;
#pragma unroll
    for (int j = 0; j < 64; j += 4) {
      float4 x = src ? *reinterpret_cast<const float4*>(src + j) : make_float4(0.f, 0.f, 0.f, 0.f);
      S[j] = x.x; S[j + 1] = x.y; S[j + 2] = x.z; S[j + 3] = x.w;
    }
  }
  const ColAddr ca = col_prep(64, tid);
  bool ok = true;
  for (int step = 0; step < NT && ok; ++step) {
    const int ci = BWD ? NT - 1 - step : step;
    const int s = step & 1;
    uint8_t* xs = smem + s * STAGE;
    uint8_t* gs = xs + TILE64;
    uint8_t* ys = xs + 2 * TILE64;
    ok = __syncthreads_and(mbar_wait(&full[s], (step >> 1) & 1));
    if (!ok) { fail(1); break; }
    // gate the x operand; this thread owns channel `tid`
    float gn = 0.f;
#pragma unroll 8
    for (int i = 0; i < C; ++i) gn += ld_bf16(gs, ca.at(i));
    float run = 0.f;
#pragma unroll 8
    for (int i = 0; i < C; ++i) {
      run += ld_bf16(gs, ca.at(i));
      float x = ld_bf16(xs, ca.at(i));
      float y = BWD ? x * p.scale * __expf(run) : x * __expf(gn - run);
      st_bf16(xg, ca.at(i), y);
    }
    const float decay = __expf(gn);
    fence_async_smem();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      const uint32_t xa = smem_u32(xg), ya = smem_u32(ys);
#pragma unroll
      for (int k0 = 0; k0 < C; k0 += 16)
        umma_bf16(tm, desc_mnmajor(xa, 64, k0, 0), desc_mnmajor(ya, 64, k0, 0), umma_idesc(128, 64, 1, 1), k0 > 0);
      umma_commit(&mma_bar);
    }
    // record the state this chunk starts from (bf16), while the tensor core works
    {
      __nv_bfloat16* dst = p.states + ((((size_t)b * NT + ci) * p.H + h) * D + tid) * D + vh * 64;
#pragma unroll
      for (int j = 0; j < 64; j += 8) {
        uint4 u;
        u.x = pack_bf16(S[j], S[j + 1]); u.y = pack_bf16(S[j + 2], S[j + 3]);
        u.z = pack_bf16(S[j + 4], S[j + 5]); u.w = pack_bf16(S[j + 6], S[j + 7]);
        *reinterpret_cast<uint4*>(dst + j) = u;
      }
    }
    ok = __syncthreads_and(mbar_wait(&mma_bar, step & 1));
    if (!ok) { fail(2); break; }
    tc_fence_after();
#pragma unroll
    for (int j = 0; j < 64; j += 32) {
      float d[32];
      tmem_ld32(tmem_addr(tm, warp * 32, j), d);
#pragma unroll
      for (int t = 0; t < 32; ++t) S[j + t] = fmaf(S[j + t], decay, d[t]);
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && step + 2 < NT) issue(step + 2);
  }
  if (ok && p.s_final) {
    float* dst = p.s_final + ((size_t)bh * D + tid) * D + vh * 64;
#pragma unroll
    for (int j = 0; j < 64; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(S[j], S[j + 1], S[j + 2], S[j + 3]);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 64);
}

// ===========================================================================
// Forward output
// ===========================================================================
struct FwdOParams {
  CUtensorMap mq, mk, mg, mv, mh;
  __nv_bfloat16* o;
  int T, H, NT;
  float scale;
};

__global__ void __launch_bounds__(NTHREADS) k_fwd_o(const __grid_constant__ FwdOParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* qs = smem;                 // q -> q~ in place
  uint8_t* ks = qs + TILE64;          // k -> k~ in place
  uint8_t* gs = ks + TILE64;          // g; later the bf16 intra matrix (first 8 KB)
  uint8_t* vs = gs + TILE64;
  uint8_t* hs = vs + TILE64;          // h_c, 128 x 128; row k scaled in place by exp(mid_k) scale
  __shared__ uint64_t bar_load, bar_a, bar_o;
  __shared__ uint32_t tmem_slot;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ci = blockIdx.x, bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int row = b * p.T + ci * C;

  if (tid == 0) {
    mbar_init(&bar_load, 1); mbar_init(&bar_a, 1); mbar_init(&bar_o, 1);
    fence_barrier_init();
    mbar_expect_tx(&bar_load, 4 * TILE64 + TILE128);
    tma_load_3d(qs, &p.mq, &bar_load, 0, h, row); tma_load_3d(qs + SLAB64, &p.mq, &bar_load, 64, h, row);
    tma_load_3d(ks, &p.mk, &bar_load, 0, h, row); tma_load_3d(ks + SLAB64, &p.mk, &bar_load, 64, h, row);
    tma_load_3d(gs, &p.mg, &bar_load, 0, h, row); tma_load_3d(gs + SLAB64, &p.mg, &bar_load, 64, h, row);
    tma_load_3d(vs, &p.mv, &bar_load, 0, h, row); tma_load_3d(vs + SLAB64, &p.mv, &bar_load, 64, h, row);
    const int hrow = ((b * p.NT + ci) * p.H + h) * D;
    tma_load_2d(hs, &p.mh, &bar_load, 0, hrow); tma_load_2d(hs + TILE128 / 2, &p.mh, &bar_load, 64, hrow);
  }
  if (warp == 0) { tmem_alloc(&tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_slot;
  bool ok = __syncthreads_and(mbar_wait(&bar_load, 0));
  if (!ok) fail(3);
  if (ok) {
    const ColAddr ca = col_prep(64, tid);
    float g0 = ld_bf16(gs, ca.at(0)), gn = 0.f;
#pragma unroll 8
    for (int i = 0; i < C; ++i) gn += ld_bf16(gs, ca.at(i));
    const float mid = 0.5f * (g0 + gn);
    const float qscale = __expf(mid) * p.scale;
    float run = 0.f;
#pragma unroll 8
    for (int i = 0; i < C; ++i) {
      run += ld_bf16(gs, ca.at(i));
      const float e = __expf(run - mid);
      const float q = ld_bf16(qs, ca.at(i)), k = ld_bf16(ks, ca.at(i));
      st_bf16(qs, ca.at(i), q * e);
      st_bf16(ks, ca.at(i), __fdividef(k, e));
    }
    // q exp(G) scale = q~ (exp(mid) scale): fold the per-channel factor into row `tid` of h_c
#pragma unroll 4
    for (int c8 = 0; c8 < D; c8 += 8) {
      uint4* ph = reinterpret_cast<uint4*>(hs + tile_off(128, tid, c8));
      uint4 a = *ph;
      __nv_bfloat162* pa = reinterpret_cast<__nv_bfloat162*>(&a);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        float2 f = __bfloat1622float2(pa[t]);
        pa[t] = __floats2bfloat162_rn(f.x * qscale, f.y * qscale);
      }
      *ph = a;
    }
    fence_async_smem();
  }
  __syncthreads();
  if (ok && tid == 0) {
    tc_fence_after();
    const uint32_t qa = smem_u32(qs), ka = smem_u32(ks), ha = smem_u32(hs);
#pragma unroll
    for (int k0 = 0; k0 < D; k0 += 16)   // A = q~ k~^T  -> columns [0,64)
      umma_bf16(tm, desc_kmajor(qa, 64, 0, k0), desc_kmajor(ka, 64, 0, k0), umma_idesc(64, 64, 0, 0), k0 > 0);
    umma_commit(&bar_a);
#pragma unroll
    for (int k0 = 0; k0 < D; k0 += 16)   // o = q~ h'  -> columns [64,192)
      umma_bf16(tm + 64, desc_kmajor(qa, 64, 0, k0), desc_mnmajor(ha, 128, k0, 0), umma_idesc(64, 128, 0, 1), k0 > 0);
  }
  if (ok) {
    ok = __syncthreads_and(mbar_wait(&bar_a, 0));
    if (!ok) fail(4);
  }
  if (ok) {
    tc_fence_after();
    // rows of an M = 64 accumulator sit in lanes 0..15 of each warp's 32-lane window
    const int i = 16 * warp + lane;
#pragma unroll
    for (int j0 = 0; j0 < C; j0 += 32) {
      float a[32];
      tmem_ld32(tmem_addr(tm, warp * 32, j0), a);
      if (lane < 16) {
#pragma unroll
        for (int c8 = 0; c8 < 32; c8 += 8) {
          uint32_t w[4];
#pragma unroll
          for (int t = 0; t < 8; t += 2) {
            const int j = j0 + c8 + t;
            w[t >> 1] = pack_bf16(j <= i ? a[c8 + t] * p.scale : 0.f, j + 1 <= i ? a[c8 + t + 1] * p.scale : 0.f);
          }
          *reinterpret_cast<uint4*>(gs + slab_off(i, j0 + c8)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
    fence_async_smem();
    tc_fence_before();
  }
  __syncthreads();
  if (ok && tid == 0) {
    tc_fence_after();
    const uint32_t pa = smem_u32(gs), va = smem_u32(vs);
#pragma unroll
    for (int k0 = 0; k0 < C; k0 += 16)   // o += A v
      umma_bf16(tm + 64, desc_kmajor(pa, 64, 0, k0), desc_mnmajor(va, 64, k0, 0), umma_idesc(64, 128, 0, 1), 1);
    umma_commit(&bar_o);
  }
  if (ok) {
    ok = __syncthreads_and(mbar_wait(&bar_o, 0));
    if (!ok) fail(5);
  }
  if (ok) {
    tc_fence_after();
    const int i = 16 * warp + lane;
    __nv_bfloat16* dst = p.o + ((size_t)(row + i) * p.H + h) * D;
#pragma unroll
    for (int c0 = 0; c0 < D; c0 += 32) {
      float a[32];
      tmem_ld32(tmem_addr(tm, warp * 32, 64 + c0), a);
      if (lane < 16) {
#pragma unroll
        for (int t = 0; t < 32; t += 8)
          *reinterpret_cast<uint4*>(dst + c0 + t) = make_uint4(pack_bf16(a[t], a[t + 1]), pack_bf16(a[t + 2], a[t + 3]),
                                                               pack_bf16(a[t + 4], a[t + 5]), pack_bf16(a[t + 6], a[t + 7]));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 256);
}

// ===========================================================================
// Backward of one chunk
// ===========================================================================
struct BwdParams {
  CUtensorMap mq, mk, mg, mv, mdo, mh, mdh;
  float *dq, *dk, *dg;   // [B,T,H,K] fp32 (dg may be null)
  __nv_bfloat16* dv;     // [B,T,H,V]
  int T, H, NT;
  float scale;
};

__global__ void __launch_bounds__(NTHREADS) k_bwd_main(const __grid_constant__ BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* qs = smem;
  uint8_t* ks = qs + TILE64;
  uint8_t* gs = ks + TILE64;
  uint8_t* vs = gs + TILE64;
  uint8_t* dos = vs + TILE64;
  uint8_t* hs = dos + TILE64;         // h_c   128 x 128
  uint8_t* dhs = hs + TILE128;        // dh_c  128 x 128
  uint8_t* qt = dhs + TILE128;        // q exp(G - mid)      (later: fp32 dg staging, with kt)
  uint8_t* kt = qt + TILE64;          // k exp(mid - G)
  uint8_t* kg = kt + TILE64;          // k exp(G_n - G)
  uint8_t* Ps = kg + TILE64;          // tril(A) scale, bf16 64 x 64
  uint8_t* dAs = Ps + SLAB64;         // tril(dA) scale, bf16 64 x 64
  __shared__ uint64_t bar_load, bar1, bar2, bar3;
  __shared__ uint32_t tmem_slot;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ci = blockIdx.x, bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int row = b * p.T + ci * C;

  if (tid == 0) {
    mbar_init(&bar_load, 1); mbar_init(&bar1, 1); mbar_init(&bar2, 1); mbar_init(&bar3, 1);
    fence_barrier_init();
    mbar_expect_tx(&bar_load, 5 * TILE64 + 2 * TILE128);
    tma_load_3d(qs, &p.mq, &bar_load, 0, h, row); tma_load_3d(qs + SLAB64, &p.mq, &bar_load, 64, h, row);
    tma_load_3d(ks, &p.mk, &bar_load, 0, h, row); tma_load_3d(ks + SLAB64, &p.mk, &bar_load, 64, h, row);
    tma_load_3d(gs, &p.mg, &bar_load, 0, h, row); tma_load_3d(gs + SLAB64, &p.mg, &bar_load, 64, h, row);
    tma_load_3d(vs, &p.mv, &bar_load, 0, h, row); tma_load_3d(vs + SLAB64, &p.mv, &bar_load, 64, h, row);
    tma_load_3d(dos, &p.mdo, &bar_load, 0, h, row); tma_load_3d(dos + SLAB64, &p.mdo, &bar_load, 64, h, row);
    const int hrow = ((b * p.NT + ci) * p.H + h) * D;
    tma_load_2d(hs, &p.mh, &bar_load, 0, hrow); tma_load_2d(hs + TILE128 / 2, &p.mh, &bar_load, 64, hrow);
    tma_load_2d(dhs, &p.mdh, &bar_load, 0, hrow); tma_load_2d(dhs + TILE128 / 2, &p.mdh, &bar_load, 64, hrow);
  }
  if (warp == 0) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_slot;
  // tensor-memory columns
  constexpr uint32_t cA = 0, cdA = 64, cdq2 = 128, cdk2 = 192, cdv = 256, cdq1 = 320, cdk1 = 384;

  const ColAddr ca = col_prep(64, tid);
  float mid = 0.f, gn = 0.f, hdh = 0.f;
  bool ok = __syncthreads_and(mbar_wait(&bar_load, 0));
  if (!ok) fail(6);
  if (ok) {
    const float g0 = ld_bf16(gs, ca.at(0));
#pragma unroll 8
    for (int i = 0; i < C; ++i) gn += ld_bf16(gs, ca.at(i));
    mid = 0.5f * (g0 + gn);
    const float tail = __expf(gn - mid);
    float run = 0.f;
#pragma unroll 8
    for (int i = 0; i < C; ++i) {
      run += ld_bf16(gs, ca.at(i));
      const float e = __expf(run - mid);
      const float q = ld_bf16(qs, ca.at(i)), k = ld_bf16(ks, ca.at(i));
      const float kn = __fdividef(k, e);
      st_bf16(qt, ca.at(i), q * e);
      st_bf16(kt, ca.at(i), kn);
      st_bf16(kg, ca.at(i), kn * tail);
    }
    // sum_v h[k][v] dh[k][v] for k = tid
#pragma unroll 4
    for (int c8 = 0; c8 < D; c8 += 8) {
      const uint32_t off = tile_off(128, tid, c8);
      const uint4 a = *reinterpret_cast<const uint4*>(hs + off), d = *reinterpret_cast<const uint4*>(dhs + off);
      const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* pd = reinterpret_cast<const __nv_bfloat162*>(&d);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 fa = __bfloat1622float2(pa[t]), fd = __bfloat1622float2(pd[t]);
        hdh = fmaf(fa.x, fd.x, hdh);
        hdh = fmaf(fa.y, fd.y, hdh);
      }
    }
    fence_async_smem();
  }
  __syncthreads();
  if (ok && tid == 0) {
    tc_fence_after();
    const uint32_t qta = smem_u32(qt), kta = smem_u32(kt), kga = smem_u32(kg), va = smem_u32(vs), doa = smem_u32(dos),
                   ha = smem_u32(hs), dha = smem_u32(dhs);
#pragma unroll
    for (int k0 = 0; k0 < D; k0 += 16)   // A[i][j] = q~ k~^T
      umma_bf16(tm + cA, desc_kmajor(qta, 64, 0, k0), desc_kmajor(kta, 64, 0, k0), umma_idesc(64, 64, 0, 0), k0 > 0);
#pragma unroll
    for (int k0 = 0; k0 < D; k0 += 16)   // dA[i][j] = do v^T
      umma_bf16(tm + cdA, desc_kmajor(doa, 64, 0, k0), desc_kmajor(va, 64, 0, k0), umma_idesc(64, 64, 0, 0), k0 > 0);
    umma_commit(&bar1);
#pragma unroll
    for (int k0 = 0; k0 < D; k0 += 16)   // dq_inter^T[k][i] = h do^T
      umma_bf16(tm + cdq2, desc_kmajor(ha, 128, 0, k0), desc_kmajor(doa, 64, 0, k0), umma_idesc(128, 64, 0, 0), k0 > 0);
#pragma unroll
    for (int k0 = 0; k0 < D; k0 += 16)   // dk_inter^T[k][j] = dh v^T
      umma_bf16(tm + cdk2, desc_kmajor(dha, 128, 0, k0), desc_kmajor(va, 64, 0, k0), umma_idesc(128, 64, 0, 0), k0 > 0);
#pragma unroll
    for (int k0 = 0; k0 < D; k0 += 16)   // dv^T[v][j] = dh^T kg^T
      umma_bf16(tm + cdv, desc_mnmajor(dha, 128, k0, 0), desc_kmajor(kga, 64, 0, k0), umma_idesc(128, 64, 1, 0), k0 > 0);
    umma_commit(&bar2);
  }
  if (ok) {
    ok = __syncthreads_and(mbar_wait(&bar1, 0));
    if (!ok) fail(7);
  }
  if (ok) {
    tc_fence_after();
    const int i = 16 * warp + lane;
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      uint8_t* dst = which ? dAs : Ps;
#pragma unroll
      for (int j0 = 0; j0 < C; j0 += 32) {
        float a[32];
        tmem_ld32(tmem_addr(tm, warp * 32, (which ? cdA : cA) + j0), a);
        if (lane < 16) {
#pragma unroll
          for (int c8 = 0; c8 < 32; c8 += 8) {
            uint32_t w[4];
#pragma unroll
            for (int t = 0; t < 8; t += 2) {
              const int j = j0 + c8 + t;
              w[t >> 1] = pack_bf16(j <= i ? a[c8 + t] * p.scale : 0.f, j + 1 <= i ? a[c8 + t + 1] * p.scale : 0.f);
            }
            *reinterpret_cast<uint4*>(dst + slab_off(i, j0 + c8)) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
    fence_async_smem();
    tc_fence_before();
  }
  __syncthreads();
  if (ok && tid == 0) {
    tc_fence_after();
    const uint32_t qta = smem_u32(qt), kta = smem_u32(kt), doa = smem_u32(dos), pa = smem_u32(Ps), daa = smem_u32(dAs);
#pragma unroll
    for (int k0 = 0; k0 < C; k0 += 16)   // dq_intra^T[k][i] = sum_j k~[j][k] dA[i][j]
      umma_bf16(tm + cdq1, desc_mnmajor(kta, 64, k0, 0), desc_kmajor(daa, 64, 0, k0), umma_idesc(128, 64, 1, 0), k0 > 0);
#pragma unroll
    for (int k0 = 0; k0 < C; k0 += 16)   // dk_intra^T[k][j] = sum_i q~[i][k] dA[i][j]
      umma_bf16(tm + cdk1, desc_mnmajor(qta, 64, k0, 0), desc_mnmajor(daa, 64, k0, 0), umma_idesc(128, 64, 1, 1), k0 > 0);
#pragma unroll
    for (int k0 = 0; k0 < C; k0 += 16)   // dv^T[v][j] += sum_i do[i][v] A[i][j]
      umma_bf16(tm + cdv, desc_mnmajor(doa, 64, k0, 0), desc_mnmajor(pa, 64, k0, 0), umma_idesc(128, 64, 1, 1), 1);
    umma_commit(&bar3);
  }
  if (ok) {
    ok = __syncthreads_and(mbar_wait(&bar3, 0));
    if (!ok) fail(8);
  }
  if (ok) {
    tc_fence_after();
    // dv: this thread owns value channel `tid`
    {
      __nv_bfloat16* dst = p.dv + ((size_t)row * p.H + h) * D + tid;
#pragma unroll
      for (int j0 = 0; j0 < C; j0 += 32) {
        float a[32];
        tmem_ld32(tmem_addr(tm, warp * 32, cdv + j0), a);
#pragma unroll
        for (int t = 0; t < 32; ++t) dst[(size_t)(j0 + t) * p.H * D] = __float2bfloat16_rn(a[t]);
      }
    }
    // dq, dk, dg: this thread owns key channel `tid`; walk time backwards so the
    // suffix sum of the gate gradient stays in a register
    float* stage = reinterpret_cast<float*>(qt);  // [64][128] fp32 over qt + kt (both consumed)
    const float c1 = p.scale * __expf(mid), c2 = __expf(gn - mid);
    float grun = gn, run = 0.f, tail = 0.f;
    const size_t obase = ((size_t)row * p.H + h) * D + tid;
    const size_t ostride = (size_t)p.H * D;
#pragma unroll 1
    for (int i0 = C - 16; i0 >= 0; i0 -= 16) {
      float dq1[16], dq2[16], dk1[16], dk2[16];
      tmem_ld16(tmem_addr(tm, warp * 32, cdq1 + i0), dq1);
      tmem_ld16(tmem_addr(tm, warp * 32, cdq2 + i0), dq2);
      tmem_ld16(tmem_addr(tm, warp * 32, cdk1 + i0), dk1);
      tmem_ld16(tmem_addr(tm, warp * 32, cdk2 + i0), dk2);
#pragma unroll
      for (int t = 15; t >= 0; --t) {
        const int i = i0 + t;
        const float e = __expf(grun - mid);
        const float r = __fdividef(1.f, e);
        const float dq = e * fmaf(c1, dq2[t], dq1[t]);
        const float dkin = r * c2 * dk2[t];
        const float dk = fmaf(r, dk1[t], dkin);
        p.dq[obase + i * ostride] = dq;
        p.dk[obase + i * ostride] = dk;
        const float q = ld_bf16(qs, ca.at(i)), k = ld_bf16(ks, ca.at(i));
        run += q * dq - k * dk;
        tail = fmaf(dkin, k, tail);
        stage[i * D + tid] = run;
        grun -= ld_bf16(gs, ca.at(i));
      }
    }
    if (p.dg) {
      const float cst = tail + __expf(gn) * hdh;
#pragma unroll 8
      for (int i = 0; i < C; ++i) p.dg[obase + i * ostride] = stage[i * D + tid] + cst;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 512);
}

// ===========================================================================
// host side
// ===========================================================================
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
  });
  return fn;
}

// [B*T, H, 128] bf16 activations: box = 64 channels x 1 head x 64 tokens
int act_map(CUtensorMap* m, const void* ptr, int BT, int H) {
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)BT};
  cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)H * D * 2};
  cuuint32_t box[3] = {64, 1, 64};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = encode_fn()(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, es,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? TOPS_OK : TOPS_E_CUDA;
}
// [rows, 128] bf16 chunk states: box = 64 columns x 128 rows
int state_map(CUtensorMap* m, const void* ptr, size_t rows) {
  cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)D * 2};
  cuuint32_t box[2] = {64, 128};
  cuuint32_t es[2] = {1, 1};
  CUresult r = encode_fn()(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, es,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? TOPS_OK : TOPS_E_CUDA;
}

bool device_is_sm100() {
  static int cached = -1;
  if (cached < 0) {
    int dev = 0, major = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    cached = (major == 10) ? 1 : 0;
  }
  return cached == 1;
}

constexpr size_t SCAN_SMEM = 2 * (2 * TILE64 + SLAB64) + TILE64 + 1024;
constexpr size_t FWD_O_SMEM = 4 * TILE64 + TILE128 + 1024;
constexpr size_t BWD_SMEM = 8 * TILE64 + 2 * TILE128 + 2 * SLAB64 + 1024;

template <class F>
int opt_in_smem(F f, size_t bytes) {
  return cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) == cudaSuccess ? TOPS_OK
                                                                                                         : TOPS_E_CUDA;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int run_scan(bool bwd, const tops_chunk_problem& pb, const void* x, const void* g, const void* y, const float* s0,
             void* states, float* s_final, cudaStream_t st) {
  ScanParams sp;
  const int BT = pb.B * pb.T;
  int rc;
  if ((rc = act_map(&sp.mx, x, BT, pb.H)) || (rc = act_map(&sp.mg, g, BT, pb.H)) || (rc = act_map(&sp.my, y, BT, pb.H)))
    return rc;
  sp.s0 = s0; sp.states = reinterpret_cast<__nv_bfloat16*>(states); sp.s_final = s_final;
  sp.T = pb.T; sp.H = pb.H; sp.NT = pb.T / C; sp.scale = pb.scale;
  dim3 grid(2, pb.B * pb.H);
  if (bwd) {
    if ((rc = opt_in_smem(k_scan<true>, SCAN_SMEM))) return rc;
    KernelScope ks("sm100_bwd_dh", st);
    k_scan<true><<<grid, NTHREADS, SCAN_SMEM, st>>>(sp);
    return post_launch();
  }
  if ((rc = opt_in_smem(k_scan<false>, SCAN_SMEM))) return rc;
  KernelScope ks("sm100_fwd_h", st);
  k_scan<false><<<grid, NTHREADS, SCAN_SMEM, st>>>(sp);
  return post_launch();
}

}  // namespace

bool supported(const tops_chunk_problem& pb) {
  if (pb.dtype != TOPS_BF16 || pb.gate_dtype != TOPS_BF16 || pb.gate_kind != TOPS_GATE_PER_CHANNEL) return false;
  if (pb.K != D || pb.V != D || pb.chunk != C || pb.T % C != 0 || pb.cu_seqlens) return false;
  if ((size_t)pb.B * pb.T >= (1u << 31)) return false;
  return device_is_sm100() && encode_fn() != nullptr;
}

static size_t state_bytes(const tops_chunk_problem& pb) {
  return align_up((size_t)pb.B * (pb.T / C) * pb.H * D * D * 2);
}

size_t fwd_workspace_bytes(const tops_chunk_fwd_params& p) { return (p.h_out ? 0 : state_bytes(p.pb)) + 256; }

int chunk_fwd(const tops_chunk_fwd_params& p, void* ws, size_t, cudaStream_t st) {
  const tops_chunk_problem& pb = p.pb;
  if (p.g_cumsum_out || p.A_out) return TOPS_E_UNSUPPORTED;
  if (!aligned16(p.q) || !aligned16(p.k) || !aligned16(p.v) || !aligned16(p.g) || !aligned16(p.o) ||
      !aligned16(p.h0) || !aligned16(p.ht) || !aligned16(ws))
    return TOPS_E_ALIGN;
  void* h = p.h_out ? p.h_out : ws;
  int rc = run_scan(false, pb, p.k, p.g, p.v, p.h0, h, p.ht, st);
  if (rc) return rc;
  FwdOParams fp;
  const int BT = pb.B * pb.T, NT = pb.T / C;
  if ((rc = act_map(&fp.mq, p.q, BT, pb.H)) || (rc = act_map(&fp.mk, p.k, BT, pb.H)) ||
      (rc = act_map(&fp.mg, p.g, BT, pb.H)) || (rc = act_map(&fp.mv, p.v, BT, pb.H)) ||
      (rc = state_map(&fp.mh, h, (size_t)pb.B * NT * pb.H * D)))
    return rc;
  fp.o = reinterpret_cast<__nv_bfloat16*>(p.o); fp.T = pb.T; fp.H = pb.H; fp.NT = NT; fp.scale = pb.scale;
  if ((rc = opt_in_smem(k_fwd_o, FWD_O_SMEM))) return rc;
  KernelScope ks("sm100_fwd_o", st);
  k_fwd_o<<<dim3(NT, pb.B * pb.H), NTHREADS, FWD_O_SMEM, st>>>(fp);
  return post_launch();
}

size_t bwd_workspace_bytes(const tops_chunk_bwd_params& p) { return 2 * state_bytes(p.pb) + 256; }

int chunk_bwd(const tops_chunk_bwd_params& p, void* ws, size_t, cudaStream_t st) {
  const tops_chunk_problem& pb = p.pb;
  if (p.grad_dtype != TOPS_F32) return TOPS_E_UNSUPPORTED;
  if (!aligned16(p.q) || !aligned16(p.k) || !aligned16(p.v) || !aligned16(p.g) || !aligned16(p.do_) ||
      !aligned16(p.h0) || !aligned16(p.dht) || !aligned16(p.dh0) || !aligned16(ws))
    return TOPS_E_ALIGN;
  char* h = reinterpret_cast<char*>(ws);
  char* dh = h + state_bytes(pb);
  int rc = run_scan(false, pb, p.k, p.g, p.v, p.h0, h, nullptr, st);
  if (rc) return rc;
  if ((rc = run_scan(true, pb, p.q, p.g, p.do_, p.dht, dh, p.dh0, st))) return rc;
  BwdParams bp;
  const int BT = pb.B * pb.T, NT = pb.T / C;
  const size_t rows = (size_t)pb.B * NT * pb.H * D;
  if ((rc = act_map(&bp.mq, p.q, BT, pb.H)) || (rc = act_map(&bp.mk, p.k, BT, pb.H)) ||
      (rc = act_map(&bp.mg, p.g, BT, pb.H)) || (rc = act_map(&bp.mv, p.v, BT, pb.H)) ||
      (rc = act_map(&bp.mdo, p.do_, BT, pb.H)) || (rc = state_map(&bp.mh, h, rows)) ||
      (rc = state_map(&bp.mdh, dh, rows)))
    return rc;
  bp.dq = reinterpret_cast<float*>(p.dq); bp.dk = reinterpret_cast<float*>(p.dk); bp.dg = p.dg;
  bp.dv = reinterpret_cast<__nv_bfloat16*>(p.dv); bp.T = pb.T; bp.H = pb.H; bp.NT = NT; bp.scale = pb.scale;
  if ((rc = opt_in_smem(k_bwd_main, BWD_SMEM))) return rc;
  KernelScope ks("sm100_bwd_main", st);
  k_bwd_main<<<dim3(NT, pb.B * pb.H), NTHREADS, BWD_SMEM, st>>>(bp);
  return post_launch();
}

int device_error(int* out) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_error, sizeof(int)) != cudaSuccess) return TOPS_E_CUDA;
  *out = v;
  return TOPS_OK;
}

}  // namespace sm100
}  // namespace tops
