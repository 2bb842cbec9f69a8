// Chunked KDA (gated delta rule, WY / UT-transform form) on the 5th-generation tensor cores.
//
// Shapes taken here: bf16 q/k/v/g/beta, K = V = 128, chunk 64, T a multiple of 64, dense batch.
// Everything else runs on the token-serial kernels of kda.cu.
//
// Per chunk of one head, with G the chunk-local cumulative gate (natural log), mid = (G_0 + G_n) / 2
// per channel, E = G - mid, and the chunk-start state kept as h' = h exp(mid):
//     q~ = q exp(E) scale      k^ = k exp(E)      k~ = k exp(-E)
//     Aqk = tril(q~ k~^T)                                  (the scale rides on q~)
//     L   = stril(diag(beta) k^ k~^T)        T = (I + L)^-1          (unit lower triangular, 64 x 64)
//     v'  = T (beta (v - k^ h'))                            (= u - w h of the reference, u = T beta v, w = T beta k exp(G))
//     o   = q~ h' + Aqk v'
//     h  <- h exp(G_n) + exp(G_n - mid) (k~^T v')
// The cumulative gates are a tensor-core product of the gate tile with a constant 0 / +-1/2 / 1 pattern
// (sm100_tiles.cuh), every contraction is a tcgen05.mma on bf16 tiles in shared memory with fp32
// accumulators in tensor memory, the running state is fp32 in registers, and the 64 x 64 triangular
// inverse is computed in fp32 on the CUDA cores: 16 x 16 diagonal blocks by forward substitution, the
// off-diagonal blocks by two levels of T_lo,hi = -T_lo,lo (L_lo,hi T_hi,hi) block products.
#include "kda_sm100.cuh"
#include "sm100_host.cuh"
#include "sm100_tiles.cuh"

namespace tops {
namespace sm100 {
namespace {

struct KdaFwdParams {
  CUtensorMap mq, mk, mg, mv;
  CUtensorMap mst;              // the states tensor as [B*NT*H*128, 128] (TMA stores); unused when states == nullptr
  const __nv_bfloat16* beta;    // [B,T,H]
  const float* s0;              // [B,H,K,V] or null (zero)
  float* s_final;               // [B,H,K,V] or null
  __nv_bfloat16* o;             // [B,T,H,V]
  __nv_bfloat16* states;        // h' [B,NT,H,K,V] or null
  __nv_bfloat16* vnew;          // v' [B,T,H,V] or null
  __nv_bfloat16* t_saved;       // T  [B,T,H,64] bf16 or null
  float* Aqk_out;               // [B,T,H,64] fp32 or null
  float* Akk_out;               // [B,T,H,64] fp32 or null
  int T, H, NT;
  float scale;
};

struct KdaFwdShared {
  uint64_t fullqkg[2], fullv, ebar, abar, pbar, vbar, sbar, obar;
  uint32_t tmem_slot;
  int abort_flag;
  float a[D], g0[D];        // G_n - mid and G_0 per channel of the current chunk
  float beta[2][C];
};

constexpr uint32_t KDA_STAGE = 3 * TILE64;   // q, k, g
constexpr size_t KDA_FWD_SMEM = 2 * KDA_STAGE + 3 * TILE64 + TILE128 + 2 * SLAB64 + 2 * SLAB64 + sizeof(KdaFwdShared);
constexpr int KDA_THREADS = NTHREADS + 32;

__device__ __forceinline__ void compute_sync() { asm volatile("bar.sync 1, %0;" ::"n"(NTHREADS) : "memory"); }

// T = (I + L)^-1 for a strictly lower triangular 64 x 64 L, fp32, row-major with row stride 64, by the
// 512 compute threads.  W: 1024 floats of scratch.
__device__ __forceinline__ void invert_unit_lower(const float* __restrict__ Lm, float* __restrict__ Tm,
                                                  float* __restrict__ W, int tid) {
  for (int idx = tid; idx < C * C; idx += NTHREADS) {
    const int i = idx >> 6, j = idx & 63;
    if ((j >> 4) > (i >> 4)) Tm[idx] = 0.f;
  }
  if (tid < 64) {   // 16 x 16 diagonal blocks: column c of block b by forward substitution
    const int b = tid >> 4, c = tid & 15;
    const float* Lb = Lm + (16 * b) * C + 16 * b;
    float x[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float s = i == c ? 1.f : 0.f;
#pragma unroll
      for (int j = 0; j < i; ++j) s = fmaf(-Lb[i * C + j], x[j], s);
      x[i] = s;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) Tm[(16 * b + i) * C + 16 * b + c] = x[i];
  }
  compute_sync();
  {   // 32 x 32 diagonal blocks: T_10 = -T_11 (L_10 T_00), T_32 = -T_33 (L_32 T_22)
    const int p = tid >> 8, i = (tid >> 4) & 15, j = tid & 15, o = 32 * p;
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) s = fmaf(Lm[(o + 16 + i) * C + o + k], Tm[(o + k) * C + o + j], s);
    W[tid] = s;
    compute_sync();
    s = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) s = fmaf(Tm[(o + 16 + i) * C + o + 16 + k], W[p * 256 + k * 16 + j], s);
    Tm[(o + 16 + i) * C + o + j] = -s;
  }
  compute_sync();
  // the 32 x 32 block below the diagonal: T_lo = -T_hh (L_lo T_00')
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int idx = tid + NTHREADS * u, i = idx >> 5, j = idx & 31;
    float s = 0.f;
#pragma unroll 8
    for (int k = 0; k < 32; ++k) s = fmaf(Lm[(32 + i) * C + k], Tm[k * C + j], s);
    W[idx] = s;
  }
  compute_sync();
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int idx = tid + NTHREADS * u, i = idx >> 5, j = idx & 31;
    float s = 0.f;
#pragma unroll 8
    for (int k = 0; k < 32; ++k) s = fmaf(Tm[(32 + i) * C + 32 + k], W[k * 32 + j], s);
    Tm[(32 + i) * C + j] = -s;
  }
  compute_sync();
}

// One block per (batch, head): 16 compute warps (state in registers: thread (q4, lane, seg) owns state row
// k = 32 q4 + lane, columns 32 seg .. + 31) and a driver warp whose first thread issues every product and
// copy.  Four block-wide barriers per chunk separate the dependent steps:
//   B1  q~, k^, k~ are in shared memory                 -> Aqk, L products
//   B2  h' is staged, L (fp32) and Aqk (bf16) are out   -> k^ h', q~ h' products (and the h' store)
//       meanwhile the compute warps invert I + L
//   B3  T (bf16) and R = beta (v - k^ h') are out        -> v' = T R
//   B4  v' is in shared memory                           -> k~^T v', o += Aqk v'; exponents of the next chunk
__global__ void __launch_bounds__(KDA_THREADS) k_kda_fwd(const __grid_constant__ KdaFwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* in = smem;                       // 2 stages x (q, k, g); the g tile later holds L in fp32
  uint8_t* vs = in + 2 * KDA_STAGE;         // v
  uint8_t* khs = vs + TILE64;               // k^
  uint8_t* rt = khs + TILE64;               // T in fp32 during the inversion, then R, then v'
  uint8_t* hst = rt + TILE64;               // h' (128 x 128)
  uint8_t* tt = hst + TILE128;              // T bf16 (64 x 64); scratch of the inversion before that
  uint8_t* at = tt + SLAB64;                // Aqk bf16 (64 x 64)
  uint8_t* mt = at + SLAB64;                // TRI_MID pattern, rows repeated to 128
  KdaFwdShared& sh = *reinterpret_cast<KdaFwdShared*>(mt + 2 * SLAB64);
  volatile int* abort_flag = &sh.abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool driver = warp == 16;
  const int q4 = warp & 3, seg = (warp >> 2) & 3, col = q4 * 32 + lane;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const int NT = p.NT;
  constexpr uint32_t cE = 0, cD = 128, cO = 256, cA = 384, cK = 448;   // cE later holds k^ h' and then v'
  if ((smem_u32(smem) & 1023u) != 0) {   // uniform over the block
    if (tid == 0) fail(12);
    return;
  }
  auto issue_qkg = [&](int pp) {
    uint8_t* qs = in + (pp & 1) * KDA_STAGE;
    uint8_t *ks = qs + TILE64, *gs = ks + TILE64;
    uint64_t* bar = &sh.fullqkg[pp & 1];
    const int row = b * p.T + pp * C;
    mbar_expect_tx(bar, KDA_STAGE);
    tma_load_3d(gs, &p.mg, bar, 0, h, row); tma_load_3d(gs + SLAB64, &p.mg, bar, 64, h, row);
    tma_load_3d(qs, &p.mq, bar, 0, h, row); tma_load_3d(qs + SLAB64, &p.mq, bar, 64, h, row);
    tma_load_3d(ks, &p.mk, bar, 0, h, row); tma_load_3d(ks + SLAB64, &p.mk, bar, 64, h, row);
  };
  auto issue_v = [&](int pp) {
    const int row = b * p.T + pp * C;
    mbar_expect_tx(&sh.fullv, TILE64);
    tma_load_3d(vs, &p.mv, &sh.fullv, 0, h, row); tma_load_3d(vs + SLAB64, &p.mv, &sh.fullv, 64, h, row);
  };
  auto load_beta = [&](int pp) {   // threads 0..63
    sh.beta[pp & 1][tid] = __bfloat162float(p.beta[((size_t)b * p.T + pp * C + tid) * p.H + h]);
  };
  if (tid == 0) {
    mbar_init(&sh.fullqkg[0], 1); mbar_init(&sh.fullqkg[1], 1); mbar_init(&sh.fullv, 1);
    mbar_init(&sh.ebar, 1); mbar_init(&sh.abar, 1); mbar_init(&sh.pbar, 1); mbar_init(&sh.vbar, 1);
    mbar_init(&sh.sbar, 1); mbar_init(&sh.obar, 1);
    fence_barrier_init();
    tma_prefetch_desc(&p.mq); tma_prefetch_desc(&p.mk); tma_prefetch_desc(&p.mg); tma_prefetch_desc(&p.mv);
    if (p.states) tma_prefetch_desc(&p.mst);
    sh.abort_flag = 0;
    issue_qkg(0);
    issue_v(0);
    if (NT > 1) issue_qkg(1);
  }
  __syncwarp();
  if (warp == 0) { tmem_alloc(&sh.tmem_slot, 512); tmem_relinquish(); }
  if (tid < C) load_beta(0);
  build_tri_tile(mt, 128, TRI_MID);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = sh.tmem_slot;
  const uint32_t lane_base = q4 * 32;

  if (driver) {
    // ------------------------------------------------------------------ products and copies
    auto issue_exponents = [&](int pp) {
      if (!mbar_wait(&sh.fullqkg[pp & 1], (pp >> 1) & 1)) { *abort_flag = 1; fail(3); }
      tc_fence_after();
      const uint32_t ga = smem_u32(in + (pp & 1) * KDA_STAGE + 2 * TILE64), ma = smem_u32(mt);
#pragma unroll
      for (int j0 = 0; j0 < C; j0 += 16)   // E = G - mid: [time (repeated to 128 lanes)][channel]
        umma_bf16(tm + cE, desc_kmajor(ma, 128, 0, j0), desc_mnmajor(ga, 64, j0, 0), umma_idesc(128, 128, 0, 1), j0 > 0);
      umma_commit(&sh.ebar);
    };
    if (lane == 0) issue_exponents(0);
    __syncwarp();
    for (int pp = 0; pp < NT; ++pp) {
      const uint32_t ph = pp & 1;
      uint8_t* qs = in + (pp & 1) * KDA_STAGE;
      uint8_t* ks = qs + TILE64;
      const uint32_t qa = smem_u32(qs), ka = smem_u32(ks), kha = smem_u32(khs), ha = smem_u32(hst), ra = smem_u32(rt),
                     ta = smem_u32(tt), aa = smem_u32(at);
      // the state store of the previous chunk has read its staging tile, which the compute warps refill
      // after the next barrier
      if (lane == 0) tma_store_wait_read();
      if (__syncthreads_or(*abort_flag)) break;   // B1
      if (lane == 0) {
        tc_fence_after();
#pragma unroll
        for (int k0 = 0; k0 < D; k0 += 16)   // Aqk = q~ k~^T
          umma_bf16(tm + cA, desc_kmajor(qa, 64, 0, k0), desc_kmajor(ka, 64, 0, k0), umma_idesc(64, 64, 0, 0), k0 > 0);
#pragma unroll
        for (int k0 = 0; k0 < D; k0 += 16)   // k^ k~^T
          umma_bf16(tm + cK, desc_kmajor(kha, 64, 0, k0), desc_kmajor(ka, 64, 0, k0), umma_idesc(64, 64, 0, 0), k0 > 0);
        umma_commit(&sh.abar);
      }
      if (__syncthreads_or(*abort_flag)) break;   // B2
      if (lane == 0) {
        tc_fence_after();
#pragma unroll
        for (int k0 = 0; k0 < D; k0 += 16)   // P = k^ h'
          umma_bf16(tm + cE, desc_kmajor(kha, 64, 0, k0), desc_mnmajor(ha, 128, k0, 0), umma_idesc(64, 128, 0, 1), k0 > 0);
        umma_commit(&sh.pbar);
#pragma unroll
        for (int k0 = 0; k0 < D; k0 += 16)   // o = q~ h'
          umma_bf16(tm + cO, desc_kmajor(qa, 64, 0, k0), desc_mnmajor(ha, 128, k0, 0), umma_idesc(64, 128, 0, 1), k0 > 0);
        if (p.states) {
          const int hrow = ((b * NT + pp) * p.H + h) * D;
          tma_store_2d(&p.mst, hst, 0, hrow);
          tma_store_2d(&p.mst, hst + TILE128 / 2, 64, hrow);
          tma_store_commit();
        }
      }
      if (__syncthreads_or(*abort_flag)) break;   // B3
      if (lane == 0) {
        tc_fence_after();
#pragma unroll
        for (int k0 = 0; k0 < C; k0 += 16)   // v' = T R
          umma_bf16(tm + cE, desc_kmajor(ta, 64, 0, k0), desc_mnmajor(ra, 64, k0, 0), umma_idesc(64, 128, 0, 1), k0 > 0);
        umma_commit(&sh.vbar);
        if (pp + 1 < NT) issue_v(pp + 1);    // R has been formed: the v tile is free
      }
      if (__syncthreads_or(*abort_flag)) break;   // B4
      if (lane == 0) {
        tc_fence_after();
#pragma unroll
        for (int k0 = 0; k0 < C; k0 += 16)   // D[k][v] = sum_j k~[j][k] v'[j][v]
          umma_bf16(tm + cD, desc_mnmajor(ka, 64, k0, 0), desc_mnmajor(ra, 64, k0, 0), umma_idesc(128, 128, 1, 1), k0 > 0);
        umma_commit(&sh.sbar);
#pragma unroll
        for (int k0 = 0; k0 < C; k0 += 16)   // o += Aqk v'
          umma_bf16(tm + cO, desc_kmajor(aa, 64, 0, k0), desc_mnmajor(ra, 64, k0, 0), umma_idesc(64, 128, 0, 1), 1);
        umma_commit(&sh.obar);
        if (pp + 1 < NT) issue_exponents(pp + 1);   // (v' has left tensor memory before B4)
        if (pp + 2 < NT) {                          // every tile of this stage is dead once these products are complete
          if (!mbar_wait(&sh.obar, ph)) { *abort_flag = 1; fail(5); }
          issue_qkg(pp + 2);
        }
      }
      __syncwarp();
    }
    if (lane == 0) tma_store_wait_all();
  } else {
    // ------------------------------------------------------------------ state in registers
    float S[32];
    {
      const float* src = p.s0 ? p.s0 + ((size_t)bh * D + col) * D + seg * 32 : nullptr;
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 x = src ? *reinterpret_cast<const float4*>(src + j) : make_float4(0.f, 0.f, 0.f, 0.f);
        S[j] = x.x; S[j + 1] = x.y; S[j + 2] = x.z; S[j + 3] = x.w;
      }
    }
    float* Lm = nullptr;
    float* Tm = reinterpret_cast<float*>(rt);
    float* Ws = reinterpret_cast<float*>(tt);
    const int ri = 16 * q4 + lane;   // row of an M = 64 accumulator held by lanes 0..15 of each quarter
    for (int pp = 0; pp < NT; ++pp) {
      const uint32_t ph = pp & 1;
      uint8_t* qs = in + (pp & 1) * KDA_STAGE;
      uint8_t *ks = qs + TILE64, *gs = ks + TILE64;
      Lm = reinterpret_cast<float*>(gs);
      const int row0 = b * p.T + pp * C;
      // ---- gate q and k: thread (q4, lane, seg) owns time row (32 q4 + lane) mod 64 and 16 channels
      if (!mbar_wait(&sh.fullqkg[pp & 1], (pp >> 1) & 1) || !mbar_wait(&sh.ebar, ph)) { *abort_flag = 1; fail(9); }
      tc_fence_after();
      {
        const int i = (q4 * 32 + lane) & 63;
        const int cg = (q4 >> 1) * 4 + seg;
        float em[16];
        tmem_ld16(tmem_addr(tm, lane_base, cE + cg * 16), em);
        const uint32_t rowoff = (uint32_t)(cg >> 2) * SLAB64 + (uint32_t)i * 128u;
        if (i == 63) {
#pragma unroll
          for (int t = 0; t < 16; ++t) sh.a[cg * 16 + t] = em[t];
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const uint32_t off = rowoff + (((uint32_t)((cg & 3) * 2 + u) ^ (uint32_t)i) & 7u) * 16u;
          float f[8], fs[8], r[8];
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            f[t] = fast_exp(em[8 * u + t]);
            fs[t] = f[t] * p.scale;
            r[t] = fast_exp(-em[8 * u + t]);
          }
          const uint4 kraw = *reinterpret_cast<const uint4*>(ks + off);
          if (i == 0) {   // G_0 = g_0
            const uint4 graw = *reinterpret_cast<const uint4*>(gs + off);
            const __nv_bfloat162* pg = reinterpret_cast<const __nv_bfloat162*>(&graw);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const float2 x = __bfloat1622float2(pg[t]);
              sh.g0[cg * 16 + 8 * u + 2 * t] = x.x;
              sh.g0[cg * 16 + 8 * u + 2 * t + 1] = x.y;
            }
          }
          *reinterpret_cast<uint4*>(qs + off) = scale8(*reinterpret_cast<const uint4*>(qs + off), fs);
          *reinterpret_cast<uint4*>(khs + off) = scale8(kraw, f);
          *reinterpret_cast<uint4*>(ks + off) = scale8(kraw, r);
        }
      }
      fence_async_smem();
      tc_fence_before();
      if (__syncthreads_or(*abort_flag)) break;   // B1
      // ---- per-channel factors of this thread's state row; stage h' = h exp(mid)
      const float av = sh.a[col], g0v = sh.g0[col];
      const float decay = fast_exp(2.f * av + g0v);   // exp(G_n)
      const float c2 = fast_exp(av);                  // exp(G_n - mid)
      {
        const float hscale = fast_exp(av + g0v);      // exp(mid)
#pragma unroll
        for (int j = 0; j < 32; j += 8)
          *reinterpret_cast<uint4*>(hst + tile_off(128, col, seg * 32 + j)) =
              make_uint4(pack_bf16(S[j] * hscale, S[j + 1] * hscale), pack_bf16(S[j + 2] * hscale, S[j + 3] * hscale),
                         pack_bf16(S[j + 4] * hscale, S[j + 5] * hscale), pack_bf16(S[j + 6] * hscale, S[j + 7] * hscale));
      }
      // ---- L = stril(beta k^ k~^T) in fp32 for the inversion; Aqk -> bf16 operand
      if (!mbar_wait(&sh.abar, ph)) { *abort_flag = 1; fail(4); }
      tc_fence_after();
      {
        float a[16];
        tmem_ld16(tmem_addr(tm, lane_base, cK + seg * 16), a);
        if (lane < 16) {
          const float bi = sh.beta[ph][ri];
#pragma unroll
          for (int t = 0; t < 16; t += 4) {
            const int j = seg * 16 + t;
            *reinterpret_cast<float4*>(Lm + ri * C + j) =
                make_float4(j < ri ? bi * a[t] : 0.f, j + 1 < ri ? bi * a[t + 1] : 0.f, j + 2 < ri ? bi * a[t + 2] : 0.f,
                            j + 3 < ri ? bi * a[t + 3] : 0.f);
          }
        }
        tmem_ld16(tmem_addr(tm, lane_base, cA + seg * 16), a);
        if (lane < 16) {
          store_tril16(at, ri, seg * 16, a, 1.f);
          if (p.Aqk_out) {
            float* dst = p.Aqk_out + ((size_t)(row0 + ri) * p.H + h) * C + seg * 16;
#pragma unroll
            for (int t = 0; t < 16; t += 4) {
              const int j = seg * 16 + t;
              *reinterpret_cast<float4*>(dst + t) = make_float4(j <= ri ? a[t] : 0.f, j + 1 <= ri ? a[t + 1] : 0.f,
                                                                j + 2 <= ri ? a[t + 2] : 0.f, j + 3 <= ri ? a[t + 3] : 0.f);
            }
          }
        }
      }
      fence_async_smem();
      tc_fence_before();
      if (__syncthreads_or(*abort_flag)) break;   // B2
      // ---- T = (I + L)^-1 while the tensor core forms k^ h' and q~ h'
      invert_unit_lower(Lm, Tm, Ws, tid);
      {
        const int i = tid >> 3, j0 = (tid & 7) * 8;
        const float4 x = *reinterpret_cast<const float4*>(Tm + i * C + j0);
        const float4 y = *reinterpret_cast<const float4*>(Tm + i * C + j0 + 4);
        const uint4 packed = make_uint4(pack_bf16(x.x, x.y), pack_bf16(x.z, x.w), pack_bf16(y.x, y.y), pack_bf16(y.z, y.w));
        *reinterpret_cast<uint4*>(tt + slab_off(i, j0)) = packed;
        const size_t orow = ((size_t)(row0 + i) * p.H + h) * C + j0;
        if (p.t_saved) *reinterpret_cast<uint4*>(p.t_saved + orow) = packed;
        if (p.Akk_out) {
          *reinterpret_cast<float4*>(p.Akk_out + orow) = x;
          *reinterpret_cast<float4*>(p.Akk_out + orow + 4) = y;
        }
      }
      compute_sync();   // T (fp32) has been read: its place is free for R
      // ---- R = beta (v - k^ h')
      if (!mbar_wait(&sh.fullv, ph) || !mbar_wait(&sh.pbar, ph)) { *abort_flag = 1; fail(6); }
      tc_fence_after();
      {
        float pv[32];
        tmem_ld32(tmem_addr(tm, lane_base, cE + seg * 32), pv);
        if (lane < 16) {
          const float bi = sh.beta[ph][ri];
#pragma unroll
          for (int t = 0; t < 32; t += 8) {
            const uint32_t off = tile_off(64, ri, seg * 32 + t);
            const uint4 vraw = *reinterpret_cast<const uint4*>(vs + off);
            const __nv_bfloat162* pvv = reinterpret_cast<const __nv_bfloat162*>(&vraw);
            uint32_t w[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const float2 x = __bfloat1622float2(pvv[u]);
              w[u] = pack_bf16(bi * (x.x - pv[t + 2 * u]), bi * (x.y - pv[t + 2 * u + 1]));
            }
            *reinterpret_cast<uint4*>(rt + off) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      fence_async_smem();
      tc_fence_before();
      if (__syncthreads_or(*abort_flag)) break;   // B3
      // ---- v' -> bf16 operand (in the place of R) and, for a backward pass, to global memory
      if (!mbar_wait(&sh.vbar, ph)) { *abort_flag = 1; fail(7); }
      tc_fence_after();
      {
        float nv[32];
        tmem_ld32(tmem_addr(tm, lane_base, cE + seg * 32), nv);
        if (lane < 16) {
          __nv_bfloat16* dst = p.vnew ? p.vnew + ((size_t)(row0 + ri) * p.H + h) * D + seg * 32 : nullptr;
#pragma unroll
          for (int t = 0; t < 32; t += 8) {
            const uint4 packed = make_uint4(pack_bf16(nv[t], nv[t + 1]), pack_bf16(nv[t + 2], nv[t + 3]),
                                            pack_bf16(nv[t + 4], nv[t + 5]), pack_bf16(nv[t + 6], nv[t + 7]));
            *reinterpret_cast<uint4*>(rt + tile_off(64, ri, seg * 32 + t)) = packed;
            if (dst) *reinterpret_cast<uint4*>(dst + t) = packed;
          }
        }
      }
      if (tid < C && pp + 1 < NT) load_beta(pp + 1);
      fence_async_smem();
      tc_fence_before();
      if (__syncthreads_or(*abort_flag)) break;   // B4
      // ---- state update, outputs
      if (!mbar_wait(&sh.sbar, ph)) { *abort_flag = 1; fail(2); }
      tc_fence_after();
      {
        float d[32];
        tmem_ld32(tmem_addr(tm, lane_base, cD + seg * 32), d);
#pragma unroll
        for (int t = 0; t < 32; ++t) S[t] = fmaf(S[t], decay, c2 * d[t]);
      }
      if (!mbar_wait(&sh.obar, ph)) { *abort_flag = 1; fail(5); }
      tc_fence_after();
      {
        float a[32];
        tmem_ld32(tmem_addr(tm, lane_base, cO + seg * 32), a);
        if (lane < 16) {
          __nv_bfloat16* dst = p.o + ((size_t)(row0 + ri) * p.H + h) * D + seg * 32;
#pragma unroll
          for (int t = 0; t < 32; t += 8)
            __stcs(reinterpret_cast<uint4*>(dst + t), make_uint4(pack_bf16(a[t], a[t + 1]), pack_bf16(a[t + 2], a[t + 3]),
                                                                   pack_bf16(a[t + 4], a[t + 5]), pack_bf16(a[t + 6], a[t + 7])));
        }
      }
      tc_fence_before();
    }
    if (!*abort_flag && p.s_final) {
      float* dst = p.s_final + ((size_t)bh * D + col) * D + seg * 32;
#pragma unroll
      for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(S[j], S[j + 1], S[j + 2], S[j + 3]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 512);
  if (tid == 0 && sh.abort_flag) {
    poison(p.o + ((size_t)b * p.T * p.H + h) * D);
    if (p.s_final) poison(p.s_final + (size_t)bh * D * D);
  }
}

// [B*T, H, 64] -> not needed: beta, T and the fp32 matrices move with plain loads and stores.

}  // namespace

bool kda_supported(const tops_chunk_kda_fwd_params& p) {
  if (p.dtype != TOPS_BF16 || p.gate_dtype != TOPS_BF16) return false;
  if (p.K != D || p.V != D || p.chunk != C || p.T % C != 0) return false;
  if (!(p.scale > 0.f) || !(p.scale < 1e30f)) return false;
  if ((size_t)p.B * p.T >= (1u << 31)) return false;
  return device_is_sm100() && encode_fn() != nullptr;
}

int kda_chunk_fwd(const tops_chunk_kda_fwd_params& p, cudaStream_t st) {
  if (!aligned16(p.q) || !aligned16(p.k) || !aligned16(p.v) || !aligned16(p.g) || !aligned16(p.o) || !aligned16(p.h0) ||
      !aligned16(p.ht) || !aligned16(p.saved_h) || !aligned16(p.saved_vnew) || !aligned16(p.saved_T) ||
      !aligned16(p.Aqk_out) || !aligned16(p.Akk_out))
    return TOPS_E_ALIGN;
  KdaFwdParams kp;
  const int BT = p.B * p.T, NT = p.T / C;
  int rc;
  if ((rc = act_map(&kp.mq, p.q, BT, p.H)) || (rc = act_map(&kp.mk, p.k, BT, p.H)) ||
      (rc = act_map(&kp.mg, p.g, BT, p.H)) || (rc = act_map(&kp.mv, p.v, BT, p.H)))
    return rc;
  kp.states = reinterpret_cast<__nv_bfloat16*>(p.saved_h);
  if (p.saved_h && (rc = state_map(&kp.mst, p.saved_h, (size_t)p.B * NT * p.H * D))) return rc;
  kp.beta = reinterpret_cast<const __nv_bfloat16*>(p.beta);
  kp.s0 = p.h0; kp.s_final = p.ht; kp.o = reinterpret_cast<__nv_bfloat16*>(p.o);
  kp.vnew = reinterpret_cast<__nv_bfloat16*>(p.saved_vnew);
  kp.t_saved = reinterpret_cast<__nv_bfloat16*>(p.saved_T);
  kp.Aqk_out = p.Aqk_out; kp.Akk_out = p.Akk_out;
  kp.T = p.T; kp.H = p.H; kp.NT = NT; kp.scale = p.scale;
  if ((rc = opt_in_smem(k_kda_fwd, KDA_FWD_SMEM))) return rc;
  KernelScope ks("sm100_kda_fwd", st);
  k_kda_fwd<<<p.B * p.H, KDA_THREADS, KDA_FWD_SMEM, st>>>(kp);
  return post_launch();
}

int kda_device_error(int* out) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_error, sizeof(int)) != cudaSuccess) return TOPS_E_CUDA;
  *out = v;
  return TOPS_OK;
}

int kda_device_error_set(int code) {
  return cudaMemcpyToSymbol(g_error, &code, sizeof(int)) == cudaSuccess ? TOPS_OK : TOPS_E_CUDA;
}

}  // namespace sm100
}  // namespace tops
