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
  __nv_bfloat16* rsave;         // R = beta (v - k^ h') [B,T,H,V] or null
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
__global__ void __launch_bounds__(KDA_THREADS, 1) k_kda_fwd(const __grid_constant__ KdaFwdParams p) {
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
          __nv_bfloat16* rdst = p.rsave ? p.rsave + ((size_t)(row0 + ri) * p.H + h) * D + seg * 32 : nullptr;
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
            if (rdst) *reinterpret_cast<uint4*>(rdst + t) = make_uint4(w[0], w[1], w[2], w[3]);
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

// ===========================================================================
// Backward, part A: the reverse scan of the state gradient
// ===========================================================================
// dh is the gradient with respect to the state a chunk hands on (h_next); per chunk, right to left,
// with dh^ = exp(G_n - mid) dh (per key channel) and k^b = beta k^ (rows scaled by beta):
//     dv'  = Aqk^T do + k~ dh^                         gradient of the delta-corrected values
//     dR   = T^T dv'                                    gradient of the right-hand side of the solve
//     dv   = beta dR                                    (output)        dbeta1 = sum_v dR v
//     D    = q~^T do - k^b^T dR                         gradient with respect to h' = h exp(mid)
//     dh  <- dh exp(G_n) + exp(mid) D
// dh^ (bf16, [B,NT,H,K,V]), dv' and -dR (bf16, [B,T,H,V]) are kept for the chunk-parallel kernels that
// finish dq, dk, dg and dbeta.  One block per (batch, head), dh in registers like the forward state.
struct KdaScanParams {
  CUtensorMap mq, mk, mg, mdo, mt;   // mt: T as [B*T, H, 64]
  CUtensorMap mst;                   // dh^ states as [B*NT*H*128, 128] (TMA stores)
  const __nv_bfloat16* beta;         // [B,T,H]
  const __nv_bfloat16* v;            // [B,T,H,V]
  const float* dht;                  // [B,H,K,V] or null (zero)
  float* dh0;                        // [B,H,K,V] or null
  __nv_bfloat16* dv;                 // [B,T,H,V] output
  __nv_bfloat16* dvn;                // dv'  [B,T,H,V] scratch
  __nv_bfloat16* ndr;                // -dR  [B,T,H,V] scratch
  float* dbeta1;                     // [B,T,H] scratch: sum_v dR v
  int T, H, NT;
  float scale;
};
struct KdaScanShared {
  uint64_t fullqkt[2], fullg, fulldo, ebar, abar, vbar, rbar, sbar;
  uint32_t tmem_slot;
  int abort_flag;
  float a[D], g0[D];
  float beta[2][C];
  float db[C];
};
constexpr uint32_t KDA_SCAN_STAGE = 2 * TILE64 + SLAB64;   // q, k, T
constexpr size_t KDA_SCAN_SMEM = 2 * KDA_SCAN_STAGE + 5 * TILE64 + TILE128 + SLAB64 + 2 * SLAB64 + sizeof(KdaScanShared);

__global__ void __launch_bounds__(KDA_THREADS, 1) k_kda_bwd_scan(const __grid_constant__ KdaScanParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* in = smem;                        // 2 stages x (q, k, T)
  uint8_t* gs = in + 2 * KDA_SCAN_STAGE;     // g
  uint8_t* dos = gs + TILE64;                // do
  uint8_t* khs = dos + TILE64;               // beta k^
  uint8_t* dvs = khs + TILE64;               // dv'
  uint8_t* nrs = dvs + TILE64;               // -dR
  uint8_t* dhst = nrs + TILE64;              // dh^ (128 x 128)
  uint8_t* at = dhst + TILE128;              // Aqk bf16 (64 x 64)
  uint8_t* mt = at + SLAB64;                 // TRI_MID pattern, rows repeated to 128
  KdaScanShared& sh = *reinterpret_cast<KdaScanShared*>(mt + 2 * SLAB64);
  volatile int* abort_flag = &sh.abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool driver = warp == 16;
  const int q4 = warp & 3, seg = (warp >> 2) & 3, col = q4 * 32 + lane;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const int NT = p.NT;
  constexpr uint32_t cE = 0, cD = 128, cA = 256;   // cE later holds dv' and then dR
  if ((smem_u32(smem) & 1023u) != 0) {
    if (tid == 0) fail(12);
    return;
  }
  auto chunk_of = [&](int pp) { return NT - 1 - pp; };
  auto issue_qkt = [&](int pp) {
    uint8_t* qs = in + (pp & 1) * KDA_SCAN_STAGE;
    uint8_t *ks = qs + TILE64, *ts = ks + TILE64;
    uint64_t* bar = &sh.fullqkt[pp & 1];
    const int row = b * p.T + chunk_of(pp) * C;
    mbar_expect_tx(bar, KDA_SCAN_STAGE);
    tma_load_3d(qs, &p.mq, bar, 0, h, row); tma_load_3d(qs + SLAB64, &p.mq, bar, 64, h, row);
    tma_load_3d(ks, &p.mk, bar, 0, h, row); tma_load_3d(ks + SLAB64, &p.mk, bar, 64, h, row);
    tma_load_3d(ts, &p.mt, bar, 0, h, row);
  };
  auto issue_g = [&](int pp) {
    const int row = b * p.T + chunk_of(pp) * C;
    mbar_expect_tx(&sh.fullg, TILE64);
    tma_load_3d(gs, &p.mg, &sh.fullg, 0, h, row); tma_load_3d(gs + SLAB64, &p.mg, &sh.fullg, 64, h, row);
  };
  auto issue_do = [&](int pp) {
    const int row = b * p.T + chunk_of(pp) * C;
    mbar_expect_tx(&sh.fulldo, TILE64);
    tma_load_3d(dos, &p.mdo, &sh.fulldo, 0, h, row); tma_load_3d(dos + SLAB64, &p.mdo, &sh.fulldo, 64, h, row);
  };
  auto load_beta = [&](int pp) {   // threads 0..63
    sh.beta[pp & 1][tid] = __bfloat162float(p.beta[((size_t)b * p.T + chunk_of(pp) * C + tid) * p.H + h]);
  };
  if (tid == 0) {
    mbar_init(&sh.fullqkt[0], 1); mbar_init(&sh.fullqkt[1], 1); mbar_init(&sh.fullg, 1); mbar_init(&sh.fulldo, 1);
    mbar_init(&sh.ebar, 1); mbar_init(&sh.abar, 1); mbar_init(&sh.vbar, 1); mbar_init(&sh.rbar, 1); mbar_init(&sh.sbar, 1);
    fence_barrier_init();
    tma_prefetch_desc(&p.mq); tma_prefetch_desc(&p.mk); tma_prefetch_desc(&p.mg); tma_prefetch_desc(&p.mdo);
    tma_prefetch_desc(&p.mt); tma_prefetch_desc(&p.mst);
    sh.abort_flag = 0;
    issue_qkt(0);
    issue_g(0);
    issue_do(0);
    if (NT > 1) issue_qkt(1);
  }
  __syncwarp();
  if (warp == 0) { tmem_alloc(&sh.tmem_slot, 512); tmem_relinquish(); }
  if (tid < C) { load_beta(0); sh.db[tid] = 0.f; }
  build_tri_tile(mt, 128, TRI_MID);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = sh.tmem_slot;
  const uint32_t lane_base = q4 * 32;

  if (driver) {
    auto issue_exponents = [&](int pp) {
      if (!mbar_wait(&sh.fullg, pp & 1)) { *abort_flag = 1; fail(3); }
      tc_fence_after();
      const uint32_t ga = smem_u32(gs), ma = smem_u32(mt);
#pragma unroll
      for (int j0 = 0; j0 < C; j0 += 16)   // E = G - mid: [time (repeated to 128 lanes)][channel]
        umma_bf16(tm + cE, desc_kmajor(ma, 128, 0, j0), desc_mnmajor(ga, 64, j0, 0), umma_idesc(128, 128, 0, 1), j0 > 0);
      umma_commit(&sh.ebar);
    };
    if (lane == 0) issue_exponents(0);
    __syncwarp();
    for (int pp = 0; pp < NT; ++pp) {
      const uint32_t ph = pp & 1;
      uint8_t* qs = in + (pp & 1) * KDA_SCAN_STAGE;
      uint8_t *ks = qs + TILE64, *ts = ks + TILE64;
      const uint32_t qa = smem_u32(qs), ka = smem_u32(ks), ta = smem_u32(ts), kha = smem_u32(khs), doa = smem_u32(dos),
                     dva = smem_u32(dvs), nra = smem_u32(nrs), dha = smem_u32(dhst), aa = smem_u32(at);
      if (lane == 0) tma_store_wait_read();       // the dh^ store of the previous chunk has read its tile
      if (__syncthreads_or(*abort_flag)) break;   // B1: q~, beta k^, k~ are in shared memory
      if (lane == 0) {
        tc_fence_after();
#pragma unroll
        for (int k0 = 0; k0 < D; k0 += 16)   // Aqk = q~ k~^T
          umma_bf16(tm + cA, desc_kmajor(qa, 64, 0, k0), desc_kmajor(ka, 64, 0, k0), umma_idesc(64, 64, 0, 0), k0 > 0);
        umma_commit(&sh.abar);
        if (pp + 1 < NT) issue_g(pp + 1);    // the exponent product of this chunk is complete
      }
      if (__syncthreads_or(*abort_flag)) break;   // B2: dh^ is staged, Aqk (bf16) is out
      if (lane == 0) {
        if (!mbar_wait(&sh.fulldo, ph)) { *abort_flag = 1; fail(6); }
        tc_fence_after();
#pragma unroll
        for (int k0 = 0; k0 < C; k0 += 16)   // dv'[j][v] = sum_i Aqk[i][j] do[i][v]
          umma_bf16(tm + cE, desc_mnmajor(aa, 64, k0, 0), desc_mnmajor(doa, 64, k0, 0), umma_idesc(64, 128, 1, 1), k0 > 0);
#pragma unroll
        for (int k0 = 0; k0 < D; k0 += 16)   // dv' += k~ dh^
          umma_bf16(tm + cE, desc_kmajor(ka, 64, 0, k0), desc_mnmajor(dha, 128, k0, 0), umma_idesc(64, 128, 0, 1), 1);
        umma_commit(&sh.vbar);
        const int hrow = ((b * NT + chunk_of(pp)) * p.H + h) * D;
        tma_store_2d(&p.mst, dhst, 0, hrow);
        tma_store_2d(&p.mst, dhst + TILE128 / 2, 64, hrow);
        tma_store_commit();
      }
      if (__syncthreads_or(*abort_flag)) break;   // B3: dv' (bf16) is in shared memory
      if (lane == 0) {
        tc_fence_after();
#pragma unroll
        for (int k0 = 0; k0 < C; k0 += 16)   // dR[j][v] = sum_i T[i][j] dv'[i][v]
          umma_bf16(tm + cE, desc_mnmajor(ta, 64, k0, 0), desc_mnmajor(dva, 64, k0, 0), umma_idesc(64, 128, 1, 1), k0 > 0);
        umma_commit(&sh.rbar);
      }
      if (__syncthreads_or(*abort_flag)) break;   // B4: -dR (bf16) is in shared memory
      if (lane == 0) {
        tc_fence_after();
#pragma unroll
        for (int k0 = 0; k0 < C; k0 += 16)   // D[k][v] = sum_i q~[i][k] do[i][v]
          umma_bf16(tm + cD, desc_mnmajor(qa, 64, k0, 0), desc_mnmajor(doa, 64, k0, 0), umma_idesc(128, 128, 1, 1), k0 > 0);
#pragma unroll
        for (int k0 = 0; k0 < C; k0 += 16)   // D += (beta k^)^T (-dR)
          umma_bf16(tm + cD, desc_mnmajor(kha, 64, k0, 0), desc_mnmajor(nra, 64, k0, 0), umma_idesc(128, 128, 1, 1), 1);
        umma_commit(&sh.sbar);
        if (pp + 1 < NT) issue_exponents(pp + 1);   // (dR has left tensor memory before B4)
        if (pp + 1 < NT) {
          if (!mbar_wait(&sh.sbar, ph)) { *abort_flag = 1; fail(2); }
          issue_do(pp + 1);                  // do, q~, k~, T of this chunk are dead
          if (pp + 2 < NT) issue_qkt(pp + 2);
        }
      }
      __syncwarp();
    }
    if (lane == 0) tma_store_wait_all();
  } else {
    float S[32];   // dh: row k = col, columns 32 seg .. + 31
    {
      const float* src = p.dht ? p.dht + ((size_t)bh * D + col) * D + seg * 32 : nullptr;
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 x = src ? *reinterpret_cast<const float4*>(src + j) : make_float4(0.f, 0.f, 0.f, 0.f);
        S[j] = x.x; S[j + 1] = x.y; S[j + 2] = x.z; S[j + 3] = x.w;
      }
    }
    const int ri = 16 * q4 + lane;
    for (int pp = 0; pp < NT; ++pp) {
      const uint32_t ph = pp & 1;
      uint8_t* qs = in + (pp & 1) * KDA_SCAN_STAGE;
      uint8_t* ks = qs + TILE64;
      const int row0 = b * p.T + chunk_of(pp) * C;
      // this thread's 32 values of v (rows of M = 64 accumulators sit in lanes 0..15), for dbeta1
      uint4 vreg[4];
      if (lane < 16) {
        const uint4* src = reinterpret_cast<const uint4*>(p.v + ((size_t)(row0 + ri) * p.H + h) * D + seg * 32);
#pragma unroll
        for (int t = 0; t < 4; ++t) vreg[t] = __ldg(src + t);
      }
      // ---- gate q and k
      if (!mbar_wait(&sh.fullqkt[pp & 1], (pp >> 1) & 1) || !mbar_wait(&sh.ebar, ph)) { *abort_flag = 1; fail(9); }
      tc_fence_after();
      {
        const int i = (q4 * 32 + lane) & 63;
        const int cg = (q4 >> 1) * 4 + seg;
        float em[16];
        tmem_ld16(tmem_addr(tm, lane_base, cE + cg * 16), em);
        const uint32_t rowoff = (uint32_t)(cg >> 2) * SLAB64 + (uint32_t)i * 128u;
        const float bi = sh.beta[ph][i];
        if (i == 63) {
#pragma unroll
          for (int t = 0; t < 16; ++t) sh.a[cg * 16 + t] = em[t];
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const uint32_t off = rowoff + (((uint32_t)((cg & 3) * 2 + u) ^ (uint32_t)i) & 7u) * 16u;
          float fb[8], fs[8], r[8];
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            const float f = fast_exp(em[8 * u + t]);
            fb[t] = f * bi;
            fs[t] = f * p.scale;
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
          *reinterpret_cast<uint4*>(khs + off) = scale8(kraw, fb);
          *reinterpret_cast<uint4*>(ks + off) = scale8(kraw, r);
        }
      }
      fence_async_smem();
      tc_fence_before();
      if (__syncthreads_or(*abort_flag)) break;   // B1
      // (beta of the next chunk: loaded here, stored to shared memory three barriers later)
      __nv_bfloat16 beta_in = __float2bfloat16(0.f);
      if (tid < C && pp + 1 < NT) beta_in = p.beta[((size_t)b * p.T + chunk_of(pp + 1) * C + tid) * p.H + h];
      const float av = sh.a[col], g0v = sh.g0[col];
      const float decay = fast_exp(2.f * av + g0v);   // exp(G_n)
      const float cmid = fast_exp(av + g0v);          // exp(mid)
      {
        const float c2 = fast_exp(av);                // exp(G_n - mid)
#pragma unroll
        for (int j = 0; j < 32; j += 8)
          *reinterpret_cast<uint4*>(dhst + tile_off(128, col, seg * 32 + j)) =
              make_uint4(pack_bf16(S[j] * c2, S[j + 1] * c2), pack_bf16(S[j + 2] * c2, S[j + 3] * c2),
                         pack_bf16(S[j + 4] * c2, S[j + 5] * c2), pack_bf16(S[j + 6] * c2, S[j + 7] * c2));
      }
      if (!mbar_wait(&sh.abar, ph)) { *abort_flag = 1; fail(4); }
      tc_fence_after();
      {
        float a[16];
        tmem_ld16(tmem_addr(tm, lane_base, cA + seg * 16), a);
        if (lane < 16) store_tril16(at, ri, seg * 16, a, 1.f);
      }
      fence_async_smem();
      tc_fence_before();
      if (__syncthreads_or(*abort_flag)) break;   // B2
      // ---- dv' -> bf16 operand and scratch
      if (!mbar_wait(&sh.vbar, ph)) { *abort_flag = 1; fail(7); }
      tc_fence_after();
      {
        float x[32];
        tmem_ld32(tmem_addr(tm, lane_base, cE + seg * 32), x);
        if (lane < 16) {
          __nv_bfloat16* dst = p.dvn + ((size_t)(row0 + ri) * p.H + h) * D + seg * 32;
#pragma unroll
          for (int t = 0; t < 32; t += 8) {
            const uint4 packed = make_uint4(pack_bf16(x[t], x[t + 1]), pack_bf16(x[t + 2], x[t + 3]),
                                            pack_bf16(x[t + 4], x[t + 5]), pack_bf16(x[t + 6], x[t + 7]));
            *reinterpret_cast<uint4*>(dvs + tile_off(64, ri, seg * 32 + t)) = packed;
            *reinterpret_cast<uint4*>(dst + t) = packed;
          }
        }
      }
      fence_async_smem();
      tc_fence_before();
      if (__syncthreads_or(*abort_flag)) break;   // B3
      // ---- dR: dv = beta dR (output), -dR (operand and scratch), dbeta1 = sum_v dR v
      if (!mbar_wait(&sh.rbar, ph)) { *abort_flag = 1; fail(8); }
      tc_fence_after();
      {
        float x[32];
        tmem_ld32(tmem_addr(tm, lane_base, cE + seg * 32), x);
        if (lane < 16) {
          const float bi = sh.beta[ph][ri];
          const size_t g0i = ((size_t)(row0 + ri) * p.H + h) * D + seg * 32;
          float dot = 0.f;
#pragma unroll
          for (int t = 0; t < 32; t += 8) {
            const __nv_bfloat162* pv = reinterpret_cast<const __nv_bfloat162*>(&vreg[t >> 3]);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const float2 vv = __bfloat1622float2(pv[u]);
              dot = fmaf(x[t + 2 * u], vv.x, dot);
              dot = fmaf(x[t + 2 * u + 1], vv.y, dot);
            }
            const uint4 neg = make_uint4(pack_bf16(-x[t], -x[t + 1]), pack_bf16(-x[t + 2], -x[t + 3]),
                                         pack_bf16(-x[t + 4], -x[t + 5]), pack_bf16(-x[t + 6], -x[t + 7]));
            *reinterpret_cast<uint4*>(nrs + tile_off(64, ri, seg * 32 + t)) = neg;
            *reinterpret_cast<uint4*>(p.ndr + g0i + t) = neg;
            __stcs(reinterpret_cast<uint4*>(p.dv + g0i + t),
                   make_uint4(pack_bf16(bi * x[t], bi * x[t + 1]), pack_bf16(bi * x[t + 2], bi * x[t + 3]),
                              pack_bf16(bi * x[t + 4], bi * x[t + 5]), pack_bf16(bi * x[t + 6], bi * x[t + 7])));
          }
          atomicAdd(&sh.db[ri], dot);
        }
      }
      if (tid < C && pp + 1 < NT) sh.beta[(pp + 1) & 1][tid] = __bfloat162float(beta_in);
      fence_async_smem();
      tc_fence_before();
      if (__syncthreads_or(*abort_flag)) break;   // B4
      if (tid < C) {
        p.dbeta1[((size_t)row0 + tid) * p.H + h] = sh.db[tid];
        sh.db[tid] = 0.f;
      }
      // ---- dh <- dh exp(G_n) + exp(mid) D
      if (!mbar_wait(&sh.sbar, ph)) { *abort_flag = 1; fail(2); }
      tc_fence_after();
      {
        float d[32];
        tmem_ld32(tmem_addr(tm, lane_base, cD + seg * 32), d);
#pragma unroll
        for (int t = 0; t < 32; ++t) S[t] = fmaf(S[t], decay, cmid * d[t]);
      }
      tc_fence_before();
    }
    if (!*abort_flag && p.dh0) {
      float* dst = p.dh0 + ((size_t)bh * D + col) * D + seg * 32;
#pragma unroll
      for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(S[j], S[j + 1], S[j + 2], S[j + 3]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 512);
  if (tid == 0 && sh.abort_flag) {
    poison(p.dv + ((size_t)b * p.T * p.H + h) * D);
    if (p.dh0) poison(p.dh0 + (size_t)bh * D * D);
  }
}

// ===========================================================================
// Backward, part B1: gradients of the two per-chunk matrices (one block per chunk and head)
// ===========================================================================
//     dS = tril(do v'^T)                 gradient of q~ k~^T (the scale rides on q~)
//     dL = -stril(T^T stril(dv' R^T) T^T)    gradient of L = stril(beta k^ k~^T) through T = (I + L)^-1
// Both leave as bf16 [B,T,H,64] (row i of a chunk at token i).
struct KdaIntraParams {
  CUtensorMap mdo, mvn, mdvn, mr, mt;
  __nv_bfloat16* dS;
  __nv_bfloat16* dL;
  int T, H, NT;
};

__global__ void __launch_bounds__(NTHREADS, 2) k_kda_bwd_intra(const __grid_constant__ KdaIntraParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* dos = smem;                 // do
  uint8_t* vns = dos + TILE64;         // v'
  uint8_t* dvs = vns + TILE64;         // dv'
  uint8_t* rs = dvs + TILE64;          // R
  uint8_t* ts = rs + TILE64;           // T (64 x 64)
  uint8_t* dts = ts + SLAB64;          // stril(dT) bf16
  uint8_t* wsm = dts + SLAB64;         // T^T dT bf16
  __shared__ uint64_t bar_load, bar_1, bar_2, bar_3;
  __shared__ uint32_t tmem_slot;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q4 = warp & 3, seg = warp >> 2;
  const int h = blockIdx.x, ci = blockIdx.y, b = blockIdx.z;
  const int row = b * p.T + ci * C;
  constexpr uint32_t cS = 0, cT = 64, cW = 128, cL = 192;
  if (tid == 0) {
    mbar_init(&bar_load, 1); mbar_init(&bar_1, 1); mbar_init(&bar_2, 1); mbar_init(&bar_3, 1);
    fence_barrier_init();
    mbar_expect_tx(&bar_load, 4 * TILE64 + SLAB64);
    tma_load_3d(dos, &p.mdo, &bar_load, 0, h, row); tma_load_3d(dos + SLAB64, &p.mdo, &bar_load, 64, h, row);
    tma_load_3d(vns, &p.mvn, &bar_load, 0, h, row); tma_load_3d(vns + SLAB64, &p.mvn, &bar_load, 64, h, row);
    tma_load_3d(dvs, &p.mdvn, &bar_load, 0, h, row); tma_load_3d(dvs + SLAB64, &p.mdvn, &bar_load, 64, h, row);
    tma_load_3d(rs, &p.mr, &bar_load, 0, h, row); tma_load_3d(rs + SLAB64, &p.mr, &bar_load, 64, h, row);
    tma_load_3d(ts, &p.mt, &bar_load, 0, h, row);
  }
  __syncwarp();
  if (warp == 0) { tmem_alloc(&tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_slot;
  const uint32_t lane_base = q4 * 32;
  const int ri = 16 * q4 + lane;   // rows of an M = 64 accumulator sit in lanes 0..15 of each quarter
  const size_t orow = ((size_t)(row + ri) * p.H + h) * C + seg * 16;
  bool ok = __syncthreads_and(mbar_wait(&bar_load, 0));
  if (!ok) fail(3);
  if (ok && tid == 0) {
    tc_fence_after();
    const uint32_t doa = smem_u32(dos), vna = smem_u32(vns), dva = smem_u32(dvs), ra = smem_u32(rs);
#pragma unroll
    for (int k0 = 0; k0 < D; k0 += 16)   // dS[i][j] = do v'^T
      umma_bf16(tm + cS, desc_kmajor(doa, 64, 0, k0), desc_kmajor(vna, 64, 0, k0), umma_idesc(64, 64, 0, 0), k0 > 0);
#pragma unroll
    for (int k0 = 0; k0 < D; k0 += 16)   // dT[i][j] = dv' R^T
      umma_bf16(tm + cT, desc_kmajor(dva, 64, 0, k0), desc_kmajor(ra, 64, 0, k0), umma_idesc(64, 64, 0, 0), k0 > 0);
    umma_commit(&bar_1);
  }
  __syncwarp();
  if (ok) { ok = __syncthreads_and(mbar_wait(&bar_1, 0)); if (!ok) fail(4); }
  if (ok) {
    tc_fence_after();
    float a[16];
    tmem_ld16(tmem_addr(tm, lane_base, cS + seg * 16), a);
    if (lane < 16) {
      uint32_t w[8];
#pragma unroll
      for (int t = 0; t < 16; t += 2) {
        const int j = seg * 16 + t;
        w[t >> 1] = pack_bf16(j <= ri ? a[t] : 0.f, j + 1 <= ri ? a[t + 1] : 0.f);
      }
      *reinterpret_cast<uint4*>(p.dS + orow) = make_uint4(w[0], w[1], w[2], w[3]);
      *reinterpret_cast<uint4*>(p.dS + orow + 8) = make_uint4(w[4], w[5], w[6], w[7]);
    }
    tmem_ld16(tmem_addr(tm, lane_base, cT + seg * 16), a);
    if (lane < 16) {
#pragma unroll
      for (int t = 0; t < 16; ++t) a[t] = (seg * 16 + t < ri) ? a[t] : 0.f;   // strictly below the diagonal
      store_tril16(dts, ri, seg * 16, a, 1.f);
    }
    fence_async_smem();
    tc_fence_before();
  }
  __syncthreads();
  if (ok && tid == 0) {
    tc_fence_after();
    const uint32_t ta = smem_u32(ts), dta = smem_u32(dts);
#pragma unroll
    for (int k0 = 0; k0 < C; k0 += 16)   // W[a][j] = sum_i T[i][a] dT[i][j]
      umma_bf16(tm + cW, desc_mnmajor(ta, 64, k0, 0), desc_mnmajor(dta, 64, k0, 0), umma_idesc(64, 64, 1, 1), k0 > 0);
    umma_commit(&bar_2);
  }
  __syncwarp();
  if (ok) { ok = __syncthreads_and(mbar_wait(&bar_2, 0)); if (!ok) fail(5); }
  if (ok) {
    tc_fence_after();
    float a[16];
    tmem_ld16(tmem_addr(tm, lane_base, cW + seg * 16), a);
    if (lane < 16) {
#pragma unroll
      for (int c8 = 0; c8 < 16; c8 += 8)
        *reinterpret_cast<uint4*>(wsm + slab_off(ri, seg * 16 + c8)) =
            make_uint4(pack_bf16(a[c8], a[c8 + 1]), pack_bf16(a[c8 + 2], a[c8 + 3]), pack_bf16(a[c8 + 4], a[c8 + 5]),
                       pack_bf16(a[c8 + 6], a[c8 + 7]));
    }
    fence_async_smem();
    tc_fence_before();
  }
  __syncthreads();
  if (ok && tid == 0) {
    tc_fence_after();
    const uint32_t ta = smem_u32(ts), wa = smem_u32(wsm);
#pragma unroll
    for (int k0 = 0; k0 < C; k0 += 16)   // X[a][c] = sum_j W[a][j] T[c][j]
      umma_bf16(tm + cL, desc_kmajor(wa, 64, 0, k0), desc_kmajor(ta, 64, 0, k0), umma_idesc(64, 64, 0, 0), k0 > 0);
    umma_commit(&bar_3);
  }
  __syncwarp();
  if (ok) { ok = __syncthreads_and(mbar_wait(&bar_3, 0)); if (!ok) fail(6); }
  if (ok) {
    tc_fence_after();
    float a[16];
    tmem_ld16(tmem_addr(tm, lane_base, cL + seg * 16), a);
    if (lane < 16) {
      uint32_t w[8];
#pragma unroll
      for (int t = 0; t < 16; t += 2) {
        const int j = seg * 16 + t;
        w[t >> 1] = pack_bf16(j < ri ? -a[t] : 0.f, j + 1 < ri ? -a[t + 1] : 0.f);
      }
      *reinterpret_cast<uint4*>(p.dL + orow) = make_uint4(w[0], w[1], w[2], w[3]);
      *reinterpret_cast<uint4*>(p.dL + orow + 8) = make_uint4(w[4], w[5], w[6], w[7]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 256);
  if (tid == 0 && !ok) poison(p.dL + ((size_t)row * p.H + h) * C);
}
constexpr size_t KDA_INTRA_SMEM = 4 * TILE64 + 3 * SLAB64 + 1024;

// ===========================================================================
// Backward, part B2: dq, dk, dg, dbeta of a chunk (one block per chunk and head)
// ===========================================================================
// Accumulators are channel-major (row = key channel, column = time step), so that a thread owns one channel
// over 16 time steps and the reverse cumulative sum of dg stays in registers:
//     dq~^T  = h' do^T + k~^T dS^T
//     dk~^T  = dh^ v'^T  (kept apart: its product with k~ is part of dg)  +  q~^T dS + (beta k^)^T dL
//     dk^b^T = h' (-dR)^T + k~^T dL^T                      gradient of beta k^ (= beta k exp(E))
//     dq = dq~ exp(E) scale      dk = dk~ exp(-E) + dk^b beta exp(E)      dbeta = dbeta1 + sum_k k exp(E) dk^b
//     dg = reverse cumsum over the chunk of (q~ dq~ + beta k^ dk^b - k~ dk~)
//          + sum_v h' dh^ + sum_i k~ dk~_inter          (the exp(G_n) dependence of the state update)
struct KdaBwdOutParams {
  CUtensorMap mq, mk, mg, mdo, mvn, mndr, mh, mdh, mdS, mdL;
  const __nv_bfloat16* beta;
  const float* dbeta1;
  void *dq, *dk, *dg;     // [B,T,H,K] fp32 or bf16
  void* dbeta;            // [B,T,H]   fp32 or bf16
  int T, H, NT, total;    // total = B * H * NT chunks
  float scale;
};
constexpr size_t KDA_OUT_SMEM = 7 * TILE64 + 2 * TILE128 + 2 * SLAB64 + 2 * SLAB64 + 1024;

// Persistent: block x walks chunks x, x + gridDim.x, ... (heads fastest, so the blocks in flight read whole
// token rows).  Everything of a chunk but q and k is dead once its products have completed, so the next
// chunk's g, do, v', -dR, h', dh^, dS, dL are fetched while the threads write the gradients of this one out;
// q and k (gated in place, read by the write-out) are brought into L2 meanwhile and fetched after it.
template <typename TG>
__global__ void __launch_bounds__(NTHREADS, 1) k_kda_bwd_out(const __grid_constant__ KdaBwdOutParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* qs = smem;                  // q -> q~ in place
  uint8_t* ks = qs + TILE64;           // k -> k~ in place
  uint8_t* gs = ks + TILE64;           // g
  uint8_t* khs = gs + TILE64;          // beta k^
  uint8_t* dos = khs + TILE64;         // do
  uint8_t* vns = dos + TILE64;         // v'
  uint8_t* nrs = vns + TILE64;         // -dR
  uint8_t* hs = nrs + TILE64;          // h' (128 x 128)
  uint8_t* dhs = hs + TILE128;         // dh^ (128 x 128)
  uint8_t* dSs = dhs + TILE128;        // dS (64 x 64)
  uint8_t* dLs = dSs + SLAB64;         // dL (64 x 64)
  uint8_t* mtm = dLs + SLAB64;         // TRI_MID pattern, rows repeated to 128
  // every barrier completes once per chunk (parity it & 1)
  __shared__ uint64_t bar_g, bar_qk, bar_rest, bar_e, bar_main;
  __shared__ uint32_t tmem_slot;
  __shared__ float sufsum[4][D], tails[4][D], hdh_s[D], beta_s[C], db_s[C];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q4 = warp & 3, seg = warp >> 2, col = q4 * 32 + lane;
  const int nit = (p.total - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  constexpr uint32_t cE = 0, cET = 128, cdq = 192, cdki = 256, cdkr = 320, cdkb = 384;
  auto chunk_rows = [&](int it, int& h, int& row, int& hrow) {
    const int cid = blockIdx.x + it * gridDim.x;
    const int ci = (cid / p.H) % p.NT, b = cid / (p.H * p.NT);
    h = cid % p.H;
    row = b * p.T + ci * C;
    hrow = ((b * p.NT + ci) * p.H + h) * D;
  };
  auto load_g = [&](int it) {
    int h, row, hrow;
    chunk_rows(it, h, row, hrow);
    mbar_expect_tx(&bar_g, TILE64);
    tma_load_3d(gs, &p.mg, &bar_g, 0, h, row); tma_load_3d(gs + SLAB64, &p.mg, &bar_g, 64, h, row);
  };
  auto load_qk = [&](int it) {
    int h, row, hrow;
    chunk_rows(it, h, row, hrow);
    mbar_expect_tx(&bar_qk, 2 * TILE64);
    tma_load_3d(qs, &p.mq, &bar_qk, 0, h, row); tma_load_3d(qs + SLAB64, &p.mq, &bar_qk, 64, h, row);
    tma_load_3d(ks, &p.mk, &bar_qk, 0, h, row); tma_load_3d(ks + SLAB64, &p.mk, &bar_qk, 64, h, row);
  };
  auto prefetch_qk = [&](int it) {
    int h, row, hrow;
    chunk_rows(it, h, row, hrow);
    tma_prefetch_l2_3d(&p.mq, 0, h, row); tma_prefetch_l2_3d(&p.mq, 64, h, row);
    tma_prefetch_l2_3d(&p.mk, 0, h, row); tma_prefetch_l2_3d(&p.mk, 64, h, row);
  };
  auto load_rest = [&](int it) {
    int h, row, hrow;
    chunk_rows(it, h, row, hrow);
    mbar_expect_tx(&bar_rest, 3 * TILE64 + 2 * TILE128 + 2 * SLAB64);
    tma_load_3d(dos, &p.mdo, &bar_rest, 0, h, row); tma_load_3d(dos + SLAB64, &p.mdo, &bar_rest, 64, h, row);
    tma_load_3d(vns, &p.mvn, &bar_rest, 0, h, row); tma_load_3d(vns + SLAB64, &p.mvn, &bar_rest, 64, h, row);
    tma_load_3d(nrs, &p.mndr, &bar_rest, 0, h, row); tma_load_3d(nrs + SLAB64, &p.mndr, &bar_rest, 64, h, row);
    tma_load_2d(hs, &p.mh, &bar_rest, 0, hrow); tma_load_2d(hs + TILE128 / 2, &p.mh, &bar_rest, 64, hrow);
    tma_load_2d(dhs, &p.mdh, &bar_rest, 0, hrow); tma_load_2d(dhs + TILE128 / 2, &p.mdh, &bar_rest, 64, hrow);
    tma_load_3d(dSs, &p.mdS, &bar_rest, 0, h, row);
    tma_load_3d(dLs, &p.mdL, &bar_rest, 0, h, row);
  };
  auto beta_of = [&](int it) {   // threads 0..63
    int h, row, hrow;
    chunk_rows(it, h, row, hrow);
    return p.beta[((size_t)row + tid) * p.H + h];
  };
  if (tid == 0) {
    mbar_init(&bar_g, 1); mbar_init(&bar_qk, 1); mbar_init(&bar_rest, 1); mbar_init(&bar_e, 1); mbar_init(&bar_main, 1);
    fence_barrier_init();
    if (nit > 0) { load_g(0); load_qk(0); load_rest(0); }
  }
  __syncwarp();
  if (warp == 0) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  __nv_bfloat16 beta_next = __float2bfloat16(0.f);   // threads 0..63: beta of the next chunk, as loaded
  if (tid < C && nit > 0) beta_next = beta_of(0);
  build_tri_tile(mtm, 128, TRI_MID);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_slot;
  const uint32_t lane_base = q4 * 32;
  TG* const dq_out = reinterpret_cast<TG*>(p.dq);
  TG* const dk_out = reinterpret_cast<TG*>(p.dk);
  TG* const dg_out = reinterpret_cast<TG*>(p.dg);
  const size_t ostride = (size_t)p.H * D;
  const ColAddr ca = col_prep(64, col);
  bool ok = true;
  // Every bounded wait sits at the start of a chunk's work, before any copy for the chunk after it is issued:
  // when one gives up, all copies in flight were issued before its spin began and have long landed.
  for (int it = 0; it < nit; ++it) {
    const uint32_t ph = it & 1;
    const bool more = it + 1 < nit;
    int h, row, hrow;
    chunk_rows(it, h, row, hrow);
    float db1 = 0.f;   // threads 0..63: the scan's part of dbeta (read here, used after the write-out)
    if (tid < C) {
      beta_s[tid] = __bfloat162float(beta_next);
      db_s[tid] = 0.f;
      db1 = p.dbeta1[((size_t)row + tid) * p.H + h];
    }
    ok = __syncthreads_and(mbar_wait(&bar_g, ph));
    if (!ok) { fail(3); break; }
    if (tid == 0) {
      tc_fence_after();
      const uint32_t ga = smem_u32(gs), mma = smem_u32(mtm);
#pragma unroll
      for (int j0 = 0; j0 < C; j0 += 16)   // G - mid, [time (repeated)][channel]
        umma_bf16(tm + cE, desc_kmajor(mma, 128, 0, j0), desc_mnmajor(ga, 64, j0, 0), umma_idesc(128, 128, 0, 1), j0 > 0);
#pragma unroll
      for (int j0 = 0; j0 < C; j0 += 16)   // G - mid, [channel][time]
        umma_bf16(tm + cET, desc_mnmajor(ga, 64, j0, 0), desc_kmajor(mma, 64, 0, j0), umma_idesc(128, 64, 1, 0), j0 > 0);
      umma_commit(&bar_e);
    }
    __syncwarp();
    ok = __syncthreads_and(mbar_wait(&bar_e, ph) && mbar_wait(&bar_qk, ph));
    if (!ok) { fail(9); break; }
    {   // gate: thread (q4, lane, seg) owns time row (32 q4 + lane) mod 64 and 16 channels
      tc_fence_after();
      const int i = (q4 * 32 + lane) & 63;
      const int cg = (q4 >> 1) * 4 + seg;
      float em[16];
      tmem_ld16(tmem_addr(tm, lane_base, cE + cg * 16), em);
      const uint32_t rowoff = (uint32_t)(cg >> 2) * SLAB64 + (uint32_t)i * 128u;
      const float bi = beta_s[i];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const uint32_t off = rowoff + (((uint32_t)((cg & 3) * 2 + u) ^ (uint32_t)i) & 7u) * 16u;
        float fb[8], fs[8], r[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const float f = fast_exp(em[8 * u + t]);
          fb[t] = f * bi;
          fs[t] = f * p.scale;
          r[t] = fast_exp(-em[8 * u + t]);
        }
        const uint4 kraw = *reinterpret_cast<const uint4*>(ks + off);
        *reinterpret_cast<uint4*>(qs + off) = scale8(*reinterpret_cast<const uint4*>(qs + off), fs);
        *reinterpret_cast<uint4*>(khs + off) = scale8(kraw, fb);
        *reinterpret_cast<uint4*>(ks + off) = scale8(kraw, r);
      }
      fence_async_smem();
      tc_fence_before();
    }
    ok = __syncthreads_and(mbar_wait(&bar_rest, ph));
    if (!ok) { fail(6); break; }
    if (tid == 0) {
      tc_fence_after();
      const uint32_t qa = smem_u32(qs), ka = smem_u32(ks), kha = smem_u32(khs), doa = smem_u32(dos), vna = smem_u32(vns),
                     nra = smem_u32(nrs), ha = smem_u32(hs), dha = smem_u32(dhs), dSa = smem_u32(dSs), dLa = smem_u32(dLs);
#pragma unroll
      for (int k0 = 0; k0 < D; k0 += 16)   // dq~^T[k][i] = h' do^T
        umma_bf16(tm + cdq, desc_kmajor(ha, 128, 0, k0), desc_kmajor(doa, 64, 0, k0), umma_idesc(128, 64, 0, 0), k0 > 0);
#pragma unroll
      for (int k0 = 0; k0 < C; k0 += 16)   // dq~^T[k][i] += sum_j k~[j][k] dS[i][j]
        umma_bf16(tm + cdq, desc_mnmajor(ka, 64, k0, 0), desc_kmajor(dSa, 64, 0, k0), umma_idesc(128, 64, 1, 0), 1);
#pragma unroll
      for (int k0 = 0; k0 < D; k0 += 16)   // dk~_inter^T[k][j] = dh^ v'^T
        umma_bf16(tm + cdki, desc_kmajor(dha, 128, 0, k0), desc_kmajor(vna, 64, 0, k0), umma_idesc(128, 64, 0, 0), k0 > 0);
#pragma unroll
      for (int k0 = 0; k0 < C; k0 += 16)   // dk~_rest^T[k][j] = sum_i q~[i][k] dS[i][j]
        umma_bf16(tm + cdkr, desc_mnmajor(qa, 64, k0, 0), desc_mnmajor(dSa, 64, k0, 0), umma_idesc(128, 64, 1, 1), k0 > 0);
#pragma unroll
      for (int k0 = 0; k0 < C; k0 += 16)   // dk~_rest^T[k][j] += sum_i (beta k^)[i][k] dL[i][j]
        umma_bf16(tm + cdkr, desc_mnmajor(kha, 64, k0, 0), desc_mnmajor(dLa, 64, k0, 0), umma_idesc(128, 64, 1, 1), 1);
#pragma unroll
      for (int k0 = 0; k0 < D; k0 += 16)   // dk^b^T[k][j] = h' (-dR)^T
        umma_bf16(tm + cdkb, desc_kmajor(ha, 128, 0, k0), desc_kmajor(nra, 64, 0, k0), umma_idesc(128, 64, 0, 0), k0 > 0);
#pragma unroll
      for (int k0 = 0; k0 < C; k0 += 16)   // dk^b^T[k][j] += sum_i k~[i][k] dL[j][i]
        umma_bf16(tm + cdkb, desc_mnmajor(ka, 64, k0, 0), desc_kmajor(dLa, 64, 0, k0), umma_idesc(128, 64, 1, 0), 1);
      umma_commit(&bar_main);
    }
    __syncwarp();
    {   // sum_v h'[k][v] dh^[k][v] while the products run: thread = (channel, quarter of the columns)
      const int kk = tid >> 2, part = tid & 3;
      float hd = 0.f;
#pragma unroll
      for (int c8 = 0; c8 < 32; c8 += 8) {
        const uint32_t off = tile_off(128, kk, part * 32 + c8);
        const uint4 a = *reinterpret_cast<const uint4*>(hs + off), d = *reinterpret_cast<const uint4*>(dhs + off);
        const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* pd = reinterpret_cast<const __nv_bfloat162*>(&d);
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float2 fa = __bfloat1622float2(pa[t]), fd = __bfloat1622float2(pd[t]);
          hd = fmaf(fa.x, fd.x, hd);
          hd = fmaf(fa.y, fd.y, hd);
        }
      }
      hd += __shfl_xor_sync(0xffffffffu, hd, 1);
      hd += __shfl_xor_sync(0xffffffffu, hd, 2);
      if (part == 0) hdh_s[kk] = hd;
    }
    ok = __syncthreads_and(mbar_wait(&bar_main, ph));
    if (!ok) { fail(8); break; }
    // the products are complete and no thread reads h', dh^ any more: all of this chunk but q~, k~, beta k^
    // is dead, the next chunk's tiles take their place while the gradients are written out
    if (tid == 0 && more) {
      load_g(it + 1);
      load_rest(it + 1);
      prefetch_qk(it + 1);
    }
    if (tid < C && more) beta_next = beta_of(it + 1);
    const size_t obase = ((size_t)(row + seg * SEG) * p.H + h) * D + col;
    const size_t obase4 = obase - (lane & 3) + (size_t)(lane & 3) * ostride;
    float dgl[SEG], dbl[SEG];
    float run = 0.f, tail = 0.f;
    tc_fence_after();
#pragma unroll
    for (int blk = 1; blk >= 0; --blk) {
      float et[8], dq[8], dki[8], dkr[8], dkb[8];
      const uint32_t c0 = seg * SEG + blk * 8;
      tmem_ld8(tmem_addr(tm, lane_base, cET + c0), et);
      tmem_ld8(tmem_addr(tm, lane_base, cdq + c0), dq);
      tmem_ld8(tmem_addr(tm, lane_base, cdki + c0), dki);
      tmem_ld8(tmem_addr(tm, lane_base, cdkr + c0), dkr);
      tmem_ld8(tmem_addr(tm, lane_base, cdkb + c0), dkb);
#pragma unroll
      for (int u = 7; u >= 0; --u) {
        const int t = blk * 8 + u, ti = seg * SEG + t;
        const uint32_t off = ca.at(ti);
        const float qv = ld_bf16(qs, off), kv = ld_bf16(ks, off), kbv = ld_bf16(khs, off);   // q~, k~, beta k^
        const float e = fast_exp(et[u]), r = fast_exp(-et[u]);
        const float dkt = dki[u] + dkr[u];                 // dk~
        run += qv * dq[u] + kbv * dkb[u] - kv * dkt;
        tail = fmaf(dki[u], kv, tail);
        dgl[t] = run;
        st_out(dq_out, obase + t * ostride, e * p.scale * dq[u]);
        st_out(dk_out, obase + t * ostride, r * dkt + e * beta_s[ti] * dkb[u]);
        dbl[t] = kv * e * e * dkb[u];   // dbeta2[t] = sum_k k exp(E) dk^b = sum_k k~ e^2 dk^b
      }
    }
    {   // sum over the channels: the lanes of a warp by a shuffle butterfly, the four warps of a segment by atomics
      const float mine = warp_sum16(dbl, lane);
      if (lane < SEG) atomicAdd(&db_s[seg * SEG + lane], mine);
    }
    sufsum[seg][col] = run;
    tails[seg][col] = tail;
    tc_fence_before();
    __syncthreads();   // q~, k~, beta k^ and tensor memory have been read
    if (tid == 0 && more) load_qk(it + 1);
    {
      const float later = (seg < 1 ? sufsum[1][col] : 0.f) + (seg < 2 ? sufsum[2][col] : 0.f) + (seg < 3 ? sufsum[3][col] : 0.f);
      const float cst = later + tails[0][col] + tails[1][col] + tails[2][col] + tails[3][col] + hdh_s[col];
#pragma unroll
      for (int t = 0; t < SEG; t += 4) {
        float w[4] = {dgl[t] + cst, dgl[t + 1] + cst, dgl[t + 2] + cst, dgl[t + 3] + cst};
        st_transposed4(dg_out, obase4 + t * ostride, w, lane);
      }
      if (tid < C) st_out(reinterpret_cast<TG*>(p.dbeta), ((size_t)row + tid) * p.H + h, db_s[tid] + db1);
    }
    __syncthreads();   // sufsum, tails, hdh_s, db_s, beta_s are free for the next chunk
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 512);
  if (tid == 0 && !ok) {
    int h, row, hrow;
    chunk_rows(0, h, row, hrow);
    poison(dq_out + ((size_t)row * p.H + h) * D);
  }
}

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
      !aligned16(p.ht) || !aligned16(p.saved_h) || !aligned16(p.saved_vnew) || !aligned16(p.saved_T) || !aligned16(p.saved_R) ||
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
  kp.rsave = reinterpret_cast<__nv_bfloat16*>(p.saved_R);
  kp.t_saved = reinterpret_cast<__nv_bfloat16*>(p.saved_T);
  kp.Aqk_out = p.Aqk_out; kp.Akk_out = p.Akk_out;
  kp.T = p.T; kp.H = p.H; kp.NT = NT; kp.scale = p.scale;
  if ((rc = opt_in_smem(k_kda_fwd, KDA_FWD_SMEM))) return rc;
  KernelScope ks("sm100_kda_fwd", st);
  k_kda_fwd<<<p.B * p.H, KDA_THREADS, KDA_FWD_SMEM, st>>>(kp);
  return post_launch();
}

static size_t kda_state_bytes(const tops_chunk_kda_bwd_params& p) {
  return align_up((size_t)p.B * (p.T / C) * p.H * D * D * 2);
}
static size_t kda_act_bytes(const tops_chunk_kda_bwd_params& p) { return align_up((size_t)p.B * p.T * p.H * D * 2); }
static size_t kda_mat_bytes(const tops_chunk_kda_bwd_params& p) { return align_up((size_t)p.B * p.T * p.H * C * 2); }
static size_t kda_beta_bytes(const tops_chunk_kda_bwd_params& p) { return align_up((size_t)p.B * p.T * p.H * 4); }

size_t kda_chunk_bwd_workspace_bytes(const tops_chunk_kda_bwd_params& p) {
  // [dh^] [dv'] [-dR] [dS] [dL] [dbeta1]
  return kda_state_bytes(p) + 2 * kda_act_bytes(p) + 2 * kda_mat_bytes(p) + kda_beta_bytes(p) + 256;
}

bool kda_bwd_supported(const tops_chunk_kda_bwd_params& p) {
  tops_chunk_kda_fwd_params f{};
  f.B = p.B; f.T = p.T; f.H = p.H; f.K = p.K; f.V = p.V; f.chunk = p.chunk; f.dtype = p.dtype; f.gate_dtype = p.gate_dtype;
  f.scale = p.scale;
  return kda_supported(f) && (p.grad_dtype == TOPS_F32 || p.grad_dtype == TOPS_BF16);
}

int kda_chunk_bwd(const tops_chunk_kda_bwd_params& p, void* ws, cudaStream_t st) {
  const void* ptrs[] = {p.q, p.k, p.v, p.g, p.do_, p.dht, p.saved_h, p.saved_vnew, p.saved_T, p.saved_R,
                        p.dq, p.dk, p.dv, p.dg, p.dh0, ws};
  for (const void* x : ptrs)
    if (!aligned16(x)) return TOPS_E_ALIGN;
  const int BT = p.B * p.T, NT = p.T / C;
  const size_t rows = (size_t)p.B * NT * p.H * D;
  char* w = reinterpret_cast<char*>(ws);
  __nv_bfloat16* dh = reinterpret_cast<__nv_bfloat16*>(w); w += kda_state_bytes(p);
  __nv_bfloat16* dvn = reinterpret_cast<__nv_bfloat16*>(w); w += kda_act_bytes(p);
  __nv_bfloat16* ndr = reinterpret_cast<__nv_bfloat16*>(w); w += kda_act_bytes(p);
  __nv_bfloat16* dS = reinterpret_cast<__nv_bfloat16*>(w); w += kda_mat_bytes(p);
  __nv_bfloat16* dL = reinterpret_cast<__nv_bfloat16*>(w); w += kda_mat_bytes(p);
  float* dbeta1 = reinterpret_cast<float*>(w);
  int rc;
  {
    KdaScanParams sp;
    if ((rc = act_map(&sp.mq, p.q, BT, p.H)) || (rc = act_map(&sp.mk, p.k, BT, p.H)) ||
        (rc = act_map(&sp.mg, p.g, BT, p.H)) || (rc = act_map(&sp.mdo, p.do_, BT, p.H)) ||
        (rc = mat_map(&sp.mt, p.saved_T, BT, p.H)) || (rc = state_map(&sp.mst, dh, rows)))
      return rc;
    sp.beta = reinterpret_cast<const __nv_bfloat16*>(p.beta);
    sp.v = reinterpret_cast<const __nv_bfloat16*>(p.v);
    sp.dht = p.dht; sp.dh0 = p.dh0; sp.dv = reinterpret_cast<__nv_bfloat16*>(p.dv);
    sp.dvn = dvn; sp.ndr = ndr; sp.dbeta1 = dbeta1;
    sp.T = p.T; sp.H = p.H; sp.NT = NT; sp.scale = p.scale;
    if ((rc = opt_in_smem(k_kda_bwd_scan, KDA_SCAN_SMEM))) return rc;
    KernelScope ks("sm100_kda_bwd_scan", st);
    k_kda_bwd_scan<<<p.B * p.H, KDA_THREADS, KDA_SCAN_SMEM, st>>>(sp);
    if ((rc = post_launch())) return rc;
  }
  const bool state_gradient_only = !p.dq && !p.dk && !p.dg && !p.dbeta;
  if (state_gradient_only) return TOPS_OK;
  {
    KdaIntraParams ip;
    if ((rc = act_map(&ip.mdo, p.do_, BT, p.H)) || (rc = act_map(&ip.mvn, p.saved_vnew, BT, p.H)) ||
        (rc = act_map(&ip.mdvn, dvn, BT, p.H)) || (rc = act_map(&ip.mr, p.saved_R, BT, p.H)) ||
        (rc = mat_map(&ip.mt, p.saved_T, BT, p.H)))
      return rc;
    ip.dS = dS; ip.dL = dL; ip.T = p.T; ip.H = p.H; ip.NT = NT;
    if ((rc = opt_in_smem(k_kda_bwd_intra, KDA_INTRA_SMEM))) return rc;
    KernelScope ks("sm100_kda_bwd_intra", st);
    k_kda_bwd_intra<<<dim3(p.H, NT, p.B), NTHREADS, KDA_INTRA_SMEM, st>>>(ip);
    if ((rc = post_launch())) return rc;
  }
  {
    KdaBwdOutParams op;
    if ((rc = act_map(&op.mq, p.q, BT, p.H)) || (rc = act_map(&op.mk, p.k, BT, p.H)) ||
        (rc = act_map(&op.mg, p.g, BT, p.H)) || (rc = act_map(&op.mdo, p.do_, BT, p.H)) ||
        (rc = act_map(&op.mvn, p.saved_vnew, BT, p.H)) || (rc = act_map(&op.mndr, ndr, BT, p.H)) ||
        (rc = state_map(&op.mh, p.saved_h, rows)) || (rc = state_map(&op.mdh, dh, rows)) ||
        (rc = mat_map(&op.mdS, dS, BT, p.H)) || (rc = mat_map(&op.mdL, dL, BT, p.H)))
      return rc;
    op.beta = reinterpret_cast<const __nv_bfloat16*>(p.beta);
    op.dbeta1 = dbeta1; op.dq = p.dq; op.dk = p.dk; op.dg = p.dg; op.dbeta = p.dbeta;
    op.T = p.T; op.H = p.H; op.NT = NT; op.scale = p.scale;
    op.total = p.B * p.H * NT;
    const int grid = op.total < sm_count() ? op.total : sm_count();
    KernelScope ks("sm100_kda_bwd_out", st);
    if (p.grad_dtype == TOPS_F32) {
      if ((rc = opt_in_smem(k_kda_bwd_out<float>, KDA_OUT_SMEM))) return rc;
      k_kda_bwd_out<float><<<grid, NTHREADS, KDA_OUT_SMEM, st>>>(op);
    } else {
      if ((rc = opt_in_smem(k_kda_bwd_out<__nv_bfloat16>, KDA_OUT_SMEM))) return rc;
      k_kda_bwd_out<__nv_bfloat16><<<grid, NTHREADS, KDA_OUT_SMEM, st>>>(op);
    }
    return post_launch();
  }
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
