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
// descriptors read (sm100_prims.cuh).  Chunk-start states and their gradients
// are kept as bf16 [B,NT,H,K,V] scratch in HBM, pre-multiplied by the
// per-channel factors their consumers need (h' = h exp(mid) scale,
// dh' = dh exp(G_n - mid)): they are only ever used as bf16 tensor-core
// operands; the running state itself is fp32 in registers of the scan kernels.
//
// Kernels
//   k_scan<false>  h'_c,  h <- h * exp(G_n) + (k exp(G_n - G))^T v       (forward scan)
//   k_scan<true>   dh'_c, dh <- dh * exp(G_n) + (q scale exp(G))^T do    (reverse scan)
//   k_fwd_o        A = tril(q~ k~^T) scale;  o = q~ h'_c + A v            (chunk-parallel outputs)
//   k_fwd_fused    the forward scan and the outputs in one pass, state kept on chip
//   k_bwd_main     dA, dv, dq, dk, dg of one chunk from q, k, v, g, do, h'_c, dh'_c
//   k_join_segments  chains the time segments a sequence is cut into when there are few sequences
// A forward is k_fwd_fused when there are enough (batch, head, segment) blocks to fill the GPU,
// else k_scan<false> + k_fwd_o; a backward is k_scan<true> + k_bwd_main (and k_scan<false> first
// when the caller did not keep the forward's states).
// G is the chunk-local cumulative gate and q~ = q exp(G - mid),
// k~ = k exp(mid - G), mid = (G_0 + G_n) / 2 per channel.  The cumulative
// gates themselves are tensor-core products of the gate tile with constant
// 0 / 1 / +-1/2 patterns, so the exponents arrive in tensor memory in the
// layout the gating or the write-out needs.
//
// Thread layout (scans, k_fwd_o, k_fwd_fused, write-out warps of k_bwd_main): 16 compute warps.
// Thread (col, seg) with col = (warp & 3) * 32 + lane and seg = warp >> 2:
// a warp may only touch the 32 tensor-memory lanes (warp & 3) * 32 .. + 31, so
// the thread owns accumulator row `col` and splits the accumulator columns
// with the three other warps of its lane quarter by `seg`.
#include <atomic>
#include <mutex>

#include "gla_sm100.cuh"
#include "sm100_host.cuh"
#include "sm100_tiles.cuh"

namespace tops {
namespace sm100 {


namespace {

// ===========================================================================
// State scans
// ===========================================================================
struct ScanParams {
  CUtensorMap mx, mg, my;  // x: k (fwd) / q (bwd); y: v / do
  CUtensorMap mst;         // the states tensor as [B*NT*H*128, 128] (TMA stores)
  const float* s0;         // state each block starts from: [B,H,nseg,K,V] or null (zero)
  __nv_bfloat16* states;   // h' / dh'  [B,T/64,H,K,V]; null: keep no chunk-start states (summary pass)
  float* s_final;          // state each block ends with: [B,H,nseg,K,V] or null
  float* gsum;             // summed log-gates of each block's chunks [B,H,nseg,K] or null
  int T, H, NT;            // T: tokens per sequence; NT: chunks per block (T / 64 / nseg)
  int nseg;                // time segments per sequence, one block each
  float scale;
  const __nv_bfloat16* gscalar;   // scalar gates [B,T,H] (SCALAR kernels; mg is unused then)
  int skip_xy;             // test hook: the x/y tile load of this chunk is never issued (-1: none), so that the
                           // bounded wait for it runs out and the kernel leaves through its error path
};

// One block per (batch, head): 16 compute warps and two issuing warps.  The whole K x V state lives in
// registers of the compute warps (thread (q4, lane, seg): row k = 32 q4 + lane, columns 32 seg .. + 31).
// Software pipeline over the chunks p (in scan order), one block-wide barrier per chunk:
//   compute warps, iteration p:  stage h'_p for its TMA store;  gate x(p+1) in place (its exponents
//       were put in tensor memory two iterations ago);  barrier;  wait for the state product of
//       chunk p;  state <- state * exp(G_n(p)) + D(p).
//   product thread, iteration p:  barrier;  state product of chunk p+1 -> accumulator (p+1)&1;  exponent
//       product of chunk p+3 -> exponent slot (p+1)&1.
//   copy thread, iteration p:  barrier;  TMA store of h'_p;  TMA loads of g of chunk p+4 and, once the state
//       product of chunk p has completed, of x, y of chunk p+3.
// No compute warp ever blocks on the issue of a product or a copy.  x/y and g tiles: 3 stages each;
// state staging: 2 tiles.
constexpr int SCAN_THREADS = NTHREADS + 64;    // 16 compute warps, a warp that issues the products, a warp that issues the copies
constexpr int FUSED_THREADS = NTHREADS + 32;   // 16 compute warps and one driver warp (splitting it made this kernel slower)
struct ScanShared {
  uint64_t fullg[3], fullxy[5], ebar[2], sbar[2];
  uint32_t tmem_slot;
  int abort_flag;
  float gn[2][D], e0[2][D];   // row 63 (G_n) and row 0 of the exponent tile, per channel
};

// SCALAR: one gate per head and time step (simple_gla).  No gate tile is fetched and no exponent product is
// issued: every compute warp keeps the 64 gates of the next chunk in registers and cumulates them with
// shuffles (warp_cumulate), so a thread gates its 16 channels of x with one factor.
// SUM (summary pass: no chunk-start states, zero start): only the state after the block's chunks is wanted,
//     S = sum_c [prod_{c' after c} exp(G_n(c'))] D(c),
// so the decay of all later chunks is folded into the gating of x (exponent + R, R the summed gates of the chunks
// already done) and every state product accumulates into ONE tensor-memory tile: nothing of a chunk depends on
// the chunk before it but the running sum R, the chain product -> register update -> next product is gone and a
// chunk costs its gating and its products.  The chunks are walked from the far end (forward scan: last chunk
// first; reverse scan: first chunk first), so that R is known when a chunk is gated.
template <bool BWD, bool SCALAR, bool SUM>
__global__ void __launch_bounds__(SCAN_THREADS, 1) k_scan(const __grid_constant__ ScanParams p) {
  // every shared object is carved from the dynamic allocation, whose start is 1024-byte aligned when the
  // kernel has no static shared memory (checked below: the swizzled tiles need that alignment)
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* xs = smem;                       // 3 x (64 x 128): x, gated in place
  uint8_t* ys = xs + 3 * TILE64;            // 3 x (64 x 128): y
  uint8_t* gs = ys + 3 * TILE64;            // 3 x (64 x 128): g
  uint8_t* mt = gs + 3 * TILE64;            // exponent pattern, rows repeated to 128
  uint8_t* hst = mt + 2 * SLAB64;           // 2 x (128 x 128) bf16: chunk-start states on their way to HBM
  ScanShared& sh = *reinterpret_cast<ScanShared*>(hst + 2 * TILE128);
  volatile int* abort_flag = &sh.abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool driver = warp >= 16;   // warp 16 issues the products, warp 17 the copies
  const int q4 = warp & 3, seg = (warp >> 2) & 3, col = q4 * 32 + lane;
  const int blk = blockIdx.x, sg = blk % p.nseg, bh = blk / p.nseg, b = bh / p.H, h = bh % p.H;
  const int NT = p.NT;
  const bool keep_states = p.states != nullptr;
  // tensor-memory columns: two exponent tiles, two state-product accumulators
  constexpr uint32_t cE = 0, cS = 256;
  if ((smem_u32(smem) & 1023u) != 0) {   // uniform over the block
    if (tid == 0) fail(12);
    return;
  }

  // chunk pp of this block (in the order the block walks them) within its sequence
  auto chunk_of = [&](int pp) { return sg * NT + ((BWD != SUM) ? NT - 1 - pp : pp); };
  // SUM: summed gates of the chunks already done, per channel (two copies, written for the next chunk while the
  // current one is read; in the place of e0, which a summary pass does not use) or, for scalar gates, in a
  // register of every thread
  float* const racc = &sh.e0[0][0];
  float racc_s = 0.f;
  // x / y stages: three; a summary pass, which is bound by how many bytes it keeps in flight, has two more in the
  // state staging tiles it does not use
  constexpr int NXY = SUM ? 5 : 3;
  auto x_stage = [&](int pp) { const int st = pp % NXY; return st < 3 ? xs + st * TILE64 : hst + (st - 3) * 2 * TILE64; };
  auto y_stage = [&](int pp) { const int st = pp % NXY; return st < 3 ? ys + st * TILE64 : hst + (st - 3) * 2 * TILE64 + TILE64; };
  auto xy_bar = [&](int pp) { return &sh.fullxy[pp % NXY]; };
  auto xy_parity = [&](int pp) { return (uint32_t)((pp / NXY) & 1); };
  auto chunk_row = [&](int pp) { return b * p.T + chunk_of(pp) * C; };
  auto issue_g = [&](int pp) {
    uint8_t* dst = gs + (pp % 3) * TILE64;
    mbar_expect_tx(&sh.fullg[pp % 3], TILE64);
    tma_load_3d(dst, &p.mg, &sh.fullg[pp % 3], 0, h, chunk_row(pp));
    tma_load_3d(dst + SLAB64, &p.mg, &sh.fullg[pp % 3], 64, h, chunk_row(pp));
  };
  auto issue_xy = [&](int pp) {
    uint8_t *xd = x_stage(pp), *yd = y_stage(pp);
    uint64_t* bar = xy_bar(pp);
    mbar_expect_tx(bar, 2 * TILE64);
    tma_load_3d(xd, &p.mx, bar, 0, h, chunk_row(pp));
    tma_load_3d(xd + SLAB64, &p.mx, bar, 64, h, chunk_row(pp));
    tma_load_3d(yd, &p.my, bar, 0, h, chunk_row(pp));
    tma_load_3d(yd + SLAB64, &p.my, bar, 64, h, chunk_row(pp));
  };
  if (tid == 0) {
    for (int i = 0; i < 3; ++i) mbar_init(&sh.fullg[i], 1);
    for (int i = 0; i < 5; ++i) mbar_init(&sh.fullxy[i], 1);
    mbar_init(&sh.ebar[0], 1); mbar_init(&sh.ebar[1], 1); mbar_init(&sh.sbar[0], 1); mbar_init(&sh.sbar[1], 1);
    fence_barrier_init();
    tma_prefetch_desc(&p.mx); tma_prefetch_desc(&p.my);
    if (!SCALAR) tma_prefetch_desc(&p.mg);
    if (p.states) tma_prefetch_desc(&p.mst);
    sh.abort_flag = 0;
    for (int c = 0; c < 3 && c < NT; ++c)
      if (!SCALAR) issue_g(c);
    for (int c = 0; c < NXY && c < NT; ++c) issue_xy(c);
  }
  __syncwarp();
  if (warp == 0) { tmem_alloc(&sh.tmem_slot, 512); tmem_relinquish(); }
  // SCALAR: the gates of the next chunks, fetched three chunks ahead into this warp's ring (see GateRing; the
  // rings take the place of the gate tiles, which scalar gates do not use)
  GateRing gring;
  const long long gidx0 = (long long)(chunk_row(0) + lane) * p.H + h;
  const long long gstep = (long long)(chunk_row(NT > 1 ? 1 : 0) - chunk_row(0)) * p.H;   // +-64 H elements per chunk
  auto gate_index = [&](int c) { return (size_t)(gidx0 + c * gstep); };
  auto load_gates = [&](int c) { gring.prefetch(p.gscalar, c < NT, c < NT ? gate_index(c) : 0, (size_t)32 * p.H, c, lane); };
  if (SCALAR) {
    if (!driver) {
      gring.init(gs + warp * GateRing::kBytesPerWarp);
      load_gates(0);
      load_gates(1);
      load_gates(2);
    }
  } else {
    build_tri_tile(mt, 128, BWD ? TRI_INCL : TRI_REVN);
    if (SUM && tid < 2 * D) racc[tid] = 0.f;
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = sh.tmem_slot;
  const uint32_t lane_base = q4 * 32;

  // exponents E = pattern . g of chunk pp: [time (repeated to 128 lanes)][channel]; row 63 is G_n
  auto issue_gate_mma = [&](int pp) {
    if (SCALAR) return;
    if (!mbar_wait(&sh.fullg[pp % 3], (pp / 3) & 1)) { *abort_flag = 1; fail(1); }
    tc_fence_after();
    const uint32_t ga = smem_u32(gs + (pp % 3) * TILE64);
    const uint32_t ma = smem_u32(mt);
#pragma unroll
    for (int j0 = 0; j0 < C; j0 += 16)
      umma_bf16(tm + cE + (pp & 1) * 128, desc_kmajor(ma, 128, 0, j0), desc_mnmajor(ga, 64, j0, 0),
                umma_idesc(128, 128, 0, 1), j0 > 0);
    umma_commit(&sh.ebar[pp & 1]);
  };
  auto issue_state_mma = [&](int pp) {
    const uint32_t xa = smem_u32(x_stage(pp)), ya = smem_u32(y_stage(pp));
    tc_fence_after();
#pragma unroll
    for (int k0 = 0; k0 < C; k0 += 16)   // (SUM: every chunk accumulates into the first tile)
      umma_bf16(tm + cS + (SUM ? 0 : (pp & 1) * 128), desc_mnmajor(xa, 64, k0, 0), desc_mnmajor(ya, 64, k0, 0),
                umma_idesc(128, 128, 1, 1), k0 > 0 || (SUM && pp > 0));
    umma_commit(&sh.sbar[pp & 1]);
  };
  // gate x of chunk pp in place and publish G_n (and G_n - G_0, or G_0) of its channels
  // (SCALAR: they are the same for every channel and stay in the registers gn_next, e0_next of every thread)
  float gn_next = 0.f, e0_next = 0.f;
  auto gate_chunk = [&](int pp) {
    if ((!SCALAR && !mbar_wait(&sh.ebar[pp & 1], (pp >> 1) & 1)) || !mbar_wait(xy_bar(pp), xy_parity(pp))) {
      *abort_flag = 1;
      fail(1);
    }
    tc_fence_after();
    const int i = (q4 * 32 + lane) & 63;          // time row of this thread
    const int cg = (q4 >> 1) * 4 + seg;           // its 16 channels
    if (SCALAR) {
      float g_lo, g_hi;
      gring.take(gate_index(pp), pp, lane, g_lo, g_hi);
      const WarpGates w = warp_cumulate(g_lo, g_hi, lane);
      const float Gi = (q4 & 1) ? w.hi : w.lo;
      gn_next = w.gn;
      e0_next = BWD ? w.g0 : w.gn - w.g0;
      const float f = BWD ? fast_exp(Gi + racc_s) * p.scale : fast_exp(w.gn - Gi + racc_s);
      if (SUM) racc_s += w.gn;
      uint8_t* xt = x_stage(pp);
      const uint32_t rowoff = (uint32_t)(cg >> 2) * SLAB64 + (uint32_t)i * 128u;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const uint32_t off = rowoff + (((uint32_t)((cg & 3) * 2 + u) ^ (uint32_t)i) & 7u) * 16u;
        *reinterpret_cast<uint4*>(xt + off) = scale8_by(*reinterpret_cast<const uint4*>(xt + off), f);
      }
      fence_async_smem();
      tc_fence_before();
      return;
    }
    float e[16];
    tmem_ld16(tmem_addr(tm, lane_base, cE + (pp & 1) * 128 + cg * 16), e);
    if (i == 63) {
#pragma unroll
      for (int t = 0; t < 16; ++t) sh.gn[pp & 1][cg * 16 + t] = e[t];
      if (SUM) {
#pragma unroll
        for (int t = 0; t < 16; ++t) racc[((pp + 1) & 1) * D + cg * 16 + t] = racc[(pp & 1) * D + cg * 16 + t] + e[t];
      }
      if (!BWD) {
#pragma unroll
        for (int t = 0; t < 16; ++t) e[t] = 0.f;   // row 63 of TRI_REVN carries G_n, its own exponent is 0
      }
    }
    if (i == 0 && !SUM) {   // forward: G_n - G_0; reverse: G_0 (for the scale of the stored states)
#pragma unroll
      for (int t = 0; t < 16; ++t) sh.e0[pp & 1][cg * 16 + t] = e[t];
    }
    if (SUM) {
#pragma unroll
      for (int t = 0; t < 16; ++t) e[t] += racc[(pp & 1) * D + cg * 16 + t];
    }
#pragma unroll
    for (int t = 0; t < 16; ++t) e[t] = BWD ? fast_exp(e[t]) * p.scale : fast_exp(e[t]);
    uint8_t* xt = x_stage(pp);
    const uint32_t rowoff = (uint32_t)(cg >> 2) * SLAB64 + (uint32_t)i * 128u;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const uint32_t off = rowoff + (((uint32_t)((cg & 3) * 2 + u) ^ (uint32_t)i) & 7u) * 16u;
      *reinterpret_cast<uint4*>(xt + off) = scale8(*reinterpret_cast<const uint4*>(xt + off), e + 8 * u);
    }
    fence_async_smem();
    tc_fence_before();
  };
  // forward states are stored as h * exp(mid) * scale, mid = (G_0 + G_n) / 2 = G_n - (G_n - G_0) / 2;
  // reverse states as dh * exp(G_n - mid) = dh * exp((G_n - G_0) / 2)
  auto gn_of = [&](int pp) { return SCALAR ? gn_next : sh.gn[pp & 1][col]; };   // (SCALAR: of the chunk gated last)
  auto state_scale = [&](int pp) {
    const float gnv = gn_of(pp), e0 = SCALAR ? e0_next : sh.e0[pp & 1][col];
    return BWD ? fast_exp(0.5f * (gnv - e0)) : fast_exp(gnv - 0.5f * e0) * p.scale;
  };

  if (warp == 16) {
    // ------------------------------------------------------------------ products
    // The two issuing threads run the same barriers as the compute warps and never wait for one another: the
    // product thread's time is the tensor core's (an issue takes about as long as the product before it runs),
    // the copy thread's is spent waiting for products to release tiles.
    if (lane == 0) {
      issue_gate_mma(0);
      if (NT > 1) issue_gate_mma(1);
    }
    bool ok = !__syncthreads_or(*abort_flag);   // chunk 0 is gated
    if (ok && lane == 0) {
      issue_state_mma(0);
      if (NT > 2) issue_gate_mma(2);
    }
    for (int pp = 0; ok && pp < NT; ++pp) {
      // h'_pp is staged, chunk pp+1 is gated; every thread of the block sees the same verdict, so
      // all of them leave the loop at the same barrier
      if (__syncthreads_or(*abort_flag)) break;
      if (lane == 0) {
        if (pp + 1 < NT) issue_state_mma(pp + 1);
        if (pp + 3 < NT) issue_gate_mma(pp + 3);   // its exponent slot was read by the gating of chunk pp+1
      }
      __syncwarp();
    }
  } else if (warp == 17) {
    // ------------------------------------------------------------------ copies
    bool ok = !__syncthreads_or(*abort_flag);
    if (ok && lane == 0 && !SCALAR && NT > 3) issue_g(3);    // into the stage of chunk 0, whose exponent product is complete
    for (int pp = 0; ok && pp < NT; ++pp) {
      // the store of chunk pp-1 has read its staging tile: after the barrier the compute warps may
      // overwrite it (with the state of chunk pp+1)
      if (lane == 0) tma_store_wait_read();
      if (__syncthreads_or(*abort_flag)) break;
      if (lane == 0) {
        if (keep_states) {
          const int hrow = ((b * (p.T / C) + chunk_of(pp)) * p.H + h) * D;
          tma_store_2d(&p.mst, hst + (pp & 1) * TILE128, 0, hrow);
          tma_store_2d(&p.mst, hst + (pp & 1) * TILE128 + TILE128 / 2, 64, hrow);
          tma_store_commit();
        }
        if (!SCALAR && pp + 4 < NT) issue_g(pp + 4);   // the stage of chunk pp+1, whose exponent product is complete
        if (pp + NXY < NT) {                       // the x/y stage of chunk pp is free once its state product is done
          if (!mbar_wait(&sh.sbar[pp & 1], (pp >> 1) & 1)) { *abort_flag = 1; fail(2); }
          if (pp + NXY != p.skip_xy) issue_xy(pp + NXY);
        }
      }
      __syncwarp();
    }
    if (lane == 0) tma_store_wait_all();
  } else {
    // ------------------------------------------------------------------ state in registers
    // fp32 state: row k = col, columns 32 seg .. + 31
    float S[32];
    {
      const float* src = p.s0 ? p.s0 + ((size_t)blk * D + col) * D + seg * 32 : nullptr;
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 x = src ? *reinterpret_cast<const float4*>(src + j) : make_float4(0.f, 0.f, 0.f, 0.f);
        S[j] = x.x; S[j + 1] = x.y; S[j + 2] = x.z; S[j + 3] = x.w;
      }
    }
    float gtot = 0.f;   // summed log-gates of this thread's channel over the block's chunks
    gate_chunk(0);
    if (SCALAR) load_gates(3);
    bool ok = !__syncthreads_or(*abort_flag);
    float decay = 1.f, hscale = 1.f, gn_cur = 0.f;   // of the chunk whose state product comes next
    if (ok) {
      gn_cur = gn_of(0);
      decay = fast_exp(gn_cur);
      hscale = state_scale(0);
    }
    for (int pp = 0; ok && pp < NT; ++pp) {
      // the state this chunk starts from (bf16), in the form its consumers use: staged in shared
      // memory in the tile format of the states tensor map and written out by a TMA store
      gtot += gn_cur;   // (published by the gating of this chunk, one iteration ago)
      if (keep_states) {
        uint8_t* tile = hst + (pp & 1) * TILE128;
#pragma unroll
        for (int j = 0; j < 32; j += 8)
          *reinterpret_cast<uint4*>(tile + tile_off(128, col, seg * 32 + j)) =
              make_uint4(pack_bf16(S[j] * hscale, S[j + 1] * hscale), pack_bf16(S[j + 2] * hscale, S[j + 3] * hscale),
                         pack_bf16(S[j + 4] * hscale, S[j + 5] * hscale), pack_bf16(S[j + 6] * hscale, S[j + 7] * hscale));
        fence_async_smem();
      }
      if (pp + 1 < NT) gate_chunk(pp + 1);
      if (__syncthreads_or(*abort_flag)) { ok = false; break; }
      float decay_n = 1.f, hscale_n = 1.f, gn_n = 0.f;
      if (pp + 1 < NT) {
        gn_n = gn_of(pp + 1);
        decay_n = fast_exp(gn_n);
        hscale_n = state_scale(pp + 1);
      }
      if (SCALAR) load_gates(pp + 4);
      // (SUM: the wait only keeps this thread within one phase of the barrier; the product was issued a chunk ago)
      if (!mbar_wait(&sh.sbar[pp & 1], (pp >> 1) & 1)) { *abort_flag = 1; fail(2); }
      tc_fence_after();
      if (!SUM) {
        float d[32];
        tmem_ld32(tmem_addr(tm, lane_base, cS + (pp & 1) * 128 + seg * 32), d);
#pragma unroll
        for (int t = 0; t < 32; ++t) S[t] = fmaf(S[t], decay, d[t]);
      }
      tc_fence_before();
      decay = decay_n;
      hscale = hscale_n;
      gn_cur = gn_n;
    }
    if (SUM && ok) {   // every product has completed: the accumulated tile is the state after the block's chunks
      tc_fence_after();
      tmem_ld32(tmem_addr(tm, lane_base, cS + seg * 32), S);
      tc_fence_before();
    }
    if (ok && p.s_final) {
      float* dst = p.s_final + ((size_t)blk * D + col) * D + seg * 32;
#pragma unroll
      for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(S[j], S[j + 1], S[j + 2], S[j + 3]);
    }
    if (ok && p.gsum && seg == 0) p.gsum[(size_t)blk * D + col] = gtot;
    // (a loop left early may leave gate copies of this thread in flight: they land before the block ends)
    if (SCALAR) asm volatile("cp.async.wait_all;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 512);
  if (tid == 0 && sh.abort_flag) {
    if (p.states) poison(p.states + ((size_t)(b * (p.T / C) + chunk_of(0)) * p.H + h) * D * D);
    if (p.s_final) poison(p.s_final + (size_t)blk * D * D);
    if (p.gsum) poison(p.gsum + (size_t)blk * D);
  }
}

// Joins the time segments of each (batch, head).  A segment acts on the state entering it as
// h_out = h_in * exp(P) + S, with P the summed log-gates of its chunks (per channel) and S its end
// state from a zero start.  Forward order for states, reverse order for state gradients.
//   first [BH,K,V] or null;  P [BH,nseg,K];  S [BH,nseg,K,V];  start [BH,nseg,K,V] (out);  last [BH,K,V] or null (out)
template <bool REVERSE>
__global__ void k_join_segments(const float* __restrict__ first, const float* __restrict__ P, const float* __restrict__ S,
                                float* __restrict__ start, float* __restrict__ last, int nseg) {
  // grid (batch x head, slices): a block chains one slice of the K x V elements of one (batch, head)
  // (the loads of a step do not depend on the chain: unrolled, they are all in flight together)
  const int bh = blockIdx.x;
  const int span = D * D / gridDim.y;
  for (int e = blockIdx.y * span + threadIdx.x * 4; e < (blockIdx.y + 1) * span; e += blockDim.x * 4) {
    const int k = e / D;
    float4 cur = first ? *reinterpret_cast<const float4*>(first + (size_t)bh * D * D + e) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int i = 0; i < nseg; ++i) {
      const int r = REVERSE ? nseg - 1 - i : i;
      const size_t sb = ((size_t)bh * nseg + r) * D * D + e;
      *reinterpret_cast<float4*>(start + sb) = cur;
      const float w = __expf(P[((size_t)bh * nseg + r) * D + k]);
      const float4 add = *reinterpret_cast<const float4*>(S + sb);
      cur = make_float4(fmaf(cur.x, w, add.x), fmaf(cur.y, w, add.y), fmaf(cur.z, w, add.z), fmaf(cur.w, w, add.w));
    }
    if (last) *reinterpret_cast<float4*>(last + (size_t)bh * D * D + e) = cur;
  }
}

// ===========================================================================
// Forward output
// ===========================================================================
struct FwdOParams {
  CUtensorMap mq, mk, mg, mv, mh;
  const __nv_bfloat16* gscalar;   // scalar gates [B,T,H] (SCALAR kernel; mg is unused then)
  __nv_bfloat16* o;
  int T, H, NT;
  float scale;
};

// SCALAR: no gate tile and no exponent product; every warp cumulates the chunk's 64 gates in registers.
template <bool SCALAR>
__global__ void __launch_bounds__(NTHREADS, 2) k_fwd_o(const __grid_constant__ FwdOParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* qs = smem;                 // q -> q~ in place
  uint8_t* ks = qs + TILE64;          // k -> k~ in place
  uint8_t* gs = ks + TILE64;          // g; later the bf16 intra matrix (first 8 KB)
  uint8_t* vs = gs + TILE64;
  uint8_t* hs = vs + TILE64;          // h_c exp(mid) scale, 128 x 128 (scaled by the scan kernel)
  uint8_t* mt = hs + TILE128;         // TRI_MID pattern, 64 x 64
  __shared__ uint64_t bar_load, bar_e, bar_a, bar_o;
  __shared__ uint32_t tmem_slot;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q4 = warp & 3, seg = warp >> 2;
  // heads vary fastest over the blocks in flight: together they read whole token rows of the
  // [B,T,H,D] activations (all heads of a time step are contiguous in memory)
  const int h = blockIdx.x, ci = blockIdx.y, b = blockIdx.z;
  const int row = b * p.T + ci * C;
  constexpr uint32_t cO = 0, cE = 0, cA = 128;   // E is consumed before O is produced

  if (tid == 0) {
    mbar_init(&bar_load, 1); mbar_init(&bar_e, 1); mbar_init(&bar_a, 1); mbar_init(&bar_o, 1);
    fence_barrier_init();
    mbar_expect_tx(&bar_load, (SCALAR ? 3 : 4) * TILE64 + TILE128);
    if (!SCALAR) { tma_load_3d(gs, &p.mg, &bar_load, 0, h, row); tma_load_3d(gs + SLAB64, &p.mg, &bar_load, 64, h, row); }
    tma_load_3d(qs, &p.mq, &bar_load, 0, h, row); tma_load_3d(qs + SLAB64, &p.mq, &bar_load, 64, h, row);
    tma_load_3d(ks, &p.mk, &bar_load, 0, h, row); tma_load_3d(ks + SLAB64, &p.mk, &bar_load, 64, h, row);
    tma_load_3d(vs, &p.mv, &bar_load, 0, h, row); tma_load_3d(vs + SLAB64, &p.mv, &bar_load, 64, h, row);
    const int hrow = ((b * p.NT + ci) * p.H + h) * D;
    tma_load_2d(hs, &p.mh, &bar_load, 0, hrow); tma_load_2d(hs + TILE128 / 2, &p.mh, &bar_load, 64, hrow);
  }
  __syncwarp();
  if (warp == 0) { tmem_alloc(&tmem_slot, 256); tmem_relinquish(); }
  __nv_bfloat16 greg_lo = __float2bfloat16(0.f), greg_hi = greg_lo;   // SCALAR: the gates of time steps lane and lane + 32
  if (SCALAR) {   // (one chunk per block: the loads have the whole tile fetch to land)
    const __nv_bfloat16* src = p.gscalar + (size_t)(row + lane) * p.H + h;
    greg_lo = src[0];
    greg_hi = src[(size_t)32 * p.H];
  } else {
    build_tri_tile(mt, 64, TRI_MID);
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_slot;
  const uint32_t lane_base = q4 * 32;
  bool ok = __syncthreads_and(mbar_wait(&bar_load, 0));
  if (!ok) fail(3);
  if (!SCALAR && ok && tid == 0) {
    tc_fence_after();
    const uint32_t ga = smem_u32(gs), ma = smem_u32(mt);
#pragma unroll
    for (int j0 = 0; j0 < C; j0 += 16)   // E = G - mid, [time][channel]
      umma_bf16(tm + cE, desc_kmajor(ma, 64, 0, j0), desc_mnmajor(ga, 64, j0, 0), umma_idesc(64, 128, 0, 1), j0 > 0);
    umma_commit(&bar_e);
  }
  __syncwarp();
  if (!SCALAR && ok) {
    ok = __syncthreads_and(mbar_wait(&bar_e, 0));
    if (!ok) fail(9);
  }
  if (SCALAR && ok) {
    // thread (q4, lane < 16, seg) gates 32 channels of time row 16 q4 + lane, whose cumulative gate sits in
    // lane (16 q4 + lane) mod 32 of the warp
    const WarpGates w = warp_cumulate(__bfloat162float(greg_lo), __bfloat162float(greg_hi), lane);
    const int i = 16 * q4 + (lane & 15);
    const float E = __shfl_sync(0xffffffffu, (q4 >> 1) ? w.hi : w.lo, i & 31) - w.mid();
    const float f = fast_exp(E), r = fast_exp(-E);
    if (lane < 16) {
      const uint32_t rowoff = (uint32_t)(seg >> 1) * SLAB64 + (uint32_t)i * 128u;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t off = rowoff + (((uint32_t)((seg & 1) * 4 + u) ^ (uint32_t)i) & 7u) * 16u;
        *reinterpret_cast<uint4*>(qs + off) = scale8_by(*reinterpret_cast<const uint4*>(qs + off), f);
        *reinterpret_cast<uint4*>(ks + off) = scale8_by(*reinterpret_cast<const uint4*>(ks + off), r);
      }
    }
    fence_async_smem();
    tc_fence_before();
  }
  if (!SCALAR && ok) {
    tc_fence_after();
    float e[32];
    tmem_ld32(tmem_addr(tm, lane_base, cE + seg * 32), e);
    if (lane < 16) {   // rows of an M = 64 accumulator sit in lanes 0..15 of each 32-lane quarter
      const int i = 16 * q4 + lane;
      const uint32_t rowoff = (uint32_t)(seg >> 1) * SLAB64 + (uint32_t)i * 128u;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t off = rowoff + (((uint32_t)((seg & 1) * 4 + u) ^ (uint32_t)i) & 7u) * 16u;
        float f[8], r[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) { f[t] = fast_exp(e[8 * u + t]); r[t] = fast_exp(-e[8 * u + t]); }
        *reinterpret_cast<uint4*>(qs + off) = scale8(*reinterpret_cast<const uint4*>(qs + off), f);
        *reinterpret_cast<uint4*>(ks + off) = scale8(*reinterpret_cast<const uint4*>(ks + off), r);
      }
    }
    fence_async_smem();
    tc_fence_before();
  }
  __syncthreads();
  if (ok && tid == 0) {
    tc_fence_after();
    const uint32_t qa = smem_u32(qs), ka = smem_u32(ks), ha = smem_u32(hs);
#pragma unroll
    for (int k0 = 0; k0 < D; k0 += 16)   // A = q~ k~^T
      umma_bf16(tm + cA, desc_kmajor(qa, 64, 0, k0), desc_kmajor(ka, 64, 0, k0), umma_idesc(64, 64, 0, 0), k0 > 0);
    umma_commit(&bar_a);
#pragma unroll
    for (int k0 = 0; k0 < D; k0 += 16)   // o = q~ h'
      umma_bf16(tm + cO, desc_kmajor(qa, 64, 0, k0), desc_mnmajor(ha, 128, k0, 0), umma_idesc(64, 128, 0, 1), k0 > 0);
  }
  __syncwarp();
  if (ok) {
    ok = __syncthreads_and(mbar_wait(&bar_a, 0));
    if (!ok) fail(4);
  }
  if (ok) {
    tc_fence_after();
    const int i = 16 * q4 + lane;
    float a[16];
    tmem_ld16(tmem_addr(tm, lane_base, cA + seg * 16), a);
    if (lane < 16) store_tril16(gs, i, seg * 16, a, p.scale);
    fence_async_smem();
    tc_fence_before();
  }
  __syncthreads();
  if (ok && tid == 0) {
    tc_fence_after();
    const uint32_t pa = smem_u32(gs), va = smem_u32(vs);
#pragma unroll
    for (int k0 = 0; k0 < C; k0 += 16)   // o += A v
      umma_bf16(tm + cO, desc_kmajor(pa, 64, 0, k0), desc_mnmajor(va, 64, k0, 0), umma_idesc(64, 128, 0, 1), 1);
    umma_commit(&bar_o);
  }
  __syncwarp();
  if (ok) {
    ok = __syncthreads_and(mbar_wait(&bar_o, 0));
    if (!ok) fail(5);
  }
  if (ok) {
    tc_fence_after();
    const int i = 16 * q4 + lane;
    __nv_bfloat16* dst = p.o + ((size_t)(row + i) * p.H + h) * D + seg * 32;
    float a[32];
    tmem_ld32(tmem_addr(tm, lane_base, cO + seg * 32), a);
    if (lane < 16) {
#pragma unroll
      for (int t = 0; t < 32; t += 8)
        *reinterpret_cast<uint4*>(dst + t) = make_uint4(pack_bf16(a[t], a[t + 1]), pack_bf16(a[t + 2], a[t + 3]),
                                                        pack_bf16(a[t + 4], a[t + 5]), pack_bf16(a[t + 6], a[t + 7]));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 256);
  if (tid == 0 && !ok) poison(p.o + ((size_t)row * p.H + h) * D);
}

// ===========================================================================
// Fused forward: state scan and chunk outputs in one pass
// ===========================================================================
// One block per (batch, head) walks its chunks in order with the K x V state in registers, so the
// chunk-start state never has to come back from HBM: per chunk it is staged once in shared memory
// as the bf16 operand h' = h exp(mid) scale of the output product (and, when the caller keeps the
// states for a backward pass, written out from there by a TMA store).  q, k, g, v are read once.
//   exponents  E = G - mid   [time (repeated to 128 lanes)][channel]      (pattern TRI_MID)
//              W[channel][0] = G_n,  W[channel][1] = G_n - mid            (pattern rows: ones, TRI_MID row 63)
//   gating     q~ = q exp(E), k~ = k exp(-E) in place
//   products   A = q~ k~^T;  o = q~ h' + tril(A) scale v;  D = k~^T v
//   state      h <- h exp(G_n) + exp(G_n - mid) D      (k exp(G_n - G) = k~ exp(G_n - mid), per channel)
// 16 compute warps (thread (q4, lane, seg): state row k = 32 q4 + lane, columns 32 seg .. + 31) and a
// driver warp that issues every product and copy; two block-wide barriers per chunk.
struct FusedParams {
  CUtensorMap mq, mk, mg, mv;
  CUtensorMap mst;         // the states tensor as [B*NT*H*128, 128] (TMA stores); unused when states == nullptr
  const float* s0;         // state each block starts from: [B,H,nseg,K,V] or null (zero)
  __nv_bfloat16* states;   // h' [B,T/64,H,K,V] or null
  float* s_final;          // state each block ends with: [B,H,nseg,K,V] or null
  __nv_bfloat16* o;        // [B,T,H,V]
  const __nv_bfloat16* gscalar;   // scalar gates [B,T,H] (SCALAR kernel; mg is unused then)
  int T, H, NT;            // T: tokens per sequence; NT: chunks per block (T / 64 / nseg)
  int nseg;                // time segments per sequence, one block each
  float scale;
};
struct FusedShared {
  uint64_t fullin[2], ebar, abar, sbar, obar;
  uint32_t tmem_slot;
  int abort_flag;
};
constexpr uint32_t FUSED_STAGE = 4 * TILE64;   // q, k, g, v
constexpr size_t FUSED_SMEM = 2 * FUSED_STAGE + 2 * TILE128 + 2 * SLAB64 + 2048 + TILE64 + sizeof(FusedShared);

// SCALAR: no gate tile is fetched and no exponent product issued; every compute warp cumulates the chunk's 64
// gates in registers (warp_cumulate), which gives its threads E of their time row, G_n and mid directly.
template <bool SCALAR>
__global__ void __launch_bounds__(FUSED_THREADS) k_fwd_fused(const __grid_constant__ FusedParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* in = smem;                         // 2 stages x (q, k, g, v)
  uint8_t* hst = in + 2 * FUSED_STAGE;        // 2 x (128 x 128) bf16: h' of the current chunk
  uint8_t* mt = hst + 2 * TILE128;            // TRI_MID pattern, rows repeated to 128
  uint8_t* wt = mt + 2 * SLAB64;              // 16 x 64 pattern for G_n and G_n - mid
  uint8_t* ost = wt + 2048;                   // 64 x 128 bf16: the outputs of a chunk, row-major, before they leave
  FusedShared& sh = *reinterpret_cast<FusedShared*>(ost + TILE64);
  volatile int* abort_flag = &sh.abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool driver = warp == 16;
  const int q4 = warp & 3, seg = (warp >> 2) & 3, col = q4 * 32 + lane;
  const int blk = blockIdx.x, sg = blk % p.nseg, bh = blk / p.nseg, b = bh / p.H, h = bh % p.H;
  const int NT = p.NT;
  const int c0 = sg * NT;   // first chunk of this block within its sequence
  constexpr uint32_t cE = 0, cD = 128, cO = 256, cA = 384, cW = 448;
  if ((smem_u32(smem) & 1023u) != 0) {   // uniform over the block
    if (tid == 0) fail(12);
    return;
  }
  auto issue_load = [&](int pp) {
    uint8_t* qs = in + (pp & 1) * FUSED_STAGE;
    uint8_t *ks = qs + TILE64, *gs = ks + TILE64, *vs = gs + TILE64;
    uint64_t* bar = &sh.fullin[pp & 1];
    const int row = b * p.T + (c0 + pp) * C;
    mbar_expect_tx(bar, SCALAR ? 3 * TILE64 : FUSED_STAGE);
    if (!SCALAR) { tma_load_3d(gs, &p.mg, bar, 0, h, row); tma_load_3d(gs + SLAB64, &p.mg, bar, 64, h, row); }
    tma_load_3d(qs, &p.mq, bar, 0, h, row); tma_load_3d(qs + SLAB64, &p.mq, bar, 64, h, row);
    tma_load_3d(ks, &p.mk, bar, 0, h, row); tma_load_3d(ks + SLAB64, &p.mk, bar, 64, h, row);
    tma_load_3d(vs, &p.mv, bar, 0, h, row); tma_load_3d(vs + SLAB64, &p.mv, bar, 64, h, row);
  };
  if (tid == 0) {
    mbar_init(&sh.fullin[0], 1); mbar_init(&sh.fullin[1], 1);
    mbar_init(&sh.ebar, 1); mbar_init(&sh.abar, 1); mbar_init(&sh.sbar, 1); mbar_init(&sh.obar, 1);
    fence_barrier_init();
    tma_prefetch_desc(&p.mq); tma_prefetch_desc(&p.mk); tma_prefetch_desc(&p.mv);
    if (!SCALAR) tma_prefetch_desc(&p.mg);
    sh.abort_flag = 0;
    issue_load(0);
    if (NT > 1) issue_load(1);
  }
  __syncwarp();
  if (warp == 0) { tmem_alloc(&sh.tmem_slot, 512); tmem_relinquish(); }
  // SCALAR: the gates of time steps lane and lane + 32 of the next chunk, in registers, loaded right after the
  // first barrier of the chunk before: a chunk is long enough here for the load to land before the loop's back
  // edge (where a register with a load in flight stalls the warp; the state scans, whose chunks are short, use
  // GateRing instead)
  __nv_bfloat16 greg_lo = __float2bfloat16(0.f), greg_hi = greg_lo;
  auto load_gates = [&](int c) {
    const __nv_bfloat16* src = p.gscalar + (size_t)(b * p.T + (c0 + c) * C + lane) * p.H + h;
    greg_lo = src[0];
    greg_hi = src[(size_t)32 * p.H];
  };
  if (SCALAR) {
    if (!driver) load_gates(0);
  } else {
    build_tri_tile(mt, 128, TRI_MID);
    build_w_tile(wt);
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = sh.tmem_slot;
  const uint32_t lane_base = q4 * 32;

  if (driver) {
    // ------------------------------------------------------------------ products and copies
    auto issue_exponents = [&](int pp) {
      if (SCALAR) return;
      if (!mbar_wait(&sh.fullin[pp & 1], (pp >> 1) & 1)) { *abort_flag = 1; fail(3); }
      tc_fence_after();
      const uint32_t ga = smem_u32(in + (pp & 1) * FUSED_STAGE + 2 * TILE64), ma = smem_u32(mt), wa = smem_u32(wt);
#pragma unroll
      for (int j0 = 0; j0 < C; j0 += 16)   // E: [time (repeated)][channel]
        umma_bf16(tm + cE, desc_kmajor(ma, 128, 0, j0), desc_mnmajor(ga, 64, j0, 0), umma_idesc(128, 128, 0, 1), j0 > 0);
#pragma unroll
      for (int j0 = 0; j0 < C; j0 += 16)   // W: [channel][G_n, G_n - mid, 0 ...]
        umma_bf16(tm + cW, desc_mnmajor(ga, 64, j0, 0), desc_kmajor(wa, 16, 0, j0), umma_idesc(128, 16, 1, 0), j0 > 0);
      umma_commit(&sh.ebar);
    };
    if (lane == 0) issue_exponents(0);
    __syncwarp();
    for (int pp = 0; pp < NT; ++pp) {
      const uint32_t ph = pp & 1;
      uint8_t* qs = in + (pp & 1) * FUSED_STAGE;
      uint8_t *ks = qs + TILE64, *gs = ks + TILE64, *vs = gs + TILE64;
      uint8_t* ht = hst + (pp & 1) * TILE128;
      // the state store of chunk pp-1 has read its staging tile, which the compute warps refill after
      // the next barrier (with the state of chunk pp+1)
      if (lane == 0) tma_store_wait_read();
      // B1: q~, k~ and h' of chunk pp are in shared memory, E and W have been read
      if (__syncthreads_or(*abort_flag)) break;
      if (lane == 0) {
        tc_fence_after();
        const uint32_t qa = smem_u32(qs), ka = smem_u32(ks), va = smem_u32(vs), ha = smem_u32(ht);
#pragma unroll
        for (int k0 = 0; k0 < D; k0 += 16)   // A = q~ k~^T
          umma_bf16(tm + cA, desc_kmajor(qa, 64, 0, k0), desc_kmajor(ka, 64, 0, k0), umma_idesc(64, 64, 0, 0), k0 > 0);
        umma_commit(&sh.abar);
#pragma unroll
        for (int k0 = 0; k0 < C; k0 += 16)   // D[k][v] = sum_j k~[j][k] v[j][v]
          umma_bf16(tm + cD, desc_mnmajor(ka, 64, k0, 0), desc_mnmajor(va, 64, k0, 0), umma_idesc(128, 128, 1, 1), k0 > 0);
        umma_commit(&sh.sbar);
#pragma unroll
        for (int k0 = 0; k0 < D; k0 += 16)   // o = q~ h'
          umma_bf16(tm + cO, desc_kmajor(qa, 64, 0, k0), desc_mnmajor(ha, 128, k0, 0), umma_idesc(64, 128, 0, 1), k0 > 0);
        if (p.states) {
          const int hrow = ((b * (p.T / C) + c0 + pp) * p.H + h) * D;
          tma_store_2d(&p.mst, ht, 0, hrow);
          tma_store_2d(&p.mst, ht + TILE128 / 2, 64, hrow);
          tma_store_commit();
        }
      }
      // B2: tril(A) scale is in shared memory (in the gate tile of this stage)
      if (__syncthreads_or(*abort_flag)) break;
      if (lane == 0) {
        tc_fence_after();
        const uint32_t pa = smem_u32(gs), va = smem_u32(vs);
#pragma unroll
        for (int k0 = 0; k0 < C; k0 += 16)   // o += tril(A) scale v
          umma_bf16(tm + cO, desc_kmajor(pa, 64, 0, k0), desc_mnmajor(va, 64, k0, 0), umma_idesc(64, 128, 0, 1), 1);
        umma_commit(&sh.obar);
        // exponents of the next chunk (E and W of this one were read before B1)
        if (pp + 1 < NT) issue_exponents(pp + 1);
        // every tile of this stage is dead once its products are complete
        if (pp + 2 < NT) {
          if (!mbar_wait(&sh.obar, ph)) { *abort_flag = 1; fail(5); }
          issue_load(pp + 2);
        }
      }
      __syncwarp();
    }
    __syncthreads();   // (the compute warps copy the last outputs after this barrier)
    if (lane == 0) tma_store_wait_all();
  } else {
    // ------------------------------------------------------------------ state in registers
    float S[32];
    {
      const float* src = p.s0 ? p.s0 + ((size_t)blk * D + col) * D + seg * 32 : nullptr;
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 x = src ? *reinterpret_cast<const float4*>(src + j) : make_float4(0.f, 0.f, 0.f, 0.f);
        S[j] = x.x; S[j + 1] = x.y; S[j + 2] = x.z; S[j + 3] = x.w;
      }
    }
    // Outputs leave in two steps: the accumulator rows (an M = 64 accumulator keeps 16 rows in the first
    // 16 lanes of each warp) are packed to bf16 in a shared tile; after the next block-wide barrier every
    // thread copies 32 contiguous bytes of it, so that a warp writes whole 256-byte rows.
    auto copy_out = [&](int pp) {
      const int r = tid >> 3, piece = tid & 7;   // 64 rows x 8 pieces of 16 channels
      // 16-byte pieces of a row are stored XOR-permuted by the row number (bank conflicts of the writers)
      const uint8_t* rowp = ost + r * 256;
      uint4* dst = reinterpret_cast<uint4*>(p.o + ((size_t)(b * p.T + (c0 + pp) * C + r) * p.H + h) * D + piece * 16);
      const uint4 x = *reinterpret_cast<const uint4*>(rowp + (((2 * piece) ^ r) & 15) * 16);
      const uint4 y = *reinterpret_cast<const uint4*>(rowp + (((2 * piece + 1) ^ r) & 15) * 16);
      __stcs(dst, x);
      __stcs(dst + 1, y);
    };
    bool ok = true;
    for (int pp = 0; ok && pp < NT; ++pp) {
      const uint32_t ph = pp & 1;
      uint8_t* qs = in + (pp & 1) * FUSED_STAGE;
      uint8_t *ks = qs + TILE64, *gs = ks + TILE64;
      uint8_t* ht = hst + (pp & 1) * TILE128;
      if (!mbar_wait(&sh.fullin[pp & 1], (pp >> 1) & 1) || (!SCALAR && !mbar_wait(&sh.ebar, ph))) { *abort_flag = 1; fail(9); }
      tc_fence_after();
      WarpGates wg;
      if (SCALAR) {
        wg = warp_cumulate(__bfloat162float(greg_lo), __bfloat162float(greg_hi), lane);
      }
      // per-channel factors of this thread's state row
      float decay, c2;
      float em[16];
      {
        float w[8];
        if (SCALAR) {
          w[0] = wg.gn;
          w[1] = wg.gn - wg.mid();
        } else {
          tmem_ld8(tmem_addr(tm, lane_base, cW), w);
          // (the exponents of the gating below are fetched now: their exponentials interleave with the staging)
          tmem_ld16(tmem_addr(tm, lane_base, cE + ((q4 >> 1) * 4 + seg) * 16), em);
        }
        decay = fast_exp(w[0]);                    // exp(G_n)
        c2 = fast_exp(w[1]);                       // exp(G_n - mid)
        const float hscale = fast_exp(w[0] - w[1]) * p.scale;   // exp(mid) scale
#pragma unroll
        for (int j = 0; j < 32; j += 8)
          *reinterpret_cast<uint4*>(ht + tile_off(128, col, seg * 32 + j)) =
              make_uint4(pack_bf16(S[j] * hscale, S[j + 1] * hscale), pack_bf16(S[j + 2] * hscale, S[j + 3] * hscale),
                         pack_bf16(S[j + 4] * hscale, S[j + 5] * hscale), pack_bf16(S[j + 6] * hscale, S[j + 7] * hscale));
      }
      // gate q, k: thread (q4, lane, seg) owns time row (32 q4 + lane) mod 64 and 16 channels
      if (SCALAR) {
        const int i = (q4 * 32 + lane) & 63;
        const int cg = (q4 >> 1) * 4 + seg;
        const float E = ((q4 & 1) ? wg.hi : wg.lo) - wg.mid();
        const float f = fast_exp(E), r = fast_exp(-E);
        const uint32_t rowoff = (uint32_t)(cg >> 2) * SLAB64 + (uint32_t)i * 128u;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const uint32_t off = rowoff + (((uint32_t)((cg & 3) * 2 + u) ^ (uint32_t)i) & 7u) * 16u;
          *reinterpret_cast<uint4*>(qs + off) = scale8_by(*reinterpret_cast<const uint4*>(qs + off), f);
          *reinterpret_cast<uint4*>(ks + off) = scale8_by(*reinterpret_cast<const uint4*>(ks + off), r);
        }
      } else {
        const int i = (q4 * 32 + lane) & 63;
        const int cg = (q4 >> 1) * 4 + seg;
        const uint32_t rowoff = (uint32_t)(cg >> 2) * SLAB64 + (uint32_t)i * 128u;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const uint32_t off = rowoff + (((uint32_t)((cg & 3) * 2 + u) ^ (uint32_t)i) & 7u) * 16u;
          float f[8], r[8];
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            f[t] = fast_exp(em[8 * u + t]);
            r[t] = fast_exp(-em[8 * u + t]);
          }
          *reinterpret_cast<uint4*>(qs + off) = scale8(*reinterpret_cast<const uint4*>(qs + off), f);
          *reinterpret_cast<uint4*>(ks + off) = scale8(*reinterpret_cast<const uint4*>(ks + off), r);
        }
      }
      fence_async_smem();
      tc_fence_before();
      if (__syncthreads_or(*abort_flag)) { ok = false; break; }   // B1
      if (pp > 0) copy_out(pp - 1);   // staged before the barrier; the products of this chunk run meanwhile
      if (SCALAR && pp + 1 < NT) load_gates(pp + 1);
      // tril(A) scale -> bf16 operand in the (dead) gate tile
      if (!mbar_wait(&sh.abar, ph)) { *abort_flag = 1; fail(4); }
      tc_fence_after();
      {
        const int i = 16 * q4 + lane;   // rows of an M = 64 accumulator sit in lanes 0..15 of each quarter
        float a[16];
        tmem_ld16(tmem_addr(tm, lane_base, cA + seg * 16), a);
        if (lane < 16) store_tril16(gs, i, seg * 16, a, p.scale);
      }
      fence_async_smem();
      tc_fence_before();
      if (__syncthreads_or(*abort_flag)) { ok = false; break; }   // B2
      // state update while the last output product runs
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
        const int i = 16 * q4 + lane;
        float a[32];
        tmem_ld32(tmem_addr(tm, lane_base, cO + seg * 32), a);
        if (lane < 16) {
#pragma unroll
          for (int t = 0; t < 32; t += 8)
            *reinterpret_cast<uint4*>(ost + i * 256 + (((seg * 4 + t / 8) ^ i) & 15) * 16) =
                make_uint4(pack_bf16(a[t], a[t + 1]), pack_bf16(a[t + 2], a[t + 3]), pack_bf16(a[t + 4], a[t + 5]),
                           pack_bf16(a[t + 6], a[t + 7]));
        }
      }
      tc_fence_before();
    }
    __syncthreads();   // the outputs of the last chunk are staged
    if (ok) copy_out(NT - 1);
    if (ok && p.s_final) {
      float* dst = p.s_final + ((size_t)blk * D + col) * D + seg * 32;
#pragma unroll
      for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(S[j], S[j + 1], S[j + 2], S[j + 3]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 512);
  if (tid == 0 && sh.abort_flag) {
    poison(p.o + ((size_t)(b * p.T + c0 * C) * p.H + h) * D);
    if (p.s_final) poison(p.s_final + (size_t)blk * D * D);
  }
}

// ===========================================================================
// Backward of the chunks (persistent: each block walks chunks blockIdx.x,
// blockIdx.x + gridDim.x, ... and fetches the next chunk's tiles while the
// tensor core and the epilogue of the current one are still busy)
// ===========================================================================
struct BwdParams {
  CUtensorMap mq, mk, mg, mv, mdo, mh, mdh;
  void *dq, *dk, *dg;    // [B,T,H,K] fp32 or bf16 (dg may be null)
  __nv_bfloat16* dv;     // [B,T,H,V]
  const __nv_bfloat16* gscalar;   // scalar gates [B,T,H] (SCALAR kernels; mg is unused then)
  int T, H, NT, total;   // total = B * H * NT chunks
  float scale;
};

// Warp roles: warps 0-15 gate q and k of the next chunk and write the gradients of a chunk out of
// tensor memory (thread = one channel, 16 time steps); warps 16-19 convert A and dA to bf16 operands
// and reduce sum_v h' dh'; one thread of warp 20 issues every tensor-core product, one thread of warp 21
// every TMA load.
// The roles meet only through mbarriers, so the gradient write-out of chunk n runs while the
// exponent product, the gating and the A / dA products of chunk n+1 are under way; the six
// gradient products of chunk n+1 start as soon as chunk n has left tensor memory.
constexpr int BWD_THREADS = 704;
constexpr int BWD_EPI_THREADS = 512, BWD_GATE_THREADS = 128;

// TG: type of dq and dk; TD: type of dg.
// SCALAR: the gate is one value per head and time step; no gate tile is fetched and no exponent product
// issued: every write-out warp cumulates the 64 gates of a chunk in registers (warp_cumulate) and hands the
// factors exp(+-(G - mid)) of the time steps around by shuffles.  dg is summed over the key channels inside
// the kernel and written as fp32 [B,T,H] (the scalar gate's gradient is the sum of the channels').
template <typename TG, typename TD, bool SCALAR>
__global__ void __launch_bounds__(BWD_THREADS, 1) k_bwd_main(const __grid_constant__ BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* qs = smem;                 // 2 x: q -> q exp(G - mid) in place
  uint8_t* ks = qs + 2 * TILE64;      // 2 x: k -> k exp(mid - G) in place
  uint8_t* gs = ks + 2 * TILE64;      // g
  uint8_t* vs = gs + TILE64;
  uint8_t* dos = vs + TILE64;
  uint8_t* hs = dos + TILE64;         // h_c exp(mid) scale, 128 x 128
  uint8_t* dhs = hs + TILE128;        // dh_c exp(G_n - mid), 128 x 128
  uint8_t* Ps = dhs + TILE128;        // tril(A) scale, bf16 64 x 64
  uint8_t* dAs = Ps + SLAB64;         // tril(dA) scale, bf16 64 x 64
  uint8_t* mtm = dAs + SLAB64;        // TRI_MID pattern, rows repeated to 128
  // single-slot barriers complete once per chunk (parity it & 1); two-slot ones are indexed by it & 1
  // and complete every other chunk (parity (it >> 1) & 1)
  __shared__ uint64_t full_g, full_qk[2], full_hdo, full_dhv, bar_gate, bar_A, bar_r1, bar_r2, bar_main, gated, conv_done,
      hdh_done[2], e_done[2];
  __shared__ uint32_t tmem_slot;
  __shared__ float sufsum[2][4][D];   // per-segment totals of the dg suffix sums
  __shared__ float tails[2][4][D];    // per-segment sum_i dk_inter k
  __shared__ float hdh_s[2][D];       // sum_v h' dh'
  __shared__ float dgk_s[2][C];       // SCALAR: dg of a chunk summed over the channels
  __shared__ volatile int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // tensor-memory columns: the exponent tile E_mid is consumed by the gating before A and dA take its place
  constexpr uint32_t cEm = 0, cA = 0, cdA = 64, cET = 128, cdq = 256, cdk1 = 320, cdk2 = 384, cdv = 448;
  const int nit = (p.total - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

  auto chunk_rows = [&](int it, int& h, int& row, int& hrow) {
    // heads vary fastest over the chunks in flight: together the blocks read and write whole
    // token rows of the [B,T,H,D] activations
    const int cid = blockIdx.x + it * gridDim.x;
    const int ci = (cid / p.H) % p.NT, b = cid / (p.H * p.NT);
    h = cid % p.H;
    row = b * p.T + ci * C;
    hrow = ((b * p.NT + ci) * p.H + h) * D;
  };
  // bounded wait that also gives up when another role has failed
  auto wait = [&](uint64_t* bar, uint32_t parity, int code) -> bool {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
      if ((i & 255u) == 255u && abort_flag) return false;
    }
    abort_flag = 1;
    fail(code);
    return false;
  };

  if (tid == 0) {
    mbar_init(&full_g, 1);
    mbar_init(&full_qk[0], 1); mbar_init(&full_qk[1], 1); mbar_init(&full_hdo, 1);
    mbar_init(&full_dhv, 1); mbar_init(&bar_gate, 1); mbar_init(&bar_A, 1); mbar_init(&bar_r1, 1); mbar_init(&bar_r2, 1);
    mbar_init(&bar_main, 1);
    mbar_init(&gated, BWD_EPI_THREADS); mbar_init(&conv_done, BWD_GATE_THREADS);
    mbar_init(&hdh_done[0], BWD_GATE_THREADS); mbar_init(&hdh_done[1], BWD_GATE_THREADS);
    mbar_init(&e_done[0], BWD_EPI_THREADS); mbar_init(&e_done[1], BWD_EPI_THREADS);
    fence_barrier_init();
    abort_flag = 0;
  }
  if (tid < 2 * C) dgk_s[tid >> 6][tid & 63] = 0.f;
  if (warp == 0) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  if (!SCALAR) build_tri_tile(mtm, 128, TRI_MID);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_slot;

  if (warp < 16) {
    // ------------------------------------------------------------------ gradient write-out
    const int q4 = warp & 3, seg = warp >> 2, col = q4 * 32 + lane;
    const uint32_t lane_base = q4 * 32;
    const ColAddr ca = col_prep(64, col);
    const size_t ostride = (size_t)p.H * D;
    TG* const dq_out = reinterpret_cast<TG*>(p.dq);
    TG* const dk_out = reinterpret_cast<TG*>(p.dk);
    TD* const dg_out = reinterpret_cast<TD*>(p.dg);
    // q -> q exp(G - mid), k -> k exp(mid - G) in place: thread (q4, lane, seg) owns time row
    // (32 q4 + lane) mod 64 and 16 channels
    // SCALAR: the gates of time steps lane and lane + 32 of the next chunk to be gated, and the factors
    // exp(G - mid), exp(mid - G) of time step (16 seg + lane) mod 32 + 32 (seg / 2) of the chunk gated last
    // (in registers, loaded a chunk ahead: see the note in k_fwd_fused)
    __nv_bfloat16 greg_lo = __float2bfloat16(0.f), greg_hi = greg_lo;
    float fw_next = 1.f, rw_next = 1.f;
    auto load_gates = [&](int it) {
      int h, row, hrow;
      chunk_rows(it, h, row, hrow);
      const __nv_bfloat16* src = p.gscalar + (size_t)(row + lane) * p.H + h;
      greg_lo = src[0];
      greg_hi = src[(size_t)32 * p.H];
    };
    if (SCALAR && nit > 0) load_gates(0);
    auto gate_chunk = [&](int it) -> bool {
      const int sl = it & 1;
      bool landed = (SCALAR || wait(&bar_gate, it & 1, 9)) && wait(&full_qk[sl], (it >> 1) & 1, 6);
      if (SCALAR) landed = __all_sync(0xffffffffu, landed);   // (shuffles follow: the whole warp takes one path)
      if (!landed) return false;
      tc_fence_after();
      const int i = (q4 * 32 + lane) & 63;
      const int cg = (q4 >> 1) * 4 + seg;
      if (SCALAR) {
        const WarpGates w = warp_cumulate(__bfloat162float(greg_lo), __bfloat162float(greg_hi), lane);
        const float mid = w.mid();
        const float f_lo = fast_exp(w.lo - mid), r_lo = fast_exp(mid - w.lo);
        const float f_hi = fast_exp(w.hi - mid), r_hi = fast_exp(mid - w.hi);
        fw_next = (seg >> 1) ? f_hi : f_lo;
        rw_next = (seg >> 1) ? r_hi : r_lo;
        const float f = (q4 & 1) ? f_hi : f_lo, r = (q4 & 1) ? r_hi : r_lo;
        const uint32_t rowoff = (uint32_t)sl * TILE64 + (uint32_t)(cg >> 2) * SLAB64 + (uint32_t)i * 128u;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const uint32_t off = rowoff + (((uint32_t)((cg & 3) * 2 + u) ^ (uint32_t)i) & 7u) * 16u;
          *reinterpret_cast<uint4*>(qs + off) = scale8_by(*reinterpret_cast<const uint4*>(qs + off), f);
          *reinterpret_cast<uint4*>(ks + off) = scale8_by(*reinterpret_cast<const uint4*>(ks + off), r);
        }
        fence_async_smem();
        tc_fence_before();
        mbar_arrive(&gated);
        return true;
      }
      float em[16];
      tmem_ld16(tmem_addr(tm, lane_base, cEm + cg * 16), em);
      const uint32_t rowoff = (uint32_t)sl * TILE64 + (uint32_t)(cg >> 2) * SLAB64 + (uint32_t)i * 128u;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const uint32_t off = rowoff + (((uint32_t)((cg & 3) * 2 + u) ^ (uint32_t)i) & 7u) * 16u;
        float f[8], r[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          f[t] = fast_exp(em[8 * u + t]);
          r[t] = fast_exp(-em[8 * u + t]);
        }
        *reinterpret_cast<uint4*>(qs + off) = scale8(*reinterpret_cast<const uint4*>(qs + off), f);
        *reinterpret_cast<uint4*>(ks + off) = scale8(*reinterpret_cast<const uint4*>(ks + off), r);
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&gated);
      return true;
    };
    bool live = nit > 0 && gate_chunk(0);
    if (SCALAR && nit > 1) load_gates(1);
    for (int it = 0; live && it < nit; ++it) {
      const int sl = it & 1;
      int h, row, hrow;
      chunk_rows(it, h, row, hrow);
      const float fw = fw_next, rw = rw_next;   // (SCALAR) of this chunk
      // the next chunk's gating runs while the tensor core works on this chunk's gradient products
      if (it + 1 < nit && !gate_chunk(it + 1)) break;
      if (SCALAR && it + 2 < nit) load_gates(it + 2);   // fetched where the thread waits anyway
      bool done = wait(&bar_main, it & 1, 8) && wait(&hdh_done[sl], (it >> 1) & 1, 11);
      if (SCALAR) done = __all_sync(0xffffffffu, done);   // (shuffles follow: the whole warp takes one path)
      if (!done) break;
      tc_fence_after();
      const uint8_t* qt = qs + sl * TILE64;
      const uint8_t* kt = ks + sl * TILE64;
      const size_t obase = ((size_t)(row + seg * SEG) * p.H + h) * D + col;
      const size_t obase4 = obase - (lane & 3) + (size_t)(lane & 3) * ostride;   // channel group, own time row
      float dgl[SEG];
      float run = 0.f, tail = 0.f;
#pragma unroll
      for (int blk = 1; blk >= 0; --blk) {
        float et[8] = {}, dq[8], dk1[8], dk2[8], dv[8];
        const uint32_t c0 = seg * SEG + blk * 8;
        if (!SCALAR) tmem_ld8(tmem_addr(tm, lane_base, cET + 64 * sl + c0), et);
        tmem_ld8(tmem_addr(tm, lane_base, cdq + c0), dq);
        tmem_ld8(tmem_addr(tm, lane_base, cdk1 + c0), dk1);
        tmem_ld8(tmem_addr(tm, lane_base, cdk2 + c0), dk2);
        tmem_ld8(tmem_addr(tm, lane_base, cdv + c0), dv);
#pragma unroll
        for (int u = 7; u >= 0; --u) {
          const int t = blk * 8 + u;
          const uint32_t off = ca.at(seg * SEG + t);
          const float qv = ld_bf16(qt, off), kv = ld_bf16(kt, off);   // q~, k~
          // exp(G - mid), exp(mid - G) of time step 16 seg + t
          const float e = SCALAR ? __shfl_sync(0xffffffffu, fw, (seg * SEG + t) & 31) : fast_exp(et[u]);
          const float r = SCALAR ? __shfl_sync(0xffffffffu, rw, (seg * SEG + t) & 31) : fast_exp(-et[u]);
          const float dqs = dq[u];                        // dq exp(mid - G)
          const float dki = dk2[u];                       // dk_inter exp(G - mid)
          const float dks = dk1[u] + dki;                 // dk exp(G - mid)
          run += qv * dqs - kv * dks;                     // q dq - k dk
          tail = fmaf(dki, kv, tail);                     // dk_inter k
          dgl[t] = run;
          st_out(p.dv, obase + t * ostride, dv[u]);
          st_out(dq_out, obase + t * ostride, e * dqs);
          st_out(dk_out, obase + t * ostride, r * dks);
        }
      }
      sufsum[sl][seg][col] = run;
      tails[sl][seg][col] = tail;
      tc_fence_before();
      asm volatile("bar.sync 1, %0;" ::"n"(BWD_EPI_THREADS) : "memory");
      const float later = (seg < 1 ? sufsum[sl][1][col] : 0.f) + (seg < 2 ? sufsum[sl][2][col] : 0.f) +
                          (seg < 3 ? sufsum[sl][3][col] : 0.f);
      const float cst = later + tails[sl][0][col] + tails[sl][1][col] + tails[sl][2][col] + tails[sl][3][col] +
                        hdh_s[sl][col] / p.scale;
      // (exp(G_n) sum_v h dh = sum_v h' dh' / scale)
      mbar_arrive(&e_done[sl]);   // tensor memory, the q~ / k~ tiles and hdh_s of this chunk are free
      if constexpr (SCALAR) {
        // sum over the 128 channels: the lanes of a warp by a shuffle butterfly (lane t keeps the total of time
        // step t), then the four warps that share this segment through shared memory
#pragma unroll
        for (int t = 0; t < SEG; ++t) dgl[t] += cst;
        const float mine = warp_sum16(dgl, lane);
        if (lane < SEG) atomicAdd(&dgk_s[sl][seg * SEG + lane], mine);
        asm volatile("bar.sync 1, %0;" ::"n"(BWD_EPI_THREADS) : "memory");
        if (tid < C) {
          if (p.dg) reinterpret_cast<float*>(p.dg)[(size_t)(row + tid) * p.H + h] = dgk_s[sl][tid];
          dgk_s[sl][tid] = 0.f;   // (this slot is used again two chunks on, two barriers later)
        }
      } else if (p.dg) {
        // after the accumulators are released: four time steps x four channels change hands inside each
        // group of four lanes, so that every store writes four neighbouring channels of one time step
#pragma unroll
        for (int t = 0; t < SEG; t += 4) {
          float w[4] = {dgl[t] + cst, dgl[t + 1] + cst, dgl[t + 2] + cst, dgl[t + 3] + cst};
          st_transposed4(dg_out, obase4 + t * ostride, w, lane);
        }
      }
    }
  } else if (warp < 20) {
    // ------------------------------------------------------------------ A / dA -> masked bf16 operands
    const int g4 = warp & 3;
    const uint32_t lane_base = g4 * 32;
    for (int it = 0; it < nit; ++it) {
      // rows of the M = 64 accumulators sit in lanes 0..15 of each quarter
      if (!wait(&bar_A, it & 1, 7)) break;
      tc_fence_after();
      const int ri = 16 * g4 + lane;
#pragma unroll
      for (int sg = 0; sg < 4; ++sg) {
        float a[16];
        tmem_ld16(tmem_addr(tm, lane_base, cA + sg * 16), a);
        if (lane < 16) store_tril16(Ps, ri, sg * 16, a, p.scale);
        tmem_ld16(tmem_addr(tm, lane_base, cdA + sg * 16), a);
        if (lane < 16) store_tril16(dAs, ri, sg * 16, a, p.scale);
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&conv_done);
      // sum_v h'[k][v] dh'[k][v] for k = this thread, while the gradient products read the same tiles
      if (!wait(&full_hdo, it & 1, 6) || !wait(&full_dhv, it & 1, 6)) break;
      {
        const int gt = g4 * 32 + lane;
        float hd = 0.f;
#pragma unroll 4
        for (int c8 = 0; c8 < D; c8 += 8) {
          const uint32_t off = tile_off(128, gt, c8);
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
        hdh_s[it & 1][gt] = hd;
      }
      mbar_arrive(&hdh_done[it & 1]);   // h' and dh' of this chunk are no longer read by threads
    }
  } else if (warp == 20) {
    // ------------------------------------------------------------------ tensor-core issue
    if (lane == 0) {
      const uint32_t ga = smem_u32(gs), mma = smem_u32(mtm), va = smem_u32(vs), doa = smem_u32(dos), ha = smem_u32(hs),
                     dha = smem_u32(dhs), pa = smem_u32(Ps), daa = smem_u32(dAs);
      auto issue_gate = [&](int it) {
#pragma unroll
        for (int j0 = 0; j0 < C; j0 += 16)   // G - mid, [time (repeated)][channel]
          umma_bf16(tm + cEm, desc_kmajor(mma, 128, 0, j0), desc_mnmajor(ga, 64, j0, 0), umma_idesc(128, 128, 0, 1), j0 > 0);
#pragma unroll
        for (int j0 = 0; j0 < C; j0 += 16)   // G - mid, [channel][time]
          umma_bf16(tm + cET + 64 * (it & 1), desc_mnmajor(ga, 64, j0, 0), desc_kmajor(mma, 64, 0, j0),
                    umma_idesc(128, 64, 1, 0), j0 > 0);
        umma_commit(&bar_gate);
      };
      auto issue_A = [&](int it) {
        const uint32_t qta = smem_u32(qs + (it & 1) * TILE64), kta = smem_u32(ks + (it & 1) * TILE64);
#pragma unroll
        for (int k0 = 0; k0 < D; k0 += 16)   // A[i][j] = q~ k~^T
          umma_bf16(tm + cA, desc_kmajor(qta, 64, 0, k0), desc_kmajor(kta, 64, 0, k0), umma_idesc(64, 64, 0, 0), k0 > 0);
      };
      auto issue_dA = [&]() {
#pragma unroll
        for (int k0 = 0; k0 < D; k0 += 16)   // dA[i][j] = do v^T
          umma_bf16(tm + cdA, desc_kmajor(doa, 64, 0, k0), desc_kmajor(va, 64, 0, k0), umma_idesc(64, 64, 0, 0), k0 > 0);
        umma_commit(&bar_A);
      };
      // The gradient products in two groups.  The first needs neither A nor dA, so it starts as soon as
      // the chunk's tiles have landed, while the conversion warps still work on A and dA; after it dh'
      // and v are dead and the next chunk's are fetched.  The second group needs the converted operands.
      auto issue_inter = [&](int it) {
        const uint32_t kta = smem_u32(ks + (it & 1) * TILE64);
#pragma unroll
        for (int k0 = 0; k0 < D; k0 += 16)   // dq_inter^T[k][i] = h' do^T
          umma_bf16(tm + cdq, desc_kmajor(ha, 128, 0, k0), desc_kmajor(doa, 64, 0, k0), umma_idesc(128, 64, 0, 0), k0 > 0);
#pragma unroll
        for (int k0 = 0; k0 < D; k0 += 16)   // (dk_inter exp(G - mid))^T[k][j] = dh' v^T
          umma_bf16(tm + cdk2, desc_kmajor(dha, 128, 0, k0), desc_kmajor(va, 64, 0, k0), umma_idesc(128, 64, 0, 0), k0 > 0);
#pragma unroll
        for (int k0 = 0; k0 < D; k0 += 16)   // dv^T[v][j] = dh'^T k~^T
          umma_bf16(tm + cdv, desc_mnmajor(dha, 128, k0, 0), desc_kmajor(kta, 64, 0, k0), umma_idesc(128, 64, 1, 0), k0 > 0);
        umma_commit(&bar_r2);
      };
      auto issue_intra = [&](int it) {
        const uint32_t qta = smem_u32(qs + (it & 1) * TILE64), kta = smem_u32(ks + (it & 1) * TILE64);
#pragma unroll
        for (int k0 = 0; k0 < C; k0 += 16)   // dv^T[v][j] += sum_i do[i][v] A[i][j]
          umma_bf16(tm + cdv, desc_mnmajor(doa, 64, k0, 0), desc_mnmajor(pa, 64, k0, 0), umma_idesc(128, 64, 1, 1), 1);
        umma_commit(&bar_r1);                // h' and do are dead
#pragma unroll
        for (int k0 = 0; k0 < C; k0 += 16)   // dq^T[k][i] += sum_j k~[j][k] dA[i][j]
          umma_bf16(tm + cdq, desc_mnmajor(kta, 64, k0, 0), desc_kmajor(daa, 64, 0, k0), umma_idesc(128, 64, 1, 0), 1);
#pragma unroll
        for (int k0 = 0; k0 < C; k0 += 16)   // dk_intra^T[k][j] = sum_i q~[i][k] dA[i][j]
          umma_bf16(tm + cdk1, desc_mnmajor(qta, 64, k0, 0), desc_mnmajor(daa, 64, k0, 0), umma_idesc(128, 64, 1, 1), k0 > 0);
        umma_commit(&bar_main);
      };
      bool ok = SCALAR || wait(&full_g, 0, 6);
      if (ok) {
        tc_fence_after();
        if (!SCALAR) issue_gate(0);
        ok = wait(&gated, 0, 12);
      }
      if (ok) {
        tc_fence_after();
        issue_A(0);
        ok = wait(&full_hdo, 0, 6) && wait(&full_dhv, 0, 6);
      }
      if (ok) issue_dA();
      for (int it = 0; ok && it < nit; ++it) {
        // A and dA of this chunk are issued; the previous chunk has left tensor memory
        if (it >= 1 && !wait(&e_done[(it - 1) & 1], ((it - 1) >> 1) & 1, 14)) break;
        tc_fence_after();
        issue_inter(it);
        if (!wait(&conv_done, it & 1, 13)) break;   // A and dA of this chunk are in shared memory
        tc_fence_after();
        const bool more = it + 1 < nit;
        if (more && !SCALAR) {   // the next chunk's exponents take the place of A and dA in tensor memory
          if (!wait(&full_g, (it + 1) & 1, 6)) break;
          issue_gate(it + 1);
        }
        issue_intra(it);
        if (more) {
          if (!wait(&gated, (it + 1) & 1, 12)) break;
          tc_fence_after();
          issue_A(it + 1);
          if (!wait(&full_hdo, (it + 1) & 1, 6) || !wait(&full_dhv, (it + 1) & 1, 6)) break;
          issue_dA();
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ TMA loads
    if (lane == 0) {
      auto load_g = [&](int it) {
        int h, row, hrow;
        chunk_rows(it, h, row, hrow);
        mbar_expect_tx(&full_g, TILE64);
        tma_load_3d(gs, &p.mg, &full_g, 0, h, row); tma_load_3d(gs + SLAB64, &p.mg, &full_g, 64, h, row);
      };
      auto load_qk = [&](int it) {
        int h, row, hrow;
        chunk_rows(it, h, row, hrow);
        uint64_t* bar = &full_qk[it & 1];
        uint8_t* qd = qs + (it & 1) * TILE64;
        uint8_t* kd = ks + (it & 1) * TILE64;
        mbar_expect_tx(bar, 2 * TILE64);
        tma_load_3d(qd, &p.mq, bar, 0, h, row); tma_load_3d(qd + SLAB64, &p.mq, bar, 64, h, row);
        tma_load_3d(kd, &p.mk, bar, 0, h, row); tma_load_3d(kd + SLAB64, &p.mk, bar, 64, h, row);
      };
      auto load_hdo = [&](int it) {
        int h, row, hrow;
        chunk_rows(it, h, row, hrow);
        mbar_expect_tx(&full_hdo, TILE128 + TILE64);
        tma_load_3d(dos, &p.mdo, &full_hdo, 0, h, row); tma_load_3d(dos + SLAB64, &p.mdo, &full_hdo, 64, h, row);
        tma_load_2d(hs, &p.mh, &full_hdo, 0, hrow); tma_load_2d(hs + TILE128 / 2, &p.mh, &full_hdo, 64, hrow);
      };
      auto load_dhv = [&](int it) {
        int h, row, hrow;
        chunk_rows(it, h, row, hrow);
        mbar_expect_tx(&full_dhv, TILE128 + TILE64);
        tma_load_3d(vs, &p.mv, &full_dhv, 0, h, row); tma_load_3d(vs + SLAB64, &p.mv, &full_dhv, 64, h, row);
        tma_load_2d(dhs, &p.mdh, &full_dhv, 0, hrow); tma_load_2d(dhs + TILE128 / 2, &p.mdh, &full_dhv, 64, hrow);
      };
      if (!SCALAR) load_g(0);
      load_qk(0);
      load_hdo(0);
      load_dhv(0);
      bool ok = true;
      if (nit > 1) {
        load_qk(1);
        if (!SCALAR) {
          ok = wait(&bar_gate, 0, 9);   // the exponent products of chunk 0 have read its gates
          if (ok) load_g(1);
        }
      }
      for (int it = 0; ok && it + 1 < nit; ++it) {
        // dh' and v are dead after the first group of products (and the h' dh' reduction), h' and do
        // after the first product of the second group
        if (!wait(&bar_r2, it & 1, 8) || !wait(&hdh_done[it & 1], (it >> 1) & 1, 11)) break;
        load_dhv(it + 1);
        if (!wait(&bar_r1, it & 1, 8)) break;
        load_hdo(it + 1);
        if (it + 2 < nit) {
          if (!wait(&e_done[it & 1], (it >> 1) & 1, 14)) break;
          load_qk(it + 2);
          if (!SCALAR) {
            if (!wait(&bar_gate, (it + 1) & 1, 9)) break;
            load_g(it + 2);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 512);
  if (tid == 0 && abort_flag && nit > 0) {
    int h, row, hrow;
    chunk_rows(0, h, row, hrow);
    poison(reinterpret_cast<TG*>(p.dq) + ((size_t)row * p.H + h) * D);
    poison(p.dv + ((size_t)row * p.H + h) * D);
  }
}

// ===========================================================================
// host side
// ===========================================================================
constexpr size_t SCAN_SMEM = 9 * TILE64 + 2 * SLAB64 + 2 * TILE128 + sizeof(ScanShared);
constexpr size_t FWD_O_SMEM = 4 * TILE64 + TILE128 + SLAB64 + 1024;
constexpr size_t BWD_SMEM = 7 * TILE64 + 2 * TILE128 + 2 * SLAB64 + 2 * SLAB64 + 1024;

// from this many (batch, head) pairs on, the forward runs as one fused pass (one block per pair)
// instead of a state scan followed by a chunk-parallel output kernel
constexpr int kFusedMinBlocks = 48;

std::atomic<int> g_test_skip_load{-1};

// One launch of the scan kernel over `nseg` time segments per (batch, head).  states == nullptr keeps
// no chunk-start states (a summary pass: end states and summed gates only).
int run_scan(bool bwd, const tops_chunk_problem& pb, int nseg, const void* x, const void* g, const void* y,
             const float* s0, void* states, float* s_final, float* gsum, cudaStream_t st) {
  ScanParams sp;
  const int BT = pb.B * pb.T;
  const bool scalar = pb.gate_kind == TOPS_GATE_SCALAR;
  int rc;
  if ((rc = act_map(&sp.mx, x, BT, pb.H)) || (rc = act_map(&sp.my, y, BT, pb.H))) return rc;
  if (!scalar && (rc = act_map(&sp.mg, g, BT, pb.H))) return rc;
  sp.gscalar = reinterpret_cast<const __nv_bfloat16*>(g);
  if (states && (rc = state_map(&sp.mst, states, (size_t)pb.B * (pb.T / C) * pb.H * D))) return rc;
  sp.s0 = s0; sp.states = reinterpret_cast<__nv_bfloat16*>(states); sp.s_final = s_final; sp.gsum = gsum;
  sp.T = pb.T; sp.H = pb.H; sp.NT = pb.T / C / nseg; sp.nseg = nseg; sp.scale = pb.scale;
  sp.skip_xy = g_test_skip_load.exchange(-1);   // one launch only
  dim3 grid(pb.B * pb.H * nseg);
  auto launch = [&](auto kernel, const char* label) {
    if ((rc = opt_in_smem(kernel, SCAN_SMEM))) return rc;
    KernelScope ks(label, st);
    kernel<<<grid, SCAN_THREADS, SCAN_SMEM, st>>>(sp);
    return post_launch();
  };
  // no chunk-start states and a zero start: the summary form of the kernel
  const bool sum = !states && !s0;
  if (bwd) {
    const char* label = states ? "sm100_bwd_dh" : "sm100_bwd_dh_summary";
    if (sum) return scalar ? launch(k_scan<true, true, true>, label) : launch(k_scan<true, false, true>, label);
    return scalar ? launch(k_scan<true, true, false>, label) : launch(k_scan<true, false, false>, label);
  }
  const char* label = states ? "sm100_fwd_h" : "sm100_fwd_h_summary";
  if (sum) return scalar ? launch(k_scan<false, true, true>, label) : launch(k_scan<false, false, true>, label);
  return scalar ? launch(k_scan<false, true, false>, label) : launch(k_scan<false, false, false>, label);
}

// Time segments per sequence.  The scans walk a sequence chunk by chunk with one block; when there are
// too few (batch, head) pairs to fill the GPU, each sequence is cut into segments that run as blocks of
// their own: a first pass finds what every segment does to the state entering it (end state from a zero
// start and summed gates), a small kernel chains the segments, and the real pass starts every segment
// from its true state.  At least four chunks per segment.
int pick_segments(const tops_chunk_problem& pb) {
  const int bh = pb.B * pb.H, nt = pb.T / C;
  if (2 * bh > sm_count()) return 1;
  int best = 1;
  for (int n = 2; n * bh <= sm_count() && n * 4 <= nt; ++n)
    if (nt % n == 0) best = n;
  return best;
}
// fp32 scratch of a segmented scan: end states, entry states (nseg x [B,H,K,V] each) and summed gates
size_t segment_floats(const tops_chunk_problem& pb, int nseg) {
  return nseg > 1 ? (size_t)pb.B * pb.H * nseg * (2 * D * D + D) : 0;
}
struct SegmentScratch {
  float *ends, *starts, *gsum;
  SegmentScratch(float* base, const tops_chunk_problem& pb, int nseg) {
    const size_t n = (size_t)pb.B * pb.H * nseg * D * D;
    ends = base; starts = base + n; gsum = base + 2 * n;
  }
};
// summary pass + join: leaves the state entering every segment in sc.starts and the state after the last
// (forward) / before the first (reverse) segment in `last` (may be null)
// With `have_summary` the scratch already holds the segments' end states and summed gates (a shard summary
// made by state_summary() for the same problem) and only the join runs.
int segment_starts(bool bwd, const tops_chunk_problem& pb, int nseg, const void* x, const void* g, const void* y,
                   const float* first, float* last, const SegmentScratch& sc, cudaStream_t st, bool have_summary = false) {
  int rc = have_summary ? TOPS_OK : run_scan(bwd, pb, nseg, x, g, y, nullptr, nullptr, sc.ends, sc.gsum, st);
  if (rc) return rc;
  KernelScope ks("sm100_join_segments", st);
  const dim3 grid(pb.B * pb.H, 16);   // 16 slices of 1024 elements: 256 threads x float4
  if (bwd) k_join_segments<true><<<grid, 256, 0, st>>>(first, sc.gsum, sc.ends, sc.starts, last, nseg);
  else k_join_segments<false><<<grid, 256, 0, st>>>(first, sc.gsum, sc.ends, sc.starts, last, nseg);
  return post_launch();
}

}  // namespace

bool supported(const tops_chunk_problem& pb) {
  if (pb.dtype != TOPS_BF16 || pb.gate_dtype != TOPS_BF16) return false;
  if (pb.gate_kind != TOPS_GATE_PER_CHANNEL && pb.gate_kind != TOPS_GATE_SCALAR) return false;
  if (pb.K != D || pb.V != D || pb.chunk != C || pb.T % C != 0 || pb.cu_seqlens) return false;
  if (!(pb.scale > 0.f) || !(pb.scale < 1e30f)) return false;   // states are stored multiplied by scale
  if ((size_t)pb.B * pb.T >= (1u << 31)) return false;
  return device_is_sm100() && encode_fn() != nullptr;
}

static size_t state_bytes(const tops_chunk_problem& pb) {
  return align_up((size_t)pb.B * (pb.T / C) * pb.H * D * D * 2);
}

// The fused one-pass forward keeps the chunk-start states on chip: only the two-kernel form (too few
// blocks for one per (batch, head, segment)) needs them in scratch, and only when the caller does not
// keep them itself.
static bool fwd_is_fused(const tops_chunk_problem& pb, int nseg) { return pb.B * pb.H * nseg >= kFusedMinBlocks; }

size_t fwd_workspace_bytes(const tops_chunk_fwd_params& p) {
  const int nseg = pick_segments(p.pb);
  const bool states_in_ws = !p.saved_out && !fwd_is_fused(p.pb, nseg);
  return (states_in_ws ? state_bytes(p.pb) : 0) + segment_floats(p.pb, nseg) * sizeof(float) + 256;
}

int chunk_fwd(const tops_chunk_fwd_params& p, void* ws, size_t, cudaStream_t st) {
  const tops_chunk_problem& pb = p.pb;
  if (p.g_cumsum_out || p.A_out || p.h_out) return TOPS_E_UNSUPPORTED;
  if (!aligned16(p.q) || !aligned16(p.k) || !aligned16(p.v) || !aligned16(p.g) || !aligned16(p.o) ||
      !aligned16(p.h0) || !aligned16(p.ht) || !aligned16(p.saved_out) || !aligned16(ws))
    return TOPS_E_ALIGN;
  const int BT = pb.B * pb.T, NT = pb.T / C;
  const int nseg = pick_segments(pb);
  const bool scalar = pb.gate_kind == TOPS_GATE_SCALAR;
  // workspace: [chunk-start states unless the caller keeps them] [segment scratch]
  char* wsp = reinterpret_cast<char*>(ws);
  void* h = p.saved_out ? p.saved_out : wsp;
  const bool fused = fwd_is_fused(pb, nseg);
  if (!aligned16(p.segments)) return TOPS_E_ALIGN;
  const SegmentScratch sc(p.segments ? reinterpret_cast<float*>(p.segments)
                                     : reinterpret_cast<float*>(wsp + ((p.saved_out || fused) ? 0 : state_bytes(pb))),
                          pb, nseg);
  int rc;
  const float* start = p.h0;
  float* last = p.ht;
  if (nseg > 1) {
    if ((rc = segment_starts(false, pb, nseg, p.k, p.g, p.v, p.h0, p.ht, sc, st, p.segments != nullptr))) return rc;
    start = sc.starts;
    last = nullptr;   // the join kernel has written the final state
  }
  if (fused) {
    // enough blocks to fill the GPU with one per (batch, head, segment): one pass over q, k, g, v
    FusedParams up;
    if ((rc = act_map(&up.mq, p.q, BT, pb.H)) || (rc = act_map(&up.mk, p.k, BT, pb.H)) ||
        (rc = act_map(&up.mv, p.v, BT, pb.H)))
      return rc;
    if (!scalar && (rc = act_map(&up.mg, p.g, BT, pb.H))) return rc;
    up.gscalar = reinterpret_cast<const __nv_bfloat16*>(p.g);
    up.states = nullptr;
    if (p.saved_out) {   // only a caller that keeps the states for its backward pass needs them in HBM
      if ((rc = state_map(&up.mst, p.saved_out, (size_t)pb.B * NT * pb.H * D))) return rc;
      up.states = reinterpret_cast<__nv_bfloat16*>(p.saved_out);
    }
    up.s0 = start; up.s_final = last; up.o = reinterpret_cast<__nv_bfloat16*>(p.o);
    up.T = pb.T; up.H = pb.H; up.NT = NT / nseg; up.nseg = nseg; up.scale = pb.scale;
    if ((rc = opt_in_smem(k_fwd_fused<true>, FUSED_SMEM)) || (rc = opt_in_smem(k_fwd_fused<false>, FUSED_SMEM))) return rc;
    KernelScope ks("sm100_fwd_fused", st);
    if (scalar) k_fwd_fused<true><<<pb.B * pb.H * nseg, FUSED_THREADS, FUSED_SMEM, st>>>(up);
    else k_fwd_fused<false><<<pb.B * pb.H * nseg, FUSED_THREADS, FUSED_SMEM, st>>>(up);
    return post_launch();
  }
  rc = run_scan(false, pb, nseg, p.k, p.g, p.v, start, h, last, nullptr, st);
  if (rc) return rc;
  FwdOParams fp;
  if ((rc = act_map(&fp.mq, p.q, BT, pb.H)) || (rc = act_map(&fp.mk, p.k, BT, pb.H)) ||
      (rc = act_map(&fp.mv, p.v, BT, pb.H)) || (rc = state_map(&fp.mh, h, (size_t)pb.B * NT * pb.H * D)))
    return rc;
  if (!scalar && (rc = act_map(&fp.mg, p.g, BT, pb.H))) return rc;
  fp.gscalar = reinterpret_cast<const __nv_bfloat16*>(p.g);
  fp.o = reinterpret_cast<__nv_bfloat16*>(p.o); fp.T = pb.T; fp.H = pb.H; fp.NT = NT; fp.scale = pb.scale;
  if ((rc = opt_in_smem(k_fwd_o<true>, FWD_O_SMEM)) || (rc = opt_in_smem(k_fwd_o<false>, FWD_O_SMEM))) return rc;
  KernelScope ks("sm100_fwd_o", st);
  if (scalar) k_fwd_o<true><<<dim3(pb.H, NT, pb.B), NTHREADS, FWD_O_SMEM, st>>>(fp);
  else k_fwd_o<false><<<dim3(pb.H, NT, pb.B), NTHREADS, FWD_O_SMEM, st>>>(fp);
  return post_launch();
}

size_t bwd_workspace_bytes(const tops_chunk_bwd_params& p) {
  return (p.h_saved ? 1 : 2) * state_bytes(p.pb) + segment_floats(p.pb, pick_segments(p.pb)) * sizeof(float) + 256;
}

bool bwd_dtypes_ok(const tops_chunk_bwd_params& p) {
  if (p.pb.gate_kind == TOPS_GATE_SCALAR)   // dg is the scalar gate's gradient, fp32 [B,T,H]
    return (p.grad_dtype == TOPS_F32 || p.grad_dtype == TOPS_BF16) && p.dg_dtype == TOPS_F32;
  return (p.grad_dtype == TOPS_F32 && p.dg_dtype == TOPS_F32) ||
         (p.grad_dtype == TOPS_BF16 && (p.dg_dtype == TOPS_F32 || p.dg_dtype == TOPS_BF16));
}

template <typename TG, typename TD, bool SCALAR = false>
int launch_bwd_main(const BwdParams& bp, cudaStream_t st) {
  int rc = opt_in_smem(k_bwd_main<TG, TD, SCALAR>, BWD_SMEM);
  if (rc) return rc;
  const int grid = bp.total < sm_count() ? bp.total : sm_count();
  KernelScope ks("sm100_bwd_main", st);
  k_bwd_main<TG, TD, SCALAR><<<grid, BWD_THREADS, BWD_SMEM, st>>>(bp);
  return post_launch();
}

int chunk_bwd(const tops_chunk_bwd_params& p, void* ws, size_t, cudaStream_t st) {
  const tops_chunk_problem& pb = p.pb;
  if (!bwd_dtypes_ok(p)) return TOPS_E_UNSUPPORTED;
  if (!aligned16(p.q) || !aligned16(p.k) || !aligned16(p.v) || !aligned16(p.g) || !aligned16(p.do_) ||
      !aligned16(p.h0) || !aligned16(p.dht) || !aligned16(p.dh0) || !aligned16(p.dq) || !aligned16(p.dk) ||
      !aligned16(p.dv) || !aligned16(p.dg) || !aligned16(p.h_saved) || !aligned16(p.rev_segments) || !aligned16(ws))
    return TOPS_E_ALIGN;
  // workspace: [dh'] [h' unless the forward kept it] [segment scratch]
  const int nseg = pick_segments(pb);
  const char* h = reinterpret_cast<const char*>(p.h_saved);
  char* dh = reinterpret_cast<char*>(ws);
  const SegmentScratch sc(reinterpret_cast<float*>(dh + (h ? 1 : 2) * state_bytes(pb)), pb, nseg);
  int rc = TOPS_OK;
  if (!h) {
    char* hw = dh + state_bytes(pb);
    const float* start = p.h0;
    if (nseg > 1) {
      if ((rc = segment_starts(false, pb, nseg, p.k, p.g, p.v, p.h0, nullptr, sc, st))) return rc;
      start = sc.starts;
    }
    if ((rc = run_scan(false, pb, nseg, p.k, p.g, p.v, start, hw, nullptr, nullptr, st))) return rc;
    h = hw;
  }
  {
    const float* start = p.dht;
    float* last = p.dh0;
    if (nseg > 1) {
      const SegmentScratch rsc(p.rev_segments ? reinterpret_cast<float*>(p.rev_segments) : sc.ends, pb, nseg);
      if ((rc = segment_starts(true, pb, nseg, p.q, p.g, p.do_, p.dht, p.dh0, rsc, st, p.rev_segments != nullptr))) return rc;
      start = rsc.starts;
      last = nullptr;   // the join kernel has written dh0
    }
    if ((rc = run_scan(true, pb, nseg, p.q, p.g, p.do_, start, dh, last, nullptr, st))) return rc;
  }
  BwdParams bp;
  const int BT = pb.B * pb.T, NT = pb.T / C;
  const size_t rows = (size_t)pb.B * NT * pb.H * D;
  const bool scalar = pb.gate_kind == TOPS_GATE_SCALAR;
  if ((rc = act_map(&bp.mq, p.q, BT, pb.H)) || (rc = act_map(&bp.mk, p.k, BT, pb.H)) ||
      (rc = act_map(&bp.mv, p.v, BT, pb.H)) ||
      (rc = act_map(&bp.mdo, p.do_, BT, pb.H)) || (rc = state_map(&bp.mh, h, rows)) ||
      (rc = state_map(&bp.mdh, dh, rows)))
    return rc;
  if (!scalar && (rc = act_map(&bp.mg, p.g, BT, pb.H))) return rc;
  bp.gscalar = reinterpret_cast<const __nv_bfloat16*>(p.g);
  bp.dq = p.dq; bp.dk = p.dk; bp.dg = p.dg;
  bp.dv = reinterpret_cast<__nv_bfloat16*>(p.dv); bp.T = pb.T; bp.H = pb.H; bp.NT = NT; bp.scale = pb.scale;
  bp.total = NT * pb.B * pb.H;
  if (scalar)
    return p.grad_dtype == TOPS_F32 ? launch_bwd_main<float, float, true>(bp, st)
                                    : launch_bwd_main<__nv_bfloat16, float, true>(bp, st);
  if (p.grad_dtype == TOPS_F32) return launch_bwd_main<float, float>(bp, st);
  if (p.dg_dtype == TOPS_F32) return launch_bwd_main<__nv_bfloat16, float>(bp, st);
  return launch_bwd_main<__nv_bfloat16, __nv_bfloat16>(bp, st);
}

// The summary of one time shard for the state exchange between ranks: the state after the shard from a
// zero start (forward: x = k, y = v) or the state gradient before the shard for a zero gradient after it
// (reverse: x = q, y = do).  Uses the time-segmented summary scan when there are few (batch, head) pairs.
size_t summary_workspace_bytes(const tops_chunk_problem& pb) {
  return segment_floats(pb, pick_segments(pb)) * sizeof(float) + 256;
}

int state_summary(const tops_chunk_problem& pb, bool reverse, const void* x, const void* g, const void* y,
                  float* state_out, void* ws, cudaStream_t st) {
  if (!aligned16(x) || !aligned16(g) || !aligned16(y) || !aligned16(state_out) || !aligned16(ws)) return TOPS_E_ALIGN;
  const int nseg = pick_segments(pb);
  if (nseg == 1) return run_scan(reverse, pb, 1, x, g, y, nullptr, nullptr, state_out, nullptr, st);
  const SegmentScratch sc(reinterpret_cast<float*>(ws), pb, nseg);
  return segment_starts(reverse, pb, nseg, x, g, y, nullptr, state_out, sc, st);
}

int device_error(int* out) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_error, sizeof(int)) != cudaSuccess) return TOPS_E_CUDA;
  *out = v;
  return TOPS_OK;
}

void test_skip_load(int chunk) { g_test_skip_load.store(chunk); }

int device_error_set(int code) {
  return cudaMemcpyToSymbol(g_error, &code, sizeof(int)) == cudaSuccess ? TOPS_OK : TOPS_E_CUDA;
}

}  // namespace sm100
}  // namespace tops
