// Device-side pieces shared by the tcgen05 kernel files: tile sizes, the constant patterns that turn a
// gate tile into cumulative-gate exponents with one tensor-core product, small packing helpers, and the
// per-file error word of the bounded waits.
#pragma once
#include "sm100_prims.cuh"

namespace tops {
namespace sm100 {

// First bounded wait that gave up in a kernel of this translation unit (0 = none).
static __device__ int g_error;

namespace {

constexpr int C = 64;    // chunk
constexpr int D = 128;   // K = V
constexpr int NTHREADS = 512;
constexpr int SEG = 16;  // time steps per thread
constexpr uint32_t SLAB64 = 64 * 128;        // bytes of a 64-row slab
constexpr uint32_t TILE64 = 2 * SLAB64;      // 64 x 128 bf16 tile
constexpr uint32_t TILE128 = 2 * 128 * 128;  // 128 x 128 bf16 tile

__device__ __forceinline__ uint8_t* align1024(uint8_t* p) {
  return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~static_cast<uintptr_t>(1023));
}
__device__ __forceinline__ float ld_bf16(const uint8_t* tile, uint32_t off) {
  return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(tile + off));
}
// offset of (row i, this thread's column) in a 64-row tile
struct ColAddr {
  uint32_t base, cchunk;
  __device__ __forceinline__ uint32_t at(int i) const {
    return base + (uint32_t)i * 128u + (((cchunk ^ (uint32_t)i) & 7u) << 4);
  }
};
__device__ __forceinline__ ColAddr col_prep(int rows, int col) {
  return ColAddr{(uint32_t)((col >> 6) * rows * 128 + (col & 7) * 2), (uint32_t)((col & 63) >> 3)};
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ void fail(int code) { atomicCAS(&g_error, 0, code); }
// A block that gave up marks one element of every output it owns with NaN, so that a caller who
// never reads the error word sees a poisoned result rather than whatever the buffer held before.
__device__ __forceinline__ void poison(float* p) { if (p) *p = __int_as_float(0x7fc00000); }
__device__ __forceinline__ void poison(__nv_bfloat16* p) { if (p) *reinterpret_cast<unsigned short*>(p) = 0x7fc0; }

// Constant 64 x 64 patterns, stored as K-major bf16 tiles, that turn the gate
// tile g [time j][channel] into exponents with one tensor-core product:
//   TRI_INCL  L[i][j] = (j <= i)                 -> G_i           (inclusive cumulative gate)
//   TRI_REV   U[i][j] = (j > i)                  -> G_n - G_i
//   TRI_REVN  TRI_REV with row 63 all ones       -> G_n - G_i for i < 63 and G_n itself in row 63 (whose own
//             exponent, 0, needs no product)
//   TRI_MID   L - 1/2 [j == 0] - 1/2             -> G_i - (G_0 + G_n) / 2
// All entries (0, 1, +-1/2) are exact in bf16 and the products accumulate in fp32.
enum { TRI_INCL = 0, TRI_REV = 1, TRI_MID = 2, TRI_REVN = 3 };
__device__ __forceinline__ float tri_value(int kind, int i, int j) {
  if (kind == TRI_INCL) return j <= i ? 1.f : 0.f;
  if (kind == TRI_REV) return j > i ? 1.f : 0.f;
  if (kind == TRI_REVN) return (i == 63 || j > i) ? 1.f : 0.f;
  return j == 0 ? 0.f : (j <= i ? 0.5f : -0.5f);
}
__device__ __forceinline__ void build_tri_tile(uint8_t* tile, int rows, int kind) {
  for (int idx = threadIdx.x; idx < rows * 8; idx += blockDim.x) {
    const int r = idx >> 3, c8 = (idx & 7) * 8, i = r & 63;
    uint32_t w[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) w[t] = pack_bf16(tri_value(kind, i, c8 + 2 * t), tri_value(kind, i, c8 + 2 * t + 1));
    *reinterpret_cast<uint4*>(tile + slab_off(r, c8)) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}
// Scalar gates (one log-gate per head and time step): the exponents of a chunk are 64 numbers, not a tile, so no
// tensor-core product and no gate tile are needed.  Every warp keeps the chunk's 64 log-gates in registers
// (lane l: time steps l and l + 32) and turns them into inclusive cumulative gates with shuffles.
struct WarpGates {
  float lo, hi;   // G of time steps lane and lane + 32
  float g0, gn;   // G_0 (the first gate) and G_63 (the chunk's summed gates)
  __device__ __forceinline__ float mid() const { return 0.5f * (g0 + gn); }
};
__device__ __forceinline__ WarpGates warp_cumulate(float a, float b, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float x = __shfl_up_sync(0xffffffffu, a, o), y = __shfl_up_sync(0xffffffffu, b, o);
    if (lane >= o) { a += x; b += y; }
  }
  b += __shfl_sync(0xffffffffu, a, 31);
  WarpGates w;
  w.lo = a; w.hi = b;
  w.g0 = __shfl_sync(0xffffffffu, a, 0);
  w.gn = __shfl_sync(0xffffffffu, b, 31);
  return w;
}
// The scalar gates of the chunks a warp will gate next.  They are fetched three chunks ahead with cp.async into a
// small ring in shared memory that belongs to the warp (4 slots x 64 words; lane l owns the words of time steps l
// and l + 32), never into registers: a register that a load in flight will write, carried around the chunk loop,
// makes the warp wait for the load at the loop's back edge (measured: ~1000 cycles per chunk in every kernel that
// did so).  The gates are bf16, cp.async moves 4-byte words: a lane copies the aligned word that holds its gate
// and picks the half when it takes it.  One group is committed per chunk index, fetched or not, so that
// `wait_group 2` at chunk c always means "chunk c has landed".
struct GateRing {
  static constexpr int kBytesPerWarp = 4 * 64 * 4;
  uint32_t base = 0;
  __device__ __forceinline__ void init(uint8_t* warp_area) { base = smem_u32(warp_area); }
  // idx: element index of the gate of time step `lane` of chunk c in the [B,T,H] tensor; hi_off: elements to
  // time step lane + 32 (an even number)
  __device__ __forceinline__ void prefetch(const __nv_bfloat16* g, bool valid, size_t idx, size_t hi_off, int c, int lane) {
    if (valid) {
      const uint32_t* w = reinterpret_cast<const uint32_t*>(g);
      const uint32_t dst = base + (uint32_t)(((c & 3) * 64 + lane) * 4);
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(w + (idx >> 1)) : "memory");
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 128u), "l"(w + ((idx + hi_off) >> 1)) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  __device__ __forceinline__ void take(size_t idx, int c, int lane, float& lo, float& hi) {
    asm volatile("cp.async.wait_group 2;" ::: "memory");
    const uint32_t src = base + (uint32_t)(((c & 3) * 64 + lane) * 4);
    uint32_t a, b;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(a) : "r"(src));
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(b) : "r"(src + 128u));
    const bool upper = (idx & 1) != 0;
    lo = __uint_as_float(upper ? (a & 0xffff0000u) : (a << 16));
    hi = __uint_as_float(upper ? (b & 0xffff0000u) : (b << 16));
  }
};

// Sums 16 values per thread over the 32 lanes of a warp with 16 shuffles (a butterfly that halves the number of
// live values at every step): on return lane l holds the warp's total of v[l & 15].
__device__ __forceinline__ float warp_sum16(float (&v)[16], int lane) {
#pragma unroll
  for (int s = 8; s >= 1; s >>= 1) {
    const bool up = (lane & s) != 0;
#pragma unroll
    for (int i = 0; i < s; ++i) {
      const float send = up ? v[i] : v[i + s];
      const float keep = up ? v[i + s] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, s);
    }
  }
  return v[0] + __shfl_xor_sync(0xffffffffu, v[0], 16);
}
// multiply 8 packed bf16 by one fp32 factor
__device__ __forceinline__ uint4 scale8_by(uint4 x, float f) {
  __nv_bfloat162* px = reinterpret_cast<__nv_bfloat162*>(&x);
  uint4 y;
  uint32_t* py = reinterpret_cast<uint32_t*>(&y);
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const float2 v = __bfloat1622float2(px[t]);
    py[t] = pack_bf16(v.x * f, v.y * f);
  }
  return y;
}

// multiply 8 packed bf16 by 8 fp32 factors
__device__ __forceinline__ uint4 scale8(uint4 x, const float* f) {
  __nv_bfloat162* px = reinterpret_cast<__nv_bfloat162*>(&x);
  uint4 y;
  uint32_t* py = reinterpret_cast<uint32_t*>(&y);
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const float2 v = __bfloat1622float2(px[t]);
    py[t] = pack_bf16(v.x * f[2 * t], v.y * f[2 * t + 1]);
  }
  return y;
}

// masked, scaled bf16 copy of 16 columns [16 seg, 16 seg + 16) of row i of a
// 64 x 64 fp32 accumulator into a K-major 64 x 64 tile
__device__ __forceinline__ void store_tril16(uint8_t* dst, int i, int j0, const float (&a)[16], float scale) {
#pragma unroll
  for (int c8 = 0; c8 < 16; c8 += 8) {
    uint32_t w[4];
#pragma unroll
    for (int t = 0; t < 8; t += 2) {
      const int j = j0 + c8 + t;
      w[t >> 1] = pack_bf16(j <= i ? a[c8 + t] * scale : 0.f, j + 1 <= i ? a[c8 + t + 1] * scale : 0.f);
    }
    *reinterpret_cast<uint4*>(dst + slab_off(i, j0 + c8)) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// 16 x 64 K-major pattern: row 0 sums the gates (G_n), row 1 gives G_n - mid = (G_n - G_0) / 2
__device__ __forceinline__ void build_w_tile(uint8_t* tile) {
  for (int idx = threadIdx.x; idx < 16 * 8; idx += blockDim.x) {
    const int r = idx >> 3, c8 = (idx & 7) * 8;
    uint32_t w[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int j = c8 + 2 * t;
      const float a = r == 0 ? 1.f : (r == 1 ? (j == 0 ? 0.f : 0.5f) : 0.f);
      const float b = r == 0 ? 1.f : (r == 1 ? 0.5f : 0.f);
      w[t] = pack_bf16(a, b);
    }
    *reinterpret_cast<uint4*>(tile + slab_off(r, c8)) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}


// 4 x 4 transpose over the lanes l, l^1, l^2, l^3.  In: v[j] = value of this lane's channel at
// time t0 + j.  Out: v[j] = value of channel (lane & ~3) + j at time t0 + (lane & 3), so that a
// thread can store four neighbouring channels of one time step with one instruction.
__device__ __forceinline__ void transpose4(float (&v)[4], int lane) {
  const bool odd = lane & 1, hi = lane & 2;
  const float r0 = __shfl_xor_sync(0xffffffffu, odd ? v[0] : v[1], 1);
  const float r1 = __shfl_xor_sync(0xffffffffu, odd ? v[2] : v[3], 1);
  const float a0 = odd ? r0 : v[0], a1 = odd ? v[1] : r0;   // time t0 + odd:     channels 2m, 2m + 1
  const float b0 = odd ? r1 : v[2], b1 = odd ? v[3] : r1;   // time t0 + 2 + odd: channels 2m, 2m + 1
  const float u0 = __shfl_xor_sync(0xffffffffu, hi ? a0 : b0, 2);
  const float u1 = __shfl_xor_sync(0xffffffffu, hi ? a1 : b1, 2);
  v[0] = hi ? u0 : a0; v[1] = hi ? u1 : a1; v[2] = hi ? b0 : u0; v[3] = hi ? b1 : u1;
}
// The same exchange followed by a store of the four neighbouring channels of time step
// t0 + (lane & 3) at p[i]; the bf16 form rounds after the first stage and moves packed pairs.
__device__ __forceinline__ void st_transposed4(float* p, size_t i, float (&v)[4], int lane) {
  transpose4(v, lane);
  __stcs(reinterpret_cast<float4*>(p + i), make_float4(v[0], v[1], v[2], v[3]));
}
__device__ __forceinline__ void st_transposed4(__nv_bfloat16* p, size_t i, const float (&v)[4], int lane) {
  const bool odd = lane & 1, hi = lane & 2;
  const float r0 = __shfl_xor_sync(0xffffffffu, odd ? v[0] : v[1], 1);
  const float r1 = __shfl_xor_sync(0xffffffffu, odd ? v[2] : v[3], 1);
  const uint32_t pa = odd ? pack_bf16(r0, v[1]) : pack_bf16(v[0], r0);
  const uint32_t pb = odd ? pack_bf16(r1, v[3]) : pack_bf16(v[2], r1);
  const uint32_t u = __shfl_xor_sync(0xffffffffu, hi ? pa : pb, 2);
  __stcs(reinterpret_cast<uint2*>(p + i), hi ? make_uint2(u, pb) : make_uint2(pa, u));
}
// gradients are written once and not read again by these kernels: streaming stores
__device__ __forceinline__ void st_out(float* p, size_t i, float x) { __stcs(p + i, x); }
__device__ __forceinline__ void st_out(__nv_bfloat16* p, size_t i, float x) {
  __stcs(reinterpret_cast<unsigned short*>(p) + i, __bfloat16_as_ushort(__float2bfloat16_rn(x)));
}

}  // namespace
}  // namespace sm100
}  // namespace tops
