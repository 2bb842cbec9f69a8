// Host-side helpers shared by the tcgen05 kernel files: the driver entry point for tensor maps, cached
// tensor maps of the two tensor shapes the kernels fetch, and per-device properties.
#pragma once
#include <mutex>

#include "common.cuh"
#include "sm100_prims.cuh"

namespace tops {
namespace sm100 {

constexpr int kHeadDim = 128;   // K = V of the tcgen05 kernels

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeFn encode_fn() {
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

// Encoded tensor maps are kept per (device, pointer, shape): a training loop calls with the same
// buffers step after step, and a map depends on nothing else.
struct MapKey {
  int dev, kind;
  const void* ptr;
  uint64_t a, b;
  bool operator==(const MapKey& o) const { return dev == o.dev && kind == o.kind && ptr == o.ptr && a == o.a && b == o.b; }
};
struct MapSlot { MapKey key; CUtensorMap map; bool used; };
constexpr int kMapSlots = 64;
inline std::mutex g_map_mu;
inline MapSlot g_maps[kMapSlots];
template <class Encode>
inline int cached_map(CUtensorMap* m, int kind, const void* ptr, uint64_t a, uint64_t b, Encode encode) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return TOPS_E_CUDA; }
  const MapKey key{dev, kind, ptr, a, b};
  const size_t slot = (reinterpret_cast<uintptr_t>(ptr) >> 8) * 0x9E3779B97F4A7C15ull >> 58;   // 6 bits
  std::lock_guard<std::mutex> lk(g_map_mu);
  MapSlot& s = g_maps[(slot + (size_t)kind) % kMapSlots];
  if (!(s.used && s.key == key)) {
    // cuTensorMapEncodeTiled is a driver call and needs a current context on THIS thread; a thread that
    // has only made context-free runtime calls so far (an autograd worker on its first backward) has none.
    // Selecting the device it already has current binds the primary context without any other effect.
    if (cudaSetDevice(dev) != cudaSuccess) { cudaGetLastError(); return TOPS_E_CUDA; }
    const CUresult r = encode(&s.map);
    if (r != CUDA_SUCCESS) {
      s.used = false;
      record_cuda_error(-(int)r, "cuTensorMapEncodeTiled (driver error code negated)");
      return TOPS_E_CUDA;
    }
    s.key = key;
    s.used = true;
  }
  *m = s.map;
  return TOPS_OK;
}

// [B*T, H, 128] bf16 activations: box = 64 channels x 1 head x 64 tokens
inline int act_map(CUtensorMap* m, const void* ptr, int BT, int H) {
  return cached_map(m, 0, ptr, (uint64_t)BT, (uint64_t)H, [&](CUtensorMap* out) {
    cuuint64_t dims[3] = {(cuuint64_t)kHeadDim, (cuuint64_t)H, (cuuint64_t)BT};
    cuuint64_t strides[2] = {(cuuint64_t)kHeadDim * 2, (cuuint64_t)H * kHeadDim * 2};
    cuuint32_t box[3] = {64, 1, 64};
    cuuint32_t es[3] = {1, 1, 1};
    return encode_fn()(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, es,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  });
}
// [B*T, H, 64] bf16 per-chunk matrices (row i of a chunk at token i): box = 64 columns x 1 head x 64 tokens
inline int mat_map(CUtensorMap* m, const void* ptr, int BT, int H) {
  return cached_map(m, 2, ptr, (uint64_t)BT, (uint64_t)H, [&](CUtensorMap* out) {
    cuuint64_t dims[3] = {64, (cuuint64_t)H, (cuuint64_t)BT};
    cuuint64_t strides[2] = {64 * 2, (cuuint64_t)H * 64 * 2};
    cuuint32_t box[3] = {64, 1, 64};
    cuuint32_t es[3] = {1, 1, 1};
    return encode_fn()(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, es,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  });
}
// [rows, 128] bf16 chunk states: box = 64 columns x 128 rows
inline int state_map(CUtensorMap* m, const void* ptr, size_t rows) {
  return cached_map(m, 1, ptr, (uint64_t)rows, 0, [&](CUtensorMap* out) {
    cuuint64_t dims[2] = {(cuuint64_t)kHeadDim, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)kHeadDim * 2};
    cuuint32_t box[2] = {64, 128};
    cuuint32_t es[2] = {1, 1};
    return encode_fn()(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, es,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  });
}

// Properties of the current device, looked up once per device ordinal.
struct DeviceInfo { int sms; bool sm100; };
inline DeviceInfo device_info() {
  constexpr int kMaxDev = 64;
  static std::mutex mu;
  static DeviceInfo cache[kMaxDev];
  static bool have[kMaxDev] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return DeviceInfo{148, false}; }
  std::lock_guard<std::mutex> lk(mu);
  if (dev >= 0 && dev < kMaxDev && have[dev]) return cache[dev];
  DeviceInfo d{148, false};
  int n = 0, major = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) d.sms = n;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) == cudaSuccess) d.sm100 = major == 10;
  else cudaGetLastError();
  if (dev >= 0 && dev < kMaxDev) { cache[dev] = d; have[dev] = true; }
  return d;
}
inline int sm_count() { return device_info().sms; }
inline bool device_is_sm100() { return device_info().sm100; }

template <class F>
inline int opt_in_smem(F f, size_t bytes) {
  const cudaError_t e = cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e == cudaSuccess) return TOPS_OK;
  record_cuda_error((int)e, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize)");
  return TOPS_E_CUDA;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
}  // namespace sm100
}  // namespace tops
