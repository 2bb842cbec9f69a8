// Stand-alone measurement of what one tcgen05.mma costs for the shapes the chunk kernels issue:
// one thread issues 256 back-to-back products on tiles that are already in shared memory and
// reports clock64 cycles per instruction (issue loop, and until the commit arrives).
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I pallas-kernel_b200/csrc \
//        -o mma_cost pallas-kernel_b200/csrc/probes/mma_cost.cu && ./mma_cost
//
// Not part of the library (build.py compiles csrc/*.cu only).  Every wait is bounded.
#include <cstdio>
#include <cuda_runtime.h>
#include "sm100_prims.cuh"
using namespace tops::sm100;

template <int M, int N, bool AMN, bool BMN, int NACC>
__global__ void k(long long* out, int reps) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  const int tid = threadIdx.x;
  for (int i = tid; i < 64 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;
  if (tid == 0) { mbar_init(&bar, 1); fence_barrier_init(); }
  if (tid < 32) { tmem_alloc(&slot, 512); tmem_relinquish(); }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = slot;
  if (tid == 0) {
    const uint32_t a = smem_u32(smem), b = smem_u32(smem + 32768);
    long long t0 = clock64();
    for (int r = 0; r < reps; ++r) {
#pragma unroll
      for (int k0 = 0; k0 < 64; k0 += 16) {
        const uint64_t ad = AMN ? desc_mnmajor(a, 64, k0, 0) : desc_kmajor(a, 128, 0, k0);
        const uint64_t bd = BMN ? desc_mnmajor(b, 64, k0, 0) : desc_kmajor(b, 128, 0, k0);
        const int acc = (k0 / 16) % NACC;
        umma_bf16(tm + acc * (512 / NACC >= N ? N : 0), ad, bd, umma_idesc(M, N, AMN, BMN), 1);
      }
    }
    long long t1 = clock64();
    umma_commit(&bar);
    mbar_wait(&bar, 0);
    long long t2 = clock64();
    out[0] = t1 - t0; out[1] = t2 - t0;
  }
  tc_fence_before();
  __syncthreads();
  if (tid < 32) tmem_dealloc(tm, 512);
}

template <int M, int N, bool AMN, bool BMN, int NACC>
void run(const char* name, long long* d) {
  cudaFuncSetAttribute(k<M, N, AMN, BMN, NACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, 70 * 1024);
  const int reps = 64;
  k<M, N, AMN, BMN, NACC><<<1, 128, 70 * 1024>>>(d, reps);
  long long h[2];
  cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
  cudaError_t e = cudaDeviceSynchronize();
  printf("%-40s issue %7.1f  total %7.1f cycles/MMA  (%s)\n", name, h[0] / (reps * 4.0), h[1] / (reps * 4.0), cudaGetErrorString(e));
}

int main() {
  long long* d;
  cudaMalloc(&d, 16);
  run<128, 128, false, false, 1>("M128 N128 K-major x K-major, 1 acc", d);
  run<128, 128, false, false, 2>("M128 N128 K x K, 2 acc", d);
  run<128, 128, true, true, 1>("M128 N128 MN x MN, 1 acc", d);
  run<128, 128, false, true, 1>("M128 N128 K x MN, 1 acc", d);
  run<128, 64, false, false, 1>("M128 N64 K x K, 1 acc", d);
  run<128, 64, true, false, 1>("M128 N64 MN x K, 1 acc", d);
  run<128, 64, true, true, 1>("M128 N64 MN x MN, 1 acc", d);
  run<64, 64, false, false, 1>("M64 N64 K x K, 1 acc", d);
  run<64, 64, false, false, 4>("M64 N64 K x K, 4 acc", d);
  run<64, 128, false, true, 1>("M64 N128 K x MN, 1 acc", d);
  run<128, 16, true, false, 1>("M128 N16 MN x K, 1 acc", d);
  run<128, 256, false, false, 1>("M128 N256 K x K, 1 acc", d);
  return 0;
}
