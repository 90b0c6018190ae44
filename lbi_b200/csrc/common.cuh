// Shared device helpers for the sm_100a kernels of lbi_b200.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

namespace lbi {

// cudaFuncAttributeMaxDynamicSharedMemorySize belongs to a (kernel, device) pair, so a process that drives several
// GPUs has to set it once on each.  One static instance per kernel remembers which devices are done (bit per ordinal).
struct PerDeviceOnce {
  std::atomic<unsigned long long> done[4] = {};
  template <typename Kernel>
  cudaError_t max_dynamic_smem(Kernel kernel, int bytes) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const bool tracked = dev >= 0 && dev < 256;
    const unsigned long long bit = 1ull << (dev & 63);
    if (tracked && (done[dev >> 6].load(std::memory_order_acquire) & bit)) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess && tracked) done[dev >> 6].fetch_or(bit, std::memory_order_release);
    return e;
  }
};

// Debug build (python -m lbi_b200.build --bounds-check, extension lbi_b200._Cdbg): index checks that record the first violation
// (a site code) in a word of their translation unit and skip the access; nothing ever traps.  In the normal build the
// macro is the constant true and costs nothing.  LBI_DEFINE_BOUNDS_GETTER(fn) defines the host function that reads and
// clears the word of the translation unit it is placed in.
#ifdef LBI_BOUNDS_CHECK
static __device__ int g_bounds_site = 0;
__device__ __forceinline__ bool bounds_ok(int64_t i, int64_t n, int site) {
  if (i >= 0 && i < n) return true;
  atomicCAS(&g_bounds_site, 0, site);
  return false;
}
#define LBI_IN_RANGE(i, n, site) lbi::bounds_ok((int64_t)(i), (int64_t)(n), (site))
#define LBI_DEFINE_BOUNDS_GETTER(fn)                                                                   \
  extern "C" int fn() {                                                                                \
    int v = 0, zero = 0;                                                                               \
    if (cudaMemcpyFromSymbol(&v, lbi::g_bounds_site, sizeof(int)) != cudaSuccess) return -1;           \
    if (cudaMemcpyToSymbol(lbi::g_bounds_site, &zero, sizeof(int)) != cudaSuccess) return -1;          \
    return v;                                                                                          \
  }
#else
#define LBI_IN_RANGE(i, n, site) (true)
#define LBI_DEFINE_BOUNDS_GETTER(fn) \
  extern "C" int fn() { return 0; }
#endif

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const bf16x8& p, float* f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ bf16x8 pack8(const float* f) {
  bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

}  // namespace lbi
