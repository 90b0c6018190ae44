// Microbenchmark: cycles per tcgen05.mma for several shapes / operand layouts (A from shared memory or from TMEM), one
// issuing thread per CTA.
#include <cstdio>
#include <cuda_runtime.h>
#include "tcgen05.cuh"
using namespace lbi::tc;

struct Cfg { int n; int a_mn; int b_mn; int two_threads; int a_tmem; };

// D[tmem] (+)= A[tmem] * B[smem]: the A tile (128 lanes x 16 bf16 = 8 columns per K step) is read from tensor memory
__device__ __forceinline__ void mma_bf16_a_tmem(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <bool A_TMEM>
__global__ void __launch_bounds__(128, 1) k(Cfg c, int iters, long long* out, int* status) {
  extern __shared__ uint8_t raw[];
  uint8_t* sm = (uint8_t*)(((uintptr_t)raw + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar[2];
  __shared__ uint32_t tbase;
  __shared__ volatile int abortf;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) { abortf = 0; mbar_init(&bar[0], 1); mbar_init(&bar[1], 1); fence_barrier_init(); }
  // operands: zeros (values do not matter for timing)
  for (int i = threadIdx.x; i < 96 * 1024 / 4; i += blockDim.x) ((uint32_t*)sm)[i] = 0;
  fence_proxy_async();
  if (warp == 0) tmem_alloc(&tbase, 512);
  fence_before_sync(); __syncthreads(); fence_after_sync();
  const uint32_t tmem = tbase;
  const uint32_t idesc = make_idesc_bf16(128, c.n, c.a_mn, c.b_mn);
  const uint32_t a_addr = smem_u32(sm), b_addr = smem_u32(sm + 32 * 1024);
  const uint64_t da0 = make_smem_desc(a_addr, c.a_mn ? 16384 : 16, 1024);
  const uint64_t db0 = make_smem_desc(b_addr, c.b_mn ? 16384 : 16, 1024);
  const int astep = c.a_mn ? 128 : 2, bstep = c.b_mn ? 128 : 2;
  const int nthreads = c.two_threads ? 2 : 1;
  if (lane == 0 && warp < nthreads) {
    long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        if (A_TMEM) mma_bf16_a_tmem(tmem + warp * 256, tmem + 480 + kk * 8, db0 + bstep * kk, idesc, 1);
        else mma_bf16(tmem + warp * 256, da0 + astep * kk, db0 + bstep * kk, idesc, 1);
      }
    }
    long long t1 = clock64();
    mma_commit(&bar[warp]);
    bool ok = mbar_wait(&bar[warp], 0, &abortf, status, 1);
    long long t2 = clock64();
    if (blockIdx.x == 0) { out[warp * 2] = t1 - t0; out[warp * 2 + 1] = t2 - t0; }
    (void)ok;
  }
  fence_before_sync(); __syncthreads();
  if (warp == 0) { fence_after_sync(); tmem_dealloc(tmem, 512); }
}

int main() {
  long long* out; int* status;
  cudaMalloc(&out, 64); cudaMalloc(&status, 4); cudaMemset(status, 0, 4);
  cudaFuncSetAttribute(k<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  cudaFuncSetAttribute(k<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  Cfg cfgs[] = {{256,0,0,0,0},{128,0,0,0,0},{64,0,0,0,0},{64,0,1,0,0},{64,1,1,0,0},{128,1,1,0,0},{128,0,0,1,0},{64,0,1,1,0},{32,0,0,0,0},{16,0,0,0,0},
                {64,0,0,0,1},{64,0,1,0,1},{128,0,0,0,1},{32,0,0,0,1}};
  const int iters = 500;
  for (auto c : cfgs) {
    cudaMemset(out, 0, 64);
    if (c.a_tmem) k<true><<<148, 128, 100 * 1024>>>(c, iters, out, status);
    else k<false><<<148, 128, 100 * 1024>>>(c, iters, out, status);
    cudaError_t e = cudaDeviceSynchronize();
    long long h[4]; int st; cudaMemcpy(h, out, 32, cudaMemcpyDeviceToHost); cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost);
    const double n = iters * 4.0;
    printf("N=%3d a_mn=%d b_mn=%d a_tmem=%d threads=%d : issue %.1f cyc/mma, done %.1f cyc/mma (ideal %.0f)  [t1: issue %.1f done %.1f] err=%d status=%d\n",
           c.n, c.a_mn, c.b_mn, c.a_tmem, c.two_threads + 1, h[0] / n, h[1] / n, c.n / 2.0, h[2] / n, h[3] / n, (int)e, st);
  }
  return 0;
}
