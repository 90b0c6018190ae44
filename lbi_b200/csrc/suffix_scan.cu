// Suffix scans over per-region interface Jacobian transposes, single GPU, whole scan in one launch.
//
// lbi_suffix_scan:  out[b, k] = mats[b, k] * mats[b, k+1] * ... * mats[b, K-1],  out[b, K] = I      (R x R fp32)
//   The reference runs a Hillis-Steele scan with one cuBLAS strided-batched SGEMM per level plus copies and two
//   permutes (cuda/interface/suffix_scan.cu:70-115).  Here the recursion out[k] = mats[k] * out[k+1] is evaluated
//   right to left inside one kernel.  Column blocks of the running product are independent, so the grid is
//   (column blocks, batch): each CTA keeps its R x CB slab of the product in shared memory, streams mats[k] through
//   shared memory in R x KT tiles, and writes every prefix as it goes.  Products are exact fp32 FMA chains, which is
//   what the fp32 parity tolerances of the scan tests assume.
//
// lbi_affine_suffix_scan:  g[b, k] = offsets[b, k] + mats[b, k] * g[b, k+1],  g[b, K] = seed or 0   (vectors of R)
//   The cotangent recursion when every region owns loss terms.  One CTA per batch element; a warp owns a row.
#include "api.h"
#include "common.cuh"

namespace lbi {

constexpr int SCAN_CB = 32;   // columns of the running product per CTA
constexpr int SCAN_KT = 32;   // k-tile of the streamed matrix
constexpr int SCAN_THREADS = 256;

// dynamic smem: acc[2][R][CB] (double buffer) + tile[R][KT + 1]
__global__ void __launch_bounds__(SCAN_THREADS) suffix_scan_kernel(const float* __restrict__ mats, float* __restrict__ out,
                                                                   int k_count, int r) {
  extern __shared__ float smem[];
  float* acc0 = smem;
  float* acc1 = acc0 + (size_t)r * SCAN_CB;
  float* tile = acc1 + (size_t)r * SCAN_CB;  // [r][KT + 1]
  const int b = blockIdx.y;
  const int c0 = blockIdx.x * SCAN_CB;
  const int tid = threadIdx.x;
  const float* m_base = mats + (size_t)b * k_count * r * r;
  float* o_base = out + (size_t)b * (k_count + 1) * r * r;

  // identity slab, also written to out[K]
  for (int idx = tid; idx < r * SCAN_CB; idx += SCAN_THREADS) {
    const int row = idx / SCAN_CB, col = idx % SCAN_CB;
    const float v = (row == c0 + col) ? 1.f : 0.f;
    acc0[idx] = v;
    if (c0 + col < r) o_base[(size_t)k_count * r * r + (size_t)row * r + c0 + col] = v;
  }
  __syncthreads();

  float* cur = acc0;
  float* nxt = acc1;
  const int col = tid % SCAN_CB;         // column within the slab
  const int row_lane = tid / SCAN_CB;    // 0..7
  constexpr int ROWS_PER_PASS = SCAN_THREADS / SCAN_CB;  // 8
  for (int k = k_count - 1; k >= 0; --k) {
    const float* m = m_base + (size_t)k * r * r;
    // nxt = m * cur, rows processed in passes of ROWS_PER_PASS * 4
    for (int row0 = 0; row0 < r; row0 += ROWS_PER_PASS * 4) {
      float sum[4] = {0.f, 0.f, 0.f, 0.f};
      for (int kk0 = 0; kk0 < r; kk0 += SCAN_KT) {
        // stage m[row0 .. row0+32, kk0 .. kk0+KT] into tile (32 rows x KT)
        __syncthreads();
        for (int idx = tid; idx < ROWS_PER_PASS * 4 * SCAN_KT; idx += SCAN_THREADS) {
          const int tr = idx / SCAN_KT, tc = idx % SCAN_KT;
          const int gr = row0 + tr, gc = kk0 + tc;
          tile[tr * (SCAN_KT + 1) + tc] = (gr < r && gc < r) ? m[(size_t)gr * r + gc] : 0.f;
        }
        __syncthreads();
        const int kmax = (r - kk0) < SCAN_KT ? (r - kk0) : SCAN_KT;
        for (int kk = 0; kk < kmax; ++kk) {
          const float cv = cur[(size_t)(kk0 + kk) * SCAN_CB + col];
#pragma unroll
          for (int i = 0; i < 4; ++i) sum[i] += tile[(row_lane + i * ROWS_PER_PASS) * (SCAN_KT + 1) + kk] * cv;
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int gr = row0 + row_lane + i * ROWS_PER_PASS;
        if (gr < r) {
          nxt[(size_t)gr * SCAN_CB + col] = sum[i];
          if (c0 + col < r) o_base[(size_t)k * r * r + (size_t)gr * r + c0 + col] = sum[i];
        }
      }
    }
    __syncthreads();
    float* t = cur;
    cur = nxt;
    nxt = t;
  }
}

__global__ void __launch_bounds__(256) affine_suffix_scan_kernel(const float* __restrict__ mats,
                                                                  const float* __restrict__ offsets,
                                                                  const float* __restrict__ seed, float* __restrict__ g,
                                                                  int k_count, int r) {
  extern __shared__ float vec[];  // [2][r]
  const int b = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  float* cur = vec;
  float* nxt = vec + r;
  float* g_base = g + (size_t)b * (k_count + 1) * r;
  for (int i = threadIdx.x; i < r; i += blockDim.x) {
    const float v = seed ? seed[(size_t)b * r + i] : 0.f;
    cur[i] = v;
    g_base[(size_t)k_count * r + i] = v;
  }
  __syncthreads();
  for (int k = k_count - 1; k >= 0; --k) {
    const float* m = mats + ((size_t)b * k_count + k) * r * r;
    const float* off = offsets + ((size_t)b * k_count + k) * r;
    for (int row = warp; row < r; row += nwarps) {
      float acc = 0.f;
      for (int j = lane; j < r; j += 32) acc += m[(size_t)row * r + j] * cur[j];
      acc = warp_sum(acc);
      if (lane == 0) {
        const float v = off[row] + acc;
        nxt[row] = v;
        g_base[(size_t)k * r + row] = v;
      }
    }
    __syncthreads();
    float* t = cur;
    cur = nxt;
    nxt = t;
  }
}

// Frobenius and spectral norm of each R x R matrix (interface-Jacobian diagnostics).  One CTA per matrix; the spectral
// norm is the square root of the top eigenvalue of A^T A found by power iteration from a fixed non-degenerate start
// vector, with the Rayleigh quotient of the last iterate as the estimate.  Dynamic smem: 2 * r floats.
__global__ void __launch_bounds__(256) matrix_norms_kernel(const float* __restrict__ mats, float* __restrict__ spec,
                                                           float* __restrict__ frob, int r, int iters) {
  extern __shared__ float sm[];
  __shared__ float scratch[33];
  float* v = sm;        // current iterate (unit norm)
  float* w = sm + r;    // A v
  const float* a = mats + (size_t)blockIdx.x * r * r;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  float part = 0.f;
  for (int i = threadIdx.x; i < r * r; i += blockDim.x) part += a[i] * a[i];
  const float f2 = block_sum(part, scratch);
  if (threadIdx.x == 0) frob[blockIdx.x] = sqrtf(f2);
  for (int i = threadIdx.x; i < r; i += blockDim.x) v[i] = rsqrtf((float)r) * (1.f + 0.37f * __sinf(1.7f * (float)i + 0.3f));
  __syncthreads();
  float sigma2 = 0.f;
  for (int it = 0; it < iters; ++it) {
    for (int row = warp; row < r; row += nwarps) {   // w = A v
      float acc = 0.f;
      for (int j = lane; j < r; j += 32) acc += a[(size_t)row * r + j] * v[j];
      acc = warp_sum(acc);
      if (lane == 0) w[row] = acc;
    }
    __syncthreads();
    part = 0.f;
    for (int i = threadIdx.x; i < r; i += blockDim.x) part += w[i] * w[i];
    const float vv = block_sum(part, scratch);     // |A v|^2 with |v| = 1: Rayleigh quotient of A^T A
    sigma2 = vv;
    __syncthreads();
    for (int col = threadIdx.x; col < r; col += blockDim.x) {   // v = A^T w (column access: coalesced over threads)
      float acc = 0.f;
      for (int i = 0; i < r; ++i) acc += a[(size_t)i * r + col] * w[i];
      v[col] = acc;
    }
    __syncthreads();
    part = 0.f;
    for (int i = threadIdx.x; i < r; i += blockDim.x) part += v[i] * v[i];
    const float n2 = block_sum(part, scratch);
    const float inv = n2 > 0.f ? rsqrtf(n2) : 0.f;
    for (int i = threadIdx.x; i < r; i += blockDim.x) v[i] *= inv;
    __syncthreads();
  }
  if (threadIdx.x == 0) spec[blockIdx.x] = sqrtf(sigma2);
}

}  // namespace lbi

extern "C" {

int lbi_matrix_norms(const float* mats, float* spec, float* frob, int count, int r, int iters, cudaStream_t st) {
  using namespace lbi;
  if (count == 0) return 0;
  if (r <= 0 || r > 4096 || iters <= 0) return (int)cudaErrorInvalidValue;
  matrix_norms_kernel<<<count, 256, 2 * r * sizeof(float), st>>>(mats, spec, frob, r, iters);
  return (int)cudaGetLastError();
}

int lbi_suffix_scan(const float* mats, float* out, int batch, int k, int r, cudaStream_t st) {
  using namespace lbi;
  if (batch == 0) return 0;
  const size_t smem = ((size_t)2 * r * SCAN_CB + (size_t)32 * (SCAN_KT + 1)) * sizeof(float);
  cudaError_t e = cudaFuncSetAttribute(suffix_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid((r + SCAN_CB - 1) / SCAN_CB, batch);
  suffix_scan_kernel<<<grid, SCAN_THREADS, smem, st>>>(mats, out, k, r);
  return (int)cudaGetLastError();
}

int lbi_affine_suffix_scan(const float* mats, const float* offsets, const float* seed, float* g, int batch, int k, int r,
                           cudaStream_t st) {
  using namespace lbi;
  if (batch == 0) return 0;
  affine_suffix_scan_kernel<<<batch, 256, 2 * r * sizeof(float), st>>>(mats, offsets, seed, g, k, r);
  return (int)cudaGetLastError();
}

}  // extern "C"
