// Jacobian products of the interface maps over a basis of directions, fp32.
//
// The interface of a region is built from small maps (Linear or Linear -> act -> Linear heads, LayerNorm) whose
// Jacobians are needed applied to P directions at once: cotangents for the backward scan, tangents for the forward
// provider.  For a head evaluated at x with pre-activation h = W1 x + b1 and d = act'(h):
//     J^T g = W1^T (d o (W2^T g))          J t = W2 (d o (W1 t))
// Both are "two skinny GEMMs around a per-sample diagonal"; one kernel serves both with the weights given row-major
// as wa [din, hidden] and wb [hidden, dout] (the transposed case passes transposed copies):
//     out[b, p, :] = ((g[b, p, :] @ wa) o d[b, :]) @ wb        (wb null: out = (g @ wa) o d, d null: no diagonal)
// The LayerNorm kernel applies the closed form  (u - mean(u) - xhat mean(u xhat)) rstd  with the weight on the input
// side (J^T) or on the output side (J).  The products stay fp32 on the SIMT pipes: they feed R x R Jacobians whose
// chain products lose the scan's accuracy in reduced precision, and they amount to a few GFLOP per step.
// Reference: interfaces/vector_mlp.py:34-122 (torch einsums, one per factor).
#include "api.h"
#include "common.cuh"

namespace lbi {
namespace iface {

constexpr int PT = 8;          // directions per CTA
constexpr int THREADS = 256;

// grid (ceil(P / PT), B).  Shared memory: PT * din floats (g tile) + PT * hidden floats (hidden tile).
__global__ void __launch_bounds__(THREADS) mlp_jac_kernel(const float* __restrict__ g, const float* __restrict__ wa,
                                                          const float* __restrict__ d, const float* __restrict__ wb,
                                                          float* __restrict__ out, int p_total, int din, int hidden, int dout,
                                                          float in_scale) {
  extern __shared__ float smem[];
  float* gt = smem;                 // [PT][din]
  float* ht = smem + PT * din;      // [PT][hidden]
  const int b = blockIdx.y, p0 = blockIdx.x * PT;
  const int np = min(PT, p_total - p0);
  for (int i = threadIdx.x; i < PT * din; i += THREADS) {
    const int pp = i / din, c = i - pp * din;
    gt[i] = pp < np ? g[((int64_t)b * p_total + p0 + pp) * din + c] * in_scale : 0.f;
  }
  __syncthreads();
  for (int j = threadIdx.x; j < hidden; j += THREADS) {
    float acc[PT];
#pragma unroll
    for (int pp = 0; pp < PT; ++pp) acc[pp] = 0.f;
    for (int o = 0; o < din; ++o) {
      const float w = wa[(int64_t)o * hidden + j];
#pragma unroll
      for (int pp = 0; pp < PT; ++pp) acc[pp] = fmaf(gt[pp * din + o], w, acc[pp]);
    }
    const float dj = d ? d[(int64_t)b * hidden + j] : 1.f;
    if (wb) {
#pragma unroll
      for (int pp = 0; pp < PT; ++pp) ht[pp * hidden + j] = acc[pp] * dj;
    } else {
#pragma unroll
      for (int pp = 0; pp < PT; ++pp)
        if (pp < np) out[((int64_t)b * p_total + p0 + pp) * hidden + j] = acc[pp] * dj;
    }
  }
  if (!wb) return;
  __syncthreads();
  for (int i = threadIdx.x; i < dout; i += THREADS) {
    float acc[PT];
#pragma unroll
    for (int pp = 0; pp < PT; ++pp) acc[pp] = 0.f;
    for (int j = 0; j < hidden; ++j) {
      const float w = wb[(int64_t)j * dout + i];
#pragma unroll
      for (int pp = 0; pp < PT; ++pp) acc[pp] = fmaf(ht[pp * hidden + j], w, acc[pp]);
    }
#pragma unroll
    for (int pp = 0; pp < PT; ++pp)
      if (pp < np) out[((int64_t)b * p_total + p0 + pp) * dout + i] = acc[pp];
  }
}

// One warp per direction row.  x [B, R]; g, out [B, P, R]; weight [R] or null.
__global__ void __launch_bounds__(THREADS) layernorm_jac_kernel(const float* __restrict__ x, const float* __restrict__ weight,
                                                                const float* __restrict__ g, float* __restrict__ out,
                                                                int64_t rows, int p_total, int r, float eps, int transpose,
                                                                float out_scale) {
  const int64_t row = (int64_t)blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const float* xr = x + (row / p_total) * r;
  const float* gr = g + row * r;
  float s = 0.f;
  for (int c = lane; c < r; c += 32) s += xr[c];
  const float mu = warp_sum(s) / r;
  float v = 0.f;
  for (int c = lane; c < r; c += 32) {
    const float t = xr[c] - mu;
    v = fmaf(t, t, v);
  }
  const float rstd = rsqrtf(warp_sum(v) / r + eps);
  float su = 0.f, sux = 0.f;
  for (int c = lane; c < r; c += 32) {
    const float u = gr[c] * ((transpose && weight) ? weight[c] : 1.f);
    su += u;
    sux = fmaf(u, (xr[c] - mu) * rstd, sux);
  }
  const float mean_u = warp_sum(su) / r, mean_ux = warp_sum(sux) / r;
  for (int c = lane; c < r; c += 32) {
    const float u = gr[c] * ((transpose && weight) ? weight[c] : 1.f);
    float o = (u - mean_u - (xr[c] - mu) * rstd * mean_ux) * rstd;
    if (!transpose && weight) o *= weight[c];
    out[row * r + c] = o * out_scale;
  }
}

}  // namespace iface
}  // namespace lbi

extern "C" int lbi_interface_mlp_jac(const float* g, const float* wa, const float* d, const float* wb, float* out, int batch,
                                     int p_total, int din, int hidden, int dout, float in_scale, cudaStream_t st) {
  using namespace lbi::iface;
  if (batch <= 0 || p_total <= 0 || din <= 0 || hidden <= 0 || (wb && dout <= 0)) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)PT * (din + (wb ? hidden : 0)) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  int rc = (int)cudaFuncSetAttribute(mlp_jac_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (rc) return rc;
  mlp_jac_kernel<<<dim3((p_total + PT - 1) / PT, batch), THREADS, smem, st>>>(g, wa, d, wb, out, p_total, din, hidden, dout, in_scale);
  return (int)cudaGetLastError();
}

extern "C" int lbi_layernorm_jac(const float* x, const float* weight, const float* g, float* out, int batch, int p_total, int r,
                                 float eps, int transpose, float out_scale, cudaStream_t st) {
  using namespace lbi::iface;
  if (batch <= 0 || p_total <= 0 || r <= 0) return (int)cudaErrorInvalidValue;
  const int64_t rows = (int64_t)batch * p_total;
  const int per = THREADS / 32;
  layernorm_jac_kernel<<<(unsigned)((rows + per - 1) / per), THREADS, 0, st>>>(x, weight, g, out, rows, p_total, r, eps, transpose,
                                                                              out_scale);
  return (int)cudaGetLastError();
}
