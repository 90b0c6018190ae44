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

// ------------------------------------------------------------------------------------------------ skinny linear maps
// The interface maps themselves act on a handful of rows (one per batch element): y = act(x W^T + b), its input
// cotangent and its parameter gradients.  Three fp32 kernels cover them, so that neither the forward of the region chain
// nor the local VJPs call a library GEMM or autograd for these maps (reference: nn.Linear inside
// interfaces/vector_mlp.py:125-161 and torch.autograd.grad in backward/local_vjp.py:137-168).
namespace lbi {
namespace iface {

__device__ __forceinline__ float act_apply(float v, int act) {
  if (act == 1) return v * sigmoidf_(v);                                            // SiLU
  if (act == 2) return 0.5f * v * (1.f + erff(v * 0.7071067811865476f));            // GELU (erf form)
  return v;
}

// y[b, o] = act(sum_i x[b, i] w[o, i] + bias[o]); pre (optional) keeps the value before the activation.  One warp per output.
__global__ void __launch_bounds__(256) small_linear_fwd_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                               const float* __restrict__ bias, float* __restrict__ y,
                                                               float* __restrict__ pre, int batch, int din, int dout, int act) {
  const int lane = threadIdx.x & 31;
  const int64_t widx = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (widx >= (int64_t)batch * dout) return;
  const int o = (int)(widx % dout), b = (int)(widx / dout);
  const float* xr = x + (int64_t)b * din;
  const float* wr = w + (int64_t)o * din;
  float acc = 0.f;
  for (int i = lane; i < din; i += 32) acc = fmaf(xr[i], wr[i], acc);
  acc = warp_sum(acc);
  if (lane == 0) {
    acc += bias ? bias[o] : 0.f;
    if (pre) pre[widx] = acc;
    y[widx] = act_apply(acc, act);
  }
}

// gx[b, i] = sum_o g[b, o] w[o, i]
__global__ void __launch_bounds__(256) small_linear_dgrad_kernel(const float* __restrict__ g, const float* __restrict__ w,
                                                                 float* __restrict__ gx, int batch, int din, int dout) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)batch * din) return;
  const int i = (int)(idx % din), b = (int)(idx / din);
  const float* gr = g + (int64_t)b * dout;
  float acc = 0.f;
  for (int o = 0; o < dout; ++o) acc = fmaf(gr[o], w[(int64_t)o * din + i], acc);
  gx[idx] = acc;
}

// dw[o, i] += sum_b g[b, o] x[b, i];  db[o] += sum_b g[b, o]   (db may be null)
__global__ void __launch_bounds__(256) small_linear_wgrad_kernel(const float* __restrict__ g, const float* __restrict__ x,
                                                                 float* __restrict__ dw, float* __restrict__ db, int batch, int din,
                                                                 int dout) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)dout * din) return;
  const int i = (int)(idx % din), o = (int)(idx / din);
  float acc = 0.f, accb = 0.f;
  for (int b = 0; b < batch; ++b) {
    const float gv = g[(int64_t)b * dout + o];
    acc = fmaf(gv, x[(int64_t)b * din + i], acc);
    accb += gv;
  }
  dw[idx] += acc;
  if (db && i == 0) db[o] += accb;
}

}  // namespace iface
}  // namespace lbi

extern "C" int lbi_small_linear_fwd(const float* x, const float* w, const float* bias, float* y, float* pre, int batch, int din,
                                    int dout, int act, cudaStream_t st) {
  using namespace lbi::iface;
  if (batch <= 0 || din <= 0 || dout <= 0 || act < 0 || act > 2) return (int)cudaErrorInvalidValue;
  const int64_t warps = (int64_t)batch * dout;
  small_linear_fwd_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, st>>>(x, w, bias, y, pre, batch, din, dout, act);
  return (int)cudaGetLastError();
}

extern "C" int lbi_small_linear_dgrad(const float* g, const float* w, float* gx, int batch, int din, int dout, cudaStream_t st) {
  using namespace lbi::iface;
  if (batch <= 0 || din <= 0 || dout <= 0) return (int)cudaErrorInvalidValue;
  const int64_t total = (int64_t)batch * din;
  small_linear_dgrad_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(g, w, gx, batch, din, dout);
  return (int)cudaGetLastError();
}

extern "C" int lbi_small_linear_wgrad(const float* g, const float* x, float* dw, float* db, int batch, int din, int dout,
                                      cudaStream_t st) {
  using namespace lbi::iface;
  if (batch <= 0 || din <= 0 || dout <= 0) return (int)cudaErrorInvalidValue;
  const int64_t total = (int64_t)dout * din;
  small_linear_wgrad_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(g, x, dw, db, batch, din, dout);
  return (int)cudaGetLastError();
}
