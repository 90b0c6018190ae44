// RMSNorm with an optional SiLU gate and optional groups, forward and backward (the Mamba block norms).
//
//   u = x * silu(z)   (gate first, Mamba-2)      or   u = x                (gate last, Mamba-3; or no gate)
//   y = u * rstd * w  with rstd = rsqrt(mean_group(u^2) + eps)             then  y *= silu(z)  when the gate comes last
//
// One warp owns one (row, group) at a time and walks rows with a fixed group, so that the weight gradient of its
// columns accumulates privately (shared memory, one slice per warp) and leaves as one row of a partials buffer that
// the caller sums: no atomics, deterministic.  Inputs and outputs are bf16 or fp32 (template), statistics fp32.
// Replaces the reference's Triton pair _layer_norm_fwd_1pass_kernel / _layer_norm_bwd_kernel
// (backbones/mamba2/ops/triton/layernorm_gated.py:45-271) for the RMS case without bias.
#include "api.h"
#include "common.cuh"

namespace lbi {
namespace gnorm {

constexpr int THREADS = 256;
constexpr int WARPS = THREADS / 32;

template <typename T>
__device__ __forceinline__ float ldf(const T* p, int64_t i) {
  return static_cast<float>(p[i]);
}
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) {
  return __bfloat162float(p[i]);
}
template <typename T>
__device__ __forceinline__ void stf(T* p, int64_t i, float v) {
  p[i] = static_cast<T>(v);
}
template <>
__device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) {
  p[i] = __float2bfloat16(v);
}

__device__ __forceinline__ float sigmoidf(float v) { return 1.f / (1.f + __expf(-v)); }

template <typename T>
__global__ void __launch_bounds__(THREADS) gated_rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ z,
                                                                    const float* __restrict__ w, T* __restrict__ y,
                                                                    float* __restrict__ rstd_out, int64_t rows, int dim, int gs,
                                                                    float eps, int gate_first) {
  const int ngroups = dim / gs;
  const int64_t vrows = rows * ngroups;
  const int lane = threadIdx.x & 31;
  for (int64_t vr = (int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5); vr < vrows; vr += (int64_t)gridDim.x * WARPS) {
    const int64_t base = (vr / ngroups) * dim + (vr % ngroups) * gs;
    const int col0 = (int)(vr % ngroups) * gs;
    float ss = 0.f;
    for (int c = lane; c < gs; c += 32) {
      float u = ldf(x, base + c);
      if (z && gate_first) {
        const float zz = ldf(z, base + c);
        u *= zz * sigmoidf(zz);
      }
      ss = fmaf(u, u, ss);
    }
    const float rstd = rsqrtf(warp_sum(ss) / gs + eps);
    if (lane == 0) rstd_out[vr] = rstd;
    for (int c = lane; c < gs; c += 32) {
      float u = ldf(x, base + c);
      float gate = 1.f;
      if (z) {
        const float zz = ldf(z, base + c);
        gate = zz * sigmoidf(zz);
      }
      if (z && gate_first) u *= gate;
      float o = u * rstd * w[col0 + c];
      if (z && !gate_first) o *= gate;
      stf(y, base + c, o);
    }
  }
}

// dw_partials [gridDim.x * WARPS / ngroups, dim]: slot s of group g holds the sum over the rows walked by that warp.
template <typename T>
__global__ void __launch_bounds__(THREADS) gated_rmsnorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                                    const T* __restrict__ z, const float* __restrict__ w,
                                                                    const float* __restrict__ rstd_in, T* __restrict__ dx,
                                                                    T* __restrict__ dz, float* __restrict__ dw_partials,
                                                                    int64_t rows, int dim, int gs, int gate_first) {
  extern __shared__ float dw_acc[];   // [WARPS][gs]
  const int ngroups = dim / gs;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* acc = dw_acc + (int64_t)warp * gs;
  for (int c = lane; c < gs; c += 32) acc[c] = 0.f;
  const int64_t gw = (int64_t)blockIdx.x * WARPS + warp;          // the launch makes the warp count a multiple of ngroups
  const int g = (int)(gw % ngroups);
  const int64_t slot = gw / ngroups, nslots = (int64_t)gridDim.x * WARPS / ngroups;
  const int col0 = g * gs;
  for (int64_t row = slot; row < rows; row += nslots) {
    const int64_t base = row * dim + col0;
    const float rstd = rstd_in[row * ngroups + g];
    float dot = 0.f;
    for (int c = lane; c < gs; c += 32) {
      float u = ldf(x, base + c), dyn = ldf(dy, base + c);
      if (z) {
        const float zz = ldf(z, base + c);
        const float gate = zz * sigmoidf(zz);
        if (gate_first) u *= gate; else dyn *= gate;
      }
      dot = fmaf(dyn * w[col0 + c], u * rstd, dot);
    }
    const float mean_gu = warp_sum(dot) / gs;
    for (int c = lane; c < gs; c += 32) {
      const float xv = ldf(x, base + c), dyv = ldf(dy, base + c), wv = w[col0 + c];
      float u = xv, dyn = dyv, gate = 1.f, dgate = 0.f;
      if (z) {
        const float zz = ldf(z, base + c);
        const float sg = sigmoidf(zz);
        gate = zz * sg;
        dgate = sg * (1.f + zz * (1.f - sg));
        if (gate_first) u *= gate; else dyn *= gate;
      }
      const float uhat = u * rstd;
      acc[c] = fmaf(dyn, uhat, acc[c]);
      const float du = rstd * (dyn * wv - uhat * mean_gu);
      if (z && gate_first) {
        stf(dx, base + c, du * gate);
        stf(dz, base + c, du * xv * dgate);
      } else {
        stf(dx, base + c, du);
        if (z) stf(dz, base + c, dyv * uhat * wv * dgate);
      }
    }
  }
  __syncwarp();
  for (int c = lane; c < gs; c += 32) dw_partials[slot * dim + col0 + c] = acc[c];
}

static int grid_for(int64_t rows, int ngroups, int* nslots) {
  // warps per grid: a multiple of ngroups and of WARPS, about two CTAs per SM, never more slots than rows
  int64_t slots = (2 * 148 * WARPS + ngroups - 1) / ngroups;
  if (slots > rows) slots = rows;
  if (slots < 1) slots = 1;
  int64_t warps = slots * ngroups;
  while (warps % WARPS != 0) warps += ngroups, ++slots;
  *nslots = (int)slots;
  return (int)(warps / WARPS);
}

template <typename T>
static int fwd(const void* x, const void* z, const float* w, void* y, float* rstd, int64_t rows, int dim, int gs, float eps,
               int gate_first, cudaStream_t st) {
  const int ngroups = dim / gs;
  int64_t blocks = (rows * ngroups + WARPS - 1) / WARPS;
  if (blocks > 148 * 8) blocks = 148 * 8;
  gated_rmsnorm_fwd_kernel<T><<<(unsigned)blocks, THREADS, 0, st>>>((const T*)x, (const T*)z, w, (T*)y, rstd, rows, dim, gs, eps,
                                                                   gate_first);
  return (int)cudaGetLastError();
}

template <typename T>
static int bwd(const void* dy, const void* x, const void* z, const float* w, const float* rstd, void* dx, void* dz,
               float* dw_partials, int64_t rows, int dim, int gs, int gate_first, cudaStream_t st) {
  int nslots = 0;
  const int blocks = grid_for(rows, dim / gs, &nslots);
  const size_t smem = (size_t)WARPS * gs * sizeof(float);
  int rc = (int)cudaFuncSetAttribute(gated_rmsnorm_bwd_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (rc) return rc;
  gated_rmsnorm_bwd_kernel<T><<<blocks, THREADS, smem, st>>>((const T*)dy, (const T*)x, (const T*)z, w, rstd, (T*)dx, (T*)dz,
                                                            dw_partials, rows, dim, gs, gate_first);
  return (int)cudaGetLastError();
}

}  // namespace gnorm
}  // namespace lbi

extern "C" int lbi_gated_rmsnorm_slots(int64_t rows, int dim, int group_size) {
  int nslots = 0;
  if (rows <= 0 || dim <= 0 || group_size <= 0 || dim % group_size != 0) return 0;
  lbi::gnorm::grid_for(rows, dim / group_size, &nslots);
  return nslots;
}

extern "C" int lbi_gated_rmsnorm_fwd(const void* x, const void* z_or_null, const float* weight, void* y, float* rstd, int64_t rows,
                                     int dim, int group_size, float eps, int gate_first, int is_bf16, cudaStream_t st) {
  if (rows <= 0 || dim <= 0 || group_size <= 0 || dim % group_size != 0) return (int)cudaErrorInvalidValue;
  return is_bf16 ? lbi::gnorm::fwd<__nv_bfloat16>(x, z_or_null, weight, y, rstd, rows, dim, group_size, eps, gate_first, st)
                 : lbi::gnorm::fwd<float>(x, z_or_null, weight, y, rstd, rows, dim, group_size, eps, gate_first, st);
}

extern "C" int lbi_gated_rmsnorm_bwd(const void* dy, const void* x, const void* z_or_null, const float* weight, const float* rstd,
                                     void* dx, void* dz_or_null, float* dw_partials, int64_t rows, int dim, int group_size,
                                     int gate_first, int is_bf16, cudaStream_t st) {
  if (rows <= 0 || dim <= 0 || group_size <= 0 || dim % group_size != 0 || group_size > 6144) return (int)cudaErrorInvalidValue;
  return is_bf16 ? lbi::gnorm::bwd<__nv_bfloat16>(dy, x, z_or_null, weight, rstd, dx, dz_or_null, dw_partials, rows, dim, group_size,
                                                  gate_first, st)
                 : lbi::gnorm::bwd<float>(dy, x, z_or_null, weight, rstd, dx, dz_or_null, dw_partials, rows, dim, group_size,
                                          gate_first, st);
}
