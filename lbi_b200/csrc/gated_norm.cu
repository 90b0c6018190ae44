// RMSNorm with an optional SiLU gate and optional groups, forward and backward (the Mamba block norms).
//
//   u = x * silu(z)   (gate first, Mamba-2)      or   u = x                (gate last, Mamba-3; or no gate)
//   y = u * rstd * w  with rstd = rsqrt(mean_group(u^2) + eps)             then  y *= silu(z)  when the gate comes last
//
// Every lane moves 16 bytes per access (8 bf16 or 4 fp32).  A group of `gs` elements is shared by LPG lanes (a power of
// two, at most 32) that each walk IT vectors, so a warp holds 32 / LPG groups at a time and group statistics are
// sub-warp shuffle reductions: a 64-wide group of the Mamba-3 norm takes 8 lanes and one access per lane and operand.
// The weight gradient accumulates in shared memory per block and leaves as one row of a partials buffer that the
// caller sums.  Statistics and arithmetic are fp32.
// Replaces the reference's Triton pair _layer_norm_fwd_1pass_kernel / _layer_norm_bwd_kernel
// (backbones/mamba2/ops/triton/layernorm_gated.py:45-271) for the RMS case without bias.
#include "api.h"
#include "common.cuh"

namespace lbi {
namespace gnorm {

constexpr int THREADS = 256;
constexpr int WARPS = THREADS / 32;

template <typename T>
struct Vec;
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* f) {
    const bf16x8 v = *reinterpret_cast<const bf16x8*>(p);
    unpack8(v, f);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* f) { *reinterpret_cast<bf16x8*>(p) = pack8(f); }
};
template <>
struct Vec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* f) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
};

__device__ __forceinline__ float sigmoidf(float v) { return 1.f / (1.f + __expf(-v)); }

__device__ __forceinline__ float group_sum(float v, int lpg) {
  for (int off = lpg >> 1; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

template <typename T>
__global__ void __launch_bounds__(THREADS) gated_rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ z,
                                                                    const float* __restrict__ w, T* __restrict__ y,
                                                                    float* __restrict__ rstd_out, int64_t vrows, int dim, int gs,
                                                                    float eps, int gate_first, int lpg, int iters) {
  constexpr int V = Vec<T>::N;
  const int ngroups = dim / gs, gpw = 32 / lpg;
  const int lane = threadIdx.x & 31, sub = lane / lpg, li = lane % lpg;
  for (int64_t v0 = ((int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5)) * gpw; v0 < vrows; v0 += (int64_t)gridDim.x * WARPS * gpw) {
    const int64_t vr = v0 + sub;
    const bool live = vr < vrows;
    const int g = live ? (int)(vr % ngroups) : 0;
    const int64_t base = live ? (vr / ngroups) * dim + (int64_t)g * gs : 0;
    float ss = 0.f;
    for (int it = 0; it < iters; ++it) {
      const int c = (it * lpg + li) * V;
      float xv[V], zv[V];
      if (live) {
        Vec<T>::load(x + base + c, xv);
        if (z && gate_first) Vec<T>::load(z + base + c, zv);
#pragma unroll
        for (int e = 0; e < V; ++e) {
          const float u = (z && gate_first) ? xv[e] * zv[e] * sigmoidf(zv[e]) : xv[e];
          ss = fmaf(u, u, ss);
        }
      }
    }
    const float rstd = rsqrtf(group_sum(ss, lpg) / gs + eps);
    if (live && li == 0) rstd_out[vr] = rstd;
    if (!live) continue;
    for (int it = 0; it < iters; ++it) {
      const int c = (it * lpg + li) * V;
      float xv[V], zv[V], wv[V], o[V];
      Vec<T>::load(x + base + c, xv);
      if (z) Vec<T>::load(z + base + c, zv);
#pragma unroll
      for (int e = 0; e < V; e += 4) {
        const float4 t = *reinterpret_cast<const float4*>(w + g * gs + c + e);
        wv[e] = t.x; wv[e + 1] = t.y; wv[e + 2] = t.z; wv[e + 3] = t.w;
      }
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const float gate = z ? zv[e] * sigmoidf(zv[e]) : 1.f;
        const float u = (z && gate_first) ? xv[e] * gate : xv[e];
        o[e] = u * rstd * wv[e] * ((z && !gate_first) ? gate : 1.f);
      }
      Vec<T>::store(y + base + c, o);
    }
  }
}

// dw_partials [gridDim.x][dim]
template <typename T>
__global__ void __launch_bounds__(THREADS) gated_rmsnorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                                    const T* __restrict__ z, const float* __restrict__ w,
                                                                    const float* __restrict__ rstd_in, T* __restrict__ dx,
                                                                    T* __restrict__ dz, float* __restrict__ dw_partials,
                                                                    int64_t vrows, int64_t fvrows, int dim, int gs, int gate_first,
                                                                    int lpg, int iters) {
  // x, z, rstd hold fvrows (row, group) pairs shared by vrows / fvrows stacked directions of dy; dw_partials may be null
  // (a pullback pass wants no weight gradient: nothing is accumulated for it)
  constexpr int V = Vec<T>::N;
  extern __shared__ float dw_acc[];   // [dim]
  const bool want_dw = dw_partials != nullptr;
  if (want_dw) {
    for (int i = threadIdx.x; i < dim; i += THREADS) dw_acc[i] = 0.f;
    __syncthreads();
  }
  const int ngroups = dim / gs, gpw = 32 / lpg;
  const int lane = threadIdx.x & 31, sub = lane / lpg, li = lane % lpg;
  for (int64_t v0 = ((int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5)) * gpw; v0 < vrows; v0 += (int64_t)gridDim.x * WARPS * gpw) {
    const int64_t vr = v0 + sub;
    const bool live = vr < vrows;
    const int g = live ? (int)(vr % ngroups) : 0;
    const int64_t base = live ? (vr / ngroups) * dim + (int64_t)g * gs : 0;
    const int64_t fvr = live ? vr % fvrows : 0;
    const int64_t fbase = (fvr / ngroups) * dim + (int64_t)g * gs;
    const float rstd = live ? rstd_in[fvr] : 0.f;
    float dot = 0.f;
    for (int it = 0; it < iters; ++it) {
      const int c = (it * lpg + li) * V;
      if (live) {
        float xv[V], zv[V], gv[V];
        Vec<T>::load(x + fbase + c, xv);
        Vec<T>::load(dy + base + c, gv);
        if (z) Vec<T>::load(z + fbase + c, zv);
#pragma unroll
        for (int e = 0; e < V; ++e) {
          float u = xv[e], dyn = gv[e];
          if (z) {
            const float gate = zv[e] * sigmoidf(zv[e]);
            if (gate_first) u *= gate; else dyn *= gate;
          }
          dot = fmaf(dyn * w[g * gs + c + e], u * rstd, dot);
        }
      }
    }
    const float mean_gu = group_sum(dot, lpg) / gs;
    if (!live) continue;
    for (int it = 0; it < iters; ++it) {
      const int c = (it * lpg + li) * V;
      float xv[V], zv[V], gv[V], ox[V], oz[V];
      Vec<T>::load(x + fbase + c, xv);
      Vec<T>::load(dy + base + c, gv);
      if (z) Vec<T>::load(z + fbase + c, zv);
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const float wv = w[g * gs + c + e];
        float u = xv[e], dyn = gv[e], gate = 1.f, dgate = 0.f;
        if (z) {
          const float sg = sigmoidf(zv[e]);
          gate = zv[e] * sg;
          dgate = sg * (1.f + zv[e] * (1.f - sg));
          if (gate_first) u *= gate; else dyn *= gate;
        }
        const float uhat = u * rstd;
        if (want_dw) atomicAdd(dw_acc + g * gs + c + e, dyn * uhat);
        const float du = rstd * (dyn * wv - uhat * mean_gu);
        if (z && gate_first) {
          ox[e] = du * gate;
          oz[e] = du * xv[e] * dgate;
        } else {
          ox[e] = du;
          oz[e] = gv[e] * uhat * wv * dgate;
        }
      }
      Vec<T>::store(dx + base + c, ox);
      if (z) Vec<T>::store(dz + base + c, oz);
    }
  }
  if (want_dw) {
    __syncthreads();
    float* out = dw_partials + (int64_t)blockIdx.x * dim;
    for (int i = threadIdx.x; i < dim; i += THREADS) out[i] = dw_acc[i];
  }
}

// The backward for wide groups (one group of thousands of channels per row, the Mamba-2 form): a block per row.  The rows of
// dy, x and z are staged in shared memory with cp.async, two stages deep, so the next row's loads are in flight while the
// current row is reduced and written (the warp-per-group kernel above walks a wide group twice with little in flight, and
// a block that keeps its row in registers leaves two rows in flight per SM).  The thread -> channel map is fixed, so the
// weight gradient accumulates in a shared array without atomics.  dw_partials [gridDim.x][dim].
// Dynamic smem: 2 stages x 3 rows x gs elements, then dim floats.
constexpr int WIDE_THREADS = 256;
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <typename T>
__global__ void __launch_bounds__(WIDE_THREADS) gated_rmsnorm_bwd_wide_kernel(
    const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ z, const float* __restrict__ w,
    const float* __restrict__ rstd_in, T* __restrict__ dx, T* __restrict__ dz, float* __restrict__ dw_partials, int64_t vrows,
    int64_t fvrows, int dim, int gs, int gate_first) {
  constexpr int V = Vec<T>::N;
  extern __shared__ __align__(16) uint8_t wide_smem[];
  __shared__ float red[WIDE_THREADS / 32];
  T* stage = reinterpret_cast<T*>(wide_smem);                                        // [2][3][gs]
  float* dw_acc = reinterpret_cast<float*>(wide_smem + (size_t)6 * gs * sizeof(T));   // [gs]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool want_dw = dw_partials != nullptr;
  if (want_dw)
    for (int i = threadIdx.x; i < gs; i += WIDE_THREADS) dw_acc[i] = 0.f;
  auto prefetch = [&](int64_t vr, int st) {
    const int64_t fvr = vr < fvrows ? vr : vr % fvrows;
    T* sx = stage + (size_t)st * 3 * gs;
    for (int c = threadIdx.x * V; c < gs; c += WIDE_THREADS * V) {
      cp_async16(sx + c, x + fvr * gs + c);
      cp_async16(sx + gs + c, dy + vr * gs + c);
      if (z) cp_async16(sx + 2 * gs + c, z + fvr * gs + c);
    }
    cp_async_commit();
  };
  int st = 0;
  if ((int64_t)blockIdx.x < vrows) prefetch(blockIdx.x, 0);
  for (int64_t vr = blockIdx.x; vr < vrows; vr += gridDim.x, st ^= 1) {
    const int64_t nxt = vr + gridDim.x;
    if (nxt < vrows) {
      prefetch(nxt, st ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int64_t fvr = vr < fvrows ? vr : vr % fvrows;
    const float rstd = rstd_in[fvr];
    const T* sx = stage + (size_t)st * 3 * gs;
    float dot = 0.f;
    for (int c = threadIdx.x * V; c < gs; c += WIDE_THREADS * V) {
      float xv[V], zv[V], gv[V], wv[V];
      Vec<T>::load(sx + c, xv);
      Vec<T>::load(sx + gs + c, gv);
      if (z) Vec<T>::load(sx + 2 * gs + c, zv);
      Vec<float>::load(w + c, wv);
      if (V == 8) Vec<float>::load(w + c + 4, wv + 4);
#pragma unroll
      for (int e = 0; e < V; ++e) {
        float u = xv[e], dyn = gv[e];
        if (z) {
          const float gate = zv[e] * sigmoidf(zv[e]);
          if (gate_first) u *= gate; else dyn *= gate;
        }
        dot = fmaf(dyn * wv[e], u * rstd, dot);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (lane == 0) red[warp] = dot;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int q = 0; q < WIDE_THREADS / 32; ++q) total += red[q];
    const float mean_gu = total / gs;
    for (int c = threadIdx.x * V; c < gs; c += WIDE_THREADS * V) {
      float xv[V], zv[V], gv[V], ox[V], oz[V], wvec[V];
      Vec<T>::load(sx + c, xv);
      Vec<T>::load(sx + gs + c, gv);
      if (z) Vec<T>::load(sx + 2 * gs + c, zv);
      Vec<float>::load(w + c, wvec);
      if (V == 8) Vec<float>::load(w + c + 4, wvec + 4);
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const float wv = wvec[e];
        float u = xv[e], dyn = gv[e], gate = 1.f, dgate = 0.f;
        if (z) {
          const float sg = sigmoidf(zv[e]);
          gate = zv[e] * sg;
          dgate = sg * (1.f + zv[e] * (1.f - sg));
          if (gate_first) u *= gate; else dyn *= gate;
        }
        const float uhat = u * rstd;
        if (want_dw) dw_acc[c + e] += dyn * uhat;   // this thread owns column c + e in every row
        const float du = rstd * (dyn * wv - uhat * mean_gu);
        if (z && gate_first) {
          ox[e] = du * gate;
          oz[e] = du * xv[e] * dgate;
        } else {
          ox[e] = du;
          oz[e] = gv[e] * uhat * wv * dgate;
        }
      }
      Vec<T>::store(dx + vr * gs + c, ox);
      if (z) Vec<T>::store(dz + vr * gs + c, oz);
    }
    __syncthreads();   // the stage is refilled by the prefetch of the next iteration; red is rewritten
  }
  if (want_dw) {
    float* out = dw_partials + (int64_t)blockIdx.x * dim;
    for (int c = threadIdx.x * V; c < gs; c += WIDE_THREADS * V)
#pragma unroll
      for (int e = 0; e < V; ++e) out[c + e] = dw_acc[c + e];
  }
}

// lanes per group: the largest power of two <= 32 that divides the number of 16-byte vectors of a group
static bool plan(int gs, int vec, int* lpg, int* iters) {
  if (gs % vec != 0) return false;
  const int nvec = gs / vec;
  int l = 32;
  while (l > 1 && nvec % l != 0) l >>= 1;
  *lpg = l;
  *iters = nvec / l;
  return true;
}

// one group per row, wide enough to occupy a block, two staged rows of dy, x, z and the weight-gradient row within 200 KB
static bool wide_shape(int dim, int gs, int vec) {
  return dim == gs && gs % vec == 0 && gs / vec > 128 && (size_t)gs * (6 * (vec == 8 ? 2 : 4) + 4) <= 200 * 1024;
}

static int grid_for(int64_t vrows, int lpg) {
  const int64_t per_block = (int64_t)WARPS * (32 / lpg);
  int64_t blocks = (vrows + per_block - 1) / per_block;
  if (blocks > 148 * 4) blocks = 148 * 4;
  return (int)(blocks < 1 ? 1 : blocks);
}

template <typename T>
static int fwd(const void* x, const void* z, const float* w, void* y, float* rstd, int64_t rows, int dim, int gs, float eps,
               int gate_first, cudaStream_t st) {
  int lpg, iters;
  if (!plan(gs, Vec<T>::N, &lpg, &iters)) return (int)cudaErrorInvalidValue;
  const int64_t vrows = rows * (dim / gs);
  gated_rmsnorm_fwd_kernel<T><<<grid_for(vrows, lpg), THREADS, 0, st>>>((const T*)x, (const T*)z, w, (T*)y, rstd, vrows, dim, gs, eps,
                                                                        gate_first, lpg, iters);
  return (int)cudaGetLastError();
}

template <typename T>
static int bwd(const void* dy, const void* x, const void* z, const float* w, const float* rstd, void* dx, void* dz,
               float* dw_partials, int64_t rows, int64_t frows, int dim, int gs, int gate_first, cudaStream_t st) {
  int lpg, iters;
  if (!plan(gs, Vec<T>::N, &lpg, &iters)) return (int)cudaErrorInvalidValue;
  if (frows <= 0 || rows % frows != 0) return (int)cudaErrorInvalidValue;
  const int64_t vrows = rows * (dim / gs), fvrows = frows * (dim / gs);
  if (wide_shape(dim, gs, Vec<T>::N)) {
    const size_t wide = (size_t)6 * gs * sizeof(T) + (size_t)gs * sizeof(float);
    static PerDeviceOnce configured_wide;
    cudaError_t e = configured_wide.max_dynamic_smem(gated_rmsnorm_bwd_wide_kernel<T>, 200 * 1024);
    if (e != cudaSuccess) return (int)e;
    gated_rmsnorm_bwd_wide_kernel<T><<<grid_for(vrows, 32), WIDE_THREADS, wide, st>>>((const T*)dy, (const T*)x, (const T*)z, w, rstd, (T*)dx,
                                                                                   (T*)dz, dw_partials, vrows, fvrows, dim, gs, gate_first);
    return (int)cudaGetLastError();
  }
  const size_t smem = (size_t)dim * sizeof(float);
  int rc = (int)cudaFuncSetAttribute(gated_rmsnorm_bwd_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (rc) return rc;
  gated_rmsnorm_bwd_kernel<T><<<grid_for(vrows, lpg), THREADS, smem, st>>>((const T*)dy, (const T*)x, (const T*)z, w, rstd, (T*)dx, (T*)dz,
                                                                           dw_partials, vrows, fvrows, dim, gs, gate_first, lpg, iters);
  return (int)cudaGetLastError();
}

}  // namespace gnorm
}  // namespace lbi

// Rows of the weight-gradient partials buffer for this shape (0: shape not supported).  The element size decides the
// vector width, so the bf16 / fp32 answer can differ.
extern "C" int lbi_gated_rmsnorm_slots(int64_t rows, int dim, int group_size, int is_bf16) {
  using namespace lbi::gnorm;
  int lpg, iters;
  if (rows <= 0 || dim <= 0 || group_size <= 0 || dim % group_size != 0 || !plan(group_size, is_bf16 ? 8 : 4, &lpg, &iters)) return 0;
  if (wide_shape(dim, group_size, is_bf16 ? 8 : 4)) lpg = 32;   // the wide backward kernel: one row per block at a time
  return grid_for(rows * (dim / group_size), lpg);
}

extern "C" int lbi_gated_rmsnorm_fwd(const void* x, const void* z_or_null, const float* weight, void* y, float* rstd, int64_t rows,
                                     int dim, int group_size, float eps, int gate_first, int is_bf16, cudaStream_t st) {
  if (rows <= 0 || dim <= 0 || group_size <= 0 || dim % group_size != 0) return (int)cudaErrorInvalidValue;
  return is_bf16 ? lbi::gnorm::fwd<__nv_bfloat16>(x, z_or_null, weight, y, rstd, rows, dim, group_size, eps, gate_first, st)
                 : lbi::gnorm::fwd<float>(x, z_or_null, weight, y, rstd, rows, dim, group_size, eps, gate_first, st);
}

extern "C" int lbi_gated_rmsnorm_bwd(const void* dy, const void* x, const void* z_or_null, const float* weight, const float* rstd,
                                     void* dx, void* dz_or_null, float* dw_partials, int64_t rows, int64_t frows, int dim,
                                     int group_size, int gate_first, int is_bf16, cudaStream_t st) {
  if (rows <= 0 || dim <= 0 || group_size <= 0 || dim % group_size != 0 || dim > 12288) return (int)cudaErrorInvalidValue;
  return is_bf16 ? lbi::gnorm::bwd<__nv_bfloat16>(dy, x, z_or_null, weight, rstd, dx, dz_or_null, dw_partials, rows, frows, dim,
                                                  group_size, gate_first, st)
                 : lbi::gnorm::bwd<float>(dy, x, z_or_null, weight, rstd, dx, dz_or_null, dw_partials, rows, frows, dim, group_size,
                                          gate_first, st);
}
