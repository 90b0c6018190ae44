// Mamba-3 SISO preprocessing of the state-mixer operands, forward and backward, on the wide tensors.
//
// Per (batch, token, head) with Qh = Q[group] + Q_bias[head], Kh = K[group] + K_bias[head] (d_state = 128 wide):
//     qk_dot = gamma * (Qh . Kh)
//     Qr     = rot(Qh, theta)                 pairs (2i, 2i + 1), i < n_angles, turn by theta_i; the rest stays
//     Kr     = rot(Kh, theta) * scale
// gamma, scale (trapezoid weights) and theta (cumulative rotary phase) are [batch, token, head(, angle)] tensors that
// the caller forms with small PyTorch ops; what runs here is everything that touches [batch, token, head, 128].
// Backward, from dQr, dKr (fp32) and dqk:
//     dQh = rot^-1(dQr) + dqk gamma Kh         dKh = scale rot^-1(dKr) + dqk gamma Qh
//     dQ[group] = sum over heads dQh,  dQ_bias[head] = sum over (batch, token) dQh        (same for K)
//     dtheta_i = <dQr_pair, J rot(Qh)_pair> + scale <dKr_pair, J rot(Kh)_pair>,  J (a, b) = (-b, a)
//     dgamma = dqk (Qh . Kh),   dscale = dKr . rot(Kh)
// One warp owns one (batch, token, group) and walks the heads of the group: four state elements (two pairs) per lane.
// The bias gradients accumulate in shared memory per block and leave as one row of a partials buffer.
// Replaces phase 1 of the reference's mamba3_siso_fwd_kernel and its mamba3_siso_bwd_kernel_rotary_bias_angles
// (backbones/mamba3/ops/triton/mamba3/mamba3_siso_fwd.py:29, mamba3_siso_bwd.py:811) for d_state 128.
#include "api.h"
#include "common.cuh"

namespace lbi {
namespace sisoprep {

constexpr int N = 128;
constexpr int THREADS = 256;
constexpr int WARPS = THREADS / 32;

template <typename T>
__device__ __forceinline__ float4 ld4(const T* p);
template <>
__device__ __forceinline__ float4 ld4<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 ld4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st4_bf16(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 o;
  o.x = *reinterpret_cast<uint32_t*>(&a);
  o.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = o;
}

struct Rot {
  float c0, s0, c1, s1;   // cos / sin of the lane's two pairs (1, 0 where the pair is not rotated)
};

__device__ __forceinline__ Rot load_rot(const float* theta_row, int lane, int n_angles) {
  Rot r{1.f, 0.f, 1.f, 0.f};
  const int i0 = 2 * lane, i1 = 2 * lane + 1;
  if (i0 < n_angles) __sincosf(theta_row[i0], &r.s0, &r.c0);
  if (i1 < n_angles) __sincosf(theta_row[i1], &r.s1, &r.c1);
  return r;
}
__device__ __forceinline__ float4 rotate(float4 v, const Rot& r) {
  return make_float4(v.x * r.c0 - v.y * r.s0, v.x * r.s0 + v.y * r.c0, v.z * r.c1 - v.w * r.s1, v.z * r.s1 + v.w * r.c1);
}
__device__ __forceinline__ float4 rotate_back(float4 v, const Rot& r) {
  return make_float4(v.x * r.c0 + v.y * r.s0, -v.x * r.s0 + v.y * r.c0, v.z * r.c1 + v.w * r.s1, -v.z * r.s1 + v.w * r.c1);
}

// grid-stride over (batch * token * group) rows, one warp per row
template <typename T>
__global__ void __launch_bounds__(THREADS) fwd_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                      const float* __restrict__ q_bias, const float* __restrict__ k_bias,
                                                      const float* __restrict__ theta, const float* __restrict__ gamma,
                                                      const float* __restrict__ scale, __nv_bfloat16* __restrict__ qr,
                                                      __nv_bfloat16* __restrict__ kr, float* __restrict__ qk_dot, int64_t rows,
                                                      int groups, int heads, int n_angles) {
  const int lane = threadIdx.x & 31;
  const int rep = heads / groups;
  for (int64_t row = (int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5); row < rows; row += (int64_t)gridDim.x * WARPS) {
    const int g = (int)(row % groups);
    const int64_t tok = row / groups;
    const float4 qg = ld4<T>(q + row * N + lane * 4), kg = ld4<T>(k + row * N + lane * 4);
    for (int r = 0; r < rep; ++r) {
      const int h = g * rep + r;
      const int64_t hrow = tok * heads + h;
      const float4 qb = ld4<float>(q_bias + h * N + lane * 4), kb = ld4<float>(k_bias + h * N + lane * 4);
      const float4 qh = make_float4(qg.x + qb.x, qg.y + qb.y, qg.z + qb.z, qg.w + qb.w);
      const float4 kh = make_float4(kg.x + kb.x, kg.y + kb.y, kg.z + kb.z, kg.w + kb.w);
      const Rot rot = load_rot(theta + hrow * n_angles, lane, n_angles);
      const float sc = scale[hrow];
      const float4 qo = rotate(qh, rot);
      float4 ko = rotate(kh, rot);
      ko = make_float4(ko.x * sc, ko.y * sc, ko.z * sc, ko.w * sc);
      st4_bf16(qr + hrow * N + lane * 4, qo);
      st4_bf16(kr + hrow * N + lane * 4, ko);
      const float dot = warp_sum(qh.x * kh.x + qh.y * kh.y + qh.z * kh.z + qh.w * kh.w);
      if (lane == 0) qk_dot[hrow] = gamma[hrow] * dot;
    }
  }
}

// bias_partials [gridDim.x][2][heads][N]
// T: dtype of q, k; C: dtype of the cotangents dqr, dkr.  The forward tensors (q, k, theta, gamma, scale) hold `frows` rows
// (tokens x groups) and are shared by rows / frows stacked directions of the cotangents.
// What one head of one (token, group) row reads: loaded one head ahead of its use, so that the loads of head r + 1 are in
// flight while the shuffles and stores of head r run (the stores in the loop body keep the compiler from hoisting them itself).
struct HeadIn {
  float4 gq, gk, qb, kb;
  float th0, th1, sc, gm, dd;
};

template <typename C>
__device__ __forceinline__ HeadIn load_head(const float* __restrict__ q_bias, const float* __restrict__ k_bias,
                                            const float* __restrict__ theta, const float* __restrict__ gamma,
                                            const float* __restrict__ scale, const C* __restrict__ dqr, const C* __restrict__ dkr,
                                            const float* __restrict__ dqk, int64_t tok, int64_t ftok, int64_t ktok, int h, int heads,
                                            int n_angles, int lane) {
  // ktok: the row of dkr that holds token `tok` (the same token, or its place in the reversed, padded layout); computed once
  // per token by the caller (it takes a 64-bit division)
  HeadIn in;
  const int64_t hrow = tok * heads + h, fhrow = ftok * heads + h;
  const int64_t krow = ktok * heads + h;
  in.gq = ld4<C>(dqr + hrow * N + lane * 4);
  in.gk = ld4<C>(dkr + krow * N + lane * 4);
  in.qb = ld4<float>(q_bias + h * N + lane * 4);
  in.kb = ld4<float>(k_bias + h * N + lane * 4);
  in.th0 = 2 * lane < n_angles ? theta[fhrow * n_angles + 2 * lane] : 0.f;
  in.th1 = 2 * lane + 1 < n_angles ? theta[fhrow * n_angles + 2 * lane + 1] : 0.f;
  in.sc = scale[fhrow];
  in.gm = gamma[fhrow];
  in.dd = dqk[hrow];
  return in;
}

template <typename T, typename C>
__global__ void __launch_bounds__(THREADS, 3) bwd_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                      const float* __restrict__ q_bias, const float* __restrict__ k_bias,
                                                      const float* __restrict__ theta, const float* __restrict__ gamma,
                                                      const float* __restrict__ scale, const C* __restrict__ dqr,
                                                      const C* __restrict__ dkr, const float* __restrict__ dqk,
                                                      float* __restrict__ dq, float* __restrict__ dk, float* __restrict__ dtheta,
                                                      float* __restrict__ dgamma, float* __restrict__ dscale,
                                                      float* __restrict__ bias_partials, int64_t rows, int64_t frows, int groups,
                                                      int heads, int n_angles, int seq_len, int dkr_pad) {
  // dkr_pad > 0: dkr is [batch, dkr_pad, heads, N] in reversed time (token l of a sequence sits in row dkr_pad - 1 - l)
  // bias_partials == nullptr: the bias gradients are not wanted (a pullback pass) and nothing is accumulated for them
  extern __shared__ float bias_acc[];   // [2][heads][N]
  const int lane = threadIdx.x & 31;
  const int rep = heads / groups;
  const bool want_bias = bias_partials != nullptr;
  if (want_bias) {
    for (int i = threadIdx.x; i < 2 * heads * N; i += THREADS) bias_acc[i] = 0.f;
    __syncthreads();
  }
  for (int64_t row = (int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5); row < rows; row += (int64_t)gridDim.x * WARPS) {
    // 64-bit divisions cost a hundred instructions each: one group and one direction per row are the common cases
    const int g = groups == 1 ? 0 : (int)(row % groups);
    const int64_t tok = groups == 1 ? row : row / groups;
    const int64_t frow = row < frows ? row : row % frows, ftok = groups == 1 ? frow : frow / groups;
    const float4 qg = ld4<T>(q + frow * N + lane * 4), kg = ld4<T>(k + frow * N + lane * 4);
    float4 dq_sum = make_float4(0.f, 0.f, 0.f, 0.f), dk_sum = make_float4(0.f, 0.f, 0.f, 0.f);
    const int64_t ktok = dkr_pad > 0 ? (tok / seq_len) * dkr_pad + (dkr_pad - 1 - tok % seq_len) : tok;
    HeadIn cur = load_head<C>(q_bias, k_bias, theta, gamma, scale, dqr, dkr, dqk, tok, ftok, ktok, g * rep, heads, n_angles, lane);
    for (int r = 0; r < rep; ++r) {
      const int h = g * rep + r;
      const int64_t hrow = tok * heads + h;
      HeadIn nxt = cur;
      if (r + 1 < rep)
        nxt = load_head<C>(q_bias, k_bias, theta, gamma, scale, dqr, dkr, dqk, tok, ftok, ktok, h + 1, heads, n_angles, lane);
      const float4 qh = make_float4(qg.x + cur.qb.x, qg.y + cur.qb.y, qg.z + cur.qb.z, qg.w + cur.qb.w);
      const float4 kh = make_float4(kg.x + cur.kb.x, kg.y + cur.kb.y, kg.z + cur.kb.z, kg.w + cur.kb.w);
      Rot rot{1.f, 0.f, 1.f, 0.f};
      if (2 * lane < n_angles) __sincosf(cur.th0, &rot.s0, &rot.c0);
      if (2 * lane + 1 < n_angles) __sincosf(cur.th1, &rot.s1, &rot.c1);
      const float sc = cur.sc, gm = cur.gm, dd = cur.dd;
      const float4 gq = cur.gq, gk = cur.gk;
      const float4 qo = rotate(qh, rot), ko = rotate(kh, rot);   // ko without the scale
      // angle gradients: J (a, b) = (-b, a) applied to the rotated pair
      const float dth0 = (-gq.x * qo.y + gq.y * qo.x) + sc * (-gk.x * ko.y + gk.y * ko.x);
      const float dth1 = (-gq.z * qo.w + gq.w * qo.z) + sc * (-gk.z * ko.w + gk.w * ko.z);
      if ((n_angles & 1) == 0) {   // rows of an even number of angles keep the pair 8-byte aligned
        if (2 * lane < n_angles) *reinterpret_cast<float2*>(dtheta + hrow * n_angles + 2 * lane) = make_float2(dth0, dth1);
      } else {
        if (2 * lane < n_angles) dtheta[hrow * n_angles + 2 * lane] = dth0;
        if (2 * lane + 1 < n_angles) dtheta[hrow * n_angles + 2 * lane + 1] = dth1;
      }
      float dsc = gk.x * ko.x + gk.y * ko.y + gk.z * ko.z + gk.w * ko.w;
      float qk = qh.x * kh.x + qh.y * kh.y + qh.z * kh.z + qh.w * kh.w;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {   // the two reductions interleaved: independent shuffles issue back to back
        dsc += __shfl_xor_sync(0xffffffffu, dsc, o);
        qk += __shfl_xor_sync(0xffffffffu, qk, o);
      }
      if (lane == 0) {
        dscale[hrow] = dsc;
        dgamma[hrow] = dd * qk;
      }
      float4 dqh = rotate_back(gq, rot);
      float4 dkh = rotate_back(make_float4(gk.x * sc, gk.y * sc, gk.z * sc, gk.w * sc), rot);
      const float w = dd * gm;
      dqh = make_float4(dqh.x + w * kh.x, dqh.y + w * kh.y, dqh.z + w * kh.z, dqh.w + w * kh.w);
      dkh = make_float4(dkh.x + w * qh.x, dkh.y + w * qh.y, dkh.z + w * qh.z, dkh.w + w * qh.w);
      dq_sum = make_float4(dq_sum.x + dqh.x, dq_sum.y + dqh.y, dq_sum.z + dqh.z, dq_sum.w + dqh.w);
      dk_sum = make_float4(dk_sum.x + dkh.x, dk_sum.y + dkh.y, dk_sum.z + dkh.z, dk_sum.w + dkh.w);
      if (want_bias) {
        float* bq = bias_acc + (int64_t)h * N + lane * 4;
        float* bk = bias_acc + (int64_t)(heads + h) * N + lane * 4;
        atomicAdd(bq, dqh.x); atomicAdd(bq + 1, dqh.y); atomicAdd(bq + 2, dqh.z); atomicAdd(bq + 3, dqh.w);
        atomicAdd(bk, dkh.x); atomicAdd(bk + 1, dkh.y); atomicAdd(bk + 2, dkh.z); atomicAdd(bk + 3, dkh.w);
      }
      cur = nxt;
    }
    *reinterpret_cast<float4*>(dq + row * N + lane * 4) = dq_sum;
    *reinterpret_cast<float4*>(dk + row * N + lane * 4) = dk_sum;
  }
  if (want_bias) {
    __syncthreads();
    float* out = bias_partials + (int64_t)blockIdx.x * 2 * heads * N;
    for (int i = threadIdx.x; i < 2 * heads * N; i += THREADS) out[i] = bias_acc[i];
  }
}

// The same backward with two heads per warp step: lanes 0 - 15 take head 2i, lanes 16 - 31 head 2i + 1 of the row's group,
// eight elements per lane.  The per-head bookkeeping (addresses, scalar loads, the shuffle reductions, the scalar stores)
// is issued once per pair of heads and the reductions are four levels deep; the kernel above is bound by instruction issue
// (about 290 warp instructions per token and head), not by memory.  Needs an even number of heads per group and
// n_angles % 4 == 0 (a lane's four rotation pairs are read as one vector); bias gradients go through the kernel above.
template <typename Cc>
struct Raw8;
template <>
struct Raw8<__nv_bfloat16> {
  uint4 v;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { v = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void unpack(float* f) const {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.z));
    const float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.w));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
  }
};
template <>
struct Raw8<float> {
  float4 lo, hi;
  __device__ __forceinline__ void load(const float* p) {
    lo = reinterpret_cast<const float4*>(p)[0];
    hi = reinterpret_cast<const float4*>(p)[1];
  }
  __device__ __forceinline__ void unpack(float* f) const {
    f[0] = lo.x; f[1] = lo.y; f[2] = lo.z; f[3] = lo.w; f[4] = hi.x; f[5] = hi.y; f[6] = hi.z; f[7] = hi.w;
  }
};

template <typename C>
struct PairIn {        // what a lane reads per head of the cotangents and the per-head scalars, loaded one step ahead
  Raw8<C> gq, gk;
  float4 th;
  float sc, gm, dd;
};

template <typename T, typename C>
__global__ void __launch_bounds__(THREADS, 2) bwd_pair_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                              const float* __restrict__ q_bias, const float* __restrict__ k_bias,
                                                              const float* __restrict__ theta, const float* __restrict__ gamma,
                                                              const float* __restrict__ scale, const C* __restrict__ dqr,
                                                              const C* __restrict__ dkr, const float* __restrict__ dqk,
                                                              float* __restrict__ dq, float* __restrict__ dk, float* __restrict__ dtheta,
                                                              float* __restrict__ dgamma, float* __restrict__ dscale, int64_t rows,
                                                              int64_t frows, int groups, int heads, int n_angles, int seq_len,
                                                              int dkr_pad) {
  const int lane = threadIdx.x & 31, half = lane >> 4, li = lane & 15;
  const int rep = heads / groups;
  const bool turns = 4 * li < n_angles;   // this lane's four pairs are rotated
  for (int64_t row = (int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5); row < rows; row += (int64_t)gridDim.x * WARPS) {
    const int g = groups == 1 ? 0 : (int)(row % groups);
    const int64_t tok = groups == 1 ? row : row / groups;
    const int64_t frow = row < frows ? row : row % frows, ftok = groups == 1 ? frow : frow / groups;
    const int64_t ktok = dkr_pad > 0 ? (tok / seq_len) * dkr_pad + (dkr_pad - 1 - tok % seq_len) : tok;
    float qg[8], kg[8];
    {
      Raw8<T> a, b;
      a.load(q + frow * N + li * 8);
      b.load(k + frow * N + li * 8);
      a.unpack(qg);
      b.unpack(kg);
    }
    float dq_sum[8], dk_sum[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) dq_sum[e] = dk_sum[e] = 0.f;
    auto load_pair = [&](int r2) {
      PairIn<C> in;
      const int h = g * rep + 2 * r2 + half;
      const int64_t hrow = tok * heads + h, fhrow = ftok * heads + h, krow = ktok * heads + h;
      in.gq.load(dqr + hrow * N + li * 8);
      in.gk.load(dkr + krow * N + li * 8);
      in.th = turns ? *reinterpret_cast<const float4*>(theta + fhrow * n_angles + 4 * li) : make_float4(0.f, 0.f, 0.f, 0.f);
      in.sc = scale[fhrow];
      in.gm = gamma[fhrow];
      in.dd = dqk[hrow];
      return in;
    };
    PairIn<C> cur = load_pair(0);
    for (int r2 = 0; r2 < rep / 2; ++r2) {
      const int h = g * rep + 2 * r2 + half;
      const int64_t hrow = tok * heads + h;
      PairIn<C> nxt = cur;
      if (r2 + 1 < rep / 2) nxt = load_pair(r2 + 1);
      float qh[8], kh[8], gq[8], gk[8];
      {
        const float4 b0 = *reinterpret_cast<const float4*>(q_bias + h * N + li * 8), b1 = *reinterpret_cast<const float4*>(q_bias + h * N + li * 8 + 4);
        const float4 c0 = *reinterpret_cast<const float4*>(k_bias + h * N + li * 8), c1 = *reinterpret_cast<const float4*>(k_bias + h * N + li * 8 + 4);
        qh[0] = qg[0] + b0.x; qh[1] = qg[1] + b0.y; qh[2] = qg[2] + b0.z; qh[3] = qg[3] + b0.w;
        qh[4] = qg[4] + b1.x; qh[5] = qg[5] + b1.y; qh[6] = qg[6] + b1.z; qh[7] = qg[7] + b1.w;
        kh[0] = kg[0] + c0.x; kh[1] = kg[1] + c0.y; kh[2] = kg[2] + c0.z; kh[3] = kg[3] + c0.w;
        kh[4] = kg[4] + c1.x; kh[5] = kg[5] + c1.y; kh[6] = kg[6] + c1.z; kh[7] = kg[7] + c1.w;
      }
      cur.gq.unpack(gq);
      cur.gk.unpack(gk);
      float cs[4] = {1.f, 1.f, 1.f, 1.f}, sn[4] = {0.f, 0.f, 0.f, 0.f};
      if (turns) {
        __sincosf(cur.th.x, &sn[0], &cs[0]);
        __sincosf(cur.th.y, &sn[1], &cs[1]);
        __sincosf(cur.th.z, &sn[2], &cs[2]);
        __sincosf(cur.th.w, &sn[3], &cs[3]);
      }
      const float sc = cur.sc, w = cur.dd * cur.gm;
      float dth[4];
      float dsc = 0.f, qk = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float qa = qh[2 * j], qb2 = qh[2 * j + 1], ka = kh[2 * j], kb2 = kh[2 * j + 1];
        // rotated pairs (ko without the scale)
        const float qoa = qa * cs[j] - qb2 * sn[j], qob = qa * sn[j] + qb2 * cs[j];
        const float koa = ka * cs[j] - kb2 * sn[j], kob = ka * sn[j] + kb2 * cs[j];
        const float gqa = gq[2 * j], gqb = gq[2 * j + 1], gka = gk[2 * j], gkb = gk[2 * j + 1];
        dth[j] = (-gqa * qob + gqb * qoa) + sc * (-gka * kob + gkb * koa);   // J (a, b) = (-b, a) applied to the rotated pair
        dsc = fmaf(gka, koa, fmaf(gkb, kob, dsc));
        qk = fmaf(qa, ka, fmaf(qb2, kb2, qk));
        // back through the rotation, plus the q . k term
        const float dqa = gqa * cs[j] + gqb * sn[j] + w * ka, dqb = -gqa * sn[j] + gqb * cs[j] + w * kb2;
        const float dka = sc * (gka * cs[j] + gkb * sn[j]) + w * qa, dkb = sc * (-gka * sn[j] + gkb * cs[j]) + w * qb2;
        dq_sum[2 * j] += dqa; dq_sum[2 * j + 1] += dqb;
        dk_sum[2 * j] += dka; dk_sum[2 * j + 1] += dkb;
      }
      if (turns) *reinterpret_cast<float4*>(dtheta + hrow * n_angles + 4 * li) = make_float4(dth[0], dth[1], dth[2], dth[3]);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) {   // sums over the sixteen lanes of the head, the two reductions interleaved
        dsc += __shfl_xor_sync(0xffffffffu, dsc, o);
        qk += __shfl_xor_sync(0xffffffffu, qk, o);
      }
      if (li == 0) {
        dscale[hrow] = dsc;
        dgamma[hrow] = cur.dd * qk;
      }
      cur = nxt;
    }
    // the two halves hold the sums of the even and the odd heads
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      dq_sum[e] += __shfl_xor_sync(0xffffffffu, dq_sum[e], 16);
      dk_sum[e] += __shfl_xor_sync(0xffffffffu, dk_sum[e], 16);
    }
    float* dst = (half == 0 ? dq : dk) + row * N + li * 8;
    const float* src = half == 0 ? dq_sum : dk_sum;
    reinterpret_cast<float4*>(dst)[0] = make_float4(src[0], src[1], src[2], src[3]);
    reinterpret_cast<float4*>(dst)[1] = make_float4(src[4], src[5], src[6], src[7]);
  }
}

static int grid_for(int64_t rows) {
  int64_t blocks = (rows + WARPS - 1) / WARPS;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return (int)(blocks < 1 ? 1 : blocks);
}

}  // namespace sisoprep
}  // namespace lbi

extern "C" int lbi_siso_prep_blocks(int64_t rows) { return lbi::sisoprep::grid_for(rows); }

extern "C" int lbi_siso_prep_fwd(const void* q, const void* k, const float* q_bias, const float* k_bias, const float* theta,
                                 const float* gamma, const float* scale, void* qr_bf16, void* kr_bf16, float* qk_dot,
                                 int64_t tokens, int groups, int heads, int d_state, int n_angles, int is_bf16, cudaStream_t st) {
  using namespace lbi::sisoprep;
  if (d_state != N || tokens <= 0 || groups <= 0 || heads % groups != 0 || n_angles < 0 || 2 * n_angles > N) return (int)cudaErrorInvalidValue;
  const int64_t rows = tokens * groups;
  const int blocks = grid_for(rows);
  if (is_bf16)
    fwd_kernel<__nv_bfloat16><<<blocks, THREADS, 0, st>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k, q_bias, k_bias, theta, gamma,
                                                         scale, (__nv_bfloat16*)qr_bf16, (__nv_bfloat16*)kr_bf16, qk_dot, rows, groups,
                                                         heads, n_angles);
  else
    fwd_kernel<float><<<blocks, THREADS, 0, st>>>((const float*)q, (const float*)k, q_bias, k_bias, theta, gamma, scale,
                                                 (__nv_bfloat16*)qr_bf16, (__nv_bfloat16*)kr_bf16, qk_dot, rows, groups, heads, n_angles);
  return (int)cudaGetLastError();
}

namespace lbi {
namespace sisoprep {
template <typename T, typename C>
static int launch_bwd(const void* q, const void* k, const float* q_bias, const float* k_bias, const float* theta, const float* gamma,
                      const float* scale, const void* dqr, const void* dkr, const float* dqk, float* dq, float* dk, float* dtheta,
                      float* dgamma, float* dscale, float* bias_partials, int64_t rows, int64_t frows, int groups, int heads,
                      int n_angles, int seq_len, int dkr_pad, cudaStream_t st) {
  const int blocks = grid_for(rows);
  if (!bias_partials && (heads / groups) % 2 == 0 && n_angles % 4 == 0 && n_angles > 0) {
    bwd_pair_kernel<T, C><<<blocks, THREADS, 0, st>>>((const T*)q, (const T*)k, q_bias, k_bias, theta, gamma, scale, (const C*)dqr,
                                                      (const C*)dkr, dqk, dq, dk, dtheta, dgamma, dscale, rows, frows, groups, heads,
                                                      n_angles, seq_len, dkr_pad);
    return (int)cudaGetLastError();
  }
  const size_t smem = (size_t)2 * heads * N * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  static PerDeviceOnce configured;
  cudaError_t e = configured.max_dynamic_smem(bwd_kernel<T, C>, (int)(200 * 1024));
  if (e != cudaSuccess) return (int)e;
  bwd_kernel<T, C><<<blocks, THREADS, smem, st>>>((const T*)q, (const T*)k, q_bias, k_bias, theta, gamma, scale, (const C*)dqr,
                                                  (const C*)dkr, dqk, dq, dk, dtheta, dgamma, dscale, bias_partials, rows, frows, groups,
                                                  heads, n_angles, seq_len, dkr_pad);
  return (int)cudaGetLastError();
}
}  // namespace sisoprep
}  // namespace lbi

extern "C" int lbi_siso_prep_bwd(const void* q, const void* k, const float* q_bias, const float* k_bias, const float* theta,
                                 const float* gamma, const float* scale, const void* dqr, const void* dkr, const float* dqk,
                                 float* dq, float* dk, float* dtheta, float* dgamma, float* dscale, float* bias_partials,
                                 int64_t tokens, int64_t ftokens, int seq_len, int dkr_pad, int groups, int heads, int d_state,
                                 int n_angles, int is_bf16, int cot_bf16, cudaStream_t st) {
  using namespace lbi::sisoprep;
  if (seq_len <= 0 || tokens % seq_len != 0 || (dkr_pad > 0 && dkr_pad < seq_len)) return (int)cudaErrorInvalidValue;
  if (ftokens <= 0 || tokens % ftokens != 0 || ftokens % seq_len != 0) return (int)cudaErrorInvalidValue;
  if (d_state != N || tokens <= 0 || groups <= 0 || heads % groups != 0 || n_angles < 0 || 2 * n_angles > N) return (int)cudaErrorInvalidValue;
  const int64_t rows = tokens * groups, frows = ftokens * groups;
#define LBI_PREP_BWD(T, C)                                                                                                      \
  return launch_bwd<T, C>(q, k, q_bias, k_bias, theta, gamma, scale, dqr, dkr, dqk, dq, dk, dtheta, dgamma, dscale, bias_partials, \
                          rows, frows, groups, heads, n_angles, seq_len, dkr_pad, st)
  if (is_bf16 && cot_bf16) LBI_PREP_BWD(__nv_bfloat16, __nv_bfloat16);
  if (is_bf16) LBI_PREP_BWD(__nv_bfloat16, float);
  if (cot_bf16) LBI_PREP_BWD(float, __nv_bfloat16);
  LBI_PREP_BWD(float, float);
#undef LBI_PREP_BWD
}
