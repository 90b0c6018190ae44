// Mamba block glue on the small tensors: the SiLU gate and the per-token, per-head scalars of the Mamba-3 SISO mixer.
//
// 1. gate            yg = y * silu(z), and its pullback for P stacked directions that share y and z.
// 2. siso small fwd  DT = softplus(dd_dt + bias), A = min(-softplus(dd_A), -floor), ADT = A DT, the trapezoid weights
//                    gamma_t = DT_t sigmoid(trap_t), scale_t = gamma_t + DT_{t+1} (1 - sigmoid(trap_{t+1})), and the rotary phase
//                    theta_t = (sum_{i <= t} pi tanh(angle_i) DT_i) mod 2 pi  (a running sum over the tokens of a sequence).
// 3. siso small bwd  cotangents of (ADT, theta, gamma, scale) -> cotangents of the four in_proj slices (dd_dt, dd_A, trap,
//                    angles); the running sum turns into a reversed running sum of dtheta.
// One warp owns one head, its lanes the rotary angles; a block walks the tokens of one sequence.  They replace the
// reference's Triton kernels angle_dt_fwd / angle_dt_bwd (backbones/mamba3/ops/triton/mamba3/angle_dt.py:26, 234) and
// the dd_dt / trap part of its backward (mamba3_siso_bwd.py:1418).
#include "api.h"
#include "common.cuh"

namespace lbi {
namespace msmall {

constexpr float PI_F = 3.14159265358979323846f;
constexpr float TWO_PI_F = 6.28318530717958647692f;

__device__ __forceinline__ float softplus_(float v) { return v > 20.f ? v : log1pf(__expf(v)); }

// ------------------------------------------------------------------------------------------------ gate
__global__ void gate_silu_fwd_kernel(const bf16x8* __restrict__ y, const bf16x8* __restrict__ z, bf16x8* __restrict__ out, int64_t n8) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    float a[8], b[8];
    unpack8(y[i], a);
    unpack8(z[i], b);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] *= b[j] * sigmoidf_(b[j]);
    out[i] = pack8(a);
  }
}

// dyg [reps * n8]; y, z [n8] shared by the reps directions.
__global__ void gate_silu_bwd_kernel(const bf16x8* __restrict__ dyg, const bf16x8* __restrict__ y, const bf16x8* __restrict__ z,
                                     bf16x8* __restrict__ dy, bf16x8* __restrict__ dz, int64_t n8, int reps, int cols8, int64_t ld_dz8) {
  // dz rows may be strided (a column range of a wider cotangent matrix): row r of direction rep sits at
  // dz + (rep * rows + r) * ld_dz8 vectors; cols8 = vectors per row; ld_dz8 == cols8 is the contiguous case
  const int64_t rows = n8 / cols8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    float yv[8], zv[8], silu[8], slope[8];
    unpack8(y[i], yv);
    unpack8(z[i], zv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = sigmoidf_(zv[j]);
      silu[j] = zv[j] * s;
      slope[j] = yv[j] * s * (1.f + zv[j] * (1.f - s));
    }
    const int64_t row = i / cols8;
    const int col = (int)(i - row * cols8);
    for (int r = 0; r < reps; ++r) {
      float g[8], a[8], b[8];
      unpack8(dyg[(int64_t)r * n8 + i], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        a[j] = g[j] * silu[j];
        b[j] = g[j] * slope[j];
      }
      dy[(int64_t)r * n8 + i] = pack8(a);
      dz[((int64_t)r * rows + row) * ld_dz8 + col] = pack8(b);
    }
  }
}

// ------------------------------------------------------------------------------------------------ Mamba-2 step size
// dt = clamp(softplus(dt_raw + bias), lo, hi), slope = d dt / d dt_raw = sigmoid(dt_raw + bias) inside the limits, 0 outside.
// dt_raw [rows, heads] with a row stride (a column range of the in_proj output), bf16 or fp32; outputs fp32, contiguous.
template <typename T>
__global__ void softplus_dt_kernel(const T* __restrict__ dt_raw, int64_t ld, const float* __restrict__ bias, float lo, float hi,
                                   float* __restrict__ dt, float* __restrict__ slope, int64_t rows, int heads) {
  const int64_t total = rows * heads;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / heads;
    const int h = (int)(i - r * heads);
    const float pre = (float)dt_raw[r * ld + h] + bias[h];
    const float v = softplus_(pre);
    const bool inside = v >= lo && v <= hi;
    dt[i] = fminf(fmaxf(v, lo), hi);
    slope[i] = inside ? sigmoidf_(pre) : 0.f;
  }
}

// ------------------------------------------------------------------------------------------------ siso small, forward
// The running rotary phase is the only dependency along the sequence: the sequence is cut into segments of FSEG tokens, a first
// kernel sums the phase increments pi tanh(angle) DT per (sequence, segment, head, angle), and a block of the second kernel
// starts its running phase from the totals of the earlier segments (taken modulo 2 pi like the running value itself).
constexpr int FSEG = 128;   // tokens per segment (a multiple of 32)

// grid (batch, segments), block = heads * 32: seg_inc[b][seg][h][64]
__global__ void __launch_bounds__(1024) phase_segment_sums_kernel(const float* __restrict__ dd_dt, const float* __restrict__ angles,
                                                                  const float* __restrict__ dt_bias, float* __restrict__ seg_inc,
                                                                  int seq_len, int heads, int n_angles) {
  const int h = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x, seg = blockIdx.y;
  const int t_lo = seg * FSEG, t_hi = min(seq_len, t_lo + FSEG);
  const float bias = dt_bias[h];
  const bool has0 = lane < n_angles, has1 = lane + 32 < n_angles;
  const int64_t row0 = (int64_t)b * seq_len;
  float acc0 = 0.f, acc1 = 0.f;
  for (int t0 = t_lo; t0 < t_hi; t0 += 4) {
    float dts[4], a0[4], a1[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {   // the loads of four tokens go out together
      const int t = t0 + j;
      const bool ok = t < t_hi;
      dts[j] = ok ? dd_dt[(row0 + t) * heads + h] : 0.f;
      a0[j] = (ok && has0) ? angles[(row0 + t) * n_angles + lane] : 0.f;
      a1[j] = (ok && has1) ? angles[(row0 + t) * n_angles + lane + 32] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (t0 + j < t_hi) {
        const float dtv = softplus_(dts[j] + bias);
        acc0 += PI_F * tanhf(a0[j]) * dtv;
        acc1 += PI_F * tanhf(a1[j]) * dtv;
      }
    }
  }
  float* out = seg_inc + (((int64_t)b * gridDim.y + seg) * heads + h) * 64;
  out[lane] = acc0;
  out[lane + 32] = acc1;
}

// grid (batch, ceil(heads / warps), segments), block = warps * 32.  Inputs dd_dt, dd_a, trap [B * L, H], angles [B * L, S] fp32.
__global__ void siso_small_fwd_kernel(const float* __restrict__ dd_dt, const float* __restrict__ dd_a, const float* __restrict__ trap,
                                      const float* __restrict__ angles, const float* __restrict__ dt_bias, float a_floor,
                                      const float* __restrict__ seg_inc, float* __restrict__ dt_o, float* __restrict__ a_o,
                                      float* __restrict__ sig_o, float* __restrict__ adt_o, float* __restrict__ gamma_o,
                                      float* __restrict__ scale_o, float* __restrict__ tanh_o, float* __restrict__ theta_o,
                                      float* __restrict__ spdt_o, float* __restrict__ spa_o, float* __restrict__ live_o, int seq_len,
                                      int heads, int n_angles) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x, h = blockIdx.y * (blockDim.x >> 5) + warp;
  if (h >= heads) return;
  const int seg = blockIdx.z, t_lo = seg * FSEG, t_end = min(seq_len, t_lo + FSEG);
  const float bias = dt_bias[h];
  const int64_t row0 = (int64_t)b * seq_len;
  const bool writes_tanh = h == 0;
  // DT_{t+1} (1 - sig_{t+1}) seen from the last token of the segment: from the inputs of the next segment's first token
  float carry_next = 0.f;
  if (t_end < seq_len) {
    const int64_t i = (row0 + t_end) * heads + h;
    carry_next = softplus_(dd_dt[i] + bias) * (1.f - sigmoidf_(trap[i]));
  }
  // elementwise part, tokens spread over the lanes, walking backwards so that the carry is known
  for (int t0 = t_end - 32; t0 > t_lo - 32; t0 -= 32) {
    const int t = t0 + lane;
    float dt = 0.f, sg = 0.f;
    if (t >= t_lo) {
      const int64_t i = (row0 + t) * heads + h;
      const float pre = dd_dt[i] + bias;
      dt = softplus_(pre);
      const float raw_a = -softplus_(dd_a[i]);
      const float a = fminf(raw_a, -a_floor);
      sg = sigmoidf_(trap[i]);
      dt_o[i] = dt;
      a_o[i] = a;
      sig_o[i] = sg;
      adt_o[i] = a * dt;
      gamma_o[i] = dt * sg;
      spdt_o[i] = sigmoidf_(pre);
      spa_o[i] = sigmoidf_(dd_a[i]);
      live_o[i] = raw_a < -a_floor ? 1.f : 0.f;
    }
    const float mine = dt * (1.f - sg);
    float next = __shfl_down_sync(0xffffffffu, mine, 1);
    if (lane == 31) next = carry_next;
    carry_next = __shfl_sync(0xffffffffu, mine, 0);   // the first token of this group follows the last of the group before it
    if (t >= t_lo) scale_o[(row0 + t) * heads + h] = dt * sg + next;
  }
  __syncwarp();
  // rotary phase: sequential over the tokens of the segment, lanes = angles
  const bool has0 = lane < n_angles, has1 = lane + 32 < n_angles;
  float acc0 = 0.f, acc1 = 0.f;   // running phase of angles lane and lane + 32
  {
    float p0[4] = {0.f, 0.f, 0.f, 0.f}, p1[4] = {0.f, 0.f, 0.f, 0.f};
    const float* src = seg_inc + (((int64_t)b * gridDim.z) * heads + h) * 64 + lane;
    const int64_t stride = (int64_t)heads * 64;
    int sgi = 0;
    for (; sgi + 4 <= seg; sgi += 4) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        p0[u] += src[(sgi + u) * stride];
        p1[u] += src[(sgi + u) * stride + 32];
      }
    }
    for (; sgi < seg; ++sgi) {
      p0[0] += src[sgi * stride];
      p1[0] += src[sgi * stride + 32];
    }
    acc0 = (p0[0] + p0[1]) + (p0[2] + p0[3]);
    acc1 = (p1[0] + p1[1]) + (p1[2] + p1[3]);
    acc0 -= TWO_PI_F * floorf(acc0 * (1.f / TWO_PI_F));
    acc1 -= TWO_PI_F * floorf(acc1 * (1.f / TWO_PI_F));
  }
  for (int t0 = t_lo; t0 < t_end; t0 += 8) {
    float dts[8], t0v[8], t1v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int t = t0 + j;
      dts[j] = t < t_end ? dt_o[(row0 + t) * heads + h] : 0.f;
      t0v[j] = (t < t_end && has0) ? tanhf(angles[(row0 + t) * n_angles + lane]) : 0.f;
      t1v[j] = (t < t_end && has1) ? tanhf(angles[(row0 + t) * n_angles + lane + 32]) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int t = t0 + j;
      if (t >= t_end) break;
      acc0 += PI_F * t0v[j] * dts[j];
      acc1 += PI_F * t1v[j] * dts[j];
      acc0 -= TWO_PI_F * floorf(acc0 * (1.f / TWO_PI_F));
      acc1 -= TWO_PI_F * floorf(acc1 * (1.f / TWO_PI_F));
      const int64_t o = ((row0 + t) * heads + h) * n_angles;
      if (has0) theta_o[o + lane] = acc0;
      if (has1) theta_o[o + lane + 32] = acc1;
      if (writes_tanh) {
        if (has0) tanh_o[(row0 + t) * n_angles + lane] = t0v[j];
        if (has1) tanh_o[(row0 + t) * n_angles + lane + 32] = t1v[j];
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ siso small, backward
// grid (P * B, segments), block = heads * 32 (heads <= 32, n_angles <= 32).  Forward tensors are indexed by b = blockIdx.x % batch.
// The reversed running sum of dtheta is the only dependency along the sequence: the sequence is cut into segments of SEG
// tokens, a first kernel sums dtheta per (sequence, segment, head, angle), and a block of the second kernel starts its sum
// from the totals of the later segments.
constexpr int TL = 8;     // tokens per tile
constexpr int SEG = 64;   // tokens per segment (a multiple of TL)

// grid (P * B, segments), block = heads * 32: seg_sum[pb][seg][h][32]
__global__ void __launch_bounds__(1024) dtheta_segment_sums_kernel(const float* __restrict__ dtheta, float* __restrict__ seg_sum,
                                                                   int seq_len, int heads, int n_angles) {
  const int h = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pb = blockIdx.x, seg = blockIdx.y;
  const int t_lo = seg * SEG, t_hi = min(seq_len, t_lo + SEG);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  if (lane < n_angles) {
    const float* src = dtheta + (((int64_t)pb * seq_len + t_lo) * heads + h) * n_angles + lane;
    const int64_t stride = (int64_t)heads * n_angles;
    int t = t_lo;
    for (; t + 4 <= t_hi; t += 4) {   // four independent loads in flight
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[j] += src[(int64_t)(t - t_lo + j) * stride];
    }
    for (; t < t_hi; ++t) acc[0] += src[(int64_t)(t - t_lo) * stride];
  }
  seg_sum[(((int64_t)pb * gridDim.y + seg) * heads + h) * 32 + lane] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
}

template <typename OutT>
__device__ __forceinline__ void put(OutT* p, float v);
template <>
__device__ __forceinline__ void put<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void put<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

// MAXT: the largest block the instantiation is launched with (heads * 32); the smaller bound leaves room for the tile
// prefetch in registers.
template <typename OutT, int MAXT>
__global__ void __launch_bounds__(MAXT) siso_small_bwd_kernel(
    const float* __restrict__ dt, const float* __restrict__ a, const float* __restrict__ sig, const float* __restrict__ tanh_a,
    const float* __restrict__ sp_dt, const float* __restrict__ sp_a, const float* __restrict__ live,
    const float* __restrict__ dadt, const float* __restrict__ dtheta, const float* __restrict__ dgamma,
    const float* __restrict__ dscale, const float* __restrict__ seg_sum, OutT* __restrict__ d_dd_dt, OutT* __restrict__ d_dd_a,
    OutT* __restrict__ d_trap, OutT* __restrict__ d_angles, int batch, int seq_len, int heads, int n_angles) {
  extern __shared__ float contrib[];   // [TL][heads][32]: pi * (reversed running sum of dtheta) * DT per token, head, angle; then [TL][32]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = warp;
  const int pb = blockIdx.x, b = pb % batch;
  const int64_t frow0 = (int64_t)b * seq_len, crow0 = (int64_t)pb * seq_len;
  const bool has = lane < n_angles;
  const int seg = blockIdx.y, t_first = seg * SEG;
  float acc = 0.f;
  {   // totals of the later segments: independent partial sums, so that the loads are in flight together
    float part[4] = {0.f, 0.f, 0.f, 0.f};
    const float* src = seg_sum + (((int64_t)pb * gridDim.y) * heads + h) * 32 + lane;
    const int64_t stride = (int64_t)heads * 32;
    int sg = seg + 1;
    for (; sg + 4 <= (int)gridDim.y; sg += 4) {
#pragma unroll
      for (int u = 0; u < 4; ++u) part[u] += src[(sg + u) * stride];
    }
    for (; sg < (int)gridDim.y; ++sg) part[0] += src[sg * stride];
    acc = (part[0] + part[1]) + (part[2] + part[3]);
  }
  float* tanh_tile = contrib + TL * heads * 32;   // [TL][32]: tanh(angle) of the tile's tokens, for the head sum
  const int t_last = min(seq_len, t_first + SEG) - 1;
  // the loads of a tile are issued one tile ahead: a tile is bound by load latency (24 KB in flight per SM otherwise)
  float dth_n[TL], tn_n[TL], dts_n[TL];
  auto load_tile = [&](int t_hi, float* dth, float* tn, float* dts) {
#pragma unroll
    for (int j = 0; j < TL; ++j) {
      const int t = t_hi - j;
      const bool ok = t >= t_first;
      dth[j] = (ok && has) ? dtheta[((crow0 + t) * heads + h) * n_angles + lane] : 0.f;
      tn[j] = (ok && has) ? tanh_a[(frow0 + t) * n_angles + lane] : 0.f;
      dts[j] = ok ? dt[(frow0 + t) * heads + h] : 0.f;
    }
  };
  load_tile(t_last, dth_n, tn_n, dts_n);
  for (int t_hi = t_last; t_hi >= t_first; t_hi -= TL) {
    float dth[TL], tn[TL], dts[TL];
#pragma unroll
    for (int j = 0; j < TL; ++j) {
      dth[j] = dth_n[j];
      tn[j] = tn_n[j];
      dts[j] = dts_n[j];
    }
    if (t_hi - TL >= t_first) load_tile(t_hi - TL, dth_n, tn_n, dts_n);
    // lane j < TL finishes the [b, l, h]-sized cotangents of token t_hi - j
    const int t_mine = t_hi - lane;
    const bool mine_ok = lane < TL && t_mine >= t_first;
    const int64_t fi = (frow0 + t_mine) * heads + h, ci = (crow0 + t_mine) * heads + h;
    float e_dsc = 0.f, e_prev = 0.f, e_dg = 0.f, e_sg = 0.f, e_dt = 0.f, e_da = 0.f, e_a = 0.f, e_spdt = 0.f, e_spa = 0.f, e_live = 0.f;
    if (mine_ok) {
      e_dsc = dscale[ci];
      e_prev = (t_mine > 0 && LBI_IN_RANGE(ci - heads, (int64_t)gridDim.x * seq_len * heads, 94)) ? dscale[ci - heads] : 0.f;
      e_dg = dgamma[ci];
      e_sg = sig[fi];
      e_dt = dt[fi];
      e_da = dadt[ci];
      e_a = a[fi];
      e_spdt = sp_dt[fi];
      e_spa = sp_a[fi];
      e_live = live[fi];
    }
    float mine = 0.f;   // lane j keeps the rotary part of d DT of token t_hi - j
    float run[TL];
#pragma unroll
    for (int j = 0; j < TL; ++j) {
      acc += dth[j];
      run[j] = acc;
      contrib[(j * heads + h) * 32 + lane] = PI_F * acc * dts[j];
      if (h == 0) tanh_tile[j * 32 + lane] = tn[j];
    }
#pragma unroll
    for (int j = 0; j < TL; ++j) {   // the TL reductions are independent: their shuffles overlap
      const float part = PI_F * warp_sum(run[j] * tn[j]);
      if (lane == j) mine = part;
    }
    if (mine_ok) {
      const float dg_all = e_dg + e_dsc;
      const float d_dt = e_da * e_a + mine + dg_all * e_sg + e_prev * (1.f - e_sg);
      const float d_sig = e_dt * (dg_all - e_prev);
      put(d_dd_dt + ci, d_dt * e_spdt);
      put(d_dd_a + ci, -(e_da * e_dt) * e_spa * e_live);
      put(d_trap + ci, d_sig * e_sg * (1.f - e_sg));
    }
    __syncthreads();
    // sum the heads: TL * n_angles outputs
    for (int o = threadIdx.x; o < TL * 32; o += blockDim.x) {
      const int j = o >> 5, s = o & 31;
      const int t = t_hi - j;
      if (t >= t_first && s < n_angles) {
        float sum = 0.f;
        for (int hh = 0; hh < heads; ++hh) sum += contrib[(j * heads + hh) * 32 + s];
        const float tv = tanh_tile[j * 32 + s];
        put(d_angles + (crow0 + t) * n_angles + s, sum * (1.f - tv * tv));
      }
    }
    __syncthreads();
  }
}

}  // namespace msmall
}  // namespace lbi

extern "C" int lbi_gate_silu_fwd(const void* y, const void* z, void* out, int64_t numel, cudaStream_t st) {
  using namespace lbi;
  if (numel <= 0) return 0;
  if (numel % 8) return (int)cudaErrorInvalidValue;
  const int64_t n8 = numel / 8;
  const int blocks = (int)((n8 + 255) / 256 < 148 * 16 ? (n8 + 255) / 256 : 148 * 16);
  msmall::gate_silu_fwd_kernel<<<blocks, 256, 0, st>>>((const bf16x8*)y, (const bf16x8*)z, (bf16x8*)out, n8);
  return (int)cudaGetLastError();
}

extern "C" int lbi_gate_silu_bwd(const void* dyg, const void* y, const void* z, void* dy, void* dz, int64_t numel, int reps,
                                 int cols, int64_t ld_dz, cudaStream_t st) {
  using namespace lbi;
  if (numel <= 0 || reps <= 0) return 0;
  if (numel % 8 || cols <= 0 || cols % 8 || numel % cols || ld_dz % 8 || ld_dz < cols) return (int)cudaErrorInvalidValue;
  const int64_t n8 = numel / 8;
  const int blocks = (int)((n8 + 255) / 256 < 148 * 16 ? (n8 + 255) / 256 : 148 * 16);
  msmall::gate_silu_bwd_kernel<<<blocks, 256, 0, st>>>((const bf16x8*)dyg, (const bf16x8*)y, (const bf16x8*)z, (bf16x8*)dy,
                                                       (bf16x8*)dz, n8, reps, cols / 8, ld_dz / 8);
  return (int)cudaGetLastError();
}

extern "C" int lbi_softplus_dt(const void* dt_raw, int64_t ld, int is_bf16, const float* bias, float lo, float hi, float* dt,
                               float* slope, int64_t rows, int heads, cudaStream_t st) {
  using namespace lbi;
  if (rows <= 0 || heads <= 0) return 0;
  if (ld < heads) return (int)cudaErrorInvalidValue;
  const int64_t total = rows * heads;
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  if (is_bf16)
    msmall::softplus_dt_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)dt_raw, ld, bias, lo, hi, dt, slope, rows, heads);
  else
    msmall::softplus_dt_kernel<float><<<blocks, 256, 0, st>>>((const float*)dt_raw, ld, bias, lo, hi, dt, slope, rows, heads);
  return (int)cudaGetLastError();
}

extern "C" int lbi_siso_small_fwd_segments(int seq_len) { return (seq_len + lbi::msmall::FSEG - 1) / lbi::msmall::FSEG; }

extern "C" int lbi_siso_small_fwd(const float* dd_dt, const float* dd_a, const float* trap, const float* angles,
                                  const float* dt_bias, float a_floor, float* seg_inc, float* dt, float* a, float* sig, float* adt,
                                  float* gamma, float* scale, float* tanh_a, float* theta, float* sp_dt, float* sp_a, float* live,
                                  int batch, int seq_len, int heads, int n_angles, cudaStream_t st) {
  using namespace lbi;
  if (batch <= 0 || seq_len <= 0) return 0;
  if (n_angles > 64 || n_angles <= 0 || heads <= 0 || heads > 32 || !seg_inc) return (int)cudaErrorInvalidValue;
  const int segs = lbi_siso_small_fwd_segments(seq_len);
  msmall::phase_segment_sums_kernel<<<dim3(batch, segs), heads * 32, 0, st>>>(dd_dt, angles, dt_bias, seg_inc, seq_len, heads, n_angles);
  const int warps = heads < 8 ? heads : 8;
  dim3 grid(batch, (heads + warps - 1) / warps, segs);
  msmall::siso_small_fwd_kernel<<<grid, warps * 32, 0, st>>>(dd_dt, dd_a, trap, angles, dt_bias, a_floor, seg_inc, dt, a, sig, adt,
                                                             gamma, scale, tanh_a, theta, sp_dt, sp_a, live, seq_len, heads, n_angles);
  return (int)cudaGetLastError();
}

extern "C" int lbi_siso_small_segments(int seq_len) { return (seq_len + lbi::msmall::SEG - 1) / lbi::msmall::SEG; }

extern "C" int lbi_siso_small_bwd(const float* dt, const float* a, const float* sig, const float* tanh_a, const float* sp_dt,
                                  const float* sp_a, const float* live, const float* dadt, const float* dtheta,
                                  const float* dgamma, const float* dscale, float* seg_sum, void* d_dd_dt, void* d_dd_a,
                                  void* d_trap, void* d_angles, int batch, int reps, int seq_len, int heads, int n_angles,
                                  int out_bf16, cudaStream_t st) {
  using namespace lbi;
  if (batch <= 0 || reps <= 0 || seq_len <= 0) return 0;
  if (heads > 32 || heads <= 0 || n_angles > 32 || n_angles <= 0 || !seg_sum) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)msmall::TL * (heads + 1) * 32 * sizeof(float);
  const dim3 grid(batch * reps, lbi_siso_small_segments(seq_len));
  msmall::dtheta_segment_sums_kernel<<<grid, heads * 32, 0, st>>>(dtheta, seg_sum, seq_len, heads, n_angles);
#define LBI_SMALL_BWD(OutT, MAXT)                                                                                              \
  msmall::siso_small_bwd_kernel<OutT, MAXT><<<grid, heads * 32, smem, st>>>(dt, a, sig, tanh_a, sp_dt, sp_a, live, dadt, dtheta, \
                                                                            dgamma, dscale, seg_sum, (OutT*)d_dd_dt,            \
                                                                            (OutT*)d_dd_a, (OutT*)d_trap, (OutT*)d_angles,      \
                                                                            batch, seq_len, heads, n_angles)
  if (out_bf16) {
    if (heads <= 24) LBI_SMALL_BWD(__nv_bfloat16, 768);
    else LBI_SMALL_BWD(__nv_bfloat16, 1024);
  } else {
    if (heads <= 24) LBI_SMALL_BWD(float, 768);
    else LBI_SMALL_BWD(float, 1024);
  }
#undef LBI_SMALL_BWD
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ Mamba-2 conv + SiLU
// Depthwise causal conv over the xBC slice of in_proj followed by SiLU, eight channels per thread (16-byte accesses).
//   pre[t, c] = bias[c] + sum_w w[c, w] x[t - (W - 1) + w, c],   act = silu(pre)
// The kernels take the weights transposed, wt [W][C] (a tap's weights of neighbouring channels are neighbours in memory: one
// coalesced 32-byte load per thread and tap instead of eight scattered ones); the weight gradient is produced as [C][W].
// The activation leaves as three contiguous tensors (x | B | C: what the scan kernels take), the pre-activation is kept
// for the backward.  Backward for P stacked directions: the cotangents of x, B, C arrive as three tensors,
//   dpre[t', c] = dact[t', c] silu'(pre[t', c]),   din[t, c] = sum_w w[c, w] dpre[t + (W - 1) - w, c]
// and din is written with a row stride, i.e. straight into its column range of the in_proj cotangent.  The weight
// gradient dw[c, w] = sum_t dpre[t, c] x[t - (W - 1) + w, c], db[c] = sum_t dpre[t, c] accumulates per thread over a run
// of tokens and leaves with one atomic per (thread, tap).  Replaces causal_conv1d_fn / its backward in the reference's fused
// Mamba-2 path (backbones/mamba2/ops/triton/ssd_combined.py:847, 921, 970) and nn.Conv1d + SiLU in its unfused path.
namespace lbi {
namespace mconv {

constexpr int MAXW = 8;

struct Seg {          // channel c belongs to segment 0 [0, c0), 1 [c0, c0 + c1) or 2 [c0 + c1, c0 + c1 + c2)
  int c0, c1, c2;
};

__device__ __forceinline__ float silu_(float v) { return v * sigmoidf_(v); }
__device__ __forceinline__ float dsilu_(float v) {
  const float s = sigmoidf_(v);
  return s * (1.f + v * (1.f - s));
}

// grid (tokens), block 128: a block owns one token, its threads walk the 8-channel vectors (no 64-bit divisions per element).
__global__ void __launch_bounds__(128) conv_silu_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                                            const float* __restrict__ bias, __nv_bfloat16* __restrict__ pre,
                                                            __nv_bfloat16* __restrict__ o0, __nv_bfloat16* __restrict__ o1,
                                                            __nv_bfloat16* __restrict__ o2, Seg seg, int64_t tokens, int seq_len,
                                                            int width) {
  const int channels = seg.c0 + seg.c1 + seg.c2, cvecs = channels / 8;
  const int64_t tok = blockIdx.x;
  const int t = (int)(tok % seq_len);
  const int k_lo = max(0, (width - 1) - t);   // taps that reach before the first token of the sequence are skipped
  for (int cv = threadIdx.x; cv < cvecs; cv += blockDim.x) {
    const int c = cv * 8;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = bias ? bias[c + e] : 0.f;
    for (int k = k_lo; k < width; ++k) {
      const int64_t src = tok - (width - 1) + k;
      if (!LBI_IN_RANGE(src, tokens, 91)) continue;
      float xv[8];
      unpack8(*reinterpret_cast<const bf16x8*>(x + src * channels + c), xv);
      {
        const float4 w0 = *reinterpret_cast<const float4*>(w + (int64_t)k * channels + c);
        const float4 w1 = *reinterpret_cast<const float4*>(w + (int64_t)k * channels + c + 4);
        acc[0] = fmaf(w0.x, xv[0], acc[0]); acc[1] = fmaf(w0.y, xv[1], acc[1]); acc[2] = fmaf(w0.z, xv[2], acc[2]);
        acc[3] = fmaf(w0.w, xv[3], acc[3]); acc[4] = fmaf(w1.x, xv[4], acc[4]); acc[5] = fmaf(w1.y, xv[5], acc[5]);
        acc[6] = fmaf(w1.z, xv[6], acc[6]); acc[7] = fmaf(w1.w, xv[7], acc[7]);
      }
    }
    *reinterpret_cast<bf16x8*>(pre + tok * channels + c) = pack8(acc);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = silu_(acc[e]);
    __nv_bfloat16* dst = c < seg.c0 ? o0 + tok * seg.c0 + c
                                    : (c < seg.c0 + seg.c1 ? o1 + tok * seg.c1 + (c - seg.c0) : o2 + tok * seg.c2 + (c - seg.c0 - seg.c1));
    *reinterpret_cast<bf16x8*>(dst) = pack8(acc);
  }
}

template <typename D0>
__device__ __forceinline__ void load_cot(const D0* p, float* out);
template <>
__device__ __forceinline__ void load_cot<__nv_bfloat16>(const __nv_bfloat16* p, float* out) {
  unpack8(*reinterpret_cast<const bf16x8*>(p), out);
}
template <>
__device__ __forceinline__ void load_cot<float>(const float* p, float* out) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w; out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}

// dpre of eight channels at token `tok` (cotangent row) / `ftok` (forward row)
template <typename D0, typename D12>
__device__ __forceinline__ void dpre8(const D0* d0, const D12* d1, const D12* d2, const __nv_bfloat16* pre, Seg seg, int channels,
                                      int64_t tok, int64_t ftok, int c, float* out) {
  float g[8], pv[8];
  if (c < seg.c0) load_cot<D0>(d0 + tok * seg.c0 + c, g);
  else if (c < seg.c0 + seg.c1) load_cot<D12>(d1 + tok * seg.c1 + (c - seg.c0), g);
  else load_cot<D12>(d2 + tok * seg.c2 + (c - seg.c0 - seg.c1), g);
  if (!pre) {   // a plain convolution (no activation after it): the cotangent is the pre-activation cotangent
#pragma unroll
    for (int e = 0; e < 8; ++e) out[e] = g[e];
    return;
  }
  unpack8(*reinterpret_cast<const bf16x8*>(pre + ftok * channels + c), pv);
#pragma unroll
  for (int e = 0; e < 8; ++e) out[e] = g[e] * dsilu_(pv[e]);
}

// grid (sequences * runs per sequence, ceil(cvecs / 128)), block 128.  A thread owns eight channels and walks the BRUN tokens of
// its run from the last to the first with a window of the W newest dpre values in registers, so that every cotangent and
// pre-activation element is read once and its SiLU slope is evaluated once (plus W - 1 tokens of halo per run).
constexpr int BRUN = 32;
// WMAX: compile-time bound of the filter width (4 for the usual d_conv = 4, else MAXW): it sizes the register windows.
template <typename D0, typename D12, int WMAX>
__global__ void __launch_bounds__(128) conv_silu_bwd_kernel(const D0* __restrict__ d0, const D12* __restrict__ d1,
                                                            const D12* __restrict__ d2, const __nv_bfloat16* __restrict__ pre,
                                                            const float* __restrict__ w, __nv_bfloat16* __restrict__ din, int64_t ld_in,
                                                            Seg seg, int64_t tokens, int64_t ftokens, int seq_len, int width) {
  const int channels = seg.c0 + seg.c1 + seg.c2, cvecs = channels / 8;
  const int cv = blockIdx.y * 128 + threadIdx.x;
  if (cv >= cvecs) return;
  const int c = cv * 8;
  const int runs_per_seq = (seq_len + BRUN - 1) / BRUN;
  const int64_t sq = blockIdx.x / runs_per_seq;
  const int run = blockIdx.x % runs_per_seq;
  const int t0 = run * BRUN, t1 = min(seq_len, t0 + BRUN);
  const int64_t tok_base = sq * seq_len;                                  // first token of the sequence, cotangent rows
  const int64_t ftok_base = (sq % (ftokens / seq_len)) * seq_len;         // the same in the forward tensors
  // weights of the eight channels by shift: wk[s][e] = w[W - 1 - s] multiplies dpre[t + s]
  float wk[WMAX][8];
#pragma unroll
  for (int sft = 0; sft < WMAX; ++sft) {
    if (sft < width) {
      const int k = width - 1 - sft;
      const float4 w0 = *reinterpret_cast<const float4*>(w + (int64_t)k * channels + c);
      const float4 w1 = *reinterpret_cast<const float4*>(w + (int64_t)k * channels + c + 4);
      wk[sft][0] = w0.x; wk[sft][1] = w0.y; wk[sft][2] = w0.z; wk[sft][3] = w0.w;
      wk[sft][4] = w1.x; wk[sft][5] = w1.y; wk[sft][6] = w1.z; wk[sft][7] = w1.w;
    }
  }
  // win[s] = dpre[t + s], s = 0 .. W - 1; starts with the halo after the run (zeros past the end of the sequence)
  float win[WMAX][8];
#pragma unroll
  for (int sft = 1; sft < WMAX; ++sft) {
    if (sft < width) {
      const int t = t1 - 1 + sft;
      if (t < seq_len && LBI_IN_RANGE(tok_base + t, tokens, 92)) {
        dpre8<D0, D12>(d0, d1, d2, pre, seg, channels, tok_base + t, ftok_base + t, c, win[sft]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) win[sft][e] = 0.f;
      }
    }
  }
#pragma unroll 4
  for (int t = t1 - 1; t >= t0; --t) {
    dpre8<D0, D12>(d0, d1, d2, pre, seg, channels, tok_base + t, ftok_base + t, c, win[0]);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int sft = 0; sft < WMAX; ++sft) {
      if (sft < width) {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = fmaf(wk[sft][e], win[sft][e], acc[e]);
      }
    }
    *reinterpret_cast<bf16x8*>(din + (tok_base + t) * ld_in + c) = pack8(acc);
#pragma unroll
    for (int sft = WMAX - 1; sft >= 1; --sft) {
      if (sft < width) {
#pragma unroll
        for (int e = 0; e < 8; ++e) win[sft][e] = win[sft - 1][e];
      }
    }
  }
}

// grid (cvecs blocks of 32 lanes x 8 token runs per block, runs); every thread walks RUN tokens of its eight channels
constexpr int RUN = 64;
template <typename D0, typename D12>
__global__ void __launch_bounds__(256) conv_silu_wgrad_kernel(const D0* __restrict__ d0, const D12* __restrict__ d1,
                                                              const D12* __restrict__ d2, const __nv_bfloat16* __restrict__ pre,
                                                              const __nv_bfloat16* __restrict__ x, float* __restrict__ dw,
                                                              float* __restrict__ db, Seg seg, int64_t tokens, int seq_len, int width) {
  const int channels = seg.c0 + seg.c1 + seg.c2, cvecs = channels / 8;
  const int cv = blockIdx.x * 32 + (threadIdx.x & 31);
  const int64_t run = (int64_t)blockIdx.y * 8 + (threadIdx.x >> 5);
  if (cv >= cvecs) return;
  const int c = cv * 8;
  float accw[MAXW][8], accb[8];
#pragma unroll
  for (int k = 0; k < MAXW; ++k)
#pragma unroll
    for (int e = 0; e < 8; ++e) accw[k][e] = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) accb[e] = 0.f;
  const int64_t t_lo = run * RUN, t_hi = t_lo + RUN < tokens ? t_lo + RUN : tokens;
  for (int64_t tok = t_lo; tok < t_hi; ++tok) {
    const int t = (int)(tok % seq_len);
    float dp[8];
    dpre8<D0, D12>(d0, d1, d2, pre, seg, channels, tok, tok, c, dp);
#pragma unroll
    for (int e = 0; e < 8; ++e) accb[e] += dp[e];
#pragma unroll
    for (int k = 0; k < MAXW; ++k) {
      if (k >= width) break;
      const int tt = t - (width - 1) + k;
      if (tt < 0) continue;
      if (!LBI_IN_RANGE(tok + (tt - t), tokens, 93)) continue;
      float xv[8];
      unpack8(*reinterpret_cast<const bf16x8*>(x + (tok + (tt - t)) * channels + c), xv);
#pragma unroll
      for (int e = 0; e < 8; ++e) accw[k][e] = fmaf(dp[e], xv[e], accw[k][e]);
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    atomicAdd(db + c + e, accb[e]);
#pragma unroll
    for (int k = 0; k < MAXW; ++k)
      if (k < width) atomicAdd(dw + (c + e) * width + k, accw[k][e]);
  }
}

}  // namespace mconv
}  // namespace lbi

extern "C" int lbi_conv_silu_fwd(const void* x, const float* w, const float* bias, void* pre, void* o0, void* o1, void* o2, int c0,
                                 int c1, int c2, int64_t tokens, int seq_len, int width, cudaStream_t st) {
  using namespace lbi::mconv;
  if (tokens <= 0) return 0;
  if (c0 % 8 || c1 % 8 || c2 % 8 || c0 + c1 + c2 <= 0 || width <= 0 || width > MAXW || seq_len <= 0 || tokens % seq_len)
    return (int)cudaErrorInvalidValue;
  if (tokens > 2147483647ll) return (int)cudaErrorInvalidValue;
  conv_silu_fwd_kernel<<<(unsigned)tokens, 128, 0, st>>>((const __nv_bfloat16*)x, w, bias, (__nv_bfloat16*)pre,
                                                                        (__nv_bfloat16*)o0, (__nv_bfloat16*)o1, (__nv_bfloat16*)o2,
                                                                        Seg{c0, c1, c2}, tokens, seq_len, width);
  return (int)cudaGetLastError();
}

extern "C" int lbi_conv_silu_bwd(const void* d0, int d0_fp32, const void* d1, const void* d2, int d12_fp32, const void* pre,
                                 const float* w, void* din, int64_t ld_in, int c0, int c1, int c2, int64_t tokens, int64_t ftokens,
                                 int seq_len, int width, cudaStream_t st) {
  using namespace lbi::mconv;
  if (tokens <= 0) return 0;
  if (c0 % 8 || c1 % 8 || c2 % 8 || c0 + c1 + c2 <= 0 || width <= 0 || width > MAXW || seq_len <= 0 || ftokens <= 0 ||
      tokens % ftokens || ftokens % seq_len || ld_in % 8 || ld_in < c0 + c1 + c2)
    return (int)cudaErrorInvalidValue;
  const int64_t runs = (tokens / seq_len) * ((seq_len + BRUN - 1) / BRUN);
  if (runs > 2147483647ll) return (int)cudaErrorInvalidValue;
  const dim3 blocks((unsigned)runs, (unsigned)(((c0 + c1 + c2) / 8 + 127) / 128));
  const Seg seg{c0, c1, c2};
#define LBI_CONV_BWD(A, B)                                                                                                          \
  do {                                                                                                                              \
    if (width <= 4)                                                                                                                 \
      conv_silu_bwd_kernel<A, B, 4><<<blocks, 128, 0, st>>>((const A*)d0, (const B*)d1, (const B*)d2, (const __nv_bfloat16*)pre, w, \
                                                            (__nv_bfloat16*)din, ld_in, seg, tokens, ftokens, seq_len, width);    \
    else                                                                                                                            \
      conv_silu_bwd_kernel<A, B, MAXW><<<blocks, 128, 0, st>>>((const A*)d0, (const B*)d1, (const B*)d2, (const __nv_bfloat16*)pre, \
                                                               w, (__nv_bfloat16*)din, ld_in, seg, tokens, ftokens, seq_len, width); \
  } while (0)
  if (d0_fp32 && d12_fp32) LBI_CONV_BWD(float, float);
  else if (d0_fp32) LBI_CONV_BWD(float, __nv_bfloat16);
  else if (d12_fp32) LBI_CONV_BWD(__nv_bfloat16, float);
  else LBI_CONV_BWD(__nv_bfloat16, __nv_bfloat16);
#undef LBI_CONV_BWD
  return (int)cudaGetLastError();
}

// dw [C, W] and db [C] must be zeroed by the caller (the kernel adds).
extern "C" int lbi_conv_silu_wgrad(const void* d0, int d0_fp32, const void* d1, const void* d2, int d12_fp32, const void* pre,
                                   const void* x, float* dw, float* db, int c0, int c1, int c2, int64_t tokens, int seq_len, int width,
                                   cudaStream_t st) {
  using namespace lbi::mconv;
  if (tokens <= 0) return 0;
  if (c0 % 8 || c1 % 8 || c2 % 8 || c0 + c1 + c2 <= 0 || width <= 0 || width > MAXW || seq_len <= 0 || tokens % seq_len)
    return (int)cudaErrorInvalidValue;
  const int cvecs = (c0 + c1 + c2) / 8;
  const int64_t runs = (tokens + RUN - 1) / RUN;
  const dim3 grid((unsigned)((cvecs + 31) / 32), (unsigned)((runs + 7) / 8));
  const Seg seg{c0, c1, c2};
#define LBI_CONV_WG(A, B)                                                                                                      \
  conv_silu_wgrad_kernel<A, B><<<grid, 256, 0, st>>>((const A*)d0, (const B*)d1, (const B*)d2, (const __nv_bfloat16*)pre,      \
                                                     (const __nv_bfloat16*)x, dw, db, seg, tokens, seq_len, width)
  if (d0_fp32 && d12_fp32) LBI_CONV_WG(float, float);
  else if (d0_fp32) LBI_CONV_WG(float, __nv_bfloat16);
  else if (d12_fp32) LBI_CONV_WG(__nv_bfloat16, float);
  else LBI_CONV_WG(__nv_bfloat16, __nv_bfloat16);
#undef LBI_CONV_WG
  return (int)cudaGetLastError();
}

LBI_DEFINE_BOUNDS_GETTER(lbi_bounds_site_mamba_small)
