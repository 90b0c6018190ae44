// Mamba-2 state-space-duality (SSD) chunk scan, forward, on tcgen05 / TMEM / TMA.
//
//   h_t = exp(dt_t A) h_{t-1} + dt_t x_t B_t^T ,   y_t = h_t C_t + D x_t          (per head; B, C shared per group)
//
// evaluated chunk-wise (chunk L = 128 tokens) in four kernels:
//   1. cumsum        dt = softplus(dt_raw + bias) (optional), dA = dt A, inclusive in-chunk cumulative sum
//   2. chunk state   S_c[(h,p), n] = sum_l x[l,(h,p)] exp(total - cum_l) dt_l B[l, n]        one tcgen05 GEMM per
//                    (batch, chunk, pair of heads): M = 2 heads x 64, N = d_state, K = 128; x is scaled in place in
//                    shared memory by the compute warps after TMA delivered it
//   3. state passing sequential over chunks (elementwise): incoming state of every chunk (bf16) and the final state
//   4. chunk scan    per (batch, chunk, head):  G = C B^T (128 x 128, K = d_state) -> TMEM;  W = G o decay o dt (causal)
//                    written as bf16 into shared memory;  Y = W X (K = 128) and Y += (C o exp(cum)) H_in^T (K = d_state)
//                    accumulate in TMEM;  epilogue adds D x and stores y.
// This replaces the reference's Triton kernels _chunk_cumsum_fwd, _chunk_state_fwd, _state_passing_fwd, _bmm_chunk_fwd
// and _chunk_scan_fwd (backbones/mamba2/ops/triton/ssd_combined.py:343-393), fusing the last two.
//
// Shapes: head_dim 64, d_state 64 or 128, seq_len a multiple of 128, an even number of heads per group.
// x [B*L, H*64] bf16, Bm / Cm [B*L, G*N] bf16, dt / cum [B, H, L] fp32, states [B, C, H, 64, N] fp32,
// prev [B, C, H, 64, N] bf16, y [B*L, H*64] bf16.  Every mbarrier wait is bounded (tcgen05.cuh).
#include <cuda_bf16.h>

#include <mutex>

#include "api_ssd.h"
#include "common.cuh"
#include "tcgen05.cuh"

namespace lbi {
namespace ssd {

using namespace tc;

constexpr int L = 128;            // chunk length
constexpr int P = 64;             // head dimension
constexpr int PANEL = L * 128;    // 128 rows x 128 bytes
constexpr int THREADS = 160;      // 4 compute warps + 1 control warp
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ float2 unpack2(uint32_t v) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v)); }
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// Multiply the 64 bf16 of row `row` of a 128-byte-row panel by f, in place (the swizzle only permutes the chunks).
__device__ __forceinline__ void scale_row(uint32_t panel, int row, float f) {
  const uint32_t base = panel + row * 128;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint4 v = lds128(base + c * 16);
    float2 a = unpack2(v.x), b = unpack2(v.y), cc = unpack2(v.z), d = unpack2(v.w);
    v.x = pack2(a.x * f, a.y * f);
    v.y = pack2(b.x * f, b.y * f);
    v.z = pack2(cc.x * f, cc.y * f);
    v.w = pack2(d.x * f, d.y * f);
    sts128(base + c * 16, v);
  }
}

// ------------------------------------------------------------------------------------------------ 1. cumsum
// grid (C, H, B), 128 threads.  dt_raw [B, L_total, H] fp32; outputs dt_out, cum [B, H, L_total] fp32.
__global__ void __launch_bounds__(128) cumsum_kernel(const float* __restrict__ dt_raw, const float* __restrict__ dt_bias,
                                                     const float* __restrict__ a_log_neg, float* __restrict__ dt_out,
                                                     float* __restrict__ cum, int seq_len, int heads, int softplus,
                                                     float dt_min, float dt_max) {
  __shared__ float warp_tot[4];
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z, t = threadIdx.x;
  const int64_t tok = (int64_t)b * seq_len + c * L + t;
  float v = dt_raw[tok * heads + h];
  if (softplus) {
    v += dt_bias ? dt_bias[h] : 0.f;
    v = v > 20.f ? v : log1pf(__expf(v));
    v = fminf(fmaxf(v, dt_min), dt_max);
  }
  float acc = v * a_log_neg[h];
  const int lane = t & 31, w = t >> 5;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const float o = __shfl_up_sync(0xffffffffu, acc, off);
    if (lane >= off) acc += o;
  }
  if (lane == 31) warp_tot[w] = acc;
  __syncthreads();
  float pre = 0.f;
  for (int i = 0; i < w; ++i) pre += warp_tot[i];
  const int64_t o = ((int64_t)b * heads + h) * seq_len + c * L + t;
  dt_out[o] = v;
  cum[o] = acc + pre;
}

// ------------------------------------------------------------------------------------------------ 2. chunk state
// PH ("per head"): B and C are given per head (Mamba-3 after its rotary / bias preprocessing) instead of per group.  Then
// one CTA owns one head, the product is taken as S^T[n, p] (M = d_state = 128) and states are stored [n][p].
template <int N>
struct SmemState {
  alignas(1024) uint8_t xs[2][PANEL];          // x of two heads (PH: of one head): [l][64 p] per panel
  alignas(1024) uint8_t bt[N / 64][PANEL];     // B: [l][64 n] per panel
  uint64_t bar_full, bar_scaled, bar_done;
  uint32_t tmem_base;
  volatile int abort_flag;
};

struct StateParams {
  int seq_len, heads, groups, chunks;
  int v_div, v_mod;     // head h reads the 64-column block (h / v_div) * v_mod + h % v_mod of the v matrix (1, 1: block h)
  const float* dt;      // [B, H, L_total]
  const float* cum;     // [B, H, L_total]
  float* states;        // [B, C, H, 64, N]
  int* status;
  int rev;              // 1: cotangent form, rows scaled by exp(cum_l) (no weight) instead of exp(total - cum_l) dt_l
  int bmod;             // the B operand, dt and cum belong to batch b % bmod (forward tensors shared by stacked directions)
};

template <int N, bool PH>
__global__ void __launch_bounds__(THREADS) chunk_state_kernel(const __grid_constant__ CUtensorMap map_x,
                                                              const __grid_constant__ CUtensorMap map_b, const StateParams p) {
  extern __shared__ uint8_t raw_smem[];
  SmemState<N>& s = *reinterpret_cast<SmemState<N>*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x, hp = blockIdx.y, b = blockIdx.z;
  const int h0 = PH ? hp : 2 * hp;
  const int g = PH ? h0 : h0 / (p.heads / p.groups);
  const int row0 = b * p.seq_len + c * L;
  const int fb = b % p.bmod;
  const int frow0 = fb * p.seq_len + c * L;
  constexpr uint32_t TMEM_COLS = PH ? 64 : N;   // a power of two >= 32

  if (threadIdx.x == 0) {
    s.abort_flag = 0;
    mbar_init(&s.bar_full, 1);
    mbar_init(&s.bar_scaled, 4);
    mbar_init(&s.bar_done, 1);
    fence_barrier_init();
    prefetch_tmap(&map_x);
    prefetch_tmap(&map_b);
  }
  if (warp == 4) tmem_alloc(&s.tmem_base, TMEM_COLS);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = s.tmem_base;
  volatile int* abortp = &s.abort_flag;

  if (warp == 4) {
    if (lane == 0) {
      mbar_arrive_expect_tx(&s.bar_full, ((PH ? 1 : 2) + N / 64) * PANEL);
      tma_load_2d(s.xs[0], &map_x, &s.bar_full, ((h0 / p.v_div) * p.v_mod + h0 % p.v_mod) * P, row0);
      if (!PH) tma_load_2d(s.xs[1], &map_x, &s.bar_full, (((h0 + 1) / p.v_div) * p.v_mod + (h0 + 1) % p.v_mod) * P, row0);
      for (int q = 0; q < N / 64; ++q) tma_load_2d(s.bt[q], &map_b, &s.bar_full, g * N + q * 64, frow0);
      bool ok = mbar_wait(&s.bar_scaled, 0, abortp, p.status, 51);
      if (ok) {
        fence_after_sync();
        // D[(h, p), n] = sum_l xs[l, (h, p)] * bt[l, n]: both operands have the reduction index as their row
        // (PH: D[n, p] = sum_l bt[l, n] * xs[l, p], the roles of the two tiles swapped)
        const uint32_t idesc = make_idesc_bf16(128, PH ? 64 : N, 1, 1);
        const uint64_t da = make_smem_desc(smem_u32(PH ? s.bt[0] : s.xs[0]), PANEL, 1024);
        const uint64_t db = make_smem_desc(smem_u32(PH ? s.xs[0] : s.bt[0]), PANEL, 1024);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) mma_bf16(tmem, da + 128 * kk, db + 128 * kk, idesc, kk);
        mma_commit(&s.bar_done);
      }
    }
  } else {
    const int l = warp * 32 + lane;   // token of the chunk handled in the scaling pass; row (h, p) in the epilogue
    const int64_t base0 = ((int64_t)fb * p.heads + h0) * p.seq_len + c * L;
    const int64_t base1 = base0 + p.seq_len;
    const float f0 = p.rev ? ex2(p.cum[base0 + l] * LOG2E)
                           : ex2((p.cum[base0 + L - 1] - p.cum[base0 + l]) * LOG2E) * (p.dt ? p.dt[base0 + l] : 1.f);
    const float f1 = PH ? 0.f
                        : (p.rev ? ex2(p.cum[base1 + l] * LOG2E)
                                 : ex2((p.cum[base1 + L - 1] - p.cum[base1 + l]) * LOG2E) * (p.dt ? p.dt[base1 + l] : 1.f));
    bool ok = mbar_wait(&s.bar_full, 0, abortp, p.status, 52);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      scale_row(smem_u32(s.xs[0]), l, f0);
      if (!PH) scale_row(smem_u32(s.xs[1]), l, f1);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.bar_scaled);
      ok = mbar_wait(&s.bar_done, 0, abortp, p.status, 53);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      fence_after_sync();
      // rows of D: (head, p) with N columns, or (PH) n with 64 columns
      const int h = PH ? h0 : h0 + (l >> 6), pp = l & 63;
      float* dst = PH ? p.states + ((((int64_t)b * p.chunks + c) * p.heads + h) * N + l) * P
                      : p.states + ((((int64_t)b * p.chunks + c) * p.heads + h) * P + pp) * N;
#pragma unroll
      for (int q = 0; q < (PH ? P : N) / 32; ++q) {
        uint32_t r[32];
        tmem_ld_32x32(tmem + ((uint32_t)(warp * 32) << 16) + q * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 8; ++e)
          reinterpret_cast<float4*>(dst + q * 32)[e] = make_float4(__uint_as_float(r[4 * e]), __uint_as_float(r[4 * e + 1]),
                                                                  __uint_as_float(r[4 * e + 2]), __uint_as_float(r[4 * e + 3]));
      }
    }
  }
  __syncwarp();
  if (s.abort_flag) {
    const unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    fence_after_sync();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------------ 3. state passing
// One thread per state element (b, h, e), e in [0, 64 * N); walks the chunks.
__global__ void state_passing_kernel(const float* __restrict__ states, const float* __restrict__ cum,
                                     const float* __restrict__ init, __nv_bfloat16* __restrict__ prev,
                                     float* __restrict__ final_state, int batch, int heads, int chunks, int seq_len,
                                     int elems) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)batch * heads * elems) return;
  const int e = (int)(idx % elems);
  const int h = (int)((idx / elems) % heads);
  const int b = (int)(idx / ((int64_t)elems * heads));
  float st = init ? init[idx] : 0.f;
  const float* cum_bh = cum + ((int64_t)b * heads + h) * seq_len;
  for (int c = 0; c < chunks; ++c) {
    const int64_t o = (((int64_t)b * chunks + c) * heads + h) * elems + e;
    prev[o] = __float2bfloat16(st);
    st = st * ex2(cum_bh[c * L + L - 1] * LOG2E) + states[o];
  }
  final_state[idx] = st;
}

// ------------------------------------------------------------------------------------------------ 4. chunk scan
template <int N>
struct SmemScan {
  alignas(1024) uint8_t ct[N / 64][PANEL];     // C: [l][64 n] per panel (K-major A of G and of the state term)
  alignas(1024) uint8_t bw[2][PANEL];          // first B ([l'][64 n] per panel, N / 64 panels), then W ([l][64 l'] x 2)
  alignas(1024) uint8_t xt[PANEL];             // x: [l'][64 p]
  alignas(1024) uint8_t pv[N / 64][P * 128];   // incoming state: [p][64 n] per panel
  float cum2[L];                               // cum * log2(e)
  float dtv[L];
  uint64_t bar_full, bar_g, bar_w, bar_y;
  uint32_t tmem_base;
  volatile int abort_flag;
};

struct ScanParams {
  int seq_len, heads, groups, chunks;
  int v_div, v_mod;       // as in StateParams
  const float* dt;        // null: weight 1 (already folded into B)
  const float* cum;
  const float* d_skip;    // [H] or null
  const float* skip_tok;  // [B, H, L] per-token skip coefficient added to d_skip, or null
  int strict;             // 1: token l sees tokens j < l through the scores (its own term comes with the skip)
  __nv_bfloat16* y;       // [B*L, H*64]
  float* y32;             // when set, the result is written here in fp32 instead of `y`
  int* status;
};

template <int N, bool PH>
__global__ void __launch_bounds__(THREADS) chunk_scan_kernel(const __grid_constant__ CUtensorMap map_x,
                                                             const __grid_constant__ CUtensorMap map_b,
                                                             const __grid_constant__ CUtensorMap map_c,
                                                             const __grid_constant__ CUtensorMap map_prev, const ScanParams p) {
  extern __shared__ uint8_t raw_smem[];
  SmemScan<N>& s = *reinterpret_cast<SmemScan<N>*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int g = PH ? h : h / (p.heads / p.groups);
  const int row0 = b * p.seq_len + c * L;
  constexpr int KS = N / 16;           // K = 16 slices over d_state
  constexpr uint32_t PANEL16 = PANEL >> 4, PV16 = (P * 128) >> 4;

  if (threadIdx.x == 0) {
    s.abort_flag = 0;
    mbar_init(&s.bar_full, 1);
    mbar_init(&s.bar_g, 1);
    mbar_init(&s.bar_w, 4);
    mbar_init(&s.bar_y, 1);
    fence_barrier_init();
    prefetch_tmap(&map_x);
    prefetch_tmap(&map_b);
    prefetch_tmap(&map_c);
    prefetch_tmap(&map_prev);
  }
  if (warp == 4) tmem_alloc(&s.tmem_base, 256);   // G: columns [0, 128), Y: [128, 192)
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = s.tmem_base;
  volatile int* abortp = &s.abort_flag;

  if (warp == 4) {
    if (lane == 0) {
      mbar_arrive_expect_tx(&s.bar_full, (2 * (N / 64) + 1) * PANEL + (N / 64) * P * 128);
      for (int q = 0; q < N / 64; ++q) {
        tma_load_2d(s.ct[q], &map_c, &s.bar_full, g * N + q * 64, row0);
        tma_load_2d(s.bw[q], &map_b, &s.bar_full, g * N + q * 64, row0);
        if (!PH) tma_load_2d(s.pv[q], &map_prev, &s.bar_full, q * 64, (int)((((int64_t)b * p.chunks + c) * p.heads + h) * P));
      }
      if (PH)  // incoming state stored [n][p]: one 128-row tile
        tma_load_2d(s.pv[0], &map_prev, &s.bar_full, 0, (int)((((int64_t)b * p.chunks + c) * p.heads + h) * N));
      tma_load_2d(s.xt, &map_x, &s.bar_full, ((h / p.v_div) * p.v_mod + h % p.v_mod) * P, row0);
      const uint64_t kmajor0 = make_smem_desc(0, 16, 1024), mnmajor0 = make_smem_desc(0, PANEL, 1024);
      const uint32_t ct16 = smem_u32(s.ct[0]) >> 4, bw16 = smem_u32(s.bw[0]) >> 4, xt16 = smem_u32(s.xt) >> 4,
                     pv16 = smem_u32(s.pv[0]) >> 4;
      bool ok = mbar_wait(&s.bar_full, 0, abortp, p.status, 54);
      if (ok) {
        fence_after_sync();
        const uint32_t idesc_g = make_idesc_bf16(128, 128, 0, 0);
#pragma unroll
        for (int kk = 0; kk < KS; ++kk)
          mma_bf16(tmem, kmajor0 + ct16 + (kk >> 2) * PANEL16 + (kk & 3) * 2, kmajor0 + bw16 + (kk >> 2) * PANEL16 + (kk & 3) * 2,
                   idesc_g, kk);
        mma_commit(&s.bar_g);
        ok = mbar_wait(&s.bar_w, 0, abortp, p.status, 55);
      }
      if (ok) {
        fence_after_sync();
        const uint32_t idesc_y = make_idesc_bf16(128, 64, 0, 1);   // W (K-major) x X (rows are the reduction index)
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          mma_bf16(tmem + 128, kmajor0 + bw16 + (kk >> 2) * PANEL16 + (kk & 3) * 2, mnmajor0 + xt16 + 128 * kk, idesc_y, kk);
        // scaled C (K-major) x incoming state: [p][n] K-major, or (PH) [n][p] with the reduction index as the row
        const uint32_t idesc_s = make_idesc_bf16(128, 64, 0, PH ? 1 : 0);
#pragma unroll
        for (int kk = 0; kk < KS; ++kk)
          mma_bf16(tmem + 128, kmajor0 + ct16 + (kk >> 2) * PANEL16 + (kk & 3) * 2,
                   PH ? mnmajor0 + pv16 + 128 * kk : kmajor0 + pv16 + (kk >> 2) * PV16 + (kk & 3) * 2, idesc_s, 1);
        mma_commit(&s.bar_y);
      }
    }
  } else {
    const int l = warp * 32 + lane;
    const int64_t base = ((int64_t)b * p.heads + h) * p.seq_len + c * L;
    const float my_cum2 = p.cum[base + l] * LOG2E;
    s.cum2[l] = my_cum2;
    s.dtv[l] = p.dt ? p.dt[base + l] : 1.f;
    named_barrier_sync(1, 128);
    bool ok = mbar_wait(&s.bar_g, 0, abortp, p.status, 56);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      fence_after_sync();
      // W[l, j] = G[l, j] exp(cum_l - cum_j) dt_j for j <= l, else 0; bf16, K-major, two 64-column panels
      const uint32_t w_base = smem_u32(s.bw[0]);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t r[32];
        tmem_ld_32x32(tmem + ((uint32_t)(warp * 32) << 16) + q * 32, r);
        tmem_ld_wait();
        const uint32_t panel = w_base + (q >> 1) * PANEL + l * 128;
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          uint32_t w[4];
#pragma unroll
          for (int e2 = 0; e2 < 4; ++e2) {
            const int j = q * 32 + c8 * 8 + e2 * 2;
            float a = __uint_as_float(r[c8 * 8 + e2 * 2]) * ex2(my_cum2 - s.cum2[j]) * s.dtv[j];
            float bb = __uint_as_float(r[c8 * 8 + e2 * 2 + 1]) * ex2(my_cum2 - s.cum2[j + 1]) * s.dtv[j + 1];
            if (j + p.strict > l) a = 0.f;
            if (j + 1 + p.strict > l) bb = 0.f;
            w[e2] = pack2(a, bb);
          }
          const int chunk = (q & 1) * 4 + c8;
          sts128(panel + ((chunk ^ (l & 7)) << 4), make_uint4(w[0], w[1], w[2], w[3]));
        }
      }
      // C row l scaled by exp(cum_l) for the incoming-state term
      const float fc = ex2(my_cum2);
#pragma unroll
      for (int q = 0; q < N / 64; ++q) scale_row(smem_u32(s.ct[q]), l, fc);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.bar_w);
      ok = mbar_wait(&s.bar_y, 0, abortp, p.status, 57);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      fence_after_sync();
      uint32_t r0[32], r1[32];
      tmem_ld_32x32(tmem + ((uint32_t)(warp * 32) << 16) + 128, r0);
      tmem_ld_32x32(tmem + ((uint32_t)(warp * 32) << 16) + 160, r1);
      tmem_ld_wait();
      const float dsk = (p.d_skip ? p.d_skip[h] : 0.f) + (p.skip_tok ? p.skip_tok[base + l] : 0.f);
      const uint32_t xrow = smem_u32(s.xt) + l * 128;
      const int64_t out_off = ((int64_t)row0 + l) * (p.heads * P) + h * P;
      uint4* dst = reinterpret_cast<uint4*>(p.y + out_off);
      float4* dst32 = reinterpret_cast<float4*>(p.y32 + out_off);
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        const uint4 xv = lds128(xrow + ((ch ^ (l & 7)) << 4));
        const uint32_t* rr = ch < 4 ? r0 + ch * 8 : r1 + (ch - 4) * 8;
        const float2 x0 = unpack2(xv.x), x1 = unpack2(xv.y), x2 = unpack2(xv.z), x3 = unpack2(xv.w);
        const float o0 = __uint_as_float(rr[0]) + dsk * x0.x, o1 = __uint_as_float(rr[1]) + dsk * x0.y,
                    o2 = __uint_as_float(rr[2]) + dsk * x1.x, o3 = __uint_as_float(rr[3]) + dsk * x1.y,
                    o4 = __uint_as_float(rr[4]) + dsk * x2.x, o5 = __uint_as_float(rr[5]) + dsk * x2.y,
                    o6 = __uint_as_float(rr[6]) + dsk * x3.x, o7 = __uint_as_float(rr[7]) + dsk * x3.y;
        if (p.y32) {
          dst32[2 * ch] = make_float4(o0, o1, o2, o3);
          dst32[2 * ch + 1] = make_float4(o4, o5, o6, o7);
        } else {
          dst[ch] = make_uint4(pack2(o0, o1), pack2(o2, o3), pack2(o4, o5), pack2(o6, o7));
        }
      }
    }
  }
  __syncwarp();
  if (s.abort_flag) {
    const unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    fence_after_sync();
    tmem_dealloc(tmem, 256);
  }
}


// ------------------------------------------------------------------------------------------------ 5. decay gradient
// da_u = d loss / d a_u for the log-decay a_u of token u, given the output cotangent gy: the sum of
//   E_ts = e^{c_t - c_s} (cq_t . bk_s) w_s (gy_t . v_s)      over all pairs s < u <= t.
// Taken as differences of row sums (cq . dcq - bk . dbk) the pairs on one side of u cancel only in exact arithmetic;
// here every pair is counted once.  Per (batch, chunk, head), with H_in the state entering the chunk and dH_out the
// cotangent of the state leaving it (the incoming state of the time-reversed pass at the mirrored chunk, times the
// decay of the first token after the chunk, which that pass applies inside its chunk):
//   pairs inside the chunk     G1 = cq bk^T, G2 = gy v^T in TMEM; e = G1 o G2 o decay o w is formed once in fp32, its row
//                              sums R_t and (through a shared-memory transpose) column sums K_s give the block sums as
//                              sum_{u' >= u} (R_u' - K_u'): exact cancellation, since both sums see the same e
//   s before, t inside         sum_{t >= u} e^{c_t} gy_t . (cq_t H_in^T)
//   s inside, t after          sum_{s < u}  w_s e^{c_end - c_s} v_s . (bk_s dH_out^T)
//   s before, t after          e^{c_end} <H_in, dH_out>
// Replaces the reference's _chunk_scan_bwd_ddAcs_stable_kernel and the ddA parts of its dc / db / dstates kernels
// (backbones/mamba2/ops/triton/ssd_chunk_scan.py:1098, ssd_chunk_state.py:398, ssd_state_passing.py:102).
template <int N>
struct SmemDda {
  alignas(1024) uint8_t ct[N / 64][PANEL];
  alignas(1024) uint8_t bt[N / 64][PANEL];
  alignas(1024) uint8_t gyt[PANEL];
  alignas(1024) uint8_t xt[PANEL];
  alignas(1024) uint8_t hin[N / 64][P * 128];
  alignas(1024) uint8_t dho[N / 64][P * 128];
  float cum2[L];
  float wv[L];
  float r2[L];
  float r3[L];
  float red[4];
  float et[L][L + 1];   // e[t][s], padded rows: conflict-free row writes and column reads
  uint64_t bar_full, bar_mma, bar_rows;
  uint32_t tmem_base;
  volatile int abort_flag;
};

struct DdaParams {
  int seq_len, heads, groups, chunks;
  const float* weight;   // [B, H, L] or null
  const float* cum;      // [B, H, L]
  float* da;             // [B, H, L]
  int* status;
};

__device__ __forceinline__ float dot_row64(uint32_t row_addr, int l, const uint32_t* r0, const uint32_t* r1) {
  float acc = 0.f;
#pragma unroll
  for (int ch = 0; ch < 8; ++ch) {
    const uint4 v = lds128(row_addr + ((ch ^ (l & 7)) << 4));
    const uint32_t* rr = ch < 4 ? r0 + ch * 8 : r1 + (ch - 4) * 8;
    const float2 a = unpack2(v.x), b = unpack2(v.y), c = unpack2(v.z), d = unpack2(v.w);
    acc = fmaf(a.x, __uint_as_float(rr[0]), acc);
    acc = fmaf(a.y, __uint_as_float(rr[1]), acc);
    acc = fmaf(b.x, __uint_as_float(rr[2]), acc);
    acc = fmaf(b.y, __uint_as_float(rr[3]), acc);
    acc = fmaf(c.x, __uint_as_float(rr[4]), acc);
    acc = fmaf(c.y, __uint_as_float(rr[5]), acc);
    acc = fmaf(d.x, __uint_as_float(rr[6]), acc);
    acc = fmaf(d.y, __uint_as_float(rr[7]), acc);
  }
  return acc;
}

template <int N, bool PH>
__global__ void __launch_bounds__(THREADS) dda_kernel(const __grid_constant__ CUtensorMap map_x,
                                                      const __grid_constant__ CUtensorMap map_gy,
                                                      const __grid_constant__ CUtensorMap map_b,
                                                      const __grid_constant__ CUtensorMap map_c,
                                                      const __grid_constant__ CUtensorMap map_hin,
                                                      const __grid_constant__ CUtensorMap map_dho, const DdaParams p) {
  extern __shared__ uint8_t raw_smem[];
  SmemDda<N>& s = *reinterpret_cast<SmemDda<N>*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int g = PH ? h : h / (p.heads / p.groups);
  const int row0 = b * p.seq_len + c * L;
  constexpr int KS = N / 16;
  constexpr uint32_t PANEL16 = PANEL >> 4, PV16 = (P * 128) >> 4;
  constexpr uint32_t TMEM_COLS = 512;   // G1 [0, 128), G2 [128, 256), cq H_in^T [256, 320), bk dH_out^T [320, 384)

  if (threadIdx.x == 0) {
    s.abort_flag = 0;
    mbar_init(&s.bar_full, 1);
    mbar_init(&s.bar_mma, 1);
    mbar_init(&s.bar_rows, 4);
    fence_barrier_init();
    prefetch_tmap(&map_x);
    prefetch_tmap(&map_gy);
    prefetch_tmap(&map_b);
    prefetch_tmap(&map_c);
    prefetch_tmap(&map_hin);
    prefetch_tmap(&map_dho);
  }
  if (warp == 4) tmem_alloc(&s.tmem_base, TMEM_COLS);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = s.tmem_base;
  volatile int* abortp = &s.abort_flag;

  if (warp == 4) {
    if (lane == 0) {
      mbar_arrive_expect_tx(&s.bar_full, (2 * (N / 64) + 2) * PANEL + 2 * (N / 64) * P * 128);
      const int st_in = (int)((((int64_t)b * p.chunks + c) * p.heads + h) * (PH ? N : P));
      const int st_out = (int)((((int64_t)b * p.chunks + (p.chunks - 1 - c)) * p.heads + h) * (PH ? N : P));
      for (int q = 0; q < N / 64; ++q) {
        tma_load_2d(s.ct[q], &map_c, &s.bar_full, g * N + q * 64, row0);
        tma_load_2d(s.bt[q], &map_b, &s.bar_full, g * N + q * 64, row0);
        if (!PH) {
          tma_load_2d(s.hin[q], &map_hin, &s.bar_full, q * 64, st_in);
          tma_load_2d(s.dho[q], &map_dho, &s.bar_full, q * 64, st_out);
        }
      }
      if (PH) {
        tma_load_2d(s.hin[0], &map_hin, &s.bar_full, 0, st_in);
        tma_load_2d(s.dho[0], &map_dho, &s.bar_full, 0, st_out);
      }
      tma_load_2d(s.gyt, &map_gy, &s.bar_full, h * P, row0);
      tma_load_2d(s.xt, &map_x, &s.bar_full, h * P, row0);
      const uint64_t kmajor0 = make_smem_desc(0, 16, 1024), mnmajor0 = make_smem_desc(0, PANEL, 1024);
      const uint32_t ct16 = smem_u32(s.ct[0]) >> 4, bt16 = smem_u32(s.bt[0]) >> 4, gy16 = smem_u32(s.gyt) >> 4,
                     xt16 = smem_u32(s.xt) >> 4, hin16 = smem_u32(s.hin[0]) >> 4, dho16 = smem_u32(s.dho[0]) >> 4;
      const bool ok = mbar_wait(&s.bar_full, 0, abortp, p.status, 61);
      if (ok) {
        fence_after_sync();
        const uint32_t idesc_g = make_idesc_bf16(128, 128, 0, 0);
#pragma unroll
        for (int kk = 0; kk < KS; ++kk)
          mma_bf16(tmem, kmajor0 + ct16 + (kk >> 2) * PANEL16 + (kk & 3) * 2, kmajor0 + bt16 + (kk >> 2) * PANEL16 + (kk & 3) * 2,
                   idesc_g, kk);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) mma_bf16(tmem + 128, kmajor0 + gy16 + kk * 2, kmajor0 + xt16 + kk * 2, idesc_g, kk);
        const uint32_t idesc_s = make_idesc_bf16(128, 64, 0, PH ? 1 : 0);
#pragma unroll
        for (int kk = 0; kk < KS; ++kk)
          mma_bf16(tmem + 256, kmajor0 + ct16 + (kk >> 2) * PANEL16 + (kk & 3) * 2,
                   PH ? mnmajor0 + hin16 + 128 * kk : kmajor0 + hin16 + (kk >> 2) * PV16 + (kk & 3) * 2, idesc_s, kk);
#pragma unroll
        for (int kk = 0; kk < KS; ++kk)
          mma_bf16(tmem + 320, kmajor0 + bt16 + (kk >> 2) * PANEL16 + (kk & 3) * 2,
                   PH ? mnmajor0 + dho16 + 128 * kk : kmajor0 + dho16 + (kk >> 2) * PV16 + (kk & 3) * 2, idesc_s, kk);
        mma_commit(&s.bar_mma);
      }
    }
  } else {
    const int l = warp * 32 + lane;
    const int64_t base = ((int64_t)b * p.heads + h) * p.seq_len + c * L;
    const float my_cum2 = p.cum[base + l] * LOG2E;
    s.cum2[l] = my_cum2;
    s.wv[l] = p.weight ? p.weight[base + l] : 1.f;
    // decay of the first token of the next chunk (its first in-chunk cumulative value); 1 past the last chunk
    const float next_decay = c + 1 < p.chunks ? ex2(p.cum[base + L] * LOG2E) : 1.f;
    named_barrier_sync(1, 128);
    bool ok = mbar_wait(&s.bar_mma, 0, abortp, p.status, 62);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      fence_after_sync();
      const uint32_t trow = tmem + ((uint32_t)(warp * 32) << 16);
      // pairs inside the chunk: e[t][s] for s < t, row sum kept, the tile stored for the column sums
      float row_sum = 0.f;
      for (int q = 0; q <= warp; ++q) {
        uint32_t g1[32], g2[32];
        tmem_ld_32x32(trow + q * 32, g1);
        tmem_ld_32x32(trow + 128 + q * 32, g2);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int sidx = q * 32 + j;
          const float e = sidx < l ? __uint_as_float(g1[j]) * __uint_as_float(g2[j]) * ex2(my_cum2 - s.cum2[sidx]) * s.wv[sidx] : 0.f;
          row_sum += e;
          s.et[l][sidx] = e;
        }
      }
      // state terms
      uint32_t r0[32], r1[32];
      tmem_ld_32x32(trow + 256, r0);
      tmem_ld_32x32(trow + 288, r1);
      tmem_ld_wait();
      const float r2 = ex2(my_cum2) * dot_row64(smem_u32(s.gyt) + l * 128, l, r0, r1);
      tmem_ld_32x32(trow + 320, r0);
      tmem_ld_32x32(trow + 352, r1);
      tmem_ld_wait();
      const float cum_end2 = s.cum2[L - 1];
      s.r3[l] = next_decay * s.wv[l] * ex2(cum_end2 - my_cum2) * dot_row64(smem_u32(s.xt) + l * 128, l, r0, r1);
      // <H_in, dH_out>: both tiles have the same layout, so the product runs over raw 16-byte pieces
      float hd = 0.f;
      const uint32_t hin_a = smem_u32(s.hin[0]), dho_a = smem_u32(s.dho[0]);
      for (int off = l * 16; off < (N / 64) * P * 128; off += 128 * 16) {
        const uint4 a = lds128(hin_a + off), d = lds128(dho_a + off);
        const float2 a0 = unpack2(a.x), a1 = unpack2(a.y), a2 = unpack2(a.z), a3 = unpack2(a.w);
        const float2 d0 = unpack2(d.x), d1 = unpack2(d.y), d2 = unpack2(d.z), d3 = unpack2(d.w);
        hd += a0.x * d0.x + a0.y * d0.y + a1.x * d1.x + a1.y * d1.y + a2.x * d2.x + a2.y * d2.y + a3.x * d3.x + a3.y * d3.y;
      }
      hd = warp_sum(hd);
      if (lane == 0) s.red[warp] = hd;
      // every warp's tile rows must be in shared memory before the column sums: bounded waits, not bar.sync, so that a
      // warp that gave up above cannot strand the others
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.bar_rows);
      ok = mbar_wait(&s.bar_rows, 0, abortp, p.status, 63);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        float col_sum = 0.f;   // K_l = sum_{t > l} e[t][l]
        for (int t = l + 1; t < L; ++t) col_sum += s.et[t][l];
        s.r2[l] = r2 + row_sum - col_sum;
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.bar_rows);
        ok = mbar_wait(&s.bar_rows, 1, abortp, p.status, 64);
        ok = __all_sync(0xffffffffu, ok);
      }
    }
    if (ok) {
      const float cum_end2 = s.cum2[L - 1];
      float tail2 = 0.f, head3 = 0.f;
      for (int t = l; t < L; ++t) tail2 += s.r2[t];
      for (int t = 0; t < l; ++t) head3 += s.r3[t];
      const float through = next_decay * ex2(cum_end2) * (s.red[0] + s.red[1] + s.red[2] + s.red[3]);
      p.da[base + l] = tail2 + head3 + through;
    }
  }
  __syncwarp();
  if (s.abort_flag) {
    const unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    fence_after_sync();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}


// ------------------------------------------------------------------------------------------------ 5b. fused chunk backward
// All input cotangents of the scan
//   y_t = sum_{s <= t} e^{c_t - c_s} (cq_t . bk_s) w_s v_s + e^{c_t} cq_t . S_in        (s < t when `strict`)
// for one (direction, chunk, head) per CTA, from one pass over the tiles.  With W[t, s] = e^{c_t - c_s} on the causal
// mask, G1 = cq bk^T, G2 = gy v^T (both in TMEM, as in the decay-gradient kernel above):
//   M   = W o G1                  bf16 tile [t][s] in shared memory
//   dGw = W o G2 o w_s            bf16 tile [t][s] in shared memory
//   dX_s   = sum_t M[t, s] gy_t + e^{c_end - c_s} bk_s . D_out                         (cotangent of w_s v_s)
//   dcq_t  = sum_s dGw[t, s] bk_s + e^{c_t} gy_t . S_in
//   dbk_s  = sum_t dGw[t, s] cq_t + w_s e^{c_end - c_s} v_s . D_out
//   da_u   = the decay gradient (pairs s < u <= t; E = G1 o dGw, row and column sums; state terms through S_in, D_out)
//   dskip_t = gy_t . v_t = G2[t, t]
// S_in is the state entering the chunk (cached by the forward), D_out the cotangent of the state leaving it, produced by
// the reversed state passing below from the per-chunk sums sum_t e^{c_t} gy_t cq_t^T (chunk_state_kernel with `rev`).
// Forward operands (cq, bk, v, S_in, cum, w, skip) are indexed by batch b % bmod, so P stacked cotangent directions read one
// copy of them (from L2 after the first direction).  TMEM: G1 -> dcq [0, 128), G2 -> dbk [128, 256), cq S_in^T [256, 320),
// bk D_out^T [320, 384), dX [384, 448).  Replaces the reference's _chunk_scan_chunk_state_bwd_dx, _chunk_state_bwd_db,
// _chunk_scan_bwd_dc, _chunk_scan_bwd_dcb, _bmm_chunk_bwd and ddAcs kernels (backbones/mamba2/ops/triton/ssd_combined.py:396-513)
// and the Mamba-3 dqkv kernel (backbones/mamba3/ops/triton/mamba3/mamba3_siso_bwd.py:202-594).
constexpr int BWD_WARPS = 16;                       // compute warps: TMEM lane quarter = warp % 4, 32-column slice = warp / 4
constexpr int BWD_THREADS = (BWD_WARPS + 1) * 32;   // + one control warp (TMA, MMA issue)

template <int N>
struct SmemBwd {
  alignas(1024) uint8_t ct[N / 64][PANEL];      // cq [t][64 n] per panel
  alignas(1024) uint8_t bt[N / 64][PANEL];      // bk [s][64 n] per panel
  alignas(1024) uint8_t gyt[PANEL];             // gy [t][64 p]
  alignas(1024) uint8_t gys[PANEL];             // gy rows scaled by e^{c_t} (the A operand of the state term of dcq)
  alignas(1024) uint8_t xt[PANEL];              // v  [s][64 p]; rows scaled by w_s e^{c_end - c_s}
  alignas(1024) uint8_t hin[N / 64][P * 128];   // S_in
  alignas(1024) uint8_t dho[N / 64][P * 128];   // D_out
  alignas(1024) uint8_t mt[2][PANEL];           // M   [t][64 s] per panel
  alignas(1024) uint8_t gt[2][PANEL];           // dGw [t][64 s] per panel
  float colpart[4][L];                          // column sums of E per row quarter
  float rowpart[4][L];                          // row sums of E per column slice
  float cum2[L];
  float wv[L];
  float r2[L];
  float r3[L];
  float red[BWD_WARPS];
  uint64_t bar_full, bar_mma, bar_st, bar_w, bar_y, bar_rows;
  uint32_t tmem_base;
  volatile int abort_flag;
};

struct BwdParams {
  int seq_len, heads, groups, chunks, bmod, strict;
  const float* weight;     // [Bf, H, L] or null
  const float* cum;        // [Bf, H, L]
  const float* skip_tok;   // [Bf, H, L] or null: dv += skip * gy
  const float* d_skip;     // [H] or null: dv += d_skip[h] * gy
  float* da;               // [B, H, L]
  float* dskip;            // [B, H, L] or null
  float* dv32;             // [B * L, H * 64], one of dv32 / dv16
  __nv_bfloat16* dv16;
  float* dcq32;            // [B * L, H * N], one of the fp32 / bf16 pairs
  float* dbk32;
  __nv_bfloat16* dcq16;
  __nv_bfloat16* dbk16;
  int* status;
};

__device__ __forceinline__ void store_row(float* dst32, __nv_bfloat16* dst16, const uint32_t* r, int n) {
  if (dst32) {
    for (int e = 0; e < n / 4; ++e)
      reinterpret_cast<float4*>(dst32)[e] = make_float4(__uint_as_float(r[4 * e]), __uint_as_float(r[4 * e + 1]),
                                                        __uint_as_float(r[4 * e + 2]), __uint_as_float(r[4 * e + 3]));
  } else {
    for (int e = 0; e < n / 8; ++e)
      reinterpret_cast<uint4*>(dst16)[e] =
          make_uint4(pack2(__uint_as_float(r[8 * e]), __uint_as_float(r[8 * e + 1])),
                     pack2(__uint_as_float(r[8 * e + 2]), __uint_as_float(r[8 * e + 3])),
                     pack2(__uint_as_float(r[8 * e + 4]), __uint_as_float(r[8 * e + 5])),
                     pack2(__uint_as_float(r[8 * e + 6]), __uint_as_float(r[8 * e + 7])));
  }
}

// Columns [32 * half, 32 * half + 32) of row `row` of a 128-byte-row swizzled panel <- 32 fp32 values as bf16 (the layout a
// TMA store with the 128-byte swizzle reads).
__device__ __forceinline__ void stage_half_row(uint32_t panel, int row, int half, const uint32_t* r) {
  const uint32_t base = panel + row * 128;
#pragma unroll
  for (int c = 0; c < 4; ++c)
    sts128(base + (((half * 4 + c) ^ (row & 7)) << 4),
           make_uint4(pack2(__uint_as_float(r[8 * c]), __uint_as_float(r[8 * c + 1])),
                      pack2(__uint_as_float(r[8 * c + 2]), __uint_as_float(r[8 * c + 3])),
                      pack2(__uint_as_float(r[8 * c + 4]), __uint_as_float(r[8 * c + 5])),
                      pack2(__uint_as_float(r[8 * c + 6]), __uint_as_float(r[8 * c + 7]))));
}

// Lane j of the warp ends with sum over the 32 lanes of their v[j] (a transposing butterfly: 31 shuffles, no shared memory).
__device__ __forceinline__ float warp_column_sums(float* v, int lane) {
#pragma unroll
  for (int step = 16, n = 32; step >= 1; step >>= 1, n >>= 1) {
    const bool upper = (lane & step) != 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if (i < n / 2) {
        const float send = upper ? v[i] : v[i + n / 2];
        const float keep = upper ? v[i + n / 2] : v[i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, step);
      }
    }
  }
  return v[0];
}

// Partial dot product of a 64-column bf16 row (128-byte swizzled) with 32 fp32 values: columns [32 * half, 32 * half + 32).
__device__ __forceinline__ float dot_row32(uint32_t row_addr, int l, int half, const uint32_t* r) {
  float acc = 0.f;
#pragma unroll
  for (int ch = 0; ch < 4; ++ch) {
    const uint4 v = lds128(row_addr + (((half * 4 + ch) ^ (l & 7)) << 4));
    const uint32_t* rr = r + ch * 8;
    const float2 a = unpack2(v.x), b = unpack2(v.y), c = unpack2(v.z), d = unpack2(v.w);
    acc = fmaf(a.x, __uint_as_float(rr[0]), acc);
    acc = fmaf(a.y, __uint_as_float(rr[1]), acc);
    acc = fmaf(b.x, __uint_as_float(rr[2]), acc);
    acc = fmaf(b.y, __uint_as_float(rr[3]), acc);
    acc = fmaf(c.x, __uint_as_float(rr[4]), acc);
    acc = fmaf(c.y, __uint_as_float(rr[5]), acc);
    acc = fmaf(d.x, __uint_as_float(rr[6]), acc);
    acc = fmaf(d.y, __uint_as_float(rr[7]), acc);
  }
  return acc;
}

// Multiply columns [32 * half, 32 * half + 32) of row `row` of a 128-byte-row panel by f, in place.
__device__ __forceinline__ void scale_half_row(uint32_t panel, int row, int half, float f) {
  const uint32_t base = panel + row * 128;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint32_t addr = base + (((half * 4 + c) ^ (row & 7)) << 4);
    uint4 v = lds128(addr);
    float2 a = unpack2(v.x), b = unpack2(v.y), cc = unpack2(v.z), d = unpack2(v.w);
    v.x = pack2(a.x * f, a.y * f);
    v.y = pack2(b.x * f, b.y * f);
    v.z = pack2(cc.x * f, cc.y * f);
    v.w = pack2(d.x * f, d.y * f);
    sts128(addr, v);
  }
}

// One half (16 columns) of a 32 x 32 block of the two Gram tiles: thread = row l.  Reads G1 = cq bk^T and G2 = gy v^T from
// TMEM, forms W = e^{c_t - c_s} (masked to s + strict <= t when MASKED), writes M = W o G1 and dGw = W o G2 o w_s as bf16
// into the swizzled operand panels, and leaves E = G1 o dGw (s < t) in ev for the row / column sums.
template <bool MASKED>
__device__ __forceinline__ void tile_half(uint32_t trow, int q, int hf, int l, float my_cum2, int strict, const float* cum2,
                                          const float* wv, uint32_t m_row, uint32_t g_row, float* ev, float& row_sum,
                                          float& diag_g2) {
  uint32_t g1[16], g2[16];
  tmem_ld_32x16(trow + q * 32 + hf * 16, g1);
  tmem_ld_32x16(trow + 128 + q * 32 + hf * 16, g2);
  tmem_ld_wait();
  const float4* c4 = reinterpret_cast<const float4*>(cum2 + q * 32 + hf * 16);   // every lane reads the same words
  const float4* w4 = reinterpret_cast<const float4*>(wv + q * 32 + hf * 16);
#pragma unroll
  for (int j4 = 0; j4 < 4; ++j4) {
    const float4 cv = c4[j4], wv4 = w4[j4];
    const float cj[4] = {cv.x, cv.y, cv.z, cv.w}, wj[4] = {wv4.x, wv4.y, wv4.z, wv4.w};
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = 4 * j4 + u;
      const int sidx = q * 32 + hf * 16 + j;
      float wdec = ex2(my_cum2 - cj[u]);
      if (MASKED) wdec = sidx + strict <= l ? wdec : 0.f;
      const float m = __uint_as_float(g1[j]) * wdec;
      const float dg = __uint_as_float(g2[j]) * wdec * wj[u];
      float e = __uint_as_float(g1[j]) * dg;
      if (MASKED) {
        e = sidx < l ? e : 0.f;
        if (sidx == l) diag_g2 = __uint_as_float(g2[j]);
      }
      row_sum += e;
      ev[hf * 16 + j] = e;
      g1[j] = __float_as_uint(m);
      g2[j] = __float_as_uint(dg);
    }
  }
#pragma unroll
  for (int c8 = 0; c8 < 2; ++c8) {
    const int chunk = (q & 1) * 4 + hf * 2 + c8;
    const uint32_t* a = g1 + c8 * 8;
    const uint32_t* d = g2 + c8 * 8;
    sts128(m_row + ((chunk ^ (l & 7)) << 4),
           make_uint4(pack2(__uint_as_float(a[0]), __uint_as_float(a[1])), pack2(__uint_as_float(a[2]), __uint_as_float(a[3])),
                      pack2(__uint_as_float(a[4]), __uint_as_float(a[5])), pack2(__uint_as_float(a[6]), __uint_as_float(a[7]))));
    sts128(g_row + ((chunk ^ (l & 7)) << 4),
           make_uint4(pack2(__uint_as_float(d[0]), __uint_as_float(d[1])), pack2(__uint_as_float(d[2]), __uint_as_float(d[3])),
                      pack2(__uint_as_float(d[4]), __uint_as_float(d[5])), pack2(__uint_as_float(d[6]), __uint_as_float(d[7]))));
  }
}

// The same into another panel: dst row <- f * src row, columns [32 * half, 32 * half + 32).
__device__ __forceinline__ void scale_half_row_to(uint32_t src_panel, uint32_t dst_panel, int row, int half, float f) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint32_t off = row * 128 + (((half * 4 + c) ^ (row & 7)) << 4);
    uint4 v = lds128(src_panel + off);
    float2 a = unpack2(v.x), b = unpack2(v.y), cc = unpack2(v.z), d = unpack2(v.w);
    v.x = pack2(a.x * f, a.y * f);
    v.y = pack2(b.x * f, b.y * f);
    v.z = pack2(cc.x * f, cc.y * f);
    v.w = pack2(d.x * f, d.y * f);
    sts128(dst_panel + off, v);
  }
}

template <int N, bool PH>
__global__ void __launch_bounds__(BWD_THREADS, 1) bwd_chunk_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                   const __grid_constant__ CUtensorMap map_gy,
                                                                   const __grid_constant__ CUtensorMap map_b,
                                                                   const __grid_constant__ CUtensorMap map_c,
                                                                   const __grid_constant__ CUtensorMap map_hin,
                                                                   const __grid_constant__ CUtensorMap map_dho,
                                                                   const __grid_constant__ CUtensorMap map_dv,
                                                                   const __grid_constant__ CUtensorMap map_dcq,
                                                                   const __grid_constant__ CUtensorMap map_dbk, const BwdParams p) {
  extern __shared__ uint8_t raw_smem[];
  SmemBwd<N>& s = *reinterpret_cast<SmemBwd<N>*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int fb = b % p.bmod;
  const int g = PH ? h : h / (p.heads / p.groups);
  const int row0 = b * p.seq_len + c * L, frow0 = fb * p.seq_len + c * L;
  constexpr int KS = N / 16;
  constexpr uint32_t PANEL16 = PANEL >> 4, PV16 = (P * 128) >> 4;
  constexpr uint32_t TMEM_COLS = 512;

  if (warp == BWD_WARPS) {
    if (lane == 0) {   // the loads go out before the CTA-wide sync: their latency covers the TMEM allocation and the setup
      s.abort_flag = 0;
      mbar_init(&s.bar_full, 1);
      mbar_init(&s.bar_mma, 1);
      mbar_init(&s.bar_st, 1);
      mbar_init(&s.bar_w, BWD_WARPS);
      mbar_init(&s.bar_y, 1);
      mbar_init(&s.bar_rows, BWD_WARPS);
      fence_barrier_init();
      mbar_arrive_expect_tx(&s.bar_full, (2 * (N / 64) + 2) * PANEL + 2 * (N / 64) * P * 128);
      const int st_in = (int)((((int64_t)fb * p.chunks + c) * p.heads + h) * (PH ? N : P));
      const int st_out = (int)((((int64_t)b * p.chunks + c) * p.heads + h) * (PH ? N : P));
      for (int q = 0; q < N / 64; ++q) {
        tma_load_2d(s.ct[q], &map_c, &s.bar_full, g * N + q * 64, frow0);
        tma_load_2d(s.bt[q], &map_b, &s.bar_full, g * N + q * 64, frow0);
      }
      tma_load_2d(s.gyt, &map_gy, &s.bar_full, h * P, row0);
      tma_load_2d(s.xt, &map_x, &s.bar_full, h * P, frow0);
      for (int q = 0; q < N / 64; ++q) {
        if (!PH) {
          tma_load_2d(s.hin[q], &map_hin, &s.bar_full, q * 64, st_in);
          tma_load_2d(s.dho[q], &map_dho, &s.bar_full, q * 64, st_out);
        }
      }
      if (PH) {
        tma_load_2d(s.hin[0], &map_hin, &s.bar_full, 0, st_in);
        tma_load_2d(s.dho[0], &map_dho, &s.bar_full, 0, st_out);
      }
      prefetch_tmap(&map_dv);
      prefetch_tmap(&map_dcq);
      prefetch_tmap(&map_dbk);
    }
    __syncwarp();
    tmem_alloc(&s.tmem_base, TMEM_COLS);
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = s.tmem_base;
  volatile int* abortp = &s.abort_flag;

  if (warp == BWD_WARPS) {
    if (lane == 0) {
      const uint64_t kmajor0 = make_smem_desc(0, 16, 1024), mnmajor0 = make_smem_desc(0, PANEL, 1024),
                     mnstate0 = make_smem_desc(0, P * 128, 1024);
      const uint32_t ct16 = smem_u32(s.ct[0]) >> 4, bt16 = smem_u32(s.bt[0]) >> 4, gy16 = smem_u32(s.gyt) >> 4, gys16 = smem_u32(s.gys) >> 4,
                     xt16 = smem_u32(s.xt) >> 4, hin16 = smem_u32(s.hin[0]) >> 4, dho16 = smem_u32(s.dho[0]) >> 4,
                     mt16 = smem_u32(s.mt[0]) >> 4, gt16 = smem_u32(s.gt[0]) >> 4;
      bool ok = mbar_wait(&s.bar_full, 0, abortp, p.status, 71);
      if (ok) {
        fence_after_sync();
        const uint32_t idesc_g = make_idesc_bf16(128, 128, 0, 0);
#pragma unroll
        for (int kk = 0; kk < KS; ++kk)
          mma_bf16(tmem, kmajor0 + ct16 + (kk >> 2) * PANEL16 + (kk & 3) * 2, kmajor0 + bt16 + (kk >> 2) * PANEL16 + (kk & 3) * 2,
                   idesc_g, kk);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) mma_bf16(tmem + 128, kmajor0 + gy16 + kk * 2, kmajor0 + xt16 + kk * 2, idesc_g, kk);
        mma_commit(&s.bar_mma);   // the compute warps start on the two Gram tiles while the state products run
        const uint32_t idesc_s = make_idesc_bf16(128, 64, 0, PH ? 1 : 0);
#pragma unroll
        for (int kk = 0; kk < KS; ++kk)
          mma_bf16(tmem + 256, kmajor0 + ct16 + (kk >> 2) * PANEL16 + (kk & 3) * 2,
                   PH ? mnmajor0 + hin16 + 128 * kk : kmajor0 + hin16 + (kk >> 2) * PV16 + (kk & 3) * 2, idesc_s, kk);
#pragma unroll
        for (int kk = 0; kk < KS; ++kk)
          mma_bf16(tmem + 320, kmajor0 + bt16 + (kk >> 2) * PANEL16 + (kk & 3) * 2,
                   PH ? mnmajor0 + dho16 + 128 * kk : kmajor0 + dho16 + (kk >> 2) * PV16 + (kk & 3) * 2, idesc_s, kk);
        mma_commit(&s.bar_st);
        ok = mbar_wait(&s.bar_w, 0, abortp, p.status, 72);
      }
      if (ok) {
        fence_after_sync();
        // dX[s, p] = sum_t M[t, s] gy[t, p]: both operands have the reduction index t as their row
        const uint32_t idesc_x = make_idesc_bf16(128, 64, 1, 1);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) mma_bf16(tmem + 384, mnmajor0 + mt16 + 128 * kk, mnmajor0 + gy16 + 128 * kk, idesc_x, kk);
        // dcq[t, n] = sum_s dGw[t, s] bk[s, n]
        const uint32_t idesc_q = make_idesc_bf16(128, N, 0, 1);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          mma_bf16(tmem, kmajor0 + gt16 + (kk >> 2) * PANEL16 + (kk & 3) * 2, mnmajor0 + bt16 + 128 * kk, idesc_q, kk);
        // dbk[s, n] = sum_t dGw[t, s] cq[t, n] + sum_p v'[s, p] D_out[p, n]
        const uint32_t idesc_k = make_idesc_bf16(128, N, 1, 1);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) mma_bf16(tmem + 128, mnmajor0 + gt16 + 128 * kk, mnmajor0 + ct16 + 128 * kk, idesc_k, kk);
        const uint32_t idesc_st = make_idesc_bf16(128, N, 0, PH ? 0 : 1);   // state [n][p]: K-major B; [p][n]: rows are the reduction index
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          mma_bf16(tmem + 128, kmajor0 + xt16 + kk * 2, PH ? kmajor0 + dho16 + kk * 2 : mnstate0 + dho16 + 128 * kk, idesc_st, 1);
        // dcq[t, n] += sum_p gy'[t, p] S_in[p, n], gy' = e^{c_t} gy from the scaled copy
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          mma_bf16(tmem, kmajor0 + gys16 + kk * 2, PH ? kmajor0 + hin16 + kk * 2 : mnstate0 + hin16 + 128 * kk, idesc_st, 1);
        mma_commit(&s.bar_y);
      }
    }
  } else {
    // 16 compute warps: row l of the tile (TMEM lane) and the 32-column slice q of it
    const int rg = warp & 3, q = warp >> 2;
    const int l = rg * 32 + lane;
    const int64_t base = ((int64_t)b * p.heads + h) * p.seq_len + c * L;
    const int64_t fbase = ((int64_t)fb * p.heads + h) * p.seq_len + c * L;
    const float my_cum2 = p.cum[fbase + l] * LOG2E;
    const float my_w = p.weight ? p.weight[fbase + l] : 1.f;
    const float sk = (p.d_skip ? p.d_skip[h] : 0.f) + (p.skip_tok ? p.skip_tok[fbase + l] : 0.f);
    if (q == 0) {
      s.cum2[l] = my_cum2;
      s.wv[l] = my_w;
    }
    named_barrier_sync(1, BWD_WARPS * 32);
    const float cum_end2 = s.cum2[L - 1];
    const float f_end = ex2(cum_end2 - my_cum2);
    const uint32_t trow = tmem + ((uint32_t)(rg * 32) << 16);
    float diag_g2 = 0.f, state_part = 0.f;
    bool ok = mbar_wait(&s.bar_mma, 0, abortp, p.status, 74);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      fence_after_sync();
      const uint32_t m_row = smem_u32(s.mt[0]) + (q >> 1) * PANEL + l * 128, g_row = smem_u32(s.gt[0]) + (q >> 1) * PANEL + l * 128;
      if (q > rg) {   // this 32 x 32 block lies above the diagonal for every row of the warp
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          const int chunk = (q & 1) * 4 + c8;
          sts128(m_row + ((chunk ^ (l & 7)) << 4), make_uint4(0, 0, 0, 0));
          sts128(g_row + ((chunk ^ (l & 7)) << 4), make_uint4(0, 0, 0, 0));
        }
        s.colpart[rg][q * 32 + lane] = 0.f;
        s.rowpart[q][l] = 0.f;
      } else {
        // two halves of 16 columns: both Gram slices of a half, the decay, the two products, packed and stored; only the
        // fp32 products E stay live for the column sums.  Blocks strictly below the diagonal take the form without masks.
        float ev[32];
        float row_sum = 0.f;
        if (q < rg) {
          tile_half<false>(trow, q, 0, l, my_cum2, p.strict, s.cum2, s.wv, m_row, g_row, ev, row_sum, diag_g2);
          tile_half<false>(trow, q, 1, l, my_cum2, p.strict, s.cum2, s.wv, m_row, g_row, ev, row_sum, diag_g2);
        } else {
          tile_half<true>(trow, q, 0, l, my_cum2, p.strict, s.cum2, s.wv, m_row, g_row, ev, row_sum, diag_g2);
          tile_half<true>(trow, q, 1, l, my_cum2, p.strict, s.cum2, s.wv, m_row, g_row, ev, row_sum, diag_g2);
        }
        s.rowpart[q][l] = row_sum;
        s.colpart[rg][q * 32 + lane] = warp_column_sums(ev, lane);
        if (q == rg && p.dskip) p.dskip[base + l] = diag_g2;   // gy_t . v_t sits on the diagonal of G2
      }
      // state terms of the decay gradient (unscaled gy and v rows), split over the column slices:
      //   q = 0, 1: halves of e^{c_t} gy_t . (cq_t S_in^T);  q = 2, 3: halves of w_s e^{c_end - c_s} v_s . (bk_s D_out^T)
      ok = mbar_wait(&s.bar_st, 0, abortp, p.status, 79);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        fence_after_sync();
        uint32_t r[32];
        tmem_ld_32x32(trow + (q < 2 ? 256 : 320) + (q & 1) * 32, r);
        tmem_ld_wait();
        state_part = (q < 2 ? ex2(my_cum2) : my_w * f_end) * dot_row32(smem_u32(q < 2 ? s.gyt : s.xt) + l * 128, l, q & 1, r);
      }
      // <S_in, D_out>: both tiles have the same layout, so the product runs over raw 16-byte pieces
      {
        float hd = 0.f;
        const uint32_t hin_a = smem_u32(s.hin[0]), dho_a = smem_u32(s.dho[0]);
        for (int off = (warp * 32 + lane) * 16; off < (N / 64) * P * 128; off += BWD_WARPS * 32 * 16) {
          const uint4 a = lds128(hin_a + off), d = lds128(dho_a + off);
          const float2 a0 = unpack2(a.x), a1 = unpack2(a.y), a2 = unpack2(a.z), a3 = unpack2(a.w);
          const float2 d0 = unpack2(d.x), d1 = unpack2(d.y), d2 = unpack2(d.z), d3 = unpack2(d.w);
          hd += a0.x * d0.x + a0.y * d0.y + a1.x * d1.x + a1.y * d1.y + a2.x * d2.x + a2.y * d2.y + a3.x * d3.x + a3.y * d3.y;
        }
        hd = warp_sum(hd);
        if (lane == 0) s.red[warp] = hd;
      }
      // v rows scaled in place for the state term of dbk (slices 2 and 3 own the halves they just read); gy rows scaled by
      // e^{c_t} into a copy for the state term of dcq (dX and the skip term need the unscaled rows)
      if (ok) {
        if (q >= 2) scale_half_row(smem_u32(s.xt), l, q & 1, my_w * f_end);
        else scale_half_row_to(smem_u32(s.gyt), smem_u32(s.gys), l, q, ex2(my_cum2));
      }
    }
    // the two halves of each state term meet in r2 / r3 (shared-memory adds); the barrier is taken by every compute warp,
    // whether or not its waits succeeded, so that a warp that gave up cannot strand the others at it
    if ((q & 1) == 0) (q < 2 ? s.r2 : s.r3)[l] = 0.f;
    named_barrier_sync(2, BWD_WARPS * 32);
    if (ok) {
      atomicAdd((q < 2 ? s.r2 : s.r3) + l, state_part);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s.bar_w);
        mbar_arrive(&s.bar_rows);
      }
      ok = mbar_wait(&s.bar_rows, 0, abortp, p.status, 75);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      if (q == 0) {
        const float col_sum = s.colpart[0][l] + s.colpart[1][l] + s.colpart[2][l] + s.colpart[3][l];
        const float row_sum = s.rowpart[0][l] + s.rowpart[1][l] + s.rowpart[2][l] + s.rowpart[3][l];
        s.r2[l] += row_sum - col_sum;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.bar_rows);
      ok = mbar_wait(&s.bar_rows, 1, abortp, p.status, 76);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      if (q == 3) {   // one slice finishes the decay gradient of its row: suffix sums of r2, prefix sums of r3
        float suf = s.r2[l], pre = s.r3[l];
        float later2 = 0.f, earlier3 = 0.f;
#pragma unroll
        for (int gq = 0; gq < 4; ++gq) {   // totals of the other row quarters
          const float t2 = warp_sum(s.r2[gq * 32 + lane]), t3 = warp_sum(s.r3[gq * 32 + lane]);
          if (gq > rg) later2 += t2;
          if (gq < rg) earlier3 += t3;
        }
        const float own3 = pre;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const float d2 = __shfl_down_sync(0xffffffffu, suf, o), u3 = __shfl_up_sync(0xffffffffu, pre, o);
          if (lane + o < 32) suf += d2;
          if (lane >= o) pre += u3;
        }
        float through = 0.f;
#pragma unroll
        for (int w = 0; w < BWD_WARPS; ++w) through += s.red[w];
        p.da[base + l] = (suf + later2) + (pre - own3 + earlier3) + ex2(cum_end2) * through;
      }
      if (ok) ok = mbar_wait(&s.bar_y, 0, abortp, p.status, 78);
      ok = __all_sync(0xffffffffu, ok);
    }
    // Epilogue.  bf16 results are staged in shared memory (the operand tiles are dead once the last product has completed) in the
    // swizzled layout and leave with TMA stores: written row by row from the registers, a warp's 32 rows lie kilobytes apart
    // and every store instruction splits into 32 transactions.  fp32 results (dv of the SSD form) keep the direct stores.
    if (ok) {
      fence_after_sync();
      const int64_t tok = (int64_t)row0 + l;
      if (q < 2) {   // dX columns [32 q, 32 q + 32): intra-chunk part + state term + skip * gy
        uint32_t x0[32], t0[32];
        tmem_ld_32x32(trow + 384 + q * 32, x0);
        tmem_ld_32x32(trow + 320 + q * 32, t0);
        tmem_ld_wait();
        const uint32_t gy_row = smem_u32(s.gyt) + l * 128;   // the unscaled gy row, for the skip term
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const uint4 gv = lds128(gy_row + (((q * 4 + ch) ^ (l & 7)) << 4));
          const float2 g0 = unpack2(gv.x), g1v = unpack2(gv.y), g2v = unpack2(gv.z), g3 = unpack2(gv.w);
          const float gyv[8] = {g0.x, g0.y, g1v.x, g1v.y, g2v.x, g2v.y, g3.x, g3.y};
#pragma unroll
          for (int e = 0; e < 8; ++e)
            x0[ch * 8 + e] = __float_as_uint(__uint_as_float(x0[ch * 8 + e]) + f_end * __uint_as_float(t0[ch * 8 + e]) + sk * gyv[e]);
        }
        if (p.dv16) stage_half_row(smem_u32(s.mt[0]), l, q, x0);
        else store_row(p.dv32 + (tok * p.heads + h) * P + q * 32, nullptr, x0, 32);
      }
      if (q < N / 32) {
        const int64_t off_n = (tok * p.heads + h) * N + q * 32;
        uint32_t r[32];
        tmem_ld_32x32(trow + q * 32, r);
        tmem_ld_wait();
        if (p.dcq16) stage_half_row(smem_u32(s.ct[q >> 1]), l, q & 1, r);
        else store_row(p.dcq32 + off_n, nullptr, r, 32);
        tmem_ld_32x32(trow + 128 + q * 32, r);
        tmem_ld_wait();
        if (p.dbk16) stage_half_row(smem_u32(s.bt[q >> 1]), l, q & 1, r);
        else store_row(p.dbk32 + off_n, nullptr, r, 32);
      }
      fence_proxy_async();
    }
    // taken by every compute warp, whether or not its waits succeeded
    named_barrier_sync(1, BWD_WARPS * 32);
    if (warp == 0 && lane == 0 && !s.abort_flag) {
      if (p.dv16) tma_store_2d(&map_dv, s.mt[0], h * P, row0);
      for (int qq = 0; qq < N / 64; ++qq) {
        if (p.dcq16) tma_store_2d(&map_dcq, s.ct[qq], h * N + qq * 64, row0);
        if (p.dbk16) tma_store_2d(&map_dbk, s.bt[qq], h * N + qq * 64, row0);
      }
      tma_store_commit();
      tma_store_wait_read<0>();   // shared memory is released when the CTA exits
    }
  }
  __syncwarp();
  if (s.abort_flag) {
    const unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == BWD_WARPS) {
    fence_after_sync();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// Reversed state passing: chunk_cot [B, C, H, elems] fp32 holds sum_t e^{c_t} gy_t cq_t^T per chunk; d_out[c] (bf16) is the
// cotangent of the state leaving chunk c, d_init the cotangent of the state entering the first chunk.
__global__ void rev_state_passing_kernel(const float* __restrict__ chunk_cot, const float* __restrict__ cum,
                                         const float* __restrict__ d_final, __nv_bfloat16* __restrict__ d_out,
                                         float* __restrict__ d_init, int batch, int bmod, int heads, int chunks, int seq_len,
                                         int elems) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)batch * heads * elems) return;
  const int e = (int)(idx % elems);
  const int h = (int)((idx / elems) % heads);
  const int b = (int)(idx / ((int64_t)elems * heads));
  float st = d_final ? d_final[idx] : 0.f;
  const float* cum_bh = cum + ((int64_t)(b % bmod) * heads + h) * seq_len;
  for (int c = chunks - 1; c >= 0; --c) {
    const int64_t o = (((int64_t)b * chunks + c) * heads + h) * elems + e;
    d_out[o] = __float2bfloat16(st);
    st = st * ex2(cum_bh[c * L + L - 1] * LOG2E) + chunk_cot[o];
  }
  if (d_init) d_init[idx] = st;
}

// Reversed state passing fused with its chunk products: one CTA owns one head (PH) or two heads of a group of one batch row
// and walks the chunks from the last to the first.  Per chunk the TMA thread loads the gy and cq tiles (two stages), the
// compute warps scale the gy rows by e^{c_t} in shared memory, one thread issues the product sum_t e^{c_t} gy_t cq_t^T into
// one of two TMEM buffers, and each compute thread keeps one row of the running cotangent state in registers:
//   d_out[c] = state (bf16, written while the product runs),   state = e^{cum_end(c)} state + product(c).
// Nothing but gy, cq and d_out touches global memory (the per-chunk products and the running state stay on chip).
template <int N, bool PH>
struct SmemRev {
  alignas(1024) uint8_t xs[2][PH ? 1 : 2][PANEL];   // [stage][head]: gy [l][64 p]
  alignas(1024) uint8_t bt[2][N / 64][PANEL];       // [stage]: cq [l][64 n] per panel
  uint64_t bar_full[2], bar_scaled[2], bar_done[2], bar_free[2];
  uint32_t tmem_base;
  volatile int abort_flag;
};

struct RevParams {
  int seq_len, heads, groups, chunks, bmod;
  const float* cum;        // [bmod, H, L_total]
  const float* d_final;    // [B, H, elems] or null
  __nv_bfloat16* d_out;    // [B, C, H, elems]
  float* d_init;           // [B, H, elems] or null
  int* status;
};

template <int N, bool PH>
__global__ void __launch_bounds__(THREADS, PH ? 2 : 1) rev_state_kernel(const __grid_constant__ CUtensorMap map_g,
                                                                         const __grid_constant__ CUtensorMap map_c,
                                                                         const RevParams p) {
  extern __shared__ uint8_t raw_smem[];
  SmemRev<N, PH>& s = *reinterpret_cast<SmemRev<N, PH>*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hp = blockIdx.x, b = blockIdx.y;
  const int h0 = PH ? hp : 2 * hp;
  const int g = PH ? h0 : h0 / (p.heads / p.groups);
  const int fb = b % p.bmod;
  constexpr uint32_t COLS = PH ? 64 : N;          // TMEM columns of one product
  constexpr int ROW = PH ? P : N;                 // elements of the state row a compute thread keeps
  constexpr int ELEMS = P * N;

  if (threadIdx.x == 0) {
    s.abort_flag = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.bar_full[i], 1);
      mbar_init(&s.bar_scaled[i], 4);
      mbar_init(&s.bar_done[i], 1);
      mbar_init(&s.bar_free[i], 4);
    }
    fence_barrier_init();
    prefetch_tmap(&map_g);
    prefetch_tmap(&map_c);
  }
  if (warp == 4) tmem_alloc(&s.tmem_base, 2 * COLS);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = s.tmem_base;
  volatile int* abortp = &s.abort_flag;

  if (warp == 4) {
    if (lane == 0) {
      auto issue_loads = [&](int it) {
        const int c = p.chunks - 1 - it, st = it & 1;
        const int row0 = b * p.seq_len + c * L, frow0 = fb * p.seq_len + c * L;
        mbar_arrive_expect_tx(&s.bar_full[st], ((PH ? 1 : 2) + N / 64) * PANEL);
        tma_load_2d(s.xs[st][0], &map_g, &s.bar_full[st], h0 * P, row0);
        if (!PH) tma_load_2d(s.xs[st][PH ? 0 : 1], &map_g, &s.bar_full[st], (h0 + 1) * P, row0);
        for (int q = 0; q < N / 64; ++q) tma_load_2d(s.bt[st][q], &map_c, &s.bar_full[st], g * N + q * 64, frow0);
      };
      issue_loads(0);
      bool ok = true;
      for (int it = 0; it < p.chunks && ok; ++it) {
        const int st = it & 1, k = it >> 1;
        if (it + 1 < p.chunks) {
          // the stage of chunk it + 1 was read by the product of chunk it - 1
          if (it >= 1) ok = mbar_wait(&s.bar_done[(it + 1) & 1], ((it - 1) >> 1) & 1, abortp, p.status, 54);
          if (!ok) break;
          issue_loads(it + 1);
        }
        ok = mbar_wait(&s.bar_scaled[st], k & 1, abortp, p.status, 55);
        if (ok && it >= 2) ok = mbar_wait(&s.bar_free[st], (k - 1) & 1, abortp, p.status, 56);
        if (!ok) break;
        fence_after_sync();
        const uint32_t idesc = make_idesc_bf16(128, PH ? 64 : N, 1, 1);
        const uint64_t da = make_smem_desc(smem_u32(PH ? s.bt[st][0] : s.xs[st][0]), PANEL, 1024);
        const uint64_t db = make_smem_desc(smem_u32(PH ? s.xs[st][0] : s.bt[st][0]), PANEL, 1024);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) mma_bf16(tmem + st * COLS, da + 128 * kk, db + 128 * kk, idesc, kk);
        mma_commit(&s.bar_done[st]);
      }
    }
  } else {
    const int l = warp * 32 + lane;   // token of the chunk in the scaling pass; row of the state otherwise
    const int h = PH ? h0 : h0 + (l >> 6), pp = l & 63;
    const int64_t row_off = PH ? (int64_t)l * P : (int64_t)pp * N;
    const int64_t bh = (int64_t)b * p.heads + h;
    float stv[ROW];
    if (p.d_final) {
      const float4* src = reinterpret_cast<const float4*>(p.d_final + bh * ELEMS + row_off);
#pragma unroll
      for (int e = 0; e < ROW / 4; ++e) {
        const float4 v = src[e];
        stv[4 * e] = v.x; stv[4 * e + 1] = v.y; stv[4 * e + 2] = v.z; stv[4 * e + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int e = 0; e < ROW; ++e) stv[e] = 0.f;
    }
    bool ok = true;
    for (int it = 0; it < p.chunks && ok; ++it) {
      const int c = p.chunks - 1 - it, st = it & 1, k = it >> 1;
      const int64_t base0 = ((int64_t)fb * p.heads + h0) * p.seq_len + c * L;
      const float f0 = ex2(p.cum[base0 + l] * LOG2E);
      const float f1 = PH ? 0.f : ex2(p.cum[base0 + p.seq_len + l] * LOG2E);
      const float decay = ex2(p.cum[((int64_t)fb * p.heads + h) * p.seq_len + c * L + L - 1] * LOG2E);
      ok = mbar_wait(&s.bar_full[st], k & 1, abortp, p.status, 57);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      scale_row(smem_u32(s.xs[st][0]), l, f0);
      if (!PH) scale_row(smem_u32(s.xs[st][PH ? 0 : 1]), l, f1);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.bar_scaled[st]);
      // the state that leaves chunk c, written while the product runs
      {
        __nv_bfloat16* dst = p.d_out + (((int64_t)b * p.chunks + c) * p.heads + h) * ELEMS + row_off;
#pragma unroll
        for (int e = 0; e < ROW / 8; ++e) {
          uint4 o;
          o.x = pack2(stv[8 * e], stv[8 * e + 1]);
          o.y = pack2(stv[8 * e + 2], stv[8 * e + 3]);
          o.z = pack2(stv[8 * e + 4], stv[8 * e + 5]);
          o.w = pack2(stv[8 * e + 6], stv[8 * e + 7]);
          reinterpret_cast<uint4*>(dst)[e] = o;
        }
      }
      ok = mbar_wait(&s.bar_done[st], k & 1, abortp, p.status, 58);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      fence_after_sync();
#pragma unroll
      for (int q = 0; q < ROW / 32; ++q) {
        uint32_t r[32];
        tmem_ld_32x32(tmem + ((uint32_t)(warp * 32) << 16) + st * COLS + q * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) stv[q * 32 + e] = fmaf(stv[q * 32 + e], decay, __uint_as_float(r[e]));
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.bar_free[st]);
    }
    if (ok && p.d_init) {
      float4* dst = reinterpret_cast<float4*>(p.d_init + bh * ELEMS + row_off);
#pragma unroll
      for (int e = 0; e < ROW / 4; ++e) dst[e] = make_float4(stv[4 * e], stv[4 * e + 1], stv[4 * e + 2], stv[4 * e + 3]);
    }
  }
  __syncwarp();
  if (s.abort_flag) {
    const unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    fence_after_sync();
    tmem_dealloc(tmem, 2 * COLS);
  }
}

// ------------------------------------------------------------------------------------------------ 6. backward glue
// dx = dt * dX + D * gy,  ddt = da * A + dX . x,  dD[h] += sum gy . x        with dX read in reversed time order.
// One warp per (batch, token, head) row of 64; dD through one atomic per warp.
template <typename T>
__device__ __forceinline__ float2 ld2(const T* p);
template <>
__device__ __forceinline__ float2 ld2<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
template <>
__device__ __forceinline__ float2 ld2<float>(const float* p) {
  return *reinterpret_cast<const float2*>(p);
}
template <typename T>
__device__ __forceinline__ void st2(T* p, float a, float b);
template <>
__device__ __forceinline__ void st2<__nv_bfloat16>(__nv_bfloat16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}
template <>
__device__ __forceinline__ void st2<float>(float* p, float a, float b) {
  *reinterpret_cast<float2*>(p) = make_float2(a, b);
}

// G: dtype of dx_rev (fp32 from the role-permuted scans, bf16 from the fused chunk backward)
template <typename T, typename G>
__global__ void __launch_bounds__(256) bwd_finish_kernel(const G* __restrict__ dx_rev, const T* __restrict__ x,
                                                         const T* __restrict__ gy, const float* __restrict__ dt,
                                                         const float* __restrict__ da, const float* __restrict__ a_param,
                                                         const float* __restrict__ d_skip, T* __restrict__ dx,
                                                         float* __restrict__ ddt, float* __restrict__ dd, int64_t tokens,
                                                         int seq_len, int seq_pad, int heads, int reversed, int64_t ftokens) {
  // grid (ceil(tokens / 128), heads): a block owns one head and 128 tokens (16 per warp), so that the dD sum leaves as one
  // atomic per block.  dx_rev is [batch, seq_pad, heads, 64] (in reversed time when `reversed`); dt [b, l, h]; da [b, h, seq_pad].
  // x and dt hold `ftokens` tokens and are shared by the tokens / ftokens stacked directions of gy.
  __shared__ float warp_dd[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int h = blockIdx.y;
  const float a_h = a_param[h], dsk = d_skip ? d_skip[h] : 0.f;
  float dd_acc = 0.f;
  for (int i = 0; i < 16; ++i) {
    const int64_t bl = (int64_t)blockIdx.x * 128 + warp * 16 + i;
    if (bl >= tokens) break;
    const int l = (int)(bl % seq_len);
    const int64_t b = bl / seq_len;
    const int64_t row = bl * heads + h;
    const int64_t frow = (bl % ftokens) * heads + h;
    const int64_t rrow = (b * seq_pad + (reversed ? seq_pad - 1 - l : l)) * heads + h;
    const float2 g = ld2<G>(dx_rev + rrow * P + lane * 2);
    const float2 xv = ld2<T>(x + frow * P + lane * 2);
    const float2 gv = ld2<T>(gy + row * P + lane * 2);
    const float dtv = dt[frow];
    st2<T>(dx + row * P + lane * 2, dtv * g.x + dsk * gv.x, dtv * g.y + dsk * gv.y);
    const float dot = warp_sum(g.x * xv.x + g.y * xv.y);
    dd_acc += gv.x * xv.x + gv.y * xv.y;
    if (lane == 0) ddt[row] = da[(b * heads + h) * seq_pad + l] * a_h + dot;
  }
  if (dd) {
    dd_acc = warp_sum(dd_acc);
    if (lane == 0) warp_dd[warp] = dd_acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) t += warp_dd[w];
      atomicAdd(dd + h, t);
    }
  }
}

// out[b, l, g, n] = sum over the heads of group g of w[b, l, h] * y[b, l', h, n]   (l' = seq_pad - 1 - l when reversed; w = 1
// when null); y is [batch, seq_pad, heads, width] bf16 with the first n of every `width` columns used.
template <typename T>
__global__ void __launch_bounds__(256) group_sum_kernel(const __nv_bfloat16* __restrict__ y, const float* __restrict__ w,
                                                        T* __restrict__ out, int64_t total, int seq_len, int seq_pad, int heads,
                                                        int groups, int n, int width, int reversed) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // one thread per two outputs
  if (idx >= total) return;
  const int half_n = n / 2;
  const int c2 = (int)(idx % half_n);
  const int g = (int)((idx / half_n) % groups);
  const int64_t bl = idx / ((int64_t)half_n * groups);
  const int l = (int)(bl % seq_len);
  const int64_t b = bl / seq_len;
  const int rep = heads / groups;
  const int64_t src_tok = b * seq_pad + (reversed ? seq_pad - 1 - l : l);
  float a0 = 0.f, a1 = 0.f;
  for (int r = 0; r < rep; ++r) {
    const int h = g * rep + r;
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(y + (src_tok * heads + h) * width + c2 * 2));
    const float ww = w ? w[(b * seq_len + l) * heads + h] : 1.f;
    a0 = fmaf(ww, v.x, a0);
    a1 = fmaf(ww, v.y, a1);
  }
  st2<T>(out + ((b * seq_len + l) * groups + g) * n + c2 * 2, a0, a1);
}

// ------------------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) == cudaSuccess &&
        res == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// [rows, width] bf16 row-major, boxes of box_rows x 64 columns, 128-byte swizzle
// ld: row stride in elements (0: the rows are contiguous, ld = width)
static int make_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t width, int box_rows, int64_t ld = 0) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return 801;
  cuuint64_t dims[2] = {(cuuint64_t)width, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(ld > 0 ? ld : width) * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? 0 : 1000 + (int)rc;
}

template <typename K>
static int set_smem(K kernel, size_t bytes) {
  return (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

template <int N, bool PH>
static int run(const void* x, const void* bm, const void* cm, const float* dt, const float* cum, const float* d_skip,
               const float* skip_tok, int strict, const float* init_state, float* states, void* prev, float* final_state,
               void* y, float* y32, int batch, int seq_len, int heads, int groups, int* status, cudaStream_t st, int v_div = 1,
               int v_mod = 1) {
  const int chunks = seq_len / L;
  const int64_t rows = (int64_t)batch * seq_len;
  CUtensorMap mx, mb, mc, mp;
  const int v_blocks = ((heads - 1) / v_div) * v_mod + v_mod;   // 64-column blocks of the v matrix
  int rc = make_map(&mx, x, rows, (int64_t)v_blocks * P, L);
  if (rc) return rc;
  rc = make_map(&mb, bm, rows, (int64_t)(PH ? heads : groups) * N, L);
  if (rc) return rc;
  rc = make_map(&mc, cm, rows, (int64_t)(PH ? heads : groups) * N, L);
  if (rc) return rc;
  rc = PH ? make_map(&mp, prev, (int64_t)batch * chunks * heads * N, P, N)
          : make_map(&mp, prev, (int64_t)batch * chunks * heads * P, N, P);
  if (rc) return rc;
  {
    StateParams p{seq_len, heads, groups, chunks, v_div, v_mod, dt, cum, states, status, 0, batch};
    const size_t smem = sizeof(SmemState<N>) + 1024;
    rc = set_smem(chunk_state_kernel<N, PH>, smem);
    if (rc) return rc;
    chunk_state_kernel<N, PH><<<dim3(chunks, PH ? heads : heads / 2, batch), THREADS, smem, st>>>(mx, mb, p);
    rc = (int)cudaGetLastError();
    if (rc) return rc;
  }
  {
    const int elems = P * N;
    const int64_t total = (int64_t)batch * heads * elems;
    state_passing_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(states, cum, init_state, (__nv_bfloat16*)prev,
                                                                         final_state, batch, heads, chunks, seq_len, elems);
    rc = (int)cudaGetLastError();
    if (rc) return rc;
  }
  {
    ScanParams p{seq_len, heads, groups, chunks, v_div, v_mod, dt, cum, d_skip, skip_tok, strict, (__nv_bfloat16*)y, y32, status};
    const size_t smem = sizeof(SmemScan<N>) + 1024;
    rc = set_smem(chunk_scan_kernel<N, PH>, smem);
    if (rc) return rc;
    chunk_scan_kernel<N, PH><<<dim3(chunks, heads, batch), THREADS, smem, st>>>(mx, mb, mc, mp, p);
    rc = (int)cudaGetLastError();
  }
  return rc;
}

template <int N, bool PH>
static int run_dda(const void* x, const void* gy, const void* bm, const void* cm, const float* weight, const float* cum,
                   const void* hin, const void* dho, float* da, int batch, int seq_len, int heads, int groups, int* status,
                   cudaStream_t st) {
  const int chunks = seq_len / L;
  const int64_t rows = (int64_t)batch * seq_len;
  CUtensorMap mx, mg, mb, mc, mh, md;
  int rc = make_map(&mx, x, rows, (int64_t)heads * P, L);
  if (rc) return rc;
  rc = make_map(&mg, gy, rows, (int64_t)heads * P, L);
  if (rc) return rc;
  rc = make_map(&mb, bm, rows, (int64_t)(PH ? heads : groups) * N, L);
  if (rc) return rc;
  rc = make_map(&mc, cm, rows, (int64_t)(PH ? heads : groups) * N, L);
  if (rc) return rc;
  rc = PH ? make_map(&mh, hin, (int64_t)batch * chunks * heads * N, P, N) : make_map(&mh, hin, (int64_t)batch * chunks * heads * P, N, P);
  if (rc) return rc;
  rc = PH ? make_map(&md, dho, (int64_t)batch * chunks * heads * N, P, N) : make_map(&md, dho, (int64_t)batch * chunks * heads * P, N, P);
  if (rc) return rc;
  DdaParams p{seq_len, heads, groups, chunks, weight, cum, da, status};
  const size_t smem = sizeof(SmemDda<N>) + 1024;
  rc = set_smem(dda_kernel<N, PH>, smem);
  if (rc) return rc;
  dda_kernel<N, PH><<<dim3(chunks, heads, batch), THREADS, smem, st>>>(mx, mg, mb, mc, mh, md, p);
  return (int)cudaGetLastError();
}


template <int N, bool PH>
static int run_bwd(const void* v, const void* gy, const void* bk, const void* cq, const float* weight, const float* cum,
                   const float* skip_tok, const float* d_skip, const void* state_in, const float* d_final, float* chunk_cot,
                   void* d_out, float* d_init, float* da, float* dskip, float* dv32, void* dv16, float* dcq32, float* dbk32,
                   void* dcq16, void* dbk16, int batch, int bmod, int seq_len, int heads, int groups, int strict, int* status,
                   cudaStream_t st, int64_t dv_ld = 0) {
  const int chunks = seq_len / L;
  const int64_t rows = (int64_t)batch * seq_len, frows = (int64_t)bmod * seq_len;
  CUtensorMap mx, mg, mb, mc, mh, md, mdv, mdq, mdk;
  int rc = make_map(&mx, v, frows, (int64_t)heads * P, L);
  if (rc) return rc;
  rc = make_map(&mg, gy, rows, (int64_t)heads * P, L);
  if (rc) return rc;
  rc = make_map(&mb, bk, frows, (int64_t)(PH ? heads : groups) * N, L);
  if (rc) return rc;
  rc = make_map(&mc, cq, frows, (int64_t)(PH ? heads : groups) * N, L);
  if (rc) return rc;
  rc = PH ? make_map(&mh, state_in, (int64_t)bmod * chunks * heads * N, P, N)
          : make_map(&mh, state_in, (int64_t)bmod * chunks * heads * P, N, P);
  if (rc) return rc;
  rc = PH ? make_map(&md, d_out, (int64_t)batch * chunks * heads * N, P, N) : make_map(&md, d_out, (int64_t)batch * chunks * heads * P, N, P);
  if (rc) return rc;
  {   // cotangents of the chunk-boundary states: chunk products and the reversed passing in one kernel
    (void)chunk_cot;
    RevParams rp{seq_len, heads, groups, chunks, bmod, cum, d_final, (__nv_bfloat16*)d_out, d_init, status};
    const size_t smem = sizeof(SmemRev<N, PH>) + 1024;
    rc = set_smem(rev_state_kernel<N, PH>, smem);
    if (rc) return rc;
    rev_state_kernel<N, PH><<<dim3(PH ? heads : heads / 2, batch), THREADS, smem, st>>>(mg, mc, rp);
    rc = (int)cudaGetLastError();
    if (rc) return rc;
  }
  // bf16 results leave through TMA stores; a map of an fp32 result is never used and points at gy
  rc = make_map(&mdv, dv16 ? dv16 : gy, rows, (int64_t)heads * P, L, dv16 ? dv_ld : 0);
  if (rc) return rc;
  rc = make_map(&mdq, dcq16 ? dcq16 : gy, rows, (int64_t)heads * (dcq16 ? N : P), L);
  if (rc) return rc;
  rc = make_map(&mdk, dbk16 ? dbk16 : gy, rows, (int64_t)heads * (dbk16 ? N : P), L);
  if (rc) return rc;
  BwdParams p{seq_len, heads, groups, chunks, bmod, strict, weight, cum, skip_tok, d_skip, da, dskip, dv32, (__nv_bfloat16*)dv16,
              dcq32, dbk32, (__nv_bfloat16*)dcq16, (__nv_bfloat16*)dbk16, status};
  const size_t smem = sizeof(SmemBwd<N>) + 1024;
  rc = set_smem(bwd_chunk_kernel<N, PH>, smem);
  if (rc) return rc;
  bwd_chunk_kernel<N, PH><<<dim3(chunks, heads, batch), BWD_THREADS, smem, st>>>(mx, mg, mb, mc, mh, md, mdv, mdq, mdk, p);
  return (int)cudaGetLastError();
}

}  // namespace ssd
}  // namespace lbi

extern "C" int lbi_ssd_chunk_bwd(const void* v, const void* gy, const void* bk, const void* cq, const float* weight,
                                 const float* cum, const float* skip_tok, const float* d_skip, const void* state_in,
                                 const float* d_final, float* chunk_cot, void* d_out, float* d_init, float* da, float* dskip,
                                 float* dv32, void* dv16, float* dcq32, float* dbk32, void* dcq16, void* dbk16, int batch, int bmod,
                                 int seq_len, int heads, int groups, int d_state, int per_head, int strict, int64_t dv_ld,
                                 int* status, cudaStream_t st) {
  using namespace lbi::ssd;
  if (seq_len % L != 0 || batch <= 0 || bmod <= 0 || batch % bmod != 0) return (int)cudaErrorInvalidValue;
  if (dv_ld != 0 && (!dv16 || dv_ld % 8 != 0 || dv_ld < (int64_t)heads * P)) return (int)cudaErrorInvalidValue;
  if (!!dv32 == !!dv16 || !!dcq32 == !!dcq16 || !!dbk32 == !!dbk16) return (int)cudaErrorInvalidValue;
  if (per_head) {
    if (d_state != 128) return (int)cudaErrorInvalidValue;
    return run_bwd<128, true>(v, gy, bk, cq, weight, cum, skip_tok, d_skip, state_in, d_final, chunk_cot, d_out, d_init, da, dskip,
                              dv32, dv16, dcq32, dbk32, dcq16, dbk16, batch, bmod, seq_len, heads, groups, strict, status, st, dv_ld);
  }
  if (groups <= 0 || heads % groups != 0 || (heads / groups) % 2 != 0) return (int)cudaErrorInvalidValue;
  if (d_state == 128)
    return run_bwd<128, false>(v, gy, bk, cq, weight, cum, skip_tok, d_skip, state_in, d_final, chunk_cot, d_out, d_init, da, dskip,
                               dv32, dv16, dcq32, dbk32, dcq16, dbk16, batch, bmod, seq_len, heads, groups, strict, status, st, dv_ld);
  if (d_state == 64)
    return run_bwd<64, false>(v, gy, bk, cq, weight, cum, skip_tok, d_skip, state_in, d_final, chunk_cot, d_out, d_init, da, dskip,
                              dv32, dv16, dcq32, dbk32, dcq16, dbk16, batch, bmod, seq_len, heads, groups, strict, status, st, dv_ld);
  return (int)cudaErrorInvalidValue;
}

namespace lbi {
namespace ssd {
}  // namespace ssd
}  // namespace lbi

extern "C" int lbi_ssd_cumsum(const float* dt_raw, const float* dt_bias, const float* a, float* dt_out, float* cum, int batch,
                              int seq_len, int heads, int softplus, float dt_min, float dt_max, cudaStream_t st) {
  using namespace lbi::ssd;
  if (seq_len % L != 0 || batch <= 0 || heads <= 0) return (int)cudaErrorInvalidValue;
  cumsum_kernel<<<dim3(seq_len / L, heads, batch), 128, 0, st>>>(dt_raw, dt_bias, a, dt_out, cum, seq_len, heads, softplus,
                                                                 dt_min, dt_max);
  return (int)cudaGetLastError();
}

extern "C" int lbi_ssd_chunk_scan_fwd(const void* x, const void* bm, const void* cm, const float* dt, const float* cum,
                                      const float* d_skip, const float* init_state, float* states, void* prev,
                                      float* final_state, void* y, int batch, int seq_len, int heads, int groups, int head_dim,
                                      int d_state, int* status, cudaStream_t st) {
  using namespace lbi::ssd;
  if (head_dim != P || seq_len % L != 0 || batch <= 0 || heads <= 0 || groups <= 0 || heads % groups != 0 ||
      (heads / groups) % 2 != 0 || (int64_t)batch * seq_len >= (1ll << 31))
    return (int)cudaErrorInvalidValue;
  if (d_state == 64)
    return run<64, false>(x, bm, cm, dt, cum, d_skip, nullptr, 0, init_state, states, prev, final_state, y, nullptr, batch, seq_len,
                          heads, groups, status, st);
  if (d_state == 128)
    return run<128, false>(x, bm, cm, dt, cum, d_skip, nullptr, 0, init_state, states, prev, final_state, y, nullptr, batch, seq_len,
                           heads, groups, status, st);
  return (int)cudaErrorInvalidValue;
}

extern "C" int lbi_siso_chunk_scan_fwd(const void* v, const void* kr, const void* qr, const float* cum, const float* d_skip,
                                       const float* skip_tok, const float* init_state, float* states, void* prev,
                                       float* final_state, void* y, int batch, int seq_len, int heads, int head_dim,
                                       int d_state, int* status, cudaStream_t st) {
  using namespace lbi::ssd;
  if (head_dim != P || d_state != 128 || seq_len % L != 0 || batch <= 0 || heads <= 0 || (int64_t)batch * seq_len >= (1ll << 31))
    return (int)cudaErrorInvalidValue;
  return run<128, true>(v, kr, qr, nullptr, cum, d_skip, skip_tok, 1, init_state, states, prev, final_state, y, nullptr, batch, seq_len,
                        heads, heads, status, st);
}

extern "C" int lbi_ssd_scan_generic(const void* v, const void* bk, const void* cq, const float* weight, const float* cum,
                                    const float* d_skip, const float* skip_tok, int strict, const float* init_state,
                                    float* states, void* prev, float* final_state, void* y, float* y32, int batch, int seq_len,
                                    int heads, int groups, int d_state, int per_head, int v_div, int v_mod, int* status,
                                    cudaStream_t st) {
  using namespace lbi::ssd;
  if (seq_len % L != 0 || batch <= 0 || heads <= 0 || (int64_t)batch * seq_len >= (1ll << 31) || v_div <= 0 || v_mod <= 0)
    return (int)cudaErrorInvalidValue;
  if (per_head) {
    if (d_state != 128) return (int)cudaErrorInvalidValue;
    return run<128, true>(v, bk, cq, weight, cum, d_skip, skip_tok, strict, init_state, states, prev, final_state, y, y32, batch,
                          seq_len, heads, heads, status, st, v_div, v_mod);
  }
  if (groups <= 0 || heads % groups != 0 || (heads / groups) % 2 != 0) return (int)cudaErrorInvalidValue;
  if (d_state == 64)
    return run<64, false>(v, bk, cq, weight, cum, d_skip, skip_tok, strict, init_state, states, prev, final_state, y, y32, batch,
                          seq_len, heads, groups, status, st, v_div, v_mod);
  if (d_state == 128)
    return run<128, false>(v, bk, cq, weight, cum, d_skip, skip_tok, strict, init_state, states, prev, final_state, y, y32, batch,
                           seq_len, heads, groups, status, st, v_div, v_mod);
  return (int)cudaErrorInvalidValue;
}

extern "C" int lbi_ssd_decay_grad(const void* v, const void* gy, const void* bk, const void* cq, const float* weight,
                                  const float* cum, const void* state_in, const void* state_cot_rev, float* da, int batch,
                                  int seq_len, int heads, int groups, int d_state, int per_head, int* status, cudaStream_t st) {
  using namespace lbi::ssd;
  if (seq_len % L != 0 || batch <= 0 || heads <= 0 || (int64_t)batch * seq_len >= (1ll << 31)) return (int)cudaErrorInvalidValue;
  if (per_head) {
    if (d_state != 128) return (int)cudaErrorInvalidValue;
    return run_dda<128, true>(v, gy, bk, cq, weight, cum, state_in, state_cot_rev, da, batch, seq_len, heads, heads, status, st);
  }
  if (groups <= 0 || heads % groups != 0) return (int)cudaErrorInvalidValue;
  if (d_state == 64)
    return run_dda<64, false>(v, gy, bk, cq, weight, cum, state_in, state_cot_rev, da, batch, seq_len, heads, groups, status, st);
  if (d_state == 128)
    return run_dda<128, false>(v, gy, bk, cq, weight, cum, state_in, state_cot_rev, da, batch, seq_len, heads, groups, status, st);
  return (int)cudaErrorInvalidValue;
}

extern "C" int lbi_ssd_bwd_finish(const void* dx_rev, int dx_is_bf16, const void* x, const void* gy, const float* dt, const float* da,
                                  const float* a_param, const float* d_skip, void* dx, float* ddt, float* dd, int batch,
                                  int seq_len, int seq_pad, int heads, int is_bf16, int reversed, int fbatch, cudaStream_t st) {
  using namespace lbi::ssd;
  if (batch <= 0 || seq_len <= 0 || seq_pad < seq_len || heads <= 0 || fbatch <= 0 || batch % fbatch != 0) return (int)cudaErrorInvalidValue;
  const int64_t tokens = (int64_t)batch * seq_len, ftokens = (int64_t)fbatch * seq_len;
  const dim3 blocks((unsigned)((tokens + 127) / 128), (unsigned)heads);
#define LBI_FINISH(T, G)                                                                                                       \
  bwd_finish_kernel<T, G><<<blocks, 256, 0, st>>>((const G*)dx_rev, (const T*)x, (const T*)gy, dt, da, a_param, d_skip, (T*)dx, ddt, \
                                                  dd, tokens, seq_len, seq_pad, heads, reversed, ftokens)
  if (is_bf16 && dx_is_bf16) LBI_FINISH(__nv_bfloat16, __nv_bfloat16);
  else if (is_bf16) LBI_FINISH(__nv_bfloat16, float);
  else if (dx_is_bf16) LBI_FINISH(float, __nv_bfloat16);
  else LBI_FINISH(float, float);
#undef LBI_FINISH
  return (int)cudaGetLastError();
}

extern "C" int lbi_ssd_group_sum(const void* y_bf16, const float* w, void* out, int batch, int seq_len, int seq_pad, int heads,
                                 int groups, int n, int width, int reversed, int out_is_bf16, cudaStream_t st) {
  using namespace lbi::ssd;
  if (batch <= 0 || seq_len <= 0 || seq_pad < seq_len || heads <= 0 || groups <= 0 || heads % groups != 0 || n <= 0 || n % 2 != 0 ||
      width < n)
    return (int)cudaErrorInvalidValue;
  const int64_t total = (int64_t)batch * seq_len * groups * (n / 2);
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (out_is_bf16)
    group_sum_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)y_bf16, w, (__nv_bfloat16*)out, total, seq_len, seq_pad,
                                                           heads, groups, n, width, reversed);
  else
    group_sum_kernel<float><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)y_bf16, w, (float*)out, total, seq_len, seq_pad, heads, groups,
                                                   n, width, reversed);
  return (int)cudaGetLastError();
}
