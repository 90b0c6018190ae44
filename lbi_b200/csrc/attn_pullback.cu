// Causal-attention input pullback over a block of output-cotangent directions, on tcgen05 / TMEM / TMA.
//
// For q, k, v [T, Dh] of one (batch, head), P = softmax(mask(q k^T s)) and directions dO_p:
//     dV_p = P^T dO_p,   dP_p = dO_p v^T,   dS_p = P o (dP_p - delta_p),   dQ_p = s dS_p k,   dK_p = s dS_p^T q
// with delta_p = rowsum(dO_p o O).  Two kernels, both built from the same template:
//
//   DKDV = true   one CTA owns a 128-row key tile j and PB = 2 directions; it walks the query tiles i >= j.
//                 Per (i, j): S = Q_i K_j^T and P are computed ONCE and P is parked in shared memory; then for every
//                 direction: dP, dS, dV_p += P^T dO_p, dK_p += dS^T Q_i.  dK_p / dV_p accumulate in TMEM over all i.
//   DKDV = false  one CTA owns a 128-row query tile i and PB = 4 directions; it walks the key tiles j <= i:
//                 S and P once per (i, j), then per direction dP, dS, dQ_p += dS K_j.  dQ_p accumulates in TMEM.
//
// The reference recomputes S and P for every direction: its "pblock4" entry is a host loop over a P = 1 WMMA kernel
// (cuda/transformer/attention_pullback_mma.cu:479-515), fp16 only, T <= 1024.
//
// Layout: all tensors are token-major and packed, rows = (p * B + b) * T + t:
//   qkv [n, 3 * H * Dh] bf16 (q | k | v sections), dO [P * n, H * Dh] bf16, d_qkv [P * n, 3 * H * Dh] bf16 (output),
//   lse [B, H, T] fp32 (natural log), delta [P, B, H, T] fp32.
// Every tile is 128 rows x 64 columns of bf16 = 128-byte rows, loaded by TMA with 128-byte swizzle; such a tile can be
// fed to the tensor core both as a K-major operand (rows = M/N index) and as an MN-major operand (rows = K index), so
// Q, K, V and dO are each loaded once per use and never transposed.  P and dS are written by the compute warps into
// shared memory in the same swizzled layout ([128 q rows] x two 64-wide key panels).
//
// Pipeline.  The S and dP products of one CTA form a sequence of "jobs" (per step: S, dP_0, .., dP_{np-1}).  Job n
// writes TMEM buffer n & 1 (columns [0,128) and [128,256)); the accumulators follow from column 256, 64 columns each.
// The control thread issues job n as soon as the compute warps have consumed job n - 2, and issues the accumulating
// MMAs of job n - 2 (which need the dS tile the compute warps wrote) at the same moment, so the tensor core always has
// the next product queued while the compute warps turn the previous one into P or dS.  dS tiles are double-buffered
// in shared memory; P stays in registers (and, for DKDV, in shared memory as an MMA operand).
// Warp roles (608 threads): warps 0-15 compute (TMEM lane quarter = warp % 4, 32-column slice = warp / 4); warp 16
// lane 0 issues the S / dP products; warp 17 lane 0 issues the accumulating products and releases shared-memory
// stages; warp 18 lane 0 is the TMA producer.  A job is only four (S, dP) or eight (accumulate) tcgen05.mma, about 256
// tensor-core cycles, so the issuing threads' own instruction streams set the pace: they carry no integer division,
// no polling and no TMA issue (phase timing showed one thread doing all three spent half its time in them).  Two issuing threads because a single thread's instruction stream (descriptor
// arithmetic + about twenty tcgen05.mma per job) was measured to be the bottleneck.  Every mbarrier wait is bounded
// (tcgen05.cuh); all barrier parities are derived from job / tile counters.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "api_attn.h"
#include "common.cuh"
#include "tcgen05.cuh"

namespace lbi {
namespace attn {

using namespace tc;

constexpr int TILE = 128;       // query rows and key rows per tile
constexpr int DH = 64;          // head dimension handled by this build
constexpr int TILE_BYTES = TILE * DH * 2;   // 16 KB
constexpr int PANEL_BYTES = TILE * 128;     // one 64-column panel of P / dS: 128 rows x 128 B
constexpr int THREADS = 608;          // 16 compute warps + 2 MMA-issuing warps + 1 TMA warp
constexpr int NCOMPUTE_WARPS = 16;     // barrier arrivals are per warp: 512 same-address arrivals per job congested the
                                      // shared-memory pipe that the MMA issue also goes through
constexpr int PB_DKDV = 2;
constexpr int PB_DQ = 4;
constexpr int NDO = 4;          // dO stages in DKDV mode

struct Params {
  int batch, heads, seq_len, nbasis;
  int n_tiles;                  // seq_len / TILE
  int64_t n_rows;               // batch * seq_len
  int64_t out_ld;               // 3 * H * Dh
  float scale, scale_log2;      // softmax scale and scale * log2(e)
  const float* lse;             // [B, H, T]
  const float* delta;           // [P, B, H, T]
  __nv_bfloat16* d_qkv;         // [P * n, 3 H Dh]
  const float* rope_cos;        // [T, Dh / 2] fp32 or null: rotate dQ and dK back before they are stored
  const float* rope_sin;
  int rope_interleaved;
  int* status;
};

template <bool DKDV>
struct Smem {
  static constexpr int NFIXED = DKDV ? 2 : 1 + PB_DQ;   // DKDV: K_j, V_j ; DQ: Q_i, dO_0..3
  static constexpr int NSTREAM = DKDV ? 2 + NDO : 4;    // DKDV: Q_i x2, dO x NDO ; DQ: K_j x2, V_j x2
  alignas(1024) uint8_t fixed[NFIXED][TILE_BYTES];
  alignas(1024) uint8_t stream[NSTREAM][TILE_BYTES];
  alignas(1024) uint8_t ds_tile[2][2][PANEL_BYTES];      // [buffer][64-column panel]
  alignas(1024) uint8_t p_tile[DKDV ? 2 : 1][DKDV ? PANEL_BYTES : 1024];
  uint64_t bar_fixed;
  uint64_t bar_stream_full[NSTREAM];
  uint64_t bar_stream_empty[NSTREAM];
  uint64_t bar_ready[2];          // job result in TMEM buffer (commit)
  uint64_t bar_consumed[2];       // compute warps are done with the TMEM buffer: one arrival per warp (read by the S/dP issuer)
  uint64_t bar_written[4];        // same event for the accumulate issuer (P / dS are in shared memory), 4 slots deep
  uint64_t bar_ds_free[2];        // the MMA that read this dS buffer has finished (commit)
  uint64_t bar_p_free;            // the MMAs that read P have finished (commit)
  uint64_t bar_acc_done;          // all accumulating MMAs finished (commit)
  uint32_t tmem_base;
  volatile int abort_flag;
};

// 16-byte chunk address of row r, chunk c (8 bf16) inside a 128-byte-swizzled panel of 128-byte rows.
__device__ __forceinline__ uint32_t swz(uint32_t panel_base, int r, int c) {
  return panel_base + r * 128 + ((c ^ (r & 7)) << 4);
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
// F16 = false: bf16 operands and results; true: fp16 (the reference kernel's only dtype).  Accumulation is fp32 either way.
template <bool F16>
__device__ __forceinline__ uint32_t pack_lp(float a, float b) {
  uint32_t d;
  if (F16) asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(b), "f"(a));
  else asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(b), "f"(a));
  return d;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ float2 unpack_bf16(uint32_t v) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v));
}
// Packed pairs: two fp32 in one 64-bit register (add / sub / fma .f32x2) and two bf16 in one 32-bit register.  The
// compute warps are bound by instruction issue, so the per-element instruction count is what matters here.
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ uint64_t pack_u32x2(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ float2 unpack_f32x2(uint64_t v) {
  float2 r;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(v));
  return r;
}
__device__ __forceinline__ uint64_t sub_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("sub.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
template <bool F16>
__device__ __forceinline__ uint32_t cvt_lp_x2(uint64_t v) {   // {lo, hi} fp32 -> 16-bit pair, lo in the low half
  uint32_t d;
  if (F16) asm("{\n.reg .f32 lo, hi;\nmov.b64 {lo, hi}, %1;\ncvt.rn.f16x2.f32 %0, hi, lo;\n}" : "=r"(d) : "l"(v));
  else asm("{\n.reg .f32 lo, hi;\nmov.b64 {lo, hi}, %1;\ncvt.rn.bf16x2.f32 %0, hi, lo;\n}" : "=r"(d) : "l"(v));
  return d;
}
template <bool F16>
__device__ __forceinline__ uint32_t mul_lp_x2(uint32_t a, uint32_t b) {
  uint32_t d;
  if (F16) asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  else asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// kind::f16 instruction descriptor with fp32 D and bf16 or fp16 A / B
__host__ __device__ constexpr uint32_t make_idesc_lp(int m, int n, int a_mn_major, int b_mn_major, bool f16) {
  return f16 ? (make_idesc_bf16(m, n, a_mn_major, b_mn_major) & ~((1u << 7) | (1u << 10))) : make_idesc_bf16(m, n, a_mn_major, b_mn_major);
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <bool DKDV, bool F16>
__global__ void __launch_bounds__(THREADS, 1)
pullback_kernel(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_do,
                const __grid_constant__ CUtensorMap map_out, const Params p) {
  constexpr int PB = DKDV ? PB_DKDV : PB_DQ;
  constexpr int NSTREAM = Smem<DKDV>::NSTREAM;
  extern __shared__ uint8_t raw_smem[];
  Smem<DKDV>& s = *reinterpret_cast<Smem<DKDV>*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // tile ownership: heavy tiles first (DKDV: small j walks more query tiles; DQ: large i walks more key tiles)
  const int own = DKDV ? (int)blockIdx.x : p.n_tiles - 1 - (int)blockIdx.x;
  const int bh = blockIdx.y;
  const int b = bh / p.heads, h = bh % p.heads;
  const int p0 = blockIdx.z * PB;
  const int np = min(PB, p.nbasis - p0);
  const int n_iter = DKDV ? p.n_tiles - own : own + 1;
  const int jobs_per_iter = np + 1;
  const int total_jobs = n_iter * jobs_per_iter;
  const int hd = p.heads * DH;
  const int col_q = h * DH, col_k = hd + h * DH, col_v = 2 * hd + h * DH;
  const int row_b = b * p.seq_len;  // first token row of this batch element (within one direction)
  // TMEM columns: job buffers [0,128) and [128,256); DKDV: dK_p at 256 + 64 p, dV_p at 384 + 64 p; DQ: dQ_p at 256 + 64 p
  constexpr int ACC0 = 256, ACC_DV = 384;

  if (threadIdx.x == 0) {
    s.abort_flag = 0;
    mbar_init(&s.bar_fixed, 1);
    for (int i = 0; i < NSTREAM; ++i) {
      mbar_init(&s.bar_stream_full[i], 1);
      mbar_init(&s.bar_stream_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.bar_ready[i], 1);
      mbar_init(&s.bar_consumed[i], NCOMPUTE_WARPS);
      mbar_init(&s.bar_ds_free[i], 1);
    }
    for (int i = 0; i < 4; ++i) mbar_init(&s.bar_written[i], NCOMPUTE_WARPS);
    mbar_init(&s.bar_p_free, 1);
    mbar_init(&s.bar_acc_done, 1);
    fence_barrier_init();
    prefetch_tmap(&map_qkv);
    prefetch_tmap(&map_do);
    prefetch_tmap(&map_out);
  }
  if (warp == 16) tmem_alloc(&s.tmem_base, 512);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = s.tmem_base;
  volatile int* abortp = &s.abort_flag;

  // Descriptors are a constant template plus (address >> 4); consecutive tiles are TILE_BYTES apart.
  const uint64_t kmajor0 = make_smem_desc(0, 16, 1024);            // rows = M/N index, 64 K-elements per 128-byte row
  const uint64_t mnmajor0 = make_smem_desc(0, PANEL_BYTES, 1024);  // rows = K index, 64-wide M/N panels PANEL_BYTES apart
  const uint32_t stream0 = smem_u32(s.stream[0]) >> 4, fixed0 = smem_u32(s.fixed[0]) >> 4;
  constexpr uint32_t TILE16 = TILE_BYTES >> 4;

  if (warp == 18) {
    // ======================================================================== TMA producer
    // Streams the tiles of up to two steps ahead.  All waits are blocking here: this thread has nothing else to do,
    // and everything a stage release depends on was loaded earlier in this same order, so the waits cannot cycle.
    if (lane == 0) {
      bool ok = true;
      auto load_tile = [&](void* dst, const CUtensorMap* m, uint64_t* bar, int col, int64_t row) {
        mbar_arrive_expect_tx(bar, TILE_BYTES);
        tma_load_2d(dst, m, bar, col, (int)row);
      };
      if (DKDV) {
        mbar_arrive_expect_tx(&s.bar_fixed, 2 * TILE_BYTES);
        tma_load_2d(s.fixed[0], &map_qkv, &s.bar_fixed, col_k, row_b + own * TILE);
        tma_load_2d(s.fixed[1], &map_qkv, &s.bar_fixed, col_v, row_b + own * TILE);
      } else {
        mbar_arrive_expect_tx(&s.bar_fixed, (1 + np) * TILE_BYTES);
        tma_load_2d(s.fixed[0], &map_qkv, &s.bar_fixed, col_q, row_b + own * TILE);
        for (int pp = 0; pp < np; ++pp)
          tma_load_2d(s.fixed[1 + pp], &map_do, &s.bar_fixed, h * DH,
                      (int)((int64_t)(p0 + pp) * p.n_rows + row_b + own * TILE));
      }
      // The shared-memory ring holds the tiles of two steps, less than the DRAM latency of a dO tile is worth in steps:
      // tiles are therefore requested into L2 PF steps ahead, so that the ring refills at L2 latency.
      constexpr int PF = 4;
      auto prefetch_step = [&](int it2) {
        if (it2 >= n_iter) return;
        if (DKDV) {
          tma_prefetch_l2_2d(&map_qkv, col_q, row_b + (own + it2) * TILE);
          for (int pp = 0; pp < np; ++pp)
            tma_prefetch_l2_2d(&map_do, h * DH, (int)((int64_t)(p0 + pp) * p.n_rows + row_b + (own + it2) * TILE));
        } else {
          tma_prefetch_l2_2d(&map_qkv, col_k, row_b + it2 * TILE);
          tma_prefetch_l2_2d(&map_qkv, col_v, row_b + it2 * TILE);
        }
      };
      for (int it2 = 2; it2 < 2 + PF; ++it2) prefetch_step(it2);
      int c = 0;  // running index of dO tiles (DKDV)
      for (int it = 0; it < n_iter && ok; ++it) {
        const int st = it & 1;
        prefetch_step(it + 2 + PF);
        if (it >= 2) {
          ok = mbar_wait(&s.bar_stream_empty[st], ((it >> 1) - 1) & 1, abortp, p.status, 11);
          if (!ok) break;
        }
        if (DKDV) {
          load_tile(s.stream[st], &map_qkv, &s.bar_stream_full[st], col_q, row_b + (own + it) * TILE);
          for (int pp = 0; pp < np && ok; ++pp, ++c) {
            const int ds = 2 + (c & (NDO - 1));
            if (c >= NDO) {
              ok = mbar_wait(&s.bar_stream_empty[ds], ((c / NDO) - 1) & 1, abortp, p.status, 12);
              if (!ok) break;
            }
            load_tile(s.stream[ds], &map_do, &s.bar_stream_full[ds], h * DH,
                      (int64_t)(p0 + pp) * p.n_rows + row_b + (own + it) * TILE);
          }
        } else {
          load_tile(s.stream[st], &map_qkv, &s.bar_stream_full[st], col_k, row_b + it * TILE);
          load_tile(s.stream[2 + st], &map_qkv, &s.bar_stream_full[2 + st], col_v, row_b + it * TILE);
        }
      }
    }
  } else if (warp == 16) {
    // ======================================================================== issuer X: S and dP products
    if (lane == 0) {
      const uint32_t idesc_nn = make_idesc_lp(128, 128, 0, 0, F16);
      bool ok = true;
      ok = mbar_wait(&s.bar_fixed, 0, abortp, p.status, 16);
      int it = 0, r = 0, c = 0;   // step, job within the step (0 = S, 1.. = dP of direction r - 1), dO tile index
      for (int n = 0; n < total_jobs && ok; ++n) {
        if (n >= 2) {
          ok = mbar_wait(&s.bar_consumed[n & 1], ((n - 2) >> 1) & 1, abortp, p.status, 17);
          if (!ok) break;
        }
        uint32_t a16, b16;  // operand tile addresses >> 4
        if (r == 0) {
          ok = mbar_wait(&s.bar_stream_full[it & 1], (it >> 1) & 1, abortp, p.status, 13);
          a16 = DKDV ? stream0 + (it & 1) * TILE16 : fixed0;
          b16 = DKDV ? fixed0 : stream0 + (it & 1) * TILE16;
        } else if (DKDV) {
          ok = mbar_wait(&s.bar_stream_full[2 + (c & (NDO - 1))], (c / NDO) & 1, abortp, p.status, 15);
          a16 = stream0 + (2 + (c & (NDO - 1))) * TILE16;
          b16 = fixed0 + TILE16;
          ++c;
        } else {
          if (r == 1) ok = mbar_wait(&s.bar_stream_full[2 + (it & 1)], (it >> 1) & 1, abortp, p.status, 14);
          a16 = fixed0 + r * TILE16;
          b16 = stream0 + (2 + (it & 1)) * TILE16;
        }
        if (!ok) break;
        fence_after_sync();
        const uint32_t d_tmem = tmem + (n & 1) * 128;
        const uint64_t da = kmajor0 + a16, db = kmajor0 + b16;
        _Pragma("unroll") for (int k = 0; k < 4; ++k) mma_bf16(d_tmem, da + 2 * k, db + 2 * k, idesc_nn, k);
        mma_commit(&s.bar_ready[n & 1]);
        if (++r == jobs_per_iter) {
          r = 0;
          ++it;
        }
      }
    }
  } else if (warp == 17) {
    // ======================================================================== issuer Y: accumulating products, releases
    if (lane == 0) {
      const uint32_t idesc_acc = DKDV ? make_idesc_lp(128, 64, 1, 1, F16) : make_idesc_lp(128, 64, 0, 1, F16);
      const uint32_t idesc_dv2 = make_idesc_lp(128, 128, 1, 1, F16);  // dV of two directions in one instruction
      const uint32_t ds0 = smem_u32(s.ds_tile[0][0]) >> 4, p16 = smem_u32(s.p_tile[0]) >> 4;
      constexpr uint32_t DSBUF16 = (2 * PANEL_BYTES) >> 4, PANEL16 = PANEL_BYTES >> 4;
      bool ok = true;
      int do_waited = 0;
      int it = 0, r = -1, c0 = 0;   // step, job within the step, index of the step's first dO tile
      for (int m = 0; m < total_jobs && ok; ++m) {
        if (++r == jobs_per_iter) {
          r = 0;
          ++it;
          c0 += np;
        }
        ok = mbar_wait(&s.bar_written[m & 3], (m >> 2) & 1, abortp, p.status, 18);
        if (!ok) break;
        fence_after_sync();
        const uint32_t first = it != 0;  // accumulate onto earlier steps?
        if (r == 0) {
          if (DKDV) {  // P_it is in shared memory: dV_p += P^T dO_p for the directions of this step
            while (ok && do_waited <= c0 + np - 1) {
              ok = mbar_wait(&s.bar_stream_full[2 + (do_waited & (NDO - 1))], (do_waited / NDO) & 1, abortp, p.status, 19);
              ++do_waited;
            }
            if (!ok) break;
            const uint64_t da = mnmajor0 + p16;
            const uint64_t db = mnmajor0 + stream0 + (2 + (c0 & (NDO - 1))) * TILE16;
            if (np == 2) {  // the two dO tiles are adjacent stages: one N = 128 operand with two 64-wide panels
              _Pragma("unroll") for (int k = 0; k < 8; ++k) mma_bf16(tmem + ACC_DV, da + 128 * k, db + 128 * k, idesc_dv2, first | (k != 0));
            } else {
              _Pragma("unroll") for (int k = 0; k < 8; ++k) mma_bf16(tmem + ACC_DV, da + 128 * k, db + 128 * k, idesc_acc, first | (k != 0));
            }
            mma_commit(&s.bar_p_free);
          }
          continue;
        }
        const int pp = r - 1, d = c0 + pp, buf = d & 1;
        const uint32_t acc = tmem + ACC0 + pp * 64;
        if (DKDV) {
          const uint64_t da = mnmajor0 + ds0 + buf * DSBUF16;
          const uint64_t db = mnmajor0 + stream0 + (it & 1) * TILE16;
          _Pragma("unroll") for (int k = 0; k < 8; ++k) mma_bf16(acc, da + 128 * k, db + 128 * k, idesc_acc, first | (k != 0));
          mma_commit(&s.bar_ds_free[buf]);
                mma_commit(&s.bar_stream_empty[2 + (d & (NDO - 1))]);  // dO tile d: its dV and this dK are behind the commit, dP was consumed
        } else {
          const uint64_t da = kmajor0 + ds0 + buf * DSBUF16;
          const uint64_t db = mnmajor0 + stream0 + (it & 1) * TILE16;
          _Pragma("unroll") for (int k = 0; k < 8; ++k)
            mma_bf16(acc, da + (k >> 2) * PANEL16 + (k & 3) * 2, db + 128 * k, idesc_acc, first | (k != 0));
          mma_commit(&s.bar_ds_free[buf]);
        }
        if (pp == np - 1) mma_commit(&s.bar_stream_empty[it & 1]);  // Q_it (DKDV) or K_it and V_it (DQ) may be overwritten
      }
      if (ok) mma_commit(&s.bar_acc_done);
    }
  } else {
    // ======================================================================== compute warps 0..15
    const int quarter = warp & 3, slice = warp >> 2, half = slice >> 1;   // slice: 32 key columns, half: 64-column panel
    const int r = quarter * 32 + lane;                       // row of the tile = TMEM lane
    const uint32_t t_lane = tmem + ((uint32_t)(quarter * 32) << 16) + slice * 32;
    const uint32_t p_panel = smem_u32(s.p_tile[DKDV ? half : 0]);
    const float* lse_bh = p.lse + ((int64_t)b * p.heads + h) * p.seq_len;
    constexpr float LOG2E = 1.4426950408889634f;
    uint32_t preg[16];                                        // this thread's 32 probabilities as bf16 pairs
    // Row statistics (log-sum-exp and the per-direction row dots) are fetched one step ahead: a load issued at the
    // point of use would expose a full DRAM round trip on every job.
    const float* delta_base = p.delta + (((int64_t)p0 * p.batch + b) * p.heads + h) * p.seq_len + r;
    const int64_t delta_dir = (int64_t)p.batch * p.heads * p.seq_len;   // stride between directions
    auto load_stats = [&](int q_tile, float& lse_out, float (&delta_out)[PB]) {
      lse_out = lse_bh[q_tile * TILE + r] * LOG2E;
#pragma unroll
      for (int i = 0; i < PB; ++i) delta_out[i] = i < np ? delta_base[i * delta_dir + q_tile * TILE] : 0.f;
    };
    float lse_r, delta_cur[PB], lse_next = 0.f, delta_next[PB];
    load_stats(own, lse_r, delta_cur);                       // DKDV: first query tile is `own`; DQ: the only one
#pragma unroll
    for (int i = 0; i < PB; ++i) delta_next[i] = 0.f;
    bool ok = true;
    int it = 0, rr = -1, d0 = 0;   // step, job within the step, index of the step's first dS tile
    for (int n = 0; n < total_jobs && ok; ++n) {
      if (++rr == jobs_per_iter) {
        rr = 0;
        ++it;
        d0 += np;
      }
      const int buf = n & 1;
      const int qi = DKDV ? own + it : own;   // query tile of this step
      const int kj = DKDV ? own : it;         // key tile of this step
      const uint32_t t_buf = t_lane + buf * 128;
      if (rr == 0) {
        if (DKDV) {
          if (it > 0) {
            lse_r = lse_next;
#pragma unroll
            for (int i = 0; i < PB; ++i) delta_cur[i] = delta_next[i];
          }
          if (it + 1 < n_iter) load_stats(qi + 1, lse_next, delta_next);
        }
        ok = mbar_wait(&s.bar_ready[buf], (n >> 1) & 1, abortp, p.status, 31);
        if (DKDV && it > 0 && ok) ok = mbar_wait(&s.bar_p_free, (it - 1) & 1, abortp, p.status, 32);
        ok = __all_sync(0xffffffffu, ok); fence_after_sync();
        if (!ok) break;
        const bool diagonal = (qi == kj);
        {
          uint32_t v[32];
          tmem_ld_32x32(t_buf, v); tmem_ld_wait();
          __syncwarp(); if (lane == 0) mbar_arrive(&s.bar_consumed[buf]);  // tcgen05.wait::ld above: the loads are complete  // TMEM buffer free
          const int col0 = slice * 32;
          const uint64_t sc2 = pack_f32x2(p.scale_log2, p.scale_log2), nl2 = pack_f32x2(-lse_r, -lse_r);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float2 t = unpack_f32x2(fma_f32x2(pack_u32x2(v[2 * i], v[2 * i + 1]), sc2, nl2));
            preg[i] = cvt_lp_x2<F16>(pack_f32x2(fast_exp2(t.x), fast_exp2(t.y)));
          }
          if (diagonal) {   // warp-uniform: only the tile on the diagonal pays for the causal mask
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int col = col0 + 2 * i;
              preg[i] &= (col <= r ? 0x0000ffffu : 0u) | (col + 1 <= r ? 0xffff0000u : 0u);
            }
          }
          if (DKDV) {
#pragma unroll
            for (int g = 0; g < 4; ++g)
              st_shared_v4(swz(p_panel, r, (slice & 1) * 4 + g),
                           make_uint4(preg[g * 4], preg[g * 4 + 1], preg[g * 4 + 2], preg[g * 4 + 3]));
          }
        }
        if (DKDV) fence_proxy_async(); __syncwarp(); if (lane == 0) mbar_arrive(&s.bar_written[n & 3]);
      } else {
        const int pp = rr - 1, d = d0 + pp, dbuf = d & 1;
        float delta_r = delta_cur[0];
#pragma unroll
        for (int i = 1; i < PB; ++i) delta_r = (pp == i) ? delta_cur[i] : delta_r;
        const uint32_t ds_panel = smem_u32(s.ds_tile[dbuf][half]);
        ok = mbar_wait(&s.bar_ready[buf], (n >> 1) & 1, abortp, p.status, 33);
        if (d >= 2 && ok) ok = mbar_wait(&s.bar_ds_free[dbuf], ((d >> 1) - 1) & 1, abortp, p.status, 34);
        ok = __all_sync(0xffffffffu, ok); fence_after_sync();
        if (!ok) break;
        {
          uint32_t v[32];
          tmem_ld_32x32(t_buf, v); tmem_ld_wait();
          __syncwarp(); if (lane == 0) mbar_arrive(&s.bar_consumed[buf]);  // tcgen05.wait::ld above: the loads are complete
          // dS = P o (dP - delta): the difference in fp32 (it cancels), the product of two bf16 values in bf16
          const uint64_t delta2 = pack_f32x2(delta_r, delta_r);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              w[e] = mul_lp_x2<F16>(preg[g * 4 + e],
                                    cvt_lp_x2<F16>(sub_f32x2(pack_u32x2(v[g * 8 + e * 2], v[g * 8 + e * 2 + 1]), delta2)));
            }
            st_shared_v4(swz(ds_panel, r, (slice & 1) * 4 + g), make_uint4(w[0], w[1], w[2], w[3]));
          }
        }
        fence_proxy_async(); __syncwarp(); if (lane == 0) mbar_arrive(&s.bar_written[n & 3]);
      }
    }
    // ------------------------------------------------------------------ epilogue: accumulators -> global
    if (ok) ok = mbar_wait(&s.bar_acc_done, 0, abortp, p.status, 35);
    // the four warps of a column slice share named barrier 1 + slice below: they take one decision (a raised abort flag wins)
    named_barrier_sync(1 + slice, 128);
    ok = (s.abort_flag == 0);
    if (ok) {
      // The (direction, accumulator) items (at most four) go one to each column slice; every thread turns one 64-element
      // head row into bf16, the slice stages its 128 x 64 tile in the (now idle) dS buffers and one TMA store writes it:
      // 16-byte stores from registers, 32 different lines per instruction, made this epilogue 12 % of the kernel.  With
      // rotary tables given, dQ and dK are rotated back here (the transpose of the forward rotation).
      fence_after_sync();
      const int pos = own * TILE + r;
      constexpr int n_acc = DKDV ? 2 : 1;
      const int items = np * n_acc;
      for (int item = slice; item < items; item += 4) {
        const int pp = item / n_acc, a = item % n_acc;
        // DKDV: a = 0 -> dK (scaled), a = 1 -> dV ; DQ: dQ (scaled)
        const uint32_t acc = tmem + (a == 0 ? ACC0 : ACC_DV) + pp * 64 + ((uint32_t)(quarter * 32) << 16);
        const int col = DKDV ? (a == 0 ? col_k : col_v) : col_q;
        const float mul = (DKDV && a == 1) ? 1.f : p.scale;
        const bool rotate = p.rope_cos != nullptr && !(DKDV && a == 1);
        uint32_t lo[32], hi[32];
        tmem_ld_32x32(acc, lo);
        tmem_ld_32x32(acc + 32, hi);
        tmem_ld_wait();
        const uint32_t stage = smem_u32(s.ds_tile[0][0]) + item * PANEL_BYTES;   // 4 panels of 128 rows x 128 bytes
        auto put = [&](int chunk, uint4 val) { st_shared_v4(swz(stage, r, chunk), val); };
        if (!rotate) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 o, o2;
            o.x = pack_lp<F16>(__uint_as_float(lo[g * 8 + 0]) * mul, __uint_as_float(lo[g * 8 + 1]) * mul);
            o.y = pack_lp<F16>(__uint_as_float(lo[g * 8 + 2]) * mul, __uint_as_float(lo[g * 8 + 3]) * mul);
            o.z = pack_lp<F16>(__uint_as_float(lo[g * 8 + 4]) * mul, __uint_as_float(lo[g * 8 + 5]) * mul);
            o.w = pack_lp<F16>(__uint_as_float(lo[g * 8 + 6]) * mul, __uint_as_float(lo[g * 8 + 7]) * mul);
            o2.x = pack_lp<F16>(__uint_as_float(hi[g * 8 + 0]) * mul, __uint_as_float(hi[g * 8 + 1]) * mul);
            o2.y = pack_lp<F16>(__uint_as_float(hi[g * 8 + 2]) * mul, __uint_as_float(hi[g * 8 + 3]) * mul);
            o2.z = pack_lp<F16>(__uint_as_float(hi[g * 8 + 4]) * mul, __uint_as_float(hi[g * 8 + 5]) * mul);
            o2.w = pack_lp<F16>(__uint_as_float(hi[g * 8 + 6]) * mul, __uint_as_float(hi[g * 8 + 7]) * mul);
            put(g, o);
            put(4 + g, o2);
          }
        } else {
          const float4* c4 = reinterpret_cast<const float4*>(p.rope_cos + (int64_t)pos * (DH / 2));
          const float4* s4 = reinterpret_cast<const float4*>(p.rope_sin + (int64_t)pos * (DH / 2));
          if (!p.rope_interleaved) {   // pairs (i, i + 32): x_i <- x_i c + x_{i+32} s ,  x_{i+32} <- -x_i s + x_{i+32} c
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              float oa[8], ob[8];
#pragma unroll
              for (int q = 0; q < 2; ++q) {
                const float4 c = c4[g * 2 + q], sn = s4[g * 2 + q];
                const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float xa = __uint_as_float(lo[g * 8 + q * 4 + e]) * mul, xb = __uint_as_float(hi[g * 8 + q * 4 + e]) * mul;
                  oa[q * 4 + e] = xa * cc[e] + xb * ss[e];
                  ob[q * 4 + e] = xb * cc[e] - xa * ss[e];
                }
              }
              put(g, make_uint4(pack_lp<F16>(oa[0], oa[1]), pack_lp<F16>(oa[2], oa[3]), pack_lp<F16>(oa[4], oa[5]), pack_lp<F16>(oa[6], oa[7])));
              put(4 + g, make_uint4(pack_lp<F16>(ob[0], ob[1]), pack_lp<F16>(ob[2], ob[3]), pack_lp<F16>(ob[4], ob[5]), pack_lp<F16>(ob[6], ob[7])));
            }
          } else {                     // pairs (2 i, 2 i + 1), angle index i
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              const uint32_t* x = hh == 0 ? lo : hi;
#pragma unroll
              for (int g = 0; g < 4; ++g) {   // 8 elements = 4 pairs, angles hh * 16 + g * 4 .. + 3
                const float4 c = c4[hh * 4 + g], sn = s4[hh * 4 + g];
                const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
                float o[8];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float xa = __uint_as_float(x[g * 8 + 2 * e]) * mul, xb = __uint_as_float(x[g * 8 + 2 * e + 1]) * mul;
                  o[2 * e] = xa * cc[e] + xb * ss[e];
                  o[2 * e + 1] = xb * cc[e] - xa * ss[e];
                }
                put(hh * 4 + g, make_uint4(pack_lp<F16>(o[0], o[1]), pack_lp<F16>(o[2], o[3]), pack_lp<F16>(o[4], o[5]), pack_lp<F16>(o[6], o[7])));
              }
            }
          }
        }
        fence_proxy_async();
        named_barrier_sync(1 + slice, 128);
        if (quarter == 0 && lane == 0) {
          tma_store_2d(&map_out, &s.ds_tile[0][0][0] + item * PANEL_BYTES, col,
                       (int)((int64_t)(p0 + pp) * p.n_rows + row_b + own * TILE));
          tma_store_commit();
          tma_store_wait_read<0>();   // the staging tile must stay intact until the copy engine has read it
        }
      }
    }
  }

  // ---------------------------------------------------------------------- teardown
  __syncwarp();
  if (s.abort_flag) {
    const unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 2000000ull) __nanosleep(1000);  // let copies in flight land before smem is released
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 16) {
    fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

// delta[p, b, h, t] = sum_d dO[(p, b, t), h * Dh + d] * O[(b, t), h * Dh + d]; one warp per (row, head).
template <bool F16>
__global__ void delta_kernel(const __nv_bfloat16* __restrict__ d_o, const __nv_bfloat16* __restrict__ o,
                             float* __restrict__ delta, int64_t rows_total, int64_t n_rows, int batch, int heads,
                             int seq_len) {
  const int64_t gw = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= rows_total * heads) return;
  const int h = (int)(gw % heads);
  const int64_t row = gw / heads;          // (p * B + b) * T + t
  const int64_t arow = row % n_rows;       // b * T + t
  const int hd = heads * DH;
  float2 af, cf;
  if (F16) {
    af = __half22float2(reinterpret_cast<const __half2*>(d_o + row * hd + h * DH)[lane]);
    cf = __half22float2(reinterpret_cast<const __half2*>(o + arow * hd + h * DH)[lane]);
  } else {
    af = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(d_o + row * hd + h * DH)[lane]);
    cf = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(o + arow * hd + h * DH)[lane]);
  }
  float acc = af.x * cf.x + af.y * cf.y;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) {
    const int64_t pb = row / seq_len;      // p * B + b
    const int t = (int)(row % seq_len);
    delta[(pb * heads + h) * seq_len + t] = acc;
  }
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

// [rows, width] bf16 row-major, tiles of 128 rows x 64 columns, 128-byte swizzle
static int make_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t width, int f16 = 0) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return 801;
  cuuint64_t dims[2] = {(cuuint64_t)width, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)width * 2};
  cuuint32_t box[2] = {DH, TILE};
  cuuint32_t estr[2] = {1, 1};
  CUresult rc = fn(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? 0 : 1000 + (int)rc;
}

template <bool DKDV, bool F16>
static int launch(const CUtensorMap& mq, const CUtensorMap& md, const CUtensorMap& mo, const Params& p, cudaStream_t st) {
  constexpr int PB = DKDV ? PB_DKDV : PB_DQ;
  const size_t smem = sizeof(Smem<DKDV>) + 1024;
  static lbi::PerDeviceOnce configured;
  {
    cudaError_t e = configured.max_dynamic_smem(pullback_kernel<DKDV, F16>, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(p.n_tiles, p.batch * p.heads, (p.nbasis + PB - 1) / PB);
  pullback_kernel<DKDV, F16><<<grid, THREADS, smem, st>>>(mq, md, mo, p);
  return (int)cudaGetLastError();
}

}  // namespace attn
}  // namespace lbi

extern "C" int lbi_attn_pullback(const void* qkv, const void* d_o, const void* o, const float* lse, void* d_qkv,
                                 float* delta, int batch, int heads, int seq_len, int head_dim, int nbasis, float scale,
                                 const float* rope_cos, const float* rope_sin, int rope_interleaved, int is_fp16, int* status,
                                 cudaStream_t st) {
  using namespace lbi::attn;
  if (head_dim != DH || seq_len % TILE != 0 || batch <= 0 || heads <= 0 || nbasis <= 0) return (int)cudaErrorInvalidValue;
  const int64_t n_rows = (int64_t)batch * seq_len;
  const int64_t rows_total = n_rows * nbasis;
  if (rows_total >= (1ll << 31)) return (int)cudaErrorInvalidValue;
  {
    const int64_t warps = rows_total * heads;
    const int threads = 256;
    const int64_t blocks = (warps * 32 + threads - 1) / threads;
    if (is_fp16)
      delta_kernel<true><<<(unsigned)blocks, threads, 0, st>>>((const __nv_bfloat16*)d_o, (const __nv_bfloat16*)o, delta, rows_total,
                                                               n_rows, batch, heads, seq_len);
    else
      delta_kernel<false><<<(unsigned)blocks, threads, 0, st>>>((const __nv_bfloat16*)d_o, (const __nv_bfloat16*)o, delta, rows_total,
                                                                n_rows, batch, heads, seq_len);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
  }
  CUtensorMap mq, md, mo;
  int rc = make_map(&mq, qkv, n_rows, 3ll * heads * DH, is_fp16);
  if (rc) return rc;
  rc = make_map(&md, d_o, rows_total, (int64_t)heads * DH, is_fp16);
  if (rc) return rc;
  rc = make_map(&mo, d_qkv, rows_total, 3ll * heads * DH, is_fp16);
  if (rc) return rc;
  Params p;
  p.batch = batch; p.heads = heads; p.seq_len = seq_len; p.nbasis = nbasis;
  p.n_tiles = seq_len / TILE;
  p.n_rows = n_rows;
  p.out_ld = 3ll * heads * DH;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = lse; p.delta = delta;
  p.d_qkv = (__nv_bfloat16*)d_qkv;
  p.rope_cos = rope_cos; p.rope_sin = rope_sin; p.rope_interleaved = rope_interleaved;
  p.status = status;
  if (is_fp16) {
    rc = launch<true, true>(mq, md, mo, p, st);
    if (rc) return rc;
    return launch<false, true>(mq, md, mo, p, st);
  }
  rc = launch<true, false>(mq, md, mo, p, st);
  if (rc) return rc;
  return launch<false, false>(mq, md, mo, p, st);
}
