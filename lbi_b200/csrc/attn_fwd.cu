// Causal flash-attention forward on tcgen05 / TMEM / TMA:  O = softmax(mask(q k^T s)) v,  lse = log sum exp.
//
// One CTA owns 256 query rows of one (batch, head): two 128-row tiles, each served by its own softmax warpgroup, and
// walks the key tiles up to the diagonal.  Per key tile j and query tile g:
//     S_g = Q_g K_j^T            tcgen05.mma  M 128 x N 128 x K 64 -> TMEM columns [128 g, 128 g + 128)
//     P_g = exp2(S_g s log2e - m) by warpgroup g, one thread per query row, written as bf16 into swizzled shared memory
//     O_g = P_g V_j              tcgen05.mma  M 128 x N 64 x K 128 -> TMEM columns [256 + 64 g, ..), NOT accumulated:
//                                the warpgroup reads the tile back and keeps the running output in registers, where
//                                the rescale by exp2(m_old - m_new) costs one multiply (no TMEM read-modify-write).
// While warpgroup 0 runs its exponentials the tensor core works for warpgroup 1 and vice versa.
// Warp roles (320 threads): warps 0-3 / 4-7 softmax warpgroups, warp 8 lane 0 TMA producer (3-stage K/V ring),
// warp 9 lane 0 MMA issuer.  The reference calls flash_attn / aten SDPA here (backbones/transformer/attention.py:78-85).
//
// Layout: qkv [B*T, 3*H*64] bf16 packed q | k | v (rotary applied), out [B*T, H*64] bf16, lse [B, H, T] fp32 (natural
// log, of the scaled scores).  T must be a multiple of 128.  Every mbarrier wait is bounded (tcgen05.cuh).
#include <cuda_bf16.h>

#include <mutex>

#include "api_attn.h"
#include "common.cuh"
#include "tcgen05.cuh"

namespace lbi {
namespace attn_fwd {

using namespace tc;

constexpr int TILE = 128;
constexpr int DH = 64;
constexpr int TILE_BYTES = TILE * DH * 2;   // 16 KB
constexpr int PANEL_BYTES = TILE * 128;     // one 64-key panel of P: 128 rows x 128 B
constexpr int THREADS = 320;
constexpr int NST = 3;                      // K/V stages

struct Params {
  int batch, heads, seq_len, n_tiles;
  float scale_log2;                         // softmax scale * log2(e)
  __nv_bfloat16* out;
  float* lse;
  int* status;
};

struct Smem {
  alignas(1024) uint8_t q[2][TILE_BYTES];
  alignas(1024) uint8_t k[NST][TILE_BYTES];
  alignas(1024) uint8_t v[NST][TILE_BYTES];
  alignas(1024) uint8_t p[2][2][PANEL_BYTES];   // [warpgroup][64-key panel]
  uint64_t bar_q;
  uint64_t bar_kv_full[NST];
  uint64_t bar_kv_empty[NST];
  uint64_t bar_s_ready[2];
  uint64_t bar_p_ready[2];
  uint64_t bar_o_ready[2];
  uint32_t tmem_base;
  volatile int abort_flag;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// F16 = false: bf16 operands and output; true: fp16.  Accumulation is fp32 either way.
template <bool F16>
__device__ __forceinline__ uint32_t pack_lp(float a, float b) {
  uint32_t d;
  if (F16) asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(b), "f"(a));
  else asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(b), "f"(a));
  return d;
}
__host__ __device__ constexpr uint32_t make_idesc_lp(int m, int n, int a_mn_major, int b_mn_major, bool f16) {
  return f16 ? (make_idesc_bf16(m, n, a_mn_major, b_mn_major) & ~((1u << 7) | (1u << 10))) : make_idesc_bf16(m, n, a_mn_major, b_mn_major);
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}

template <bool F16>
__global__ void __launch_bounds__(THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_qkv, const Params p) {
  extern __shared__ uint8_t raw_smem[];
  Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // heavy blocks (late queries walk more key tiles) first
  const int qb = (int)gridDim.x - 1 - (int)blockIdx.x;
  const int bh = blockIdx.y;
  const int b = bh / p.heads, h = bh % p.heads;
  const int hd = p.heads * DH;
  const int col_q = h * DH, col_k = hd + h * DH, col_v = 2 * hd + h * DH;
  const int row_b = b * p.seq_len;
  // query tile g of this block is tile 2 qb + g; it walks key tiles 0 .. 2 qb + g (none if the tile does not exist)
  const int nkv0 = 2 * qb + 1;
  const int nkv1 = (2 * qb + 1 < p.n_tiles) ? 2 * qb + 2 : 0;
  const int n_j = max(nkv0, nkv1);

  if (threadIdx.x == 0) {
    s.abort_flag = 0;
    mbar_init(&s.bar_q, 1);
    for (int i = 0; i < NST; ++i) {
      mbar_init(&s.bar_kv_full[i], 1);
      mbar_init(&s.bar_kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.bar_s_ready[i], 1);
      mbar_init(&s.bar_p_ready[i], 4);   // one arrival per warp of the warpgroup
      mbar_init(&s.bar_o_ready[i], 1);
    }
    fence_barrier_init();
    prefetch_tmap(&map_qkv);
  }
  if (warp == 8) tmem_alloc(&s.tmem_base, 512);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = s.tmem_base;
  volatile int* abortp = &s.abort_flag;

  if (warp == 8) {
    // ======================================================================== TMA producer
    if (lane == 0) {
      const int nq = nkv1 > 0 ? 2 : 1;
      mbar_arrive_expect_tx(&s.bar_q, nq * TILE_BYTES);
      for (int g = 0; g < nq; ++g) tma_load_2d(s.q[g], &map_qkv, &s.bar_q, col_q, row_b + (2 * qb + g) * TILE);
      bool ok = true;
      for (int j = 0; j < n_j && ok; ++j) {
        const int st = j % NST;
        if (j >= NST) {
          ok = mbar_wait(&s.bar_kv_empty[st], ((j / NST) - 1) & 1, abortp, p.status, 31);
          if (!ok) break;
        }
        mbar_arrive_expect_tx(&s.bar_kv_full[st], 2 * TILE_BYTES);
        tma_load_2d(s.k[st], &map_qkv, &s.bar_kv_full[st], col_k, row_b + j * TILE);
        tma_load_2d(s.v[st], &map_qkv, &s.bar_kv_full[st], col_v, row_b + j * TILE);
      }
    }
  } else if (warp == 9) {
    // ======================================================================== MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_lp(128, 128, 0, 0, F16);   // Q (K-major) x K (K-major)
      const uint32_t idesc_o = make_idesc_lp(128, 64, 0, 1, F16);    // P (K-major) x V (MN-major: rows are the key index)
      const uint64_t kmajor0 = make_smem_desc(0, 16, 1024);
      const uint64_t mnmajor0 = make_smem_desc(0, PANEL_BYTES, 1024);
      const uint32_t q16 = smem_u32(s.q[0]) >> 4, k16 = smem_u32(s.k[0]) >> 4, v16 = smem_u32(s.v[0]) >> 4;
      const uint32_t p16 = smem_u32(s.p[0][0]) >> 4;
      constexpr uint32_t TILE16 = TILE_BYTES >> 4, PANEL16 = PANEL_BYTES >> 4;
      auto issue_s = [&](int g, int st) {
        const uint64_t da = kmajor0 + q16 + g * TILE16, db = kmajor0 + k16 + st * TILE16;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) mma_bf16(tmem + g * 128, da + 2 * kk, db + 2 * kk, idesc_s, kk);
        mma_commit(&s.bar_s_ready[g]);
      };
      bool ok = mbar_wait(&s.bar_q, 0, abortp, p.status, 32);
      ok = ok && mbar_wait(&s.bar_kv_full[0], 0, abortp, p.status, 33);
      if (ok) {
        fence_after_sync();
        issue_s(0, 0);
        if (nkv1 > 0) issue_s(1, 0);
      }
      for (int j = 0; j < n_j && ok; ++j) {
        const int st = j % NST, st_next = (j + 1) % NST;
        if (j + 1 < n_j) {
          ok = mbar_wait(&s.bar_kv_full[st_next], ((j + 1) / NST) & 1, abortp, p.status, 34);
          if (!ok) break;
        }
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          const int nkv_g = g == 0 ? nkv0 : nkv1;
          if (!ok || j >= nkv_g) continue;
          ok = mbar_wait(&s.bar_p_ready[g], j & 1, abortp, p.status, 35);
          if (!ok) break;
          fence_after_sync();
          const uint64_t da = kmajor0 + p16 + g * 2 * PANEL16, db = mnmajor0 + v16 + st * TILE16;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            mma_bf16(tmem + 256 + g * 64, da + (kk >> 2) * PANEL16 + (kk & 3) * 2, db + 128 * kk, idesc_o, kk);
          mma_commit(&s.bar_o_ready[g]);
          if (j + 1 < nkv_g) issue_s(g, st_next);
        }
        if (ok) mma_commit(&s.bar_kv_empty[st]);   // everything that read stage st has been issued before this commit
      }
    }
  } else {
    // ======================================================================== softmax warpgroups
    const int g = warp >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int nkv_g = g == 0 ? nkv0 : nkv1;
    if (nkv_g > 0) {
      const int i_g = 2 * qb + g;
      const uint32_t t_s = tmem + ((uint32_t)(quarter * 32) << 16) + g * 128;
      const uint32_t t_o = tmem + ((uint32_t)(quarter * 32) << 16) + 256 + g * 64;
      const uint32_t p_base = smem_u32(s.p[g][0]);
      float acc[DH];
#pragma unroll
      for (int e = 0; e < DH; ++e) acc[e] = 0.f;
      float m_run = -INFINITY, l_run = 0.f;
      bool ok = true;
      for (int j = 0; j < nkv_g; ++j) {
        ok = mbar_wait(&s.bar_s_ready[g], j & 1, abortp, p.status, 36);
        if (!ok) break;
        fence_after_sync();
        const bool diag = (j == i_g);
        // pass 1: row maximum of the raw scores
        float mx = -INFINITY;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_s + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const float val = __uint_as_float(r[e]);
            if (!diag || c * 32 + e <= row) mx = fmaxf(mx, val);
          }
        }
        const float m_new = fmaxf(m_run, mx * p.scale_log2);
        const float alpha = ex2(m_run - m_new);
        // pass 2: probabilities -> bf16 P in shared memory (K-major, two 64-key panels), row sum
        float sum = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_s + c * 32, r);
          tmem_ld_wait();
          const uint32_t panel = p_base + (c >> 1) * PANEL_BYTES + row * 128;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint32_t w[4];
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2) {
              const int e = q4 * 8 + e2 * 2;
              float a = ex2(fmaf(__uint_as_float(r[e]), p.scale_log2, -m_new));
              float bb = ex2(fmaf(__uint_as_float(r[e + 1]), p.scale_log2, -m_new));
              if (diag) {
                if (c * 32 + e > row) a = 0.f;
                if (c * 32 + e + 1 > row) bb = 0.f;
              }
              sum += a + bb;
              w[e2] = pack_lp<F16>(a, bb);
            }
            const int chunk = (c & 1) * 4 + q4;
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(panel + ((chunk ^ (row & 7)) << 4)), "r"(w[0]),
                         "r"(w[1]), "r"(w[2]), "r"(w[3])
                         : "memory");
          }
        }
        l_run = l_run * alpha + sum;
        m_run = m_new;
        fence_proxy_async();   // S was read with tcgen05.wait::ld above, so the TMEM reads are complete
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.bar_p_ready[g]);
#pragma unroll
        for (int e = 0; e < DH; ++e) acc[e] *= alpha;
        ok = mbar_wait(&s.bar_o_ready[g], j & 1, abortp, p.status, 37);
        if (!ok) break;
        fence_after_sync();
        {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(t_o, r0);
          tmem_ld_32x32(t_o + 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            acc[e] += __uint_as_float(r0[e]);
            acc[32 + e] += __uint_as_float(r1[e]);
          }
        }
      }
      if (ok) {
        const float inv = 1.f / l_run;
        const int64_t tok = (int64_t)row_b + i_g * TILE + row;
        uint4* dst = reinterpret_cast<uint4*>(p.out + tok * hd + h * DH);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint4 vv;
          vv.x = pack_lp<F16>(acc[8 * c] * inv, acc[8 * c + 1] * inv);
          vv.y = pack_lp<F16>(acc[8 * c + 2] * inv, acc[8 * c + 3] * inv);
          vv.z = pack_lp<F16>(acc[8 * c + 4] * inv, acc[8 * c + 5] * inv);
          vv.w = pack_lp<F16>(acc[8 * c + 6] * inv, acc[8 * c + 7] * inv);
          dst[c] = vv;
        }
        p.lse[((int64_t)b * p.heads + h) * p.seq_len + i_g * TILE + row] = (m_run + log2f(l_run)) * 0.6931471805599453f;
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
  if (warp == 8) {
    fence_after_sync();
    tmem_dealloc(tmem, 512);
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

}  // namespace attn_fwd
}  // namespace lbi

extern "C" int lbi_attn_fwd(const void* qkv, void* out, float* lse, int batch, int heads, int seq_len, int head_dim,
                            float scale, int is_fp16, int* status, cudaStream_t st) {
  using namespace lbi::attn_fwd;
  if (head_dim != DH || seq_len % TILE != 0 || batch <= 0 || heads <= 0) return (int)cudaErrorInvalidValue;
  const int64_t n_rows = (int64_t)batch * seq_len;
  if (n_rows >= (1ll << 31)) return (int)cudaErrorInvalidValue;
  EncodeTiledFn fn = encode_fn();
  if (!fn) return 801;
  CUtensorMap map;
  const int64_t width = 3ll * heads * DH;
  cuuint64_t dims[2] = {(cuuint64_t)width, (cuuint64_t)n_rows};
  cuuint64_t strides[1] = {(cuuint64_t)width * 2};
  cuuint32_t box[2] = {DH, TILE};
  cuuint32_t estr[2] = {1, 1};
  CUresult rc = fn(&map, is_fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(qkv), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return 1000 + (int)rc;
  Params p;
  p.batch = batch; p.heads = heads; p.seq_len = seq_len; p.n_tiles = seq_len / TILE;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.out = (__nv_bfloat16*)out; p.lse = lse; p.status = status;
  const size_t smem = sizeof(Smem) + 1024;
  static lbi::PerDeviceOnce configured, configured_bf16;
  {
    cudaError_t e = is_fp16 ? configured.max_dynamic_smem(attn_fwd_kernel<true>, (int)smem)
                            : configured_bf16.max_dynamic_smem(attn_fwd_kernel<false>, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((p.n_tiles + 1) / 2, batch * heads);
  if (is_fp16) attn_fwd_kernel<true><<<grid, THREADS, smem, st>>>(map, p);
  else attn_fwd_kernel<false><<<grid, THREADS, smem, st>>>(map, p);
  return (int)cudaGetLastError();
}
