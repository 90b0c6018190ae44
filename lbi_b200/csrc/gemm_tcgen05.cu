// bf16 GEMM on the 5th-generation tensor cores:  C[M, N] (+)= A[M, K] * B[N, K]^T, fp32 accumulation in TMEM.
//
// One persistent CTA per SM, 192 threads, warp-specialised:
//   warp 0        TMA producer: 128 x 64 tile of A and BN x 64 tile of B per stage, 128-byte swizzle, 4-stage ring
//   warp 1        allocates 512 TMEM columns (two BN-column accumulators) and issues tcgen05.mma (one elected lane):
//                 four K = 16 instructions per stage, tcgen05.commit frees the stage, a last commit publishes the tile
//   warps 2..5    epilogue: tcgen05.ld 32 lanes x 32 columns, convert, stage 128-byte rows in swizzled shared memory,
//                 TMA store (or TMA reduce-add for fp32 accumulation / split-K) of 128 x 128-byte boxes; runs one tile
//                 behind the MMA warp thanks to the double-buffered accumulator.  (Direct 16-byte stores from
//                 registers made the epilogue, not the main loop, the limit for K <= 1024: about 10 us per tile.)
// Each operand may be K-major (row-major [rows, K]) or MN-major (row-major [K, rows]); the latter is loaded as
// 64-row panels through a 3-D tensor map, so dgrad (dY * W) and wgrad (dY^T * X) need no transposed copies.
// Split-K (gridDim.y) spreads a long reduction over several CTAs that add into an fp32 C with vector atomics.
// Every mbarrier wait is bounded (see tcgen05.cuh); on a timeout the CTA stops, frees its TMEM and reports through
// the status word.
#include <cuda_bf16.h>

#include <mutex>

#include "api_gemm.h"
#include "common.cuh"
#include "tcgen05.cuh"

namespace lbi {
namespace gemm {

using namespace tc;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int THREADS = 192;
constexpr int UMMA_K = 16;

struct Params {
  int M, N, K;
  int out_fp32;
  int atomic_add;    // fp32 C: add to memory (TMA reduce) instead of storing
  int a_mn_major, b_mn_major;
  int k_blocks_per_split;
  int* status;
};

template <int BN>
struct Smem {
  alignas(1024) uint8_t a[STAGES][BM * BK * 2];
  alignas(1024) uint8_t b[STAGES][BN * BK * 2];
  alignas(1024) uint8_t cstage[2][BM * 128];   // epilogue staging: two boxes of 128 rows x 128 bytes
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  volatile int abort_flag;
};

template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const __grid_constant__ CUtensorMap tmap_c, const Params p) {
  extern __shared__ uint8_t raw_smem[];
  Smem<BN>& s = *reinterpret_cast<Smem<BN>*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks_total = (p.K + BK - 1) / BK;
  const int kb_begin = blockIdx.y * p.k_blocks_per_split;
  const int kb_end = min(k_blocks_total, kb_begin + p.k_blocks_per_split);
  const int num_kb = kb_end - kb_begin;

  if (threadIdx.x == 0) {
    s.abort_flag = 0;
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.tmem_full[i], 1);
      mbar_init(&s.tmem_empty[i], 4);
    }
    fence_barrier_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    prefetch_tmap(&tmap_c);
  }
  if (warp == 1) tmem_alloc(&s.tmem_base, 512);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = s.tmem_base;

  if (num_kb > 0) {
    if (warp == 0) {
      // ------------------------------------------------------------------ TMA producer
      if (elect_one()) {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
          const int m0 = (tile / tiles_n) * BM;
          const int n0 = (tile % tiles_n) * BN;
          for (int kb = kb_begin; kb < kb_end; ++kb) {
            ok = mbar_wait(&s.empty[stage], phase ^ 1, &s.abort_flag, p.status, 1);
            if (!ok) break;
            mbar_arrive_expect_tx(&s.full[stage], (BM + BN) * BK * 2);
            if (p.a_mn_major)
              tma_load_3d(s.a[stage], &tmap_a, &s.full[stage], 0, kb * BK, m0 / 64);
            else
              tma_load_2d(s.a[stage], &tmap_a, &s.full[stage], kb * BK, m0);
            if (p.b_mn_major)
              tma_load_3d(s.b[stage], &tmap_b, &s.full[stage], 0, kb * BK, n0 / 64);
            else
              tma_load_2d(s.b[stage], &tmap_b, &s.full[stage], kb * BK, n0);
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1;
            }
          }
        }
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------------ MMA issuer
      if (elect_one()) {
        const uint32_t idesc = make_idesc_bf16(BM, BN, p.a_mn_major, p.b_mn_major);
        // K-major: one K = 16 slice is 32 bytes inside the 128-byte row; MN-major: 16 k-rows = two swizzle atoms
        const uint32_t a_lbo = p.a_mn_major ? 64 * BK * 2 : 16, a_kstep = p.a_mn_major ? 2048 : 32;
        const uint32_t b_lbo = p.b_mn_major ? 64 * BK * 2 : 16, b_kstep = p.b_mn_major ? 2048 : 32;
        const uint64_t a_desc0 = make_smem_desc(smem_u32(s.a[0]), a_lbo, 1024);
        const uint64_t b_desc0 = make_smem_desc(smem_u32(s.b[0]), b_lbo, 1024);
        int stage = 0;
        uint32_t phase = 0;
        int local_tile = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
          const int buf = local_tile & 1;
          const uint32_t acc_phase = (local_tile >> 1) & 1;
          ok = mbar_wait(&s.tmem_empty[buf], acc_phase ^ 1, &s.abort_flag, p.status, 2);
          if (!ok) break;
          fence_after_sync();
          const uint32_t d_tmem = tmem_base + buf * BN;
          for (int kb = 0; kb < num_kb; ++kb) {
            ok = mbar_wait(&s.full[stage], phase, &s.abort_flag, p.status, 3);
            if (!ok) break;
            fence_after_sync();
            // descriptor = constant template + (address >> 4); a K = 16 slice advances the address field only
            const uint64_t da = a_desc0 + (uint64_t)(stage * ((BM * BK * 2) >> 4));
            const uint64_t db = b_desc0 + (uint64_t)(stage * ((BN * BK * 2) >> 4));
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              mma_bf16(d_tmem, da + k * (a_kstep >> 4), db + k * (b_kstep >> 4), idesc, (kb | k) != 0 ? 1u : 0u);
            mma_commit(&s.empty[stage]);
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1;
            }
          }
          if (ok) mma_commit(&s.tmem_full[buf]);
        }
      }
    } else {
      // ------------------------------------------------------------------ epilogue (warps 2..5)
      const int quarter = warp & 3;  // TMEM lanes [32 * quarter, 32 * quarter + 32) belong to this warp
      const int row = quarter * 32 + lane;
      const bool leader = (warp == 2 && lane == 0);
      constexpr int COLS_PER_BOX_BF16 = 64, COLS_PER_BOX_F32 = 32;
      const int cols_per_box = p.out_fp32 ? COLS_PER_BOX_F32 : COLS_PER_BOX_BF16;
      const int boxes = BN / cols_per_box;
      int local_tile = 0, box_count = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
        const int buf = local_tile & 1;
        const uint32_t acc_phase = (local_tile >> 1) & 1;
        const int m0 = (tile / tiles_n) * BM;
        const int n0 = (tile % tiles_n) * BN;
        ok = mbar_wait(&s.tmem_full[buf], acc_phase, &s.abort_flag, p.status, 4);
        // all four warps take the same decision (they share named barrier 1 below): a raised abort flag wins
        named_barrier_sync(1, 128);
        ok = (s.abort_flag == 0);
        if (!ok) break;
        fence_after_sync();
        const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
#pragma unroll 1
        for (int bx = 0; bx < boxes; ++bx, ++box_count) {
          const int half = box_count & 1;
          const uint32_t stage_row = smem_u32(s.cstage[half]) + row * 128;
          // the TMA store issued two boxes ago must have finished reading this staging half
          if (leader) tma_store_wait_read<1>();
          named_barrier_sync(1, 128);
          if (p.out_fp32) {
            uint32_t r[32];
            tmem_ld_32x32(t_row + bx * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j)
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage_row + ((j ^ (row & 7)) << 4)), "r"(r[4 * j]),
                           "r"(r[4 * j + 1]), "r"(r[4 * j + 2]), "r"(r[4 * j + 3])
                           : "memory");
          } else {
            uint32_t r[2][32];
            tmem_ld_32x32(t_row + bx * 64, r[0]);
            tmem_ld_32x32(t_row + bx * 64 + 32, r[1]);
            tmem_ld_wait();
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  __nv_bfloat162 t2 =
                      __floats2bfloat162_rn(__uint_as_float(r[hh][8 * j + 2 * e]), __uint_as_float(r[hh][8 * j + 2 * e + 1]));
                  w[e] = *reinterpret_cast<uint32_t*>(&t2);
                }
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage_row + (((hh * 4 + j) ^ (row & 7)) << 4)),
                             "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                             : "memory");
              }
            }
          }
          if (bx == boxes - 1) {  // accumulator fully read: hand the TMEM buffer back to the MMA warp
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s.tmem_empty[buf]);
          }
          fence_proxy_async();
          named_barrier_sync(1, 128);
          if (leader) {
            const int x = n0 + bx * cols_per_box;
            if (x < p.N && m0 < p.M) {
              if (p.atomic_add) tma_reduce_add_2d(&tmap_c, s.cstage[half], x, m0);
              else tma_store_2d(&tmap_c, s.cstage[half], x, m0);
            }
            tma_store_commit();
          }
        }
      }
      if (leader) tma_store_wait_all<0>();
    }
  }

  // ---------------------------------------------------------------------- teardown
  __syncwarp();
  if (s.abort_flag) {
    // give TMA copies that are still in flight time to land before shared memory is released
    const unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc(tmem_base, 512);
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

// Tensor map of one operand.  `rows` is the M (or N) extent, `k` the reduction extent, `ld` the leading dimension
// in elements of the row-major storage ([rows, k] when K-major, [k, rows] when MN-major), `tile_rows` 128 or BN.
static int make_operand_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t k, int64_t ld, int mn_major,
                            int tile_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return 801;  // cudaErrorNotSupported
  CUresult rc;
  if (!mn_major) {
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)tile_rows};
    cuuint32_t estr[2] = {1, 1};
    rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    // [k, rows] storage viewed as (64 contiguous rows-elements, k, panel): panel p starts 128 bytes after panel p-1
    cuuint64_t dims[3] = {64, (cuuint64_t)k, (cuuint64_t)(rows / 64)};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 2, 128};
    cuuint32_t box[3] = {64, (cuuint32_t)BK, (cuuint32_t)(tile_rows / 64)};
    cuuint32_t estr[3] = {1, 1, 1};
    rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  return rc == CUDA_SUCCESS ? 0 : 1000 + (int)rc;
}

// Output map: boxes of 128 rows x 128 bytes (64 bf16 or 32 fp32 columns), 128-byte swizzle like the staging buffer.
static int make_output_map(CUtensorMap* map, void* ptr, int64_t rows, int64_t cols, int64_t ld, int out_fp32) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return 801;
  const int esize = out_fp32 ? 4 : 2;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * esize};
  cuuint32_t box[2] = {(cuuint32_t)(128 / esize), (cuuint32_t)BM};
  cuuint32_t estr[2] = {1, 1};
  CUresult rc = fn(map, out_fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ptr, dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? 0 : 1000 + (int)rc;
}

template <int BN>
static int launch(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                  int a_mn, int b_mn, int out_fp32, int accumulate, int splits, int* status, int max_ctas,
                  cudaStream_t st) {
  CUtensorMap ma, mb, mc;
  int rc = make_operand_map(&ma, A, M, K, lda, a_mn, BM);
  if (rc) return rc;
  rc = make_operand_map(&mb, B, N, K, ldb, b_mn, BN);
  if (rc) return rc;
  rc = make_output_map(&mc, C, M, N, ldc, out_fp32);
  if (rc) return rc;
  const int k_blocks = (K + BK - 1) / BK;
  if (splits < 1) splits = 1;
  if (splits > k_blocks) splits = k_blocks > 0 ? k_blocks : 1;
  Params p;
  p.M = M; p.N = N; p.K = K; p.out_fp32 = out_fp32;
  p.atomic_add = (accumulate || splits > 1) ? 1 : 0;
  p.a_mn_major = a_mn; p.b_mn_major = b_mn;
  p.k_blocks_per_split = (k_blocks + splits - 1) / splits;
  p.status = status;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int ctas = max_ctas / splits;
  if (ctas < 1) ctas = 1;
  if (ctas > tiles) ctas = tiles;
  const size_t smem = sizeof(Smem<BN>) + 1024;
  static lbi::PerDeviceOnce configured;
  {
    cudaError_t e = configured.max_dynamic_smem(gemm_kernel<BN>, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(ctas, splits);
  gemm_kernel<BN><<<grid, THREADS, smem, st>>>(ma, mb, mc, p);
  return (int)cudaGetLastError();
}

}  // namespace gemm
}  // namespace lbi

extern "C" int lbi_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb,
                             int64_t ldc, int a_mn_major, int b_mn_major, int out_fp32, int accumulate, int splits,
                             int* status, int sm_count, cudaStream_t st) {
  using namespace lbi::gemm;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) {   // an empty sum: C = 0 unless the caller accumulates
    if (!accumulate) {
      const size_t esize = out_fp32 ? 4 : 2;
      cudaError_t e = cudaMemset2DAsync(C, (size_t)ldc * esize, 0, (size_t)N * esize, (size_t)M, st);
      if (e != cudaSuccess) return (int)e;
    }
    return 0;
  }
  if (N > 128)
    return launch<256>(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, out_fp32, accumulate, splits, status,
                       sm_count, st);
  return launch<128>(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, out_fp32, accumulate, splits, status,
                     sm_count, st);
}
