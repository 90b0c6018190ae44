// Peer-memory kernels: compute fused with the NVLink / NVSwitch transfer (see api_peer.h for the contracts).
//
//  * interface update + hand-off: the MLP / LayerNorm epilogue stores the new bounded state straight into the next
//    region owner's mailbox and raises its flag; the receiver's wait kernel acquires it (replaces ~10 small
//    kernels + send/recv);
//  * cross-GPU affine suffix scan: every rank peer-loads the Jacobians it needs and runs the recursion locally;
//  * gradient reduce-scatter by peer loads (or NVLS multimem.ld_reduce) with the gradient-norm partial, and
//    clip + AdamW fused with the all-gather of the new bf16 weights (peer stores).
// No TMA is used on peer memory.  Every poll on a flag is bounded and records a site code instead of hanging.
#include <cuda_bf16.h>

#include "api_peer.h"
#include "common.cuh"

namespace lbi {
namespace peer {

// Time limit of every flag wait.  Ranks of one step may legitimately be seconds apart (a rank's forward starts when the
// previous owner's regions are done), so the default is generous; tests of the failure path set it to about a second.
__device__ unsigned long long g_wait_limit_ns = 20000000000ull;

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Wait until *flag >= want (sequence numbers, wrap-safe for differences < 2^31).  False on timeout.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t want, int* status, int site) {
  // the clock is read only after a few thousand polls: %globaltimer is slow to read and most waits are short
  for (int i = 0; i < 4096; ++i) {
    if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
  }
  const unsigned long long t0 = now_ns();
  uint32_t spins = 0;
  while ((int32_t)(ld_acquire_sys(flag) - want) < 0) {
    if ((++spins & 0xff) == 0 && now_ns() - t0 > g_wait_limit_ns) {
      if (status) atomicCAS(status, 0, site);
      return false;
    }
    __nanosleep(64);
  }
  return true;
}

// ------------------------------------------------------------------------------------------------ barrier / signal
__global__ void barrier_kernel(uint32_t* const* flag_ptrs, int rank, int world, int slot_base, uint32_t seq, int* status) {
  const int t = threadIdx.x;
  if (t < world) {
    __threadfence_system();
    st_release_sys(flag_ptrs[t] + slot_base + rank, seq);
    wait_flag(flag_ptrs[rank] + slot_base + t, seq, status, 41);
  }
}

__global__ void signal_all_kernel(uint32_t* const* flag_ptrs, int rank, int world, int slot_base, uint32_t seq) {
  const int t = threadIdx.x;
  if (t < world) {
    __threadfence_system();
    st_release_sys(flag_ptrs[t] + slot_base + rank, seq);
  }
}

// ------------------------------------------------------------------------------------------------ interface hand-off
__device__ __forceinline__ float activate(float x, int act) {
  if (act == 0) return x / (1.f + __expf(-x));                       // SiLU
  return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));           // GELU (erf form)
}

// One CTA per batch row.  Dynamic smem: pooled[dim] | hidden[max(hidden, 1)] | pre[width].
__global__ void __launch_bounds__(256) interface_update_handoff_kernel(
    const float* __restrict__ state_in, const float* __restrict__ pooled, const float* __restrict__ w1,
    const float* __restrict__ b1, const float* __restrict__ w2, const float* __restrict__ b2,
    const float* __restrict__ alpha, const float* __restrict__ ln_w, const float* __restrict__ ln_b, float ln_eps, int act,
    int dim, int hidden, int width, float* __restrict__ delta_out, float* __restrict__ pre_out,
    float* __restrict__ state_out, float* peer_state, uint32_t* peer_flag, uint32_t seq, uint32_t* done_counter) {
  extern __shared__ float sm[];
  __shared__ float scratch[33];
  float* s_pooled = sm;
  float* s_hidden = sm + dim;
  float* s_pre = s_hidden + (hidden > 0 ? hidden : 1);
  const int row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) s_pooled[i] = pooled[(size_t)row * dim + i];
  __syncthreads();
  const float scale = tanhf(*alpha);
  if (hidden > 0) {
    for (int hcol = warp; hcol < hidden; hcol += nwarps) {
      const float* wrow = w1 + (size_t)hcol * dim;
      float acc = 0.f;
      for (int i = lane; i < dim; i += 32) acc += wrow[i] * s_pooled[i];
      acc = warp_sum(acc);
      if (lane == 0) s_hidden[hcol] = activate(acc + (b1 ? b1[hcol] : 0.f), act);
    }
    __syncthreads();
  }
  const float* in_vec = hidden > 0 ? s_hidden : s_pooled;
  const float* w_out = hidden > 0 ? w2 : w1;
  const float* b_out = hidden > 0 ? b2 : b1;
  const int in_dim = hidden > 0 ? hidden : dim;
  for (int rcol = warp; rcol < width; rcol += nwarps) {
    const float* wrow = w_out + (size_t)rcol * in_dim;
    float acc = 0.f;
    for (int i = lane; i < in_dim; i += 32) acc += wrow[i] * in_vec[i];
    acc = warp_sum(acc);
    if (lane == 0) {
      const float d = acc + (b_out ? b_out[rcol] : 0.f);
      const float pre = state_in[(size_t)row * width + rcol] + scale * d;
      delta_out[(size_t)row * width + rcol] = d;
      pre_out[(size_t)row * width + rcol] = pre;
      s_pre[rcol] = pre;
    }
  }
  __syncthreads();
  // LayerNorm over the interface width
  float part = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) part += s_pre[i];
  const float mean = block_sum(part, scratch) / (float)width;
  part = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float c = s_pre[i] - mean;
    part += c * c;
  }
  const float rstd = rsqrtf(block_sum(part, scratch) / (float)width + ln_eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float y = (s_pre[i] - mean) * rstd * ln_w[i] + ln_b[i];
    state_out[(size_t)row * width + i] = y;
    if (peer_state) peer_state[(size_t)row * width + i] = y;   // store into the next owner's mailbox over NVLink
  }
  if (peer_state) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t done = atomicAdd(done_counter, 1u);
      if (done == gridDim.x - 1) {       // last row to finish raises the flag
        *done_counter = 0;
        __threadfence_system();
        st_release_sys(peer_flag, seq);
      }
    }
  }
}

// The same update with the hidden layer spread over the grid: one hidden unit per warp, every CTA handles all batch rows, so
// the first weight matrix is read once (the per-row kernel above reads it once per batch row from a handful of CTAs and is
// bound by load latency).  The CTA that finishes last (ticket counter) runs the narrow second layer, the LayerNorm, the
// store into the peer's mailbox and the flag.  batch <= WIDE_MAXB.  Dynamic smem: batch * max(dim, hidden) + batch * width floats.
constexpr int WIDE_MAXB = 8;
__global__ void __launch_bounds__(256) interface_update_handoff_wide_kernel(
    const float* __restrict__ state_in, const float* __restrict__ pooled, const float* __restrict__ w1,
    const float* __restrict__ b1, const float* __restrict__ w2, const float* __restrict__ b2,
    const float* __restrict__ alpha, const float* __restrict__ ln_w, const float* __restrict__ ln_b, float ln_eps, int act,
    int batch, int dim, int hidden, int width, float* hidden_buf, float* __restrict__ delta_out, float* __restrict__ pre_out,
    float* __restrict__ state_out, float* peer_state, uint32_t* peer_flag, uint32_t seq, uint32_t* ticket) {
  extern __shared__ float sm[];
  __shared__ int is_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  float* s_in = sm;                                              // [batch][dim], later [batch][hidden]
  float* s_pre = sm + (size_t)batch * (dim > hidden ? dim : hidden);   // [batch][width]
  for (int i = threadIdx.x; i < batch * dim; i += blockDim.x) s_in[i] = pooled[i];
  __syncthreads();
  const int hcol = blockIdx.x * nwarps + warp;
  if (hcol < hidden) {
    const float* wrow = w1 + (size_t)hcol * dim;
    float acc[WIDE_MAXB];
#pragma unroll
    for (int b = 0; b < WIDE_MAXB; ++b) acc[b] = 0.f;
    for (int i = lane; i < dim; i += 32) {
      const float wv = wrow[i];
#pragma unroll
      for (int b = 0; b < WIDE_MAXB; ++b)
        if (b < batch) acc[b] = fmaf(wv, s_in[b * dim + i], acc[b]);
    }
    const float bias = b1 ? b1[hcol] : 0.f;
#pragma unroll
    for (int b = 0; b < WIDE_MAXB; ++b) {
      if (b < batch) {
        const float v = warp_sum(acc[b]);
        if (lane == 0) hidden_buf[(size_t)b * hidden + hcol] = activate(v + bias, act);
      }
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(ticket, 1u) == gridDim.x - 1 ? 1 : 0;
  __syncthreads();
  if (!is_last) return;
  if (threadIdx.x == 0) *ticket = 0;
  __threadfence();
  for (int i = threadIdx.x; i < batch * hidden; i += blockDim.x) s_in[i] = __ldcg(hidden_buf + i);
  __syncthreads();
  const float scale = tanhf(*alpha);
  for (int rcol = warp; rcol < width; rcol += nwarps) {
    const float* wrow = w2 + (size_t)rcol * hidden;
    float acc[WIDE_MAXB];
#pragma unroll
    for (int b = 0; b < WIDE_MAXB; ++b) acc[b] = 0.f;
    for (int i = lane; i < hidden; i += 32) {
      const float wv = wrow[i];
#pragma unroll
      for (int b = 0; b < WIDE_MAXB; ++b)
        if (b < batch) acc[b] = fmaf(wv, s_in[b * hidden + i], acc[b]);
    }
    const float bias = b2 ? b2[rcol] : 0.f;
#pragma unroll
    for (int b = 0; b < WIDE_MAXB; ++b) {
      if (b < batch) {
        const float d = warp_sum(acc[b]) + bias;
        if (lane == 0) {
          const float pre = state_in[(size_t)b * width + rcol] + scale * d;
          delta_out[(size_t)b * width + rcol] = d;
          pre_out[(size_t)b * width + rcol] = pre;
          s_pre[b * width + rcol] = pre;
        }
      }
    }
  }
  __syncthreads();
  // LayerNorm over the interface width: one warp per batch row
  for (int b = warp; b < batch; b += nwarps) {
    float part = 0.f;
    for (int i = lane; i < width; i += 32) part += s_pre[b * width + i];
    const float mean = warp_sum(part) / (float)width;
    part = 0.f;
    for (int i = lane; i < width; i += 32) {
      const float c = s_pre[b * width + i] - mean;
      part += c * c;
    }
    const float rstd = rsqrtf(warp_sum(part) / (float)width + ln_eps);
    for (int i = lane; i < width; i += 32) {
      const float y = (s_pre[b * width + i] - mean) * rstd * ln_w[i] + ln_b[i];
      state_out[(size_t)b * width + i] = y;
      if (peer_state) peer_state[(size_t)b * width + i] = y;   // store into the next owner's mailbox over NVLink
    }
  }
  if (peer_state) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) st_release_sys(peer_flag, seq);
  }
}

__global__ void wait_state_kernel(const float* mailbox, const uint32_t* flag, uint32_t seq, float* out, int n, int* status) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = wait_flag(flag, seq, status, 42) ? 1 : 0;
  __syncthreads();
  if (!ok) return;
  for (int i = threadIdx.x; i < n; i += blockDim.x) out[i] = __ldcv(mailbox + i);
}

// ------------------------------------------------------------------------------------------------ cross-GPU scan
// One CTA per batch element; a warp owns a row of the mat-vec.  Dynamic smem: 2 * r floats.
__global__ void __launch_bounds__(256) affine_scan_peer_kernel(const float* const* mats_ptrs, const float* const* offs_ptrs,
                                                                const uint32_t* flags, int slot_base, uint32_t seq,
                                                                float* __restrict__ g, int world, int k_local, int r,
                                                                int* status) {
  extern __shared__ float vec[];
  __shared__ int ok_all;
  const int b = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if (threadIdx.x == 0) ok_all = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    if (!wait_flag(flags + slot_base + threadIdx.x, seq, status, 43)) ok_all = 0;
  }
  __syncthreads();
  if (!ok_all) return;
  const int k_total = world * k_local;
  float* cur = vec;
  float* nxt = vec + r;
  float* g_b = g + (size_t)b * k_total * r;
  // seed: g_{K-1} = b_{K-1}
  {
    const int owner = (k_total - 1) / k_local, kl = (k_total - 1) % k_local;
    const float* off = offs_ptrs[owner] + ((size_t)b * k_local + kl) * r;
    for (int i = threadIdx.x; i < r; i += blockDim.x) {
      const float v = __ldcv(off + i);
      cur[i] = v;
      g_b[(size_t)(k_total - 1) * r + i] = v;
    }
  }
  __syncthreads();
  for (int k = k_total - 2; k >= 0; --k) {
    const int owner = k / k_local, kl = k % k_local;
    const float* m = mats_ptrs[owner] + ((size_t)b * k_local + kl) * r * r;
    const float* off = offs_ptrs[owner] + ((size_t)b * k_local + kl) * r;
    for (int row = warp; row < r; row += nwarps) {
      float acc = 0.f;
      for (int j = lane; j < r; j += 32) acc += __ldcv(m + (size_t)row * r + j) * cur[j];
      acc = warp_sum(acc);
      if (lane == 0) {
        const float v = __ldcv(off + row) + acc;
        nxt[row] = v;
        g_b[(size_t)k * r + row] = v;
      }
    }
    __syncthreads();
    float* t = cur;
    cur = nxt;
    nxt = t;
  }
}

// Basis-parallel variant: every rank holds PARTIAL Jacobian rows for all regions (zeros where another rank did the work),
// rows[k][b][j][a] = d s_out[j] / d s_in[a], and partial offsets offs[k][b][a].  The kernel sums the partials over the
// ranks while it loads them (plain peer loads) and runs g_k[a] = b_k[a] + sum_j rows_k[j][a] g_{k+1}[j] on every rank.
// One CTA per batch element; component a of the result is shared by blockDim.x / r thread groups that split the j range
// (the loads are peer loads with microseconds of latency, so many must be in flight).  Dynamic smem: (2 + groups) * r floats.
__global__ void __launch_bounds__(1024) affine_scan_peer_sum_kernel(const float* const* rows_ptrs, const float* const* offs_ptrs,
                                                                     const uint32_t* flags, int slot_base, uint32_t seq,
                                                                     float* __restrict__ g, int world, int batch, int k_total, int r,
                                                                     int* status, int flag_world) {
  // `world` buffers are summed while they are loaded; `flag_world` >= world ranks are waited for (with published rows the
  // whole matrix set already sits in this rank's own buffer: world = 1, flag_world = all ranks)
  extern __shared__ float vec[];
  __shared__ int ok_all;
  const int b = blockIdx.x;
  if (threadIdx.x == 0) ok_all = 1;
  __syncthreads();
  if (threadIdx.x < flag_world) {
    if (!wait_flag(flags + slot_base + threadIdx.x, seq, status, 45)) ok_all = 0;
  }
  __syncthreads();
  if (!ok_all) return;
  const int groups = max(1, (int)blockDim.x / r);
  const int a = threadIdx.x % r, grp = threadIdx.x / r;
  const bool active = grp < groups;
  float* cur = vec;
  float* nxt = vec + r;
  float* part = vec + 2 * r;   // [groups][r]
  float* g_b = g + (size_t)b * k_total * r;
  for (int k = k_total - 1; k >= 0; --k) {
    const size_t off_base = ((size_t)k * batch + b) * r;
    const size_t row_base = off_base * r;
    if (active) {
      float acc = 0.f;
      if (grp == 0)
        for (int w = 0; w < world; ++w) acc += __ldcg(offs_ptrs[w] + off_base + a);
      if (k < k_total - 1) {
        // sixteen loads in flight per thread: the recursion is bound by load latency, not by bandwidth.  The data was
        // complete before the flags were seen (acquire), so the loads need not be volatile; they bypass L1 only.  The
        // single-buffer form (published rows) is spelled out: with the loop over buffers between them, the add that
        // consumes a load sits before the next load in program order and an in-order warp then waits for each load in turn.
        if (world == 1) {
          const float* rows = rows_ptrs[0] + row_base + a;
          for (int j0 = grp; j0 < r; j0 += groups * 16) {
            float m[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) {
              const int j = j0 + u * groups;
              m[u] = j < r ? __ldcg(rows + (size_t)j * r) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 16; ++u) {
              const int j = j0 + u * groups;
              if (j < r) acc = fmaf(m[u], cur[j], acc);
            }
          }
        } else {
          for (int j = grp; j < r; j += groups) {
            float m = 0.f;
            for (int w = 0; w < world; ++w) m += __ldcg(rows_ptrs[w] + row_base + (size_t)j * r + a);
            acc = fmaf(m, cur[j], acc);
          }
        }
      }
      part[grp * r + a] = acc;
    }
    __syncthreads();
    if (threadIdx.x < r) {
      float acc = 0.f;
      for (int q = 0; q < groups; ++q) acc += part[q * r + threadIdx.x];
      nxt[threadIdx.x] = acc;
      g_b[(size_t)k * r + threadIdx.x] = acc;
    }
    __syncthreads();
    float* t = cur;
    cur = nxt;
    nxt = t;
  }
}

// Publish: copy segments of two local buffers (Jacobian rows, offsets) into the same place of every rank's symmetric buffer by
// peer stores, then raise this rank's flag on every peer.  Each (region, block of basis directions) was produced by exactly
// one rank, so after all ranks have published, every rank holds the complete set and scans it from local memory: no rank
// reads a matrix over NVLink more than once and nothing is summed.  segs[i] = (offset, length) in floats, multiples of 4.
// grid (chunks, n_seg_a + n_seg_b).  The flags go out from the last CTA to finish (ticket counter), after a system fence.
__global__ void __launch_bounds__(256) publish_segments_kernel(const float* __restrict__ src_a, float* const* dst_a,
                                                               const int64_t* __restrict__ segs_a, int n_a,
                                                               const float* __restrict__ src_b, float* const* dst_b,
                                                               const int64_t* __restrict__ segs_b, uint32_t* const* flag_ptrs,
                                                               int rank, int world, int slot_base, uint32_t seq,
                                                               uint32_t* done_counter) {
  const int sidx = blockIdx.y;
  const bool first = sidx < n_a;
  const float* src = first ? src_a : src_b;
  float* const* dst = first ? dst_a : dst_b;
  const int64_t* seg = first ? segs_a + 2 * sidx : segs_b + 2 * (sidx - n_a);
  const int64_t off = seg[0], nvec = seg[1] >> 2;
  const float4* s4 = reinterpret_cast<const float4*>(src + off);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    const float4 v = s4[i];
    for (int w = 0; w < world; ++w) reinterpret_cast<float4*>(dst[w] + off)[i] = v;
  }
  __threadfence_system();
  __syncthreads();
  __shared__ uint32_t ticket;
  if (threadIdx.x == 0) ticket = atomicAdd(done_counter, 1u);
  __syncthreads();
  if (ticket == gridDim.x * gridDim.y - 1) {
    if (threadIdx.x == 0) *done_counter = 0;
    __threadfence_system();
    if (threadIdx.x < world) st_release_sys(flag_ptrs[threadIdx.x] + slot_base + rank, seq);
  }
}

// ------------------------------------------------------------------------------------------------ gradient path
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}

__global__ void grad_reduce_scatter_kernel(float* const* grad_ptrs, const float* mc_grads, int rank, int world, int64_t lo,
                                           int64_t n, float* sumsq) {
  __shared__ float scratch[33];
  float acc = 0.f;
  const int64_t nvec = n >> 2;
  float4* mine = reinterpret_cast<float4*>(grad_ptrs[rank] + lo);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    float4 s;
    if (mc_grads) {
      s = multimem_ld_reduce_f32x4(mc_grads + lo + 4 * i);
    } else {
      s = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int w = 0; w < world; ++w) {
        const float4 v = __ldcv(reinterpret_cast<const float4*>(grad_ptrs[w] + lo) + i);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
    }
    mine[i] = s;
    acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  const float total = block_sum(acc, scratch);
  if (threadIdx.x == 0) atomicAdd(sumsq, total);
}

__global__ void exchange_scalar_kernel(float* const* val_ptrs, uint32_t* const* flag_ptrs, const float* mine, int rank,
                                       int world, int slot_base, uint32_t seq, int* status) {
  const int t = threadIdx.x;
  if (t < world) {
    val_ptrs[t][rank] = *mine;
    __threadfence_system();
    st_release_sys(flag_ptrs[t] + slot_base + rank, seq);
    wait_flag(flag_ptrs[rank] + slot_base + t, seq, status, 44);
  }
}

__global__ void adamw_allgather_kernel(float* __restrict__ param, const float* __restrict__ grad, float* __restrict__ m,
                                       float* __restrict__ v, __nv_bfloat16* const* shadow_ptrs, int world, int64_t lo,
                                       int64_t n, float lr, float beta1, float beta2, float eps, float weight_decay,
                                       float bias1, float bias2_sqrt, const float* __restrict__ sumsq_parts,
                                       float clip_norm) {
  float mul = 1.f;
  if (clip_norm > 0.f) {
    float total = 0.f;
    for (int w = 0; w < world; ++w) total += __ldcv(sumsq_parts + w);
    mul = fminf(1.f, clip_norm / (sqrtf(total) + 1e-6f));
  }
  const int64_t npair = n >> 1;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < npair; i += (int64_t)gridDim.x * blockDim.x) {
    float out[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int64_t idx = 2 * i + e;
      const float g = grad[idx] * mul;
      float p = param[idx] * (1.f - lr * weight_decay);
      const float mi = beta1 * m[idx] + (1.f - beta1) * g;
      const float vi = beta2 * v[idx] + (1.f - beta2) * g * g;
      m[idx] = mi;
      v[idx] = vi;
      p -= (lr / bias1) * mi / (sqrtf(vi) / bias2_sqrt + eps);
      param[idx] = p;
      out[e] = p;
    }
    const __nv_bfloat162 packed = __floats2bfloat162_rn(out[0], out[1]);
    for (int w = 0; w < world; ++w) reinterpret_cast<__nv_bfloat162*>(shadow_ptrs[w] + lo)[i] = packed;  // all-gather by peer stores
  }
}

}  // namespace peer
}  // namespace lbi

using namespace lbi::peer;

extern "C" {

int lbi_peer_set_wait_limit_ms(int ms) {
  if (ms < 1) return (int)cudaErrorInvalidValue;
  const unsigned long long ns = (unsigned long long)ms * 1000000ull;
  return (int)cudaMemcpyToSymbol(g_wait_limit_ns, &ns, sizeof(ns));
}

int lbi_peer_barrier(uint32_t* const* flag_ptrs, int rank, int world, int slot_base, uint32_t seq, int* status,
                     cudaStream_t st) {
  barrier_kernel<<<1, 32, 0, st>>>(flag_ptrs, rank, world, slot_base, seq, status);
  return (int)cudaGetLastError();
}

int lbi_peer_signal_all(uint32_t* const* flag_ptrs, int rank, int world, int slot_base, uint32_t seq, cudaStream_t st) {
  signal_all_kernel<<<1, 32, 0, st>>>(flag_ptrs, rank, world, slot_base, seq);
  return (int)cudaGetLastError();
}

int lbi_interface_update_handoff(const float* state_in, const float* pooled, const float* w1, const float* b1,
                                 const float* w2, const float* b2, const float* alpha, const float* ln_w,
                                 const float* ln_b, float ln_eps, int act, int batch, int dim, int hidden, int width,
                                 float* hidden_buf, float* delta_out, float* pre_out, float* state_out, float* peer_state,
                                 uint32_t* peer_flag, uint32_t seq, uint32_t* done_counter, cudaStream_t st) {
  if (batch <= 0) return 0;
  if (hidden > 0 && hidden_buf && batch <= WIDE_MAXB) {
    const size_t wide = ((size_t)batch * (dim > hidden ? dim : hidden) + (size_t)batch * width) * sizeof(float);
    if (wide <= 200 * 1024) {
      static lbi::PerDeviceOnce configured_wide;
      cudaError_t e = configured_wide.max_dynamic_smem(interface_update_handoff_wide_kernel, (int)(200 * 1024));
      if (e != cudaSuccess) return (int)e;
      interface_update_handoff_wide_kernel<<<(hidden + 7) / 8, 256, wide, st>>>(
          state_in, pooled, w1, b1, w2, b2, alpha, ln_w, ln_b, ln_eps, act, batch, dim, hidden, width, hidden_buf, delta_out,
          pre_out, state_out, peer_state, peer_flag, seq, done_counter);
      return (int)cudaGetLastError();
    }
  }
  const size_t smem = (size_t)(dim + (hidden > 0 ? hidden : 1) + width) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(interface_update_handoff_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  interface_update_handoff_kernel<<<batch, 256, smem, st>>>(state_in, pooled, w1, b1, w2, b2, alpha, ln_w, ln_b, ln_eps, act,
                                                            dim, hidden, width, delta_out, pre_out, state_out, peer_state,
                                                            peer_flag, seq, done_counter);
  return (int)cudaGetLastError();
}

int lbi_wait_state(const float* mailbox, const uint32_t* flag, uint32_t seq, float* out, int n, int* status,
                   cudaStream_t st) {
  wait_state_kernel<<<1, 256, 0, st>>>(mailbox, flag, seq, out, n, status);
  return (int)cudaGetLastError();
}

int lbi_affine_scan_peer(const float* const* mats_ptrs, const float* const* offs_ptrs, const uint32_t* flags,
                         int slot_base, uint32_t seq, float* g, int batch, int world, int k_local, int r, int* status,
                         cudaStream_t st) {
  if (batch <= 0) return 0;
  affine_scan_peer_kernel<<<batch, 256, 2 * r * sizeof(float), st>>>(mats_ptrs, offs_ptrs, flags, slot_base, seq, g, world,
                                                                     k_local, r, status);
  return (int)cudaGetLastError();
}

int lbi_peer_publish(const float* src_a, float* const* dst_a, const int64_t* segs_a, int n_a, const float* src_b,
                     float* const* dst_b, const int64_t* segs_b, int n_b, uint32_t* const* flag_ptrs, int rank, int world,
                     int slot_base, uint32_t seq, uint32_t* done_counter, cudaStream_t st) {
  if (n_a < 0 || n_b < 0 || n_a + n_b <= 0 || world <= 0 || world > 256) return (int)cudaErrorInvalidValue;
  publish_segments_kernel<<<dim3(8, n_a + n_b), 256, 0, st>>>(src_a, dst_a, segs_a, n_a, src_b, dst_b, segs_b, flag_ptrs, rank, world,
                                                              slot_base, seq, done_counter);
  return (int)cudaGetLastError();
}

int lbi_affine_scan_peer_sum(const float* const* rows_ptrs, const float* const* offs_ptrs, const uint32_t* flags, int slot_base,
                             uint32_t seq, float* g, int batch, int world, int k_total, int r, int flag_world, int* status,
                             cudaStream_t st) {
  if (batch <= 0) return 0;
  if (r <= 0 || r > 1024 || flag_world < world || flag_world > 1024) return (int)cudaErrorInvalidValue;
  const int threads = 1024 / r * r >= 32 ? (1024 / r) * r : r;   // a whole number of groups of r threads
  const int groups = threads / r;
  affine_scan_peer_sum_kernel<<<batch, threads, (size_t)(2 + groups) * r * sizeof(float), st>>>(rows_ptrs, offs_ptrs, flags, slot_base,
                                                                                                seq, g, world, batch, k_total, r, status,
                                                                                                flag_world);
  return (int)cudaGetLastError();
}

int lbi_grad_reduce_scatter(float* const* grad_ptrs, const float* mc_grads, int rank, int world, int64_t lo, int64_t n,
                            float* sumsq, cudaStream_t st) {
  if (n <= 0) return 0;
  if ((n & 3) != 0 || (lo & 3) != 0) return (int)cudaErrorInvalidValue;
  int blocks = (int)(((n >> 2) + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  grad_reduce_scatter_kernel<<<blocks, 256, 0, st>>>(grad_ptrs, mc_grads, rank, world, lo, n, sumsq);
  return (int)cudaGetLastError();
}

int lbi_exchange_scalar(float* const* val_ptrs, uint32_t* const* flag_ptrs, const float* mine, int rank, int world,
                        int slot_base, uint32_t seq, int* status, cudaStream_t st) {
  exchange_scalar_kernel<<<1, 32, 0, st>>>(val_ptrs, flag_ptrs, mine, rank, world, slot_base, seq, status);
  return (int)cudaGetLastError();
}

int lbi_adamw_allgather(float* param, const float* reduced_grad, float* exp_avg, float* exp_avg_sq,
                        void* const* shadow_ptrs, int world, int64_t lo, int64_t n, float lr, float beta1, float beta2,
                        float eps, float weight_decay, int step, const float* sumsq_parts, float clip_norm,
                        cudaStream_t st) {
  if (n <= 0) return 0;
  if ((n & 1) != 0 || (lo & 1) != 0) return (int)cudaErrorInvalidValue;
  int blocks = (int)(((n >> 1) + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  const float bias1 = 1.f - powf(beta1, (float)step);
  const float bias2_sqrt = sqrtf(1.f - powf(beta2, (float)step));
  adamw_allgather_kernel<<<blocks, 256, 0, st>>>(param, reduced_grad, exp_avg, exp_avg_sq,
                                                 (__nv_bfloat16* const*)shadow_ptrs, world, lo, n, lr, beta1, beta2, eps,
                                                 weight_decay, bias1, bias2_sqrt, sumsq_parts, clip_norm);
  return (int)cudaGetLastError();
}

}  // extern "C"
