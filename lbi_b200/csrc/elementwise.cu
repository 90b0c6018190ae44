// Fused memory-bound kernels: RMSNorm (+ residual add) forward / input pullback / weight gradient, RoPE on packed
// qkv, SwiGLU forward / pullback, interface glue (condition add, token pooling), embedding gather / scatter-add,
// bf16 transpose, depthwise causal conv, gradient norm, AdamW, softmax cross-entropy on logits.
//
// All of them are bandwidth-bound: 16-byte vector accesses, one pass over HBM where the row fits a block, fp32 math.
// Cotangent tensors may carry a leading basis factor: their rows are laid out basis-major (P * n rows) and cached
// activations are read at row % n, so one set of activations serves every basis direction.
#include "api.h"
#include "common.cuh"

namespace lbi {

// ------------------------------------------------------------------------------------------------ RMSNorm fwd
template <int THREADS>
__global__ void __launch_bounds__(THREADS) add_rmsnorm_fwd_kernel(const bf16x8* __restrict__ branch,
                                                                   const float4* __restrict__ stream,
                                                                   const float4* __restrict__ weight,
                                                                   bf16x8* __restrict__ normed,
                                                                   float4* __restrict__ new_stream,
                                                                   float* __restrict__ rstd_out, int dim, float eps) {
  __shared__ float scratch[33];
  const int64_t row = blockIdx.x;
  const int nvec = dim >> 3;
  const bf16x8* b = branch + row * nvec;
  const float4* s = stream ? stream + row * nvec * 2 : nullptr;
  float4* ns = new_stream + row * nvec * 2;
  float acc = 0.f;
  for (int i = threadIdx.x; i < nvec; i += THREADS) {
    float v[8];
    unpack8(b[i], v);
    if (s) {
      float4 s0 = s[2 * i], s1 = s[2 * i + 1];
      v[0] += s0.x; v[1] += s0.y; v[2] += s0.z; v[3] += s0.w;
      v[4] += s1.x; v[5] += s1.y; v[6] += s1.z; v[7] += s1.w;
    }
    ns[2 * i] = make_float4(v[0], v[1], v[2], v[3]);
    ns[2 * i + 1] = make_float4(v[4], v[5], v[6], v[7]);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += v[j] * v[j];
  }
  const float total = block_sum(acc, scratch);
  const float r = rsqrtf(total / (float)dim + eps);
  if (threadIdx.x == 0) rstd_out[row] = r;
  bf16x8* o = normed + row * nvec;
  for (int i = threadIdx.x; i < nvec; i += THREADS) {
    // same thread wrote these addresses above, so the reads see its own stores
    float4 a0 = ns[2 * i], a1 = ns[2 * i + 1];
    float4 w0 = weight[2 * i], w1 = weight[2 * i + 1];
    float v[8] = {a0.x * r * w0.x, a0.y * r * w0.y, a0.z * r * w0.z, a0.w * r * w0.w,
                  a1.x * r * w1.x, a1.y * r * w1.y, a1.z * r * w1.z, a1.w * r * w1.w};
    o[i] = pack8(v);
  }
}

// ------------------------------------------------------------------------------------------------ RMSNorm bwd (dx)
// One CTA per activation row; it walks all cotangent rows that share the row (row = p * act_rows + arow), so the
// normalised activations and the weight are staged once in shared memory (2 * dim floats) instead of being re-read per
// direction, and each thread keeps its part of the cotangent in registers between the two passes (dim <= 8 * 4 * THREADS).
template <int THREADS>
__global__ void __launch_bounds__(THREADS) rmsnorm_bwd_kernel(const bf16x8* __restrict__ d_normed,
                                                               const float4* __restrict__ x_stream,
                                                               const float* __restrict__ rstd,
                                                               const float4* __restrict__ weight,
                                                               const float4* d_stream_in, float4* d_stream_out,
                                                               bf16x8* lowp_out, int64_t rows, int64_t act_rows, int dim) {
  extern __shared__ float4 sm4[];
  __shared__ float scratch[33];
  const int64_t arow = blockIdx.x;
  const int nvec = dim >> 3;
  float4* xh = sm4;             // xhat = x * rstd, 2 float4 per vector
  float4* wv = sm4 + 2 * nvec;  // weight
  const float r = rstd[arow];
  for (int i = threadIdx.x; i < 2 * nvec; i += THREADS) {
    float4 v = x_stream[arow * nvec * 2 + i];
    v.x *= r; v.y *= r; v.z *= r; v.w *= r;
    xh[i] = v;
    wv[i] = weight[i];
  }
  __syncthreads();
  const int reps = (int)(rows / act_rows);
  constexpr int MAXV = 4;   // vectors of 8 elements per thread kept in registers
  for (int p = 0; p < reps; ++p) {
    const int64_t row = (int64_t)p * act_rows + arow;
    const bf16x8* g = d_normed + row * nvec;
    float gw[MAXV][8];
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int i = threadIdx.x + k * THREADS;
      if (i < nvec) {
        float gv[8];
        unpack8(g[i], gv);
        const float4 w0 = wv[2 * i], w1 = wv[2 * i + 1], x0 = xh[2 * i], x1 = xh[2 * i + 1];
        gw[k][0] = gv[0] * w0.x; gw[k][1] = gv[1] * w0.y; gw[k][2] = gv[2] * w0.z; gw[k][3] = gv[3] * w0.w;
        gw[k][4] = gv[4] * w1.x; gw[k][5] = gv[5] * w1.y; gw[k][6] = gv[6] * w1.z; gw[k][7] = gv[7] * w1.w;
        dot += gw[k][0] * x0.x + gw[k][1] * x0.y + gw[k][2] * x0.z + gw[k][3] * x0.w + gw[k][4] * x1.x + gw[k][5] * x1.y +
               gw[k][6] * x1.z + gw[k][7] * x1.w;
      }
    }
    // c = mean over the row of (g * w) * xhat
    const float c = block_sum(dot, scratch) / (float)dim;
    const float4* din = d_stream_in ? d_stream_in + row * nvec * 2 : nullptr;
    float4* dout = d_stream_out + row * nvec * 2;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int i = threadIdx.x + k * THREADS;
      if (i < nvec) {
        const float4 x0 = xh[2 * i], x1 = xh[2 * i + 1];
        float4 o0, o1;
        o0.x = r * (gw[k][0] - x0.x * c);
        o0.y = r * (gw[k][1] - x0.y * c);
        o0.z = r * (gw[k][2] - x0.z * c);
        o0.w = r * (gw[k][3] - x0.w * c);
        o1.x = r * (gw[k][4] - x1.x * c);
        o1.y = r * (gw[k][5] - x1.y * c);
        o1.z = r * (gw[k][6] - x1.z * c);
        o1.w = r * (gw[k][7] - x1.w * c);
        if (din) {
          const float4 p0 = din[2 * i], p1 = din[2 * i + 1];
          o0.x += p0.x; o0.y += p0.y; o0.z += p0.z; o0.w += p0.w;
          o1.x += p1.x; o1.y += p1.y; o1.z += p1.z; o1.w += p1.w;
        }
        dout[2 * i] = o0;
        dout[2 * i + 1] = o1;
        if (lowp_out) {  // the bf16 copy the next GEMM reads, written here instead of by a separate cast pass
          const float ov[8] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w};
          lowp_out[row * nvec + i] = pack8(ov);
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ RMSNorm wgrad
// Stage 1: block b sums its slab of rows for every column into partials[b, :]; stage 2 sums the partials.
__global__ void rmsnorm_wgrad_stage1(const __nv_bfloat16* __restrict__ d_normed, const float* __restrict__ x,
                                     const float* __restrict__ rstd, float* __restrict__ partials, int64_t rows,
                                     int dim) {
  const int64_t per = (rows + gridDim.x - 1) / gridDim.x;
  const int64_t r0 = per * blockIdx.x;
  const int64_t r1 = r0 + per < rows ? r0 + per : rows;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    float acc = 0.f;
    for (int64_t r = r0; r < r1; ++r) acc += __bfloat162float(d_normed[r * dim + d]) * x[r * dim + d] * rstd[r];
    partials[(int64_t)blockIdx.x * dim + d] = acc;
  }
}

__global__ void column_sum_kernel(const float* __restrict__ partials, float* __restrict__ out, int nblocks, int dim) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= dim) return;
  float acc = 0.f;
  for (int b = 0; b < nblocks; ++b) acc += partials[(int64_t)b * dim + d];
  out[d] = acc;
}

// ------------------------------------------------------------------------------------------------ RoPE
// One thread rotates 8 pairs.  Half-split layout pairs element i with i + Dh/2; interleaved pairs (2i, 2i+1).
__global__ void rope_qkv_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ cos_tab,
                                const float* __restrict__ sin_tab, int64_t rows, int n_rot_heads, int qkv_dim,
                                int head_dim, int seq_len, int interleaved, float sin_sign) {
  const int half = head_dim >> 1;
  const int groups_per_head = half >> 3;  // groups of 8 pairs
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = rows * n_rot_heads * groups_per_head;
  if (idx >= total) return;
  const int grp = (int)(idx % groups_per_head);
  const int head = (int)((idx / groups_per_head) % n_rot_heads);
  const int64_t row = idx / ((int64_t)groups_per_head * n_rot_heads);
  const int pos = (int)(row % seq_len);
  const float* c = cos_tab + (int64_t)pos * half + grp * 8;
  const float* s = sin_tab + (int64_t)pos * half + grp * 8;
  __nv_bfloat16* base = qkv + row * qkv_dim + (int64_t)head * head_dim;
  if (!interleaved) {
    bf16x8* pa = reinterpret_cast<bf16x8*>(base + grp * 8);
    bf16x8* pb = reinterpret_cast<bf16x8*>(base + half + grp * 8);
    float a[8], b[8], oa[8], ob[8];
    unpack8(*pa, a);
    unpack8(*pb, b);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float ci = c[i], si = s[i] * sin_sign;
      oa[i] = a[i] * ci - b[i] * si;
      ob[i] = a[i] * si + b[i] * ci;
    }
    *pa = pack8(oa);
    *pb = pack8(ob);
  } else {
    bf16x8* p0 = reinterpret_cast<bf16x8*>(base + grp * 16);
    bf16x8* p1 = p0 + 1;
    float v0[8], v1[8];
    unpack8(*p0, v0);
    unpack8(*p1, v1);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float ci = c[i], si = s[i] * sin_sign;
      float a = v0[2 * i], b = v0[2 * i + 1];
      v0[2 * i] = a * ci - b * si;
      v0[2 * i + 1] = a * si + b * ci;
      ci = c[4 + i];
      si = s[4 + i] * sin_sign;
      a = v1[2 * i];
      b = v1[2 * i + 1];
      v1[2 * i] = a * ci - b * si;
      v1[2 * i + 1] = a * si + b * ci;
    }
    *p0 = pack8(v0);
    *p1 = pack8(v1);
  }
}

// ------------------------------------------------------------------------------------------------ SwiGLU
__global__ void swiglu_fwd_kernel(const bf16x8* __restrict__ u, bf16x8* __restrict__ a, int64_t rows, int hvec) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * hvec) return;
  const int64_t row = idx / hvec;
  const int col = (int)(idx % hvec);
  float up[8], gate[8], o[8];
  unpack8(u[row * 2 * hvec + col], up);
  unpack8(u[row * 2 * hvec + hvec + col], gate);
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = up[i] * gate[i] * sigmoidf_(gate[i]);
  a[idx] = pack8(o);
}

// One thread owns 8 columns of one activation row and walks all cotangent rows that share it (row = p * act_rows +
// arow): the activations are read once and the two derivative factors computed once, instead of once per direction
// (with 16 directions the 92 MB activation matrix was otherwise re-read from DRAM 16 times: it does not stay in L2).
__global__ void swiglu_bwd_kernel(const bf16x8* __restrict__ da, const bf16x8* __restrict__ u, bf16x8* __restrict__ du,
                                  int64_t rows, int64_t act_rows, int hvec) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= act_rows * hvec) return;
  const int64_t arow = idx / hvec;
  const int col = (int)(idx % hvec);
  float up[8], gate[8], f_up[8], f_gate[8];
  unpack8(u[arow * 2 * hvec + col], up);
  unpack8(u[arow * 2 * hvec + hvec + col], gate);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float sg = sigmoidf_(gate[i]);
    f_up[i] = gate[i] * sg;
    f_gate[i] = up[i] * sg * (1.f + gate[i] * (1.f - sg));
  }
  const int reps = (int)(rows / act_rows);
#pragma unroll 4
  for (int p = 0; p < reps; ++p) {
    const int64_t row = (int64_t)p * act_rows + arow;
    float g[8], dup[8], dgate[8];
    unpack8(da[row * hvec + col], g);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      dup[i] = g[i] * f_up[i];
      dgate[i] = g[i] * f_gate[i];
    }
    du[row * 2 * hvec + col] = pack8(dup);
    du[row * 2 * hvec + hvec + col] = pack8(dgate);
  }
}

// ------------------------------------------------------------------------------------------------ interface glue
__global__ void add_condition_kernel(const bf16x8* __restrict__ canvas, const float4* __restrict__ cond,
                                     bf16x8* __restrict__ out, int64_t rows, int nvec, int seq_len) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * nvec) return;
  const int64_t row = idx / nvec;
  const int col = (int)(idx % nvec);
  const int64_t b = row / seq_len;
  float v[8];
  unpack8(canvas[idx], v);
  const float4 c0 = cond[(b * nvec + col) * 2], c1 = cond[(b * nvec + col) * 2 + 1];
  v[0] += c0.x; v[1] += c0.y; v[2] += c0.z; v[3] += c0.w;
  v[4] += c1.x; v[5] += c1.y; v[6] += c1.z; v[7] += c1.w;
  out[idx] = pack8(v);
}

// grid (groups, ceil(dim / blockDim.x), tsplit): each block sums a slice of the tokens of one group.
template <typename T>
__global__ void pool_tokens_kernel(const T* __restrict__ rows, float* __restrict__ out, int seq_len, int dim,
                                   float scale) {
  const int d = blockIdx.y * blockDim.x + threadIdx.x;
  if (d >= dim) return;
  const int64_t g = blockIdx.x;
  const int per = (seq_len + gridDim.z - 1) / gridDim.z;
  const int t0 = per * blockIdx.z;
  const int t1 = t0 + per < seq_len ? t0 + per : seq_len;
  const T* p = rows + (g * seq_len + t0) * (int64_t)dim + d;
  float acc = 0.f;
  for (int t = t0; t < t1; ++t, p += dim) acc += (float)(*p);
  atomicAdd(out + g * dim + d, acc * scale);
}

// ------------------------------------------------------------------------------------------------ embedding
template <typename T>
__global__ void embedding_fwd_kernel(const int64_t* __restrict__ ids, const T* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, int64_t rows, int dim, int64_t vocab, int* status) {
  // a token id outside [0, vocab) is recorded in the status word (site 81) and its row is written as zeros: bad data must
  // not become an illegal address
  const int64_t row = blockIdx.x;
  const int64_t id = ids[row];
  __nv_bfloat16* dst = out + row * dim;
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, 81);
    for (int d = threadIdx.x; d < dim; d += blockDim.x) dst[d] = __float2bfloat16(0.f);
    return;
  }
  const T* src = table + id * (int64_t)dim;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) dst[d] = __float2bfloat16((float)src[d]);
}

template <typename T>
__global__ void embedding_scatter_add_kernel(float* __restrict__ d_table, const int64_t* __restrict__ ids,
                                             const T* __restrict__ d_rows, int64_t rows, int dim, int64_t vocab, int* status) {
  const int64_t row = blockIdx.x;
  const int64_t id = ids[row];
  if (id < 0 || id >= vocab) {   // recorded (site 82) and skipped
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, 82);
    return;
  }
  float* dst = d_table + id * (int64_t)dim;
  const T* src = d_rows + row * dim;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) atomicAdd(dst + d, (float)src[d]);
}

// ------------------------------------------------------------------------------------------------ transpose
__global__ void transpose_bf16_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                      int64_t rows, int64_t cols) {
  __shared__ __nv_bfloat16 tile[64][66];
  const int64_t c0 = (int64_t)blockIdx.x * 64, r0 = (int64_t)blockIdx.y * 64;
  for (int i = threadIdx.y; i < 64; i += blockDim.y) {
    const int64_t r = r0 + i;
    for (int j = threadIdx.x; j < 64; j += blockDim.x) {
      const int64_t c = c0 + j;
      if (r < rows && c < cols) tile[i][j] = in[r * cols + c];
    }
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 64; i += blockDim.y) {
    const int64_t c = c0 + i;
    for (int j = threadIdx.x; j < 64; j += blockDim.x) {
      const int64_t r = r0 + j;
      if (r < rows && c < cols) out[c * rows + r] = tile[j][i];
    }
  }
}

// ------------------------------------------------------------------------------------------------ grouped kv heads
// Grouped-query attention on kernels that take one k / v head per q head: expand copies kv head h / group for q head h
// (packed rows [q | k | v] with H, Hkv, Hkv heads -> H, H, H heads); reduce sums the cotangents of the group's copies back
// (and copies the q part through).  16-byte pieces, head_dim a multiple of 8.
__global__ void gqa_expand_kernel(const bf16x8* __restrict__ in, bf16x8* __restrict__ out, int64_t rows, int heads, int kv_heads,
                                  int dvec) {
  const int group = heads / kv_heads;
  const int out_w = 3 * heads * dvec, in_w = (heads + 2 * kv_heads) * dvec;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < rows * out_w; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / out_w;
    const int c = (int)(i - row * out_w);
    const int part = c / (heads * dvec), within = c - part * heads * dvec;
    const int h = within / dvec, d = within - h * dvec;
    const int src = part == 0 ? within : heads * dvec + (part - 1) * kv_heads * dvec + (h / group) * dvec + d;
    out[i] = in[row * in_w + src];
  }
}

__global__ void gqa_reduce_kernel(const bf16x8* __restrict__ in, bf16x8* __restrict__ out, int64_t rows, int heads, int kv_heads,
                                  int dvec) {
  const int group = heads / kv_heads;
  const int in_w = 3 * heads * dvec, out_w = (heads + 2 * kv_heads) * dvec;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < rows * out_w; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / out_w;
    const int c = (int)(i - row * out_w);
    if (c < heads * dvec) {
      out[i] = in[row * in_w + c];
      continue;
    }
    const int rest = c - heads * dvec;
    const int part = rest / (kv_heads * dvec), within = rest - part * kv_heads * dvec;
    const int kh = within / dvec, d = within - kh * dvec;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int g = 0; g < group; ++g) {
      float v[8];
      unpack8(in[row * in_w + (1 + part) * heads * dvec + (kh * group + g) * dvec + d], v);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += v[e];
    }
    out[i] = pack8(acc);
  }
}

// ------------------------------------------------------------------------------------------------ causal conv
// y[s, t, c] = bias[c] + sum_w w[c, w] * x[s, t - (W-1) + w, c]
__global__ void causal_conv_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                       const float* __restrict__ bias, __nv_bfloat16* __restrict__ y, int64_t seqs,
                                       int seq_len, int channels, int width) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = seqs * seq_len * channels;
  if (idx >= total) return;
  const int c = (int)(idx % channels);
  const int t = (int)((idx / channels) % seq_len);
  float acc = bias ? bias[c] : 0.f;
  for (int k = 0; k < width; ++k) {
    const int tt = t - (width - 1) + k;
    if (tt >= 0 && LBI_IN_RANGE(idx + (int64_t)(tt - t) * channels, total, 95))
      acc += w[c * width + k] * __bfloat162float(x[idx + (int64_t)(tt - t) * channels]);
  }
  y[idx] = __float2bfloat16(acc);
}

// dx[s, t, c] = sum_w w[c, w] * dy[s, t + (W-1) - w, c]
__global__ void causal_conv_dgrad_kernel(const __nv_bfloat16* __restrict__ dy, const float* __restrict__ w,
                                         __nv_bfloat16* __restrict__ dx, int64_t seqs, int seq_len, int channels,
                                         int width) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = seqs * seq_len * channels;
  if (idx >= total) return;
  const int c = (int)(idx % channels);
  const int t = (int)((idx / channels) % seq_len);
  float acc = 0.f;
  for (int k = 0; k < width; ++k) {
    const int tt = t + (width - 1) - k;
    if (tt < seq_len && LBI_IN_RANGE(idx + (int64_t)(tt - t) * channels, total, 96))
      acc += w[c * width + k] * __bfloat162float(dy[idx + (int64_t)(tt - t) * channels]);
  }
  dx[idx] = __float2bfloat16(acc);
}

// ------------------------------------------------------------------------------------------------ optimizer
__global__ void sumsq_kernel(const float* __restrict__ x, int64_t n, float* __restrict__ out) {
  __shared__ float scratch[33];
  float acc = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = x[i];
    acc += v * v;
  }
  const float total = block_sum(acc, scratch);
  if (threadIdx.x == 0) atomicAdd(out, total);
}

__global__ void adamw_kernel(float* __restrict__ param, const float* __restrict__ grad, float* __restrict__ m,
                             float* __restrict__ v, __nv_bfloat16* __restrict__ shadow, int64_t n, float lr, float beta1,
                             float beta2, float eps, float weight_decay, float bias1, float bias2_sqrt, float grad_mul,
                             const float* __restrict__ sumsq, float clip_norm) {
  float mul = grad_mul;
  if (sumsq != nullptr && clip_norm > 0.f) {
    const float norm = sqrtf(*sumsq) * fabsf(grad_mul);
    mul *= fminf(1.f, clip_norm / (norm + 1e-6f));
  }
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float g = grad[i] * mul;
    float p = param[i] * (1.f - lr * weight_decay);
    const float mi = beta1 * m[i] + (1.f - beta1) * g;
    const float vi = beta2 * v[i] + (1.f - beta2) * g * g;
    m[i] = mi;
    v[i] = vi;
    p -= (lr / bias1) * mi / (sqrtf(vi) / bias2_sqrt + eps);
    param[i] = p;
    if (shadow) shadow[i] = __float2bfloat16(p);
  }
}

// ------------------------------------------------------------------------------------------------ cross-entropy
// One block per row of bf16 logits: online max / sum-exp, loss accumulation, then in-place gradient.
template <int THREADS>
__global__ void __launch_bounds__(THREADS) ce_fwd_bwd_kernel(bf16x8* __restrict__ logits,
                                                              const int64_t* __restrict__ targets,
                                                              float* __restrict__ loss_sum, int vocab, float scale) {
  __shared__ float scratch[33];
  const int64_t row = blockIdx.x;
  const int nvec = vocab >> 3;
  bf16x8* l = logits + row * nvec;
  const int64_t target = targets[row];
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < nvec; i += THREADS) {
    float v[8];
    unpack8(l[i], v);
#pragma unroll
    for (int j = 0; j < 8; ++j) mx = fmaxf(mx, v[j]);
  }
  mx = block_max(mx, scratch);
  float se = 0.f;
  for (int i = threadIdx.x; i < nvec; i += THREADS) {
    float v[8];
    unpack8(l[i], v);
#pragma unroll
    for (int j = 0; j < 8; ++j) se += __expf(v[j] - mx);
  }
  se = block_sum(se, scratch);
  const float lse = mx + __logf(se);
  const bool valid = target >= 0 && target < vocab;
  if (threadIdx.x == 0 && valid) {
    const float picked = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(l)[target]);
    atomicAdd(loss_sum, scale * (lse - picked));
  }
  const float gscale = valid ? scale : 0.f;
  for (int i = threadIdx.x; i < nvec; i += THREADS) {
    float v[8];
    unpack8(l[i], v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p = __expf(v[j] - lse);
      if ((int64_t)(i * 8 + j) == target) p -= 1.f;
      v[j] = p * gscale;
    }
    l[i] = pack8(v);
  }
}

inline int launch_status() { return (int)cudaGetLastError(); }

}  // namespace lbi

using namespace lbi;

extern "C" {

int lbi_add_rmsnorm_fwd(const void* branch, const float* stream_in, const float* weight, void* normed, float* new_stream,
                        float* rstd, int64_t rows, int dim, float eps, cudaStream_t st) {
  if (rows == 0) return 0;
  add_rmsnorm_fwd_kernel<128><<<(unsigned)rows, 128, 0, st>>>(
      (const bf16x8*)branch, (const float4*)stream_in, (const float4*)weight, (bf16x8*)normed, (float4*)new_stream, rstd,
      dim, eps);
  return launch_status();
}

int lbi_rmsnorm_bwd(const void* d_normed, const float* x_stream, const float* rstd, const float* weight,
                    const float* d_in, float* d_out, void* d_out_lowp, int64_t rows, int64_t act_rows, int dim,
                    cudaStream_t st) {
  if (rows == 0) return 0;
  if (act_rows <= 0 || rows % act_rows != 0 || dim % 8 != 0 || dim > 8 * 4 * 256) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)dim * 2 * sizeof(float);
  if (dim <= 8 * 4 * 128) {
    rmsnorm_bwd_kernel<128><<<(unsigned)act_rows, 128, smem, st>>>((const bf16x8*)d_normed, (const float4*)x_stream, rstd,
                                                                   (const float4*)weight, (const float4*)d_in, (float4*)d_out,
                                                                   (bf16x8*)d_out_lowp, rows, act_rows, dim);
  } else {
    static PerDeviceOnce configured;
    {
      cudaError_t e = configured.max_dynamic_smem(rmsnorm_bwd_kernel<256>, 64 * 1024);
      if (e != cudaSuccess) return (int)e;
    }
    rmsnorm_bwd_kernel<256><<<(unsigned)act_rows, 256, smem, st>>>((const bf16x8*)d_normed, (const float4*)x_stream, rstd,
                                                                   (const float4*)weight, (const float4*)d_in, (float4*)d_out,
                                                                   (bf16x8*)d_out_lowp, rows, act_rows, dim);
  }
  return launch_status();
}

int lbi_rmsnorm_wgrad(const void* d_normed, const float* x_stream, const float* rstd, float* partials, float* dw,
                      int64_t rows, int dim, int nblocks, cudaStream_t st) {
  rmsnorm_wgrad_stage1<<<nblocks, 256, 0, st>>>((const __nv_bfloat16*)d_normed, x_stream, rstd, partials, rows, dim);
  column_sum_kernel<<<(dim + 255) / 256, 256, 0, st>>>(partials, dw, nblocks, dim);
  return launch_status();
}

int lbi_rope_qkv(void* qkv, const float* cos_tab, const float* sin_tab, int64_t rows, int n_rot_heads, int qkv_dim,
                 int head_dim, int seq_len, int interleaved, int inverse, cudaStream_t st) {
  const int64_t total = rows * n_rot_heads * (head_dim / 16);
  if (total == 0) return 0;
  rope_qkv_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>((__nv_bfloat16*)qkv, cos_tab, sin_tab, rows,
                                                                   n_rot_heads, qkv_dim, head_dim, seq_len, interleaved,
                                                                   inverse ? -1.f : 1.f);
  return launch_status();
}

int lbi_swiglu_fwd(const void* u, void* a, int64_t rows, int hidden, cudaStream_t st) {
  const int hvec = hidden / 8;
  const int64_t total = rows * hvec;
  if (total == 0) return 0;
  swiglu_fwd_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const bf16x8*)u, (bf16x8*)a, rows, hvec);
  return launch_status();
}

int lbi_swiglu_bwd(const void* da, const void* u, void* du, int64_t rows, int64_t act_rows, int hidden,
                   cudaStream_t st) {
  const int hvec = hidden / 8;
  const int64_t total = act_rows * hvec;
  if (total == 0 || rows == 0) return 0;
  if (rows % act_rows != 0) return (int)cudaErrorInvalidValue;
  swiglu_bwd_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const bf16x8*)da, (const bf16x8*)u, (bf16x8*)du,
                                                                     rows, act_rows, hvec);
  return launch_status();
}

int lbi_add_condition(const void* canvas, const float* cond, void* out, int64_t rows, int dim, int seq_len,
                      cudaStream_t st) {
  const int nvec = dim / 8;
  const int64_t total = rows * nvec;
  if (total == 0) return 0;
  add_condition_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const bf16x8*)canvas, (const float4*)cond,
                                                                        (bf16x8*)out, rows, nvec, seq_len);
  return launch_status();
}

int lbi_pool_tokens(const void* rows, int is_bf16, float* out, int64_t groups, int seq_len, int dim, float scale,
                    cudaStream_t st) {
  if (groups == 0) return 0;
  int tsplit = 1;
  const int64_t base_blocks = groups * ((dim + 255) / 256);
  while (base_blocks * tsplit < 592 && tsplit * 64 < seq_len) tsplit *= 2;
  dim3 grid((unsigned)groups, (dim + 255) / 256, tsplit);
  if (is_bf16)
    pool_tokens_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)rows, out, seq_len, dim, scale);
  else
    pool_tokens_kernel<float><<<grid, 256, 0, st>>>((const float*)rows, out, seq_len, dim, scale);
  return launch_status();
}

int lbi_embedding_fwd(const int64_t* ids, const void* table, int table_is_bf16, void* out, int64_t rows, int dim,
                      int64_t vocab, int* status, cudaStream_t st) {
  if (rows == 0) return 0;
  if (table_is_bf16)
    embedding_fwd_kernel<__nv_bfloat16><<<(unsigned)rows, 128, 0, st>>>(ids, (const __nv_bfloat16*)table,
                                                                         (__nv_bfloat16*)out, rows, dim, vocab, status);
  else
    embedding_fwd_kernel<float><<<(unsigned)rows, 128, 0, st>>>(ids, (const float*)table, (__nv_bfloat16*)out, rows, dim, vocab, status);
  return launch_status();
}

int lbi_embedding_scatter_add(float* d_table, const int64_t* ids, const void* d_rows, int rows_is_bf16, int64_t rows,
                              int dim, int64_t vocab, int* status, cudaStream_t st) {
  if (rows == 0) return 0;
  if (rows_is_bf16)
    embedding_scatter_add_kernel<__nv_bfloat16><<<(unsigned)rows, 128, 0, st>>>(d_table, ids,
                                                                                 (const __nv_bfloat16*)d_rows, rows, dim, vocab, status);
  else
    embedding_scatter_add_kernel<float><<<(unsigned)rows, 128, 0, st>>>(d_table, ids, (const float*)d_rows, rows, dim, vocab, status);
  return launch_status();
}

int lbi_transpose_bf16(const void* in, void* out, int64_t rows, int64_t cols, cudaStream_t st) {
  if (rows == 0 || cols == 0) return 0;
  dim3 grid((unsigned)((cols + 63) / 64), (unsigned)((rows + 63) / 64));
  transpose_bf16_kernel<<<grid, dim3(32, 8), 0, st>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, rows, cols);
  return launch_status();
}

int lbi_gqa_expand(const void* in, void* out, int64_t rows, int heads, int kv_heads, int head_dim, cudaStream_t st) {
  if (rows == 0) return 0;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || head_dim % 8 != 0) return (int)cudaErrorInvalidValue;
  const int64_t total = rows * 3 * heads * (head_dim / 8);
  int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  gqa_expand_kernel<<<blocks, 256, 0, st>>>((const bf16x8*)in, (bf16x8*)out, rows, heads, kv_heads, head_dim / 8);
  return launch_status();
}

int lbi_gqa_reduce(const void* in, void* out, int64_t rows, int heads, int kv_heads, int head_dim, cudaStream_t st) {
  if (rows == 0) return 0;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || head_dim % 8 != 0) return (int)cudaErrorInvalidValue;
  const int64_t total = rows * (heads + 2 * kv_heads) * (head_dim / 8);
  int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  gqa_reduce_kernel<<<blocks, 256, 0, st>>>((const bf16x8*)in, (bf16x8*)out, rows, heads, kv_heads, head_dim / 8);
  return launch_status();
}

int lbi_causal_conv_fwd(const void* x, const float* w, const float* bias, void* y, int64_t seqs, int seq_len,
                        int channels, int width, cudaStream_t st) {
  const int64_t total = seqs * seq_len * channels;
  if (total == 0) return 0;
  causal_conv_fwd_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)x, w, bias,
                                                                          (__nv_bfloat16*)y, seqs, seq_len, channels,
                                                                          width);
  return launch_status();
}

int lbi_causal_conv_dgrad(const void* dy, const float* w, void* dx, int64_t seqs, int seq_len, int channels, int width,
                          cudaStream_t st) {
  const int64_t total = seqs * seq_len * channels;
  if (total == 0) return 0;
  causal_conv_dgrad_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)dy, w,
                                                                            (__nv_bfloat16*)dx, seqs, seq_len, channels,
                                                                            width);
  return launch_status();
}

int lbi_sumsq(const float* x, int64_t n, float* out, cudaStream_t st) {
  if (n == 0) return 0;
  int blocks = (int)((n + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  sumsq_kernel<<<blocks, 256, 0, st>>>(x, n, out);
  return launch_status();
}

int lbi_adamw_step(float* param, const float* grad, float* m, float* v, void* shadow, int64_t n, float lr, float beta1,
                   float beta2, float eps, float weight_decay, int step, float grad_mul, const float* sumsq,
                   float clip_norm, cudaStream_t st) {
  if (n == 0) return 0;
  int blocks = (int)((n + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  const float bias1 = 1.f - powf(beta1, (float)step);
  const float bias2_sqrt = sqrtf(1.f - powf(beta2, (float)step));
  adamw_kernel<<<blocks, 256, 0, st>>>(param, grad, m, v, (__nv_bfloat16*)shadow, n, lr, beta1, beta2, eps, weight_decay,
                                       bias1, bias2_sqrt, grad_mul, sumsq, clip_norm);
  return launch_status();
}

int lbi_ce_fwd_bwd(void* logits, const int64_t* targets, float* loss_sum, int64_t rows, int vocab, float scale,
                   cudaStream_t st) {
  if (rows == 0) return 0;
  ce_fwd_bwd_kernel<256><<<(unsigned)rows, 256, 0, st>>>((bf16x8*)logits, targets, loss_sum, vocab, scale);
  return launch_status();
}

}  // extern "C"

LBI_DEFINE_BOUNDS_GETTER(lbi_bounds_site_elementwise)
