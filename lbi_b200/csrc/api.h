// C entry points of the lbi_b200 CUDA kernels.  All pointers are device pointers unless noted; every
// function enqueues work on `stream` and returns the cudaError_t of the launch as an int (0 = success).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- fused elementwise / normalisation (elementwise.cu) -------------------------------------------------
// new_stream = branch (+ stream); rstd = rsqrt(mean(new_stream^2) + eps); normed = new_stream * rstd * weight.
int lbi_add_rmsnorm_fwd(const void* branch_bf16, const float* stream_or_null, const float* weight, void* normed_bf16,
                        float* new_stream, float* rstd, int64_t rows, int dim, float eps, cudaStream_t stream);
// d_stream_out = d_stream_in (or 0) + J_rmsnorm^T d_normed; activation rows are indexed by row % act_rows.
// d_stream_out_bf16 (optional) receives a bf16 copy of the result in the same pass.
int lbi_rmsnorm_bwd(const void* d_normed_bf16, const float* x_stream, const float* rstd, const float* weight,
                    const float* d_stream_in_or_null, float* d_stream_out, void* d_stream_out_bf16_or_null, int64_t rows,
                    int64_t act_rows, int dim, cudaStream_t stream);
// dw[d] = sum_r d_normed[r, d] * x[r, d] * rstd[r]; `partials` holds nblocks * dim floats.
int lbi_rmsnorm_wgrad(const void* d_normed_bf16, const float* x_stream, const float* rstd, float* partials, float* dw,
                      int64_t rows, int dim, int nblocks, cudaStream_t stream);
int lbi_rope_qkv(void* qkv_bf16, const float* cos_tab, const float* sin_tab, int64_t rows, int n_rot_heads, int qkv_dim,
                 int head_dim, int seq_len, int interleaved, int inverse, cudaStream_t stream);
// Grouped kv heads: packed rows [q (H heads) | k (Hkv) | v (Hkv)] -> [q | k | v] with H heads each (expand), and the sum of the
// cotangents of a group's copies back to the packed layout (reduce).  bf16, head_dim a multiple of 8.
int lbi_gqa_expand(const void* in_bf16, void* out_bf16, int64_t rows, int heads, int kv_heads, int head_dim, cudaStream_t stream);
int lbi_gqa_reduce(const void* in_bf16, void* out_bf16, int64_t rows, int heads, int kv_heads, int head_dim, cudaStream_t stream);
int lbi_swiglu_fwd(const void* u_bf16, void* a_bf16, int64_t rows, int hidden, cudaStream_t stream);
int lbi_swiglu_bwd(const void* da_bf16, const void* u_bf16, void* du_bf16, int64_t rows, int64_t act_rows, int hidden,
                   cudaStream_t stream);
int lbi_add_condition(const void* canvas_bf16, const float* cond, void* out_bf16, int64_t rows, int dim, int seq_len,
                      cudaStream_t stream);
// out[g, d] = scale * sum_t rows[g * seq_len + t, d]; out must be zeroed by the caller (accumulates with atomics).
int lbi_pool_tokens(const void* rows, int is_bf16, float* out, int64_t groups, int seq_len, int dim, float scale,
                    cudaStream_t stream);
// A token id outside [0, vocab) sets the status word (81 gather, 82 scatter) and is skipped (the gathered row is zeros).
int lbi_embedding_fwd(const int64_t* ids, const void* table, int table_is_bf16, void* out_bf16, int64_t rows, int dim,
                      int64_t vocab, int* status, cudaStream_t stream);
int lbi_embedding_scatter_add(float* d_table, const int64_t* ids, const void* d_rows, int rows_is_bf16, int64_t rows,
                              int dim, int64_t vocab, int* status, cudaStream_t stream);
int lbi_transpose_bf16(const void* in, void* out, int64_t rows, int64_t cols, cudaStream_t stream);
int lbi_causal_conv_fwd(const void* x_bf16, const float* w, const float* bias_or_null, void* y_bf16, int64_t seqs,
                        int seq_len, int channels, int width, cudaStream_t stream);
int lbi_causal_conv_dgrad(const void* dy_bf16, const float* w, void* dx_bf16, int64_t seqs, int seq_len, int channels,
                          int width, cudaStream_t stream);
// sumsq_out += sum(x^2) over a flat fp32 buffer (sumsq_out zeroed by the caller).
int lbi_sumsq(const float* x, int64_t n, float* sumsq_out, cudaStream_t stream);
// AdamW with decoupled weight decay on flat fp32 buffers.  The gradient is multiplied by grad_mul and, when
// sumsq_or_null is given, by the clip coefficient min(1, clip_norm / (sqrt(*sumsq * grad_mul^2) + 1e-6)).
// shadow_bf16_or_null receives the updated parameters rounded to bf16.
int lbi_adamw_step(float* param, const float* grad, float* exp_avg, float* exp_avg_sq, void* shadow_bf16_or_null,
                   int64_t n, float lr, float beta1, float beta2, float eps, float weight_decay, int step, float grad_mul,
                   const float* sumsq_or_null, float clip_norm, cudaStream_t stream);
// Per-row softmax cross-entropy over bf16 logits [rows, vocab]: loss_sum += scale * (lse - logit[target]) and
// logits are overwritten by scale * (softmax - onehot).  Rows with a negative target get zero gradient.
int lbi_ce_fwd_bwd(void* logits_bf16, const int64_t* targets, float* loss_sum, int64_t rows, int vocab, float scale,
                   cudaStream_t stream);

// ---- interface Jacobian scans (suffix_scan.cu) -----------------------------------------------------------
// out[b, k] = mats[b, k] @ mats[b, k+1] @ ... @ mats[b, K-1], out[b, K] = I;  mats [B, K, R, R] fp32 row-major.
int lbi_suffix_scan(const float* mats, float* out, int batch, int k, int r, cudaStream_t stream);
// g[b, k] = offsets[b, k] + mats[b, k] @ g[b, k+1], g[b, K] = seed (or 0);  g [B, K+1, R].
// Frobenius and spectral norms (power iteration, `iters` rounds) of `count` fp32 R x R matrices.
int lbi_matrix_norms(const float* mats, float* spec, float* frob, int count, int r, int iters, cudaStream_t stream);
int lbi_affine_suffix_scan(const float* mats, const float* offsets, const float* seed_or_null, float* g, int batch, int k,
                           int r, cudaStream_t stream);


// ---- gated / grouped RMSNorm (gated_norm.cu) --------------------------------------------------------------
// y = rmsnorm_group(x * silu(z)) * w (gate_first) or rmsnorm_group(x) * w * silu(z); z may be null.  x, z, y are bf16
// (is_bf16) or fp32 [rows, dim]; weight fp32 [dim]; rstd [rows, dim / group_size] fp32.
int lbi_gated_rmsnorm_fwd(const void* x, const void* z_or_null, const float* weight, void* y, float* rstd, int64_t rows, int dim,
                          int group_size, float eps, int gate_first, int is_bf16, cudaStream_t stream);
// dw_partials holds lbi_gated_rmsnorm_slots(rows, dim, group_size, is_bf16) rows of dim floats; the caller sums them.
// group_size must be a multiple of 8 (bf16) or 4 (fp32): every lane moves 16 bytes per access.
int lbi_gated_rmsnorm_slots(int64_t rows, int dim, int group_size, int is_bf16);
// x, z, rstd hold `frows` rows shared by rows / frows stacked directions of dy, dx, dz; dw_partials may be null (not wanted).
int lbi_gated_rmsnorm_bwd(const void* dy, const void* x, const void* z_or_null, const float* weight, const float* rstd, void* dx,
                          void* dz_or_null, float* dw_partials, int64_t rows, int64_t frows, int dim, int group_size,
                          int gate_first, int is_bf16, cudaStream_t stream);

// ---- Mamba-3 SISO preprocessing on the wide tensors (siso_prep.cu) ---------------------------------------
// q, k [tokens, groups, 128] bf16 (is_bf16) or fp32; biases [heads, 128]; theta [tokens, heads, n_angles]; gamma, scale
// [tokens, heads]  ->  qr, kr [tokens, heads, 128] bf16, qk_dot [tokens, heads].
int lbi_siso_prep_fwd(const void* q, const void* k, const float* q_bias, const float* k_bias, const float* theta,
                      const float* gamma, const float* scale, void* qr_bf16, void* kr_bf16, float* qk_dot, int64_t tokens,
                      int groups, int heads, int d_state, int n_angles, int is_bf16, cudaStream_t stream);
// Backward from dqr, dkr [tokens, heads, 128] (fp32, or bf16 when cot_bf16) and dqk [tokens, heads]: dq, dk [tokens, groups, 128]
// fp32, dtheta, dgamma, dscale, and bias_partials [lbi_siso_prep_blocks(tokens * groups)][2][heads][128] (summed by the caller:
// dq_bias, dk_bias; null: not wanted).  tokens = batch * seq_len; the forward tensors q, k, theta, gamma, scale hold `ftokens`
// tokens shared by tokens / ftokens stacked directions.  dkr_pad > 0: dkr is [batch, dkr_pad, heads, 128] in reversed time.
int lbi_siso_prep_blocks(int64_t rows);
int lbi_siso_prep_bwd(const void* q, const void* k, const float* q_bias, const float* k_bias, const float* theta,
                      const float* gamma, const float* scale, const void* dqr, const void* dkr, const float* dqk, float* dq,
                      float* dk, float* dtheta, float* dgamma, float* dscale, float* bias_partials, int64_t tokens, int64_t ftokens,
                      int seq_len, int dkr_pad, int groups, int heads, int d_state, int n_angles, int is_bf16, int cot_bf16,
                      cudaStream_t stream);

// ---- Mamba block glue on the small tensors (mamba_small.cu) ------------------------------------------------
// out = y * silu(z); bf16, numel a multiple of 8.
int lbi_gate_silu_fwd(const void* y, const void* z, void* out, int64_t numel, cudaStream_t stream);
// dyg, dy [reps * numel] bf16; y, z [numel] = [rows, cols] shared by the reps stacked directions; dz [reps * rows, cols] with
// row stride ld_dz elements (a column range of a wider matrix; ld_dz = cols when contiguous).  cols, ld_dz multiples of 8.
int lbi_gate_silu_bwd(const void* dyg, const void* y, const void* z, void* dy, void* dz, int64_t numel, int reps, int cols,
                      int64_t ld_dz, cudaStream_t stream);
// Mamba-2 step size: dt = clamp(softplus(dt_raw + bias), lo, hi) and its slope (0 outside the limits), fp32 [rows, heads];
// dt_raw [rows, heads] bf16 or fp32 with row stride ld (elements).
int lbi_softplus_dt(const void* dt_raw, int64_t ld, int is_bf16, const float* bias, float lo, float hi, float* dt, float* slope,
                    int64_t rows, int heads, cudaStream_t stream);
// Mamba-3 per-token, per-head scalars.  dd_dt, dd_a, trap [B * L, H], angles [B * L, S], dt_bias [H] (fp32) ->
// dt, a, sig, adt, gamma, scale, sp_dt, sp_a, live [B, L, H]; tanh_a [B, L, S]; theta [B, L, H, S] in [0, 2 pi).  S <= 64,
// H <= 32.  Scratch: seg_inc [B, lbi_siso_small_fwd_segments(L), H, 64] fp32 (phase increments summed per segment of the
// sequence, so that the running phase can start in every segment at once).  Two kernels on `stream`.
int lbi_siso_small_fwd_segments(int seq_len);
int lbi_siso_small_fwd(const float* dd_dt, const float* dd_a, const float* trap, const float* angles, const float* dt_bias,
                       float a_floor, float* seg_inc, float* dt, float* a, float* sig, float* adt, float* gamma, float* scale,
                       float* tanh_a, float* theta, float* sp_dt, float* sp_a, float* live, int batch, int seq_len, int heads,
                       int n_angles, cudaStream_t stream);
// Cotangents dadt, dgamma, dscale [reps * B, L, H] and dtheta [reps * B, L, H, S] -> d_dd_dt, d_dd_a, d_trap [reps * B * L, H]
// and d_angles [reps * B * L, S] (fp32 or bf16); the forward tensors [B, ...] are shared by the reps directions.
// H <= 32, S <= 32.  Scratch: seg_sum [reps * B, lbi_siso_small_segments(L), H, 32] fp32 (dtheta summed per segment of the
// sequence, so that the reversed running sum can start in every segment at once).  Two kernels on `stream`.
int lbi_siso_small_segments(int seq_len);
int lbi_siso_small_bwd(const float* dt, const float* a, const float* sig, const float* tanh_a, const float* sp_dt,
                       const float* sp_a, const float* live, const float* dadt, const float* dtheta, const float* dgamma,
                       const float* dscale, float* seg_sum, void* d_dd_dt, void* d_dd_a, void* d_trap, void* d_angles, int batch,
                       int reps, int seq_len, int heads, int n_angles, int out_bf16, cudaStream_t stream);

// Mamba-2 depthwise causal conv + SiLU over the xBC slice (channels = c0 + c1 + c2, each a multiple of 8; width <= 8).
// x [tokens, channels] bf16, wt [width, channels] (the weights TRANSPOSED), bias [channels] or null (fp32) -> pre [tokens, channels] bf16 (conv output) and
// the activation split into o0 [tokens, c0], o1 [tokens, c1], o2 [tokens, c2] bf16.
int lbi_conv_silu_fwd(const void* x, const float* wt, const float* bias, void* pre, void* o0, void* o1, void* o2, int c0, int c1,
                      int c2, int64_t tokens, int seq_len, int width, cudaStream_t stream);
// Cotangents of the three activation parts d0 [tokens, c0] (bf16 or fp32), d1, d2 [tokens, c1 / c2] (bf16 or fp32) -> cotangent of
// the conv input, written with row stride ld_in (elements) at din.  pre holds ftokens tokens shared by tokens / ftokens directions.
int lbi_conv_silu_bwd(const void* d0, int d0_fp32, const void* d1, const void* d2, int d12_fp32, const void* pre, const float* wt,
                      void* din, int64_t ld_in, int c0, int c1, int c2, int64_t tokens, int64_t ftokens, int seq_len, int width,
                      cudaStream_t stream);
// dw [channels, width] += , db [channels] += (fp32; zeroed by the caller).  One direction (tokens = ftokens).  pre may be null:
// the weight gradient of a plain convolution (no SiLU after it), with d0 its output cotangent and c1 = c2 = 0.
int lbi_conv_silu_wgrad(const void* d0, int d0_fp32, const void* d1, const void* d2, int d12_fp32, const void* pre, const void* x,
                        float* dw, float* db, int c0, int c1, int c2, int64_t tokens, int seq_len, int width, cudaStream_t stream);

// ---- interface Jacobian products over a basis (interface_jac.cu) -----------------------------------------
// out[b, p, :] = (((in_scale * g[b, p, :]) @ wa) o d[b, :]) @ wb;  g [B, P, din], wa [din, hidden], d [B, hidden] or null,
// wb [hidden, dout] or null (then out [B, P, hidden] = (g @ wa) o d).  All fp32 row-major.
int lbi_interface_mlp_jac(const float* g, const float* wa, const float* d, const float* wb, float* out, int batch, int p_total,
                          int din, int hidden, int dout, float in_scale, cudaStream_t stream);
// LayerNorm Jacobian at x [B, R] applied to g [B, P, R]: transpose = 1 gives J^T g (weight on the input side),
// transpose = 0 gives J g (weight on the output side); the result is multiplied by out_scale.
int lbi_layernorm_jac(const float* x, const float* weight, const float* g, float* out, int batch, int p_total, int r, float eps,
                      int transpose, float out_scale, cudaStream_t stream);

// Skinny fp32 linear maps of the interface (a few rows): y = act(x w^T + bias) with act 0 none / 1 SiLU / 2 GELU, `pre` (or null)
// receives the value before the activation; gx = g w; dw += g^T x, db += sum_b g (db may be null).  x [B, din], w [dout, din].
int lbi_small_linear_fwd(const float* x, const float* w, const float* bias, float* y, float* pre, int batch, int din, int dout,
                         int act, cudaStream_t stream);
int lbi_small_linear_dgrad(const float* g, const float* w, float* gx, int batch, int din, int dout, cudaStream_t stream);
int lbi_small_linear_wgrad(const float* g, const float* x, float* dw, float* db, int batch, int din, int dout, cudaStream_t stream);

// Debug build only (-DLBI_BOUNDS_CHECK): the first index-check violation (site code) of a translation unit, read and cleared;
// 0 = none.  The normal build returns 0.
int lbi_bounds_site_elementwise();
int lbi_bounds_site_mamba_small();

#ifdef __cplusplus
}
#endif
