// C entry points of the Mamba-2 SSD chunk-scan forward (ssd.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// dt_raw [B, L, H] fp32 -> dt_out, cum [B, H, L] fp32: dt = clamp(softplus(dt_raw + bias)) when `softplus`, else dt_raw;
// cum = inclusive cumulative sum of dt * a[h] inside every 128-token chunk.  L must be a multiple of 128.
int lbi_ssd_cumsum(const float* dt_raw, const float* dt_bias, const float* a, float* dt_out, float* cum, int batch, int seq_len,
                   int heads, int softplus, float dt_min, float dt_max, cudaStream_t stream);

// Chunked scan.  x [B*L, H*64] bf16, bm / cm [B*L, G*N] bf16, dt / cum from lbi_ssd_cumsum, d_skip [H] fp32 or null,
// init_state [B, H, 64, N] fp32 or null.  Scratch supplied by the caller: states [B, L/128, H, 64, N] fp32 and
// prev (same shape, bf16).  Outputs: final_state [B, H, 64, N] fp32, y [B*L, H*64] bf16.
// head_dim must be 64, d_state 64 or 128, heads / groups even.  Three kernels on `stream`.
int lbi_ssd_chunk_scan_fwd(const void* x, const void* bm, const void* cm, const float* dt, const float* cum,
                           const float* d_skip, const float* init_state, float* states, void* prev, float* final_state,
                           void* y, int batch, int seq_len, int heads, int groups, int head_dim, int d_state, int* status,
                           cudaStream_t stream);

// Mamba-3 SISO chunk scan on preprocessed operands (per-head rotated / biased / scaled):
//   h_t = exp(adt_t) h_{t-1} + v_t kr_t^T ,   y_t = qr_t . (exp(adt_t) h_{t-1}) + (d_skip[h] + skip_tok[t]) v_t
// v [B*L, H*64] bf16, kr / qr [B*L, H*128] bf16, cum [B, H, L] fp32 = in-chunk cumulative sum of adt (lbi_ssd_cumsum
// with a = 1), skip_tok [B, H, L] fp32.  States are kept [n][p]: states / prev [B, L/128, H, 128, 64], init / final
// [B, H, 128, 64].  head_dim 64, d_state 128.
int lbi_siso_chunk_scan_fwd(const void* v, const void* kr, const void* qr, const float* cum, const float* d_skip,
                            const float* skip_tok, const float* init_state, float* states, void* prev, float* final_state,
                            void* y, int batch, int seq_len, int heads, int head_dim, int d_state, int* status,
                            cudaStream_t stream);

// The chunk scan with free operand roles (the backward passes are this operator with the roles permuted):
//   y_t = sum_{s <= t} exp(c_t - c_s) (cq_t . bk_s) w_s v_s + exp(c_t) cq_t . init      (s < t when `strict`)
//   final = sum_s exp(c_end - c_s) w_s v_s bk_s^T + exp(c_end) init
// v [B*L, H*64] bf16; bk / cq [B*L, G*N] bf16 (or [B*L, H*128] when `per_head`); weight [B, H, L] fp32 or null (w = 1);
// cum [B, H, L] fp32 in-chunk cumulative sums.  The result goes to `y32` (fp32) when it is set, else to `y` (bf16).
// States are [p][n] (per_head: [n][p]).  N = 64 or 128 (per_head: 128); heads / groups even unless per_head.
// Head h reads the 64-column block (h / v_div) * v_mod + h % v_mod of v (1, 1: its own block), so that several heads can
// share columns of a narrower v matrix without a materialised copy.
int lbi_ssd_scan_generic(const void* v, const void* bk, const void* cq, const float* weight, const float* cum,
                         const float* d_skip, const float* skip_tok, int strict, const float* init_state, float* states,
                         void* prev, float* final_state, void* y, float* y32, int batch, int seq_len, int heads, int groups,
                         int d_state, int per_head, int v_div, int v_mod, int* status, cudaStream_t stream);

// Gradient of the log-decays of that scan: da_u = sum over pairs s < u <= t of e^{c_t - c_s} (cq_t . bk_s) w_s (gy_t . v_s),
// pairs that reach before the first or past the last token included through `state_in` (the bf16 incoming states of the
// forward scan, [B, L/128, H, 64, N]; per_head: [.., N, 64]) and `state_cot_rev` (the incoming states of the
// time-reversed scan that pulled gy back, same layout, chunk axis reversed).  gy like v; da [B, H, L] fp32.
int lbi_ssd_decay_grad(const void* v, const void* gy, const void* bk, const void* cq, const float* weight, const float* cum,
                       const void* state_in, const void* state_cot_rev, float* da, int batch, int seq_len, int heads,
                       int groups, int d_state, int per_head, int* status, cudaStream_t stream);

// Elementwise tail of the SSD backward.  dx_rev [B, seq_pad, H, 64] fp32 is the reversed-time scan result; x, gy, dx
// [B, L, H, 64] bf16 or fp32; dt, ddt [B, L, H]; da [B, H, seq_pad]; a_param, d_skip (or null), dd (or null, accumulated) [H].
//   dx = dt * dX + d_skip * gy,  ddt = da * a_param + dX . x,  dd[h] += sum gy . x
// `reversed`: dx_rev is in reversed time (else natural order); x and dt hold `fbatch` sequences shared by batch / fbatch
// stacked directions of gy.
int lbi_ssd_bwd_finish(const void* dx_rev, int dx_is_bf16, const void* x, const void* gy, const float* dt, const float* da,
                       const float* a_param, const float* d_skip, void* dx, float* ddt, float* dd, int batch, int seq_len,
                       int seq_pad, int heads, int is_bf16, int reversed, int fbatch, cudaStream_t stream);

// Fused chunk backward of lbi_ssd_scan_generic: every input cotangent from one pass (see bwd_chunk_kernel in ssd.cu).
// Forward operands v [Bf*L, H*64], bk / cq [Bf*L, G*N] (per_head: [Bf*L, H*128]) bf16, weight / cum / skip_tok [Bf, H, L] fp32 and
// state_in (bf16 incoming chunk states of the forward, [Bf, L/128, H, 64, N]; per_head [.., N, 64]) belong to `bmod` = Bf
// sequences and are shared by batch / bmod stacked directions of gy [B*L, H*64] bf16.  d_final (cotangent of the final state,
// fp32, layout of the states) may be null.  Scratch: d_out [B, L/128, H, 64*N] bf16 (cotangents of the chunk-boundary states);
// chunk_cot is unused (kept for callers of the earlier three-kernel form) and may be null.
// Results: d_init (or null), da, dskip (or null) [B, H, L]; dv [B*L, H*64] in dv32 or dv16 (cotangent of w_s v_s, plus
// (d_skip[h] + skip_tok) * gy when given); dcq, dbk [B*L, H*N] per head in fp32 or bf16.  dv_ld: row stride of dv16 in elements
// (a column range of a wider matrix; a multiple of 8; 0 = contiguous).  Two kernels on `stream`.
int lbi_ssd_chunk_bwd(const void* v, const void* gy, const void* bk, const void* cq, const float* weight, const float* cum,
                      const float* skip_tok, const float* d_skip, const void* state_in, const float* d_final, float* chunk_cot,
                      void* d_out, float* d_init, float* da, float* dskip, float* dv32, void* dv16, float* dcq32, float* dbk32,
                      void* dcq16, void* dbk16, int batch, int bmod, int seq_len, int heads, int groups, int d_state, int per_head,
                      int strict, int64_t dv_ld, int* status, cudaStream_t stream);
// out[b, l, g, :n] = sum over the heads h of group g of w[b, l, h] * y[b, l or seq_pad - 1 - l, h, :n]; y bf16 with rows of
// `width` columns, w [B, L, H] or null, out bf16 or fp32.
int lbi_ssd_group_sum(const void* y_bf16, const float* w, void* out, int batch, int seq_len, int seq_pad, int heads, int groups,
                      int n, int width, int reversed, int out_is_bf16, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
