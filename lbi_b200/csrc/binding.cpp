// Python bindings of the lbi_b200 CUDA kernels (module lbi_b200._C).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "api.h"
#include "api_attn.h"
#include "api_ssd.h"
#include "api_gemm.h"
#include "api_peer.h"

namespace {

using torch::Tensor;

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check(int rc, const char* what) {
  TORCH_CHECK(rc == 0, what, " failed with code ", rc, " (", rc < 1000 ? cudaGetErrorString((cudaError_t)rc) : "driver", ")");
}

#define CHECK_BF16(x) TORCH_CHECK((x).is_cuda() && (x).scalar_type() == at::kBFloat16 && (x).is_contiguous(), #x " must be a contiguous CUDA bf16 tensor")
#define CHECK_LP16(x) TORCH_CHECK((x).is_cuda() && ((x).scalar_type() == at::kBFloat16 || (x).scalar_type() == at::kHalf) && (x).is_contiguous(), #x " must be a contiguous CUDA bf16 / fp16 tensor")
#define CHECK_F32(x) TORCH_CHECK((x).is_cuda() && (x).scalar_type() == at::kFloat && (x).is_contiguous(), #x " must be a contiguous CUDA fp32 tensor")

Tensor status_word(const Tensor& like) {
  static thread_local std::vector<Tensor> words(16);
  int dev = like.get_device();
  if (!words[dev].defined()) words[dev] = torch::zeros({1}, like.options().dtype(at::kInt));
  return words[dev];
}

std::tuple<Tensor, Tensor, Tensor> add_rmsnorm_fwd(const Tensor& branch, const c10::optional<Tensor>& stream_in,
                                                   const Tensor& weight, double eps) {
  CHECK_BF16(branch);
  c10::cuda::CUDAGuard guard(branch.device());
  const int64_t rows = branch.size(0);
  const int dim = (int)branch.size(1);
  TORCH_CHECK(dim % 8 == 0, "feature dim must be a multiple of 8");
  Tensor w = weight.to(at::kFloat).contiguous();
  Tensor normed = torch::empty_like(branch);
  Tensor new_stream = torch::empty({rows, dim}, branch.options().dtype(at::kFloat));
  Tensor rstd = torch::empty({rows}, branch.options().dtype(at::kFloat));
  const float* sp = nullptr;
  if (stream_in.has_value() && stream_in->defined()) {
    CHECK_F32(*stream_in);
    sp = stream_in->data_ptr<float>();
  }
  check(lbi_add_rmsnorm_fwd(branch.data_ptr(), sp, w.data_ptr<float>(), normed.data_ptr(), new_stream.data_ptr<float>(),
                            rstd.data_ptr<float>(), rows, dim, (float)eps, cur_stream()),
        "add_rmsnorm_fwd");
  return {normed, new_stream, rstd};
}

static std::tuple<Tensor, Tensor> rmsnorm_bwd_impl(const Tensor& d_normed, const Tensor& x_stream, const Tensor& rstd,
                                                   const Tensor& weight, const c10::optional<Tensor>& d_stream, bool want_lowp) {
  CHECK_BF16(d_normed);
  CHECK_F32(x_stream);
  CHECK_F32(rstd);
  c10::cuda::CUDAGuard guard(d_normed.device());
  const int64_t rows = d_normed.size(0), act_rows = x_stream.size(0);
  const int dim = (int)d_normed.size(1);
  TORCH_CHECK(rows % act_rows == 0, "cotangent rows must be a multiple of activation rows");
  Tensor w = weight.to(at::kFloat).contiguous();
  Tensor out, lowp;
  const float* din = nullptr;
  if (d_stream.has_value() && d_stream->defined()) {
    CHECK_F32(*d_stream);
    out = *d_stream;  // accumulate in place
    din = out.data_ptr<float>();
  } else {
    out = torch::empty({rows, dim}, d_normed.options().dtype(at::kFloat));
  }
  if (want_lowp) lowp = torch::empty({rows, dim}, d_normed.options());
  check(lbi_rmsnorm_bwd(d_normed.data_ptr(), x_stream.data_ptr<float>(), rstd.data_ptr<float>(), w.data_ptr<float>(), din,
                        out.data_ptr<float>(), want_lowp ? lowp.data_ptr() : nullptr, rows, act_rows, dim, cur_stream()),
        "rmsnorm_bwd");
  return {out, lowp};
}

Tensor rmsnorm_bwd(const Tensor& d_normed, const Tensor& x_stream, const Tensor& rstd, const Tensor& weight,
                   const c10::optional<Tensor>& d_stream) {
  return std::get<0>(rmsnorm_bwd_impl(d_normed, x_stream, rstd, weight, d_stream, false));
}

// Same, and also returns the bf16 copy of the new cotangent stream (what the next GEMM reads).
std::tuple<Tensor, Tensor> rmsnorm_bwd_lowp(const Tensor& d_normed, const Tensor& x_stream, const Tensor& rstd, const Tensor& weight,
                                            const c10::optional<Tensor>& d_stream) {
  return rmsnorm_bwd_impl(d_normed, x_stream, rstd, weight, d_stream, true);
}

Tensor rmsnorm_wgrad(const Tensor& d_normed, const Tensor& x_stream, const Tensor& rstd) {
  CHECK_BF16(d_normed);
  CHECK_F32(x_stream);
  c10::cuda::CUDAGuard guard(d_normed.device());
  const int64_t rows = d_normed.size(0);
  const int dim = (int)d_normed.size(1);
  TORCH_CHECK(x_stream.size(0) == rows, "rmsnorm_wgrad takes a single cotangent");
  const int nblocks = (int)std::min<int64_t>(296, std::max<int64_t>(1, rows / 16));
  Tensor partials = torch::empty({nblocks, dim}, x_stream.options());
  Tensor dw = torch::empty({dim}, x_stream.options());
  check(lbi_rmsnorm_wgrad(d_normed.data_ptr(), x_stream.data_ptr<float>(), rstd.data_ptr<float>(),
                          partials.data_ptr<float>(), dw.data_ptr<float>(), rows, dim, nblocks, cur_stream()),
        "rmsnorm_wgrad");
  return dw;
}

Tensor rope_qkv_(Tensor qkv, const Tensor& cos_tab, const Tensor& sin_tab, int64_t n_heads, int64_t n_kv_heads,
                 int64_t head_dim, int64_t seq_len, bool interleaved, bool inverse) {
  CHECK_BF16(qkv);
  CHECK_F32(cos_tab);
  CHECK_F32(sin_tab);
  c10::cuda::CUDAGuard guard(qkv.device());
  TORCH_CHECK(head_dim % 16 == 0, "head_dim must be a multiple of 16");
  TORCH_CHECK(cos_tab.size(0) >= seq_len && cos_tab.size(1) == head_dim / 2, "rope table shape mismatch");
  check(lbi_rope_qkv(qkv.data_ptr(), cos_tab.data_ptr<float>(), sin_tab.data_ptr<float>(), qkv.size(0),
                     (int)(n_heads + n_kv_heads), (int)qkv.size(1), (int)head_dim, (int)seq_len, interleaved ? 1 : 0,
                     inverse ? 1 : 0, cur_stream()),
        "rope_qkv");
  return qkv;
}

Tensor gqa_expand(const Tensor& qkv, int64_t heads, int64_t kv_heads, int64_t head_dim) {
  CHECK_BF16(qkv);
  c10::cuda::CUDAGuard guard(qkv.device());
  TORCH_CHECK(qkv.dim() == 2 && qkv.size(1) == (heads + 2 * kv_heads) * head_dim, "gqa_expand: packed rows [q | k | v]");
  Tensor out = torch::empty({qkv.size(0), 3 * heads * head_dim}, qkv.options());
  check(lbi_gqa_expand(qkv.data_ptr(), out.data_ptr(), qkv.size(0), (int)heads, (int)kv_heads, (int)head_dim, cur_stream()), "gqa_expand");
  return out;
}

Tensor gqa_reduce(const Tensor& d_qkv, int64_t heads, int64_t kv_heads, int64_t head_dim) {
  CHECK_BF16(d_qkv);
  c10::cuda::CUDAGuard guard(d_qkv.device());
  TORCH_CHECK(d_qkv.dim() == 2 && d_qkv.size(1) == 3 * heads * head_dim, "gqa_reduce: rows [q | k | v] with H heads each");
  Tensor out = torch::empty({d_qkv.size(0), (heads + 2 * kv_heads) * head_dim}, d_qkv.options());
  check(lbi_gqa_reduce(d_qkv.data_ptr(), out.data_ptr(), d_qkv.size(0), (int)heads, (int)kv_heads, (int)head_dim, cur_stream()), "gqa_reduce");
  return out;
}

Tensor swiglu_fwd(const Tensor& u) {
  CHECK_BF16(u);
  c10::cuda::CUDAGuard guard(u.device());
  const int hidden = (int)(u.size(1) / 2);
  Tensor a = torch::empty({u.size(0), hidden}, u.options());
  check(lbi_swiglu_fwd(u.data_ptr(), a.data_ptr(), u.size(0), hidden, cur_stream()), "swiglu_fwd");
  return a;
}

Tensor swiglu_bwd(const Tensor& da, const Tensor& u) {
  CHECK_BF16(da);
  CHECK_BF16(u);
  c10::cuda::CUDAGuard guard(u.device());
  const int hidden = (int)da.size(1);
  TORCH_CHECK(u.size(1) == 2 * hidden && da.size(0) % u.size(0) == 0, "swiglu_bwd shape mismatch");
  Tensor du = torch::empty({da.size(0), 2 * hidden}, da.options());
  check(lbi_swiglu_bwd(da.data_ptr(), u.data_ptr(), du.data_ptr(), da.size(0), u.size(0), hidden, cur_stream()),
        "swiglu_bwd");
  return du;
}

Tensor add_condition(const Tensor& canvas, const Tensor& cond, int64_t seq_len) {
  CHECK_BF16(canvas);
  CHECK_F32(cond);
  c10::cuda::CUDAGuard guard(canvas.device());
  Tensor out = torch::empty_like(canvas);
  check(lbi_add_condition(canvas.data_ptr(), cond.data_ptr<float>(), out.data_ptr(), canvas.size(0), (int)canvas.size(1),
                          (int)seq_len, cur_stream()),
        "add_condition");
  return out;
}

Tensor pool_tokens(const Tensor& rows, int64_t groups, int64_t seq_len, double scale) {
  TORCH_CHECK(rows.is_cuda() && rows.is_contiguous(), "rows must be a contiguous CUDA tensor");
  c10::cuda::CUDAGuard guard(rows.device());
  const int dim = (int)rows.size(-1);
  TORCH_CHECK(rows.numel() == groups * seq_len * dim, "pool_tokens shape mismatch");
  Tensor out = torch::zeros({groups, dim}, rows.options().dtype(at::kFloat));
  check(lbi_pool_tokens(rows.data_ptr(), rows.scalar_type() == at::kBFloat16 ? 1 : 0, out.data_ptr<float>(), groups,
                        (int)seq_len, dim, (float)scale, cur_stream()),
        "pool_tokens");
  return out;
}

Tensor embedding_fwd(const Tensor& ids, const Tensor& table) {
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous(), "ids must be contiguous int64");
  TORCH_CHECK(table.is_cuda() && table.is_contiguous(), "table must be contiguous");
  c10::cuda::CUDAGuard guard(table.device());
  Tensor out = torch::empty({ids.numel(), table.size(1)}, table.options().dtype(at::kBFloat16));
  check(lbi_embedding_fwd(ids.data_ptr<int64_t>(), table.data_ptr(), table.scalar_type() == at::kBFloat16 ? 1 : 0,
                          out.data_ptr(), ids.numel(), (int)table.size(1), table.size(0), status_word(table).data_ptr<int>(), cur_stream()),
        "embedding_fwd");
  return out;
}

void embedding_scatter_add_(Tensor d_table, const Tensor& ids, const Tensor& d_rows) {
  CHECK_F32(d_table);
  c10::cuda::CUDAGuard guard(d_table.device());
  check(lbi_embedding_scatter_add(d_table.data_ptr<float>(), ids.data_ptr<int64_t>(), d_rows.data_ptr(),
                                  d_rows.scalar_type() == at::kBFloat16 ? 1 : 0, ids.numel(), (int)d_table.size(1), d_table.size(0),
                                  status_word(d_table).data_ptr<int>(), cur_stream()),
        "embedding_scatter_add");
}

Tensor transpose_bf16(const Tensor& x) {
  CHECK_BF16(x);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = torch::empty({x.size(1), x.size(0)}, x.options());
  check(lbi_transpose_bf16(x.data_ptr(), out.data_ptr(), x.size(0), x.size(1), cur_stream()), "transpose_bf16");
  return out;
}

Tensor causal_conv_fwd(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& bias, int64_t batch, int64_t seq_len) {
  CHECK_BF16(x);
  CHECK_F32(w);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty_like(x);
  const float* bp = (bias.has_value() && bias->defined()) ? bias->data_ptr<float>() : nullptr;
  check(lbi_causal_conv_fwd(x.data_ptr(), w.data_ptr<float>(), bp, y.data_ptr(), x.size(0) / seq_len, (int)seq_len,
                            (int)x.size(1), (int)w.size(1), cur_stream()),
        "causal_conv_fwd");
  return y;
}

Tensor causal_conv_dgrad(const Tensor& dy, const Tensor& w, int64_t batch, int64_t seq_len) {
  CHECK_BF16(dy);
  CHECK_F32(w);
  c10::cuda::CUDAGuard guard(dy.device());
  Tensor dx = torch::empty_like(dy);
  check(lbi_causal_conv_dgrad(dy.data_ptr(), w.data_ptr<float>(), dx.data_ptr(), dy.size(0) / seq_len, (int)seq_len,
                              (int)dy.size(1), (int)w.size(1), cur_stream()),
        "causal_conv_dgrad");
  return dx;
}

void sumsq_(const Tensor& x, Tensor out) {
  CHECK_F32(x);
  CHECK_F32(out);
  c10::cuda::CUDAGuard guard(x.device());
  check(lbi_sumsq(x.data_ptr<float>(), x.numel(), out.data_ptr<float>(), cur_stream()), "sumsq");
}

void adamw_step_(Tensor param, const Tensor& grad, Tensor m, Tensor v, const c10::optional<Tensor>& shadow, double lr,
                 double beta1, double beta2, double eps, double weight_decay, int64_t step, double grad_mul,
                 const c10::optional<Tensor>& sumsq, double clip_norm) {
  CHECK_F32(param);
  CHECK_F32(grad);
  CHECK_F32(m);
  CHECK_F32(v);
  c10::cuda::CUDAGuard guard(param.device());
  void* sh = nullptr;
  if (shadow.has_value() && shadow->defined()) {
    CHECK_BF16(*shadow);
    sh = shadow->data_ptr();
  }
  const float* sq = (sumsq.has_value() && sumsq->defined()) ? sumsq->data_ptr<float>() : nullptr;
  check(lbi_adamw_step(param.data_ptr<float>(), grad.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), sh,
                       param.numel(), (float)lr, (float)beta1, (float)beta2, (float)eps, (float)weight_decay, (int)step,
                       (float)grad_mul, sq, (float)clip_norm, cur_stream()),
        "adamw_step");
}

void ce_fwd_bwd_(Tensor logits, const Tensor& targets, Tensor loss_sum, double scale) {
  CHECK_BF16(logits);
  CHECK_F32(loss_sum);
  TORCH_CHECK(targets.scalar_type() == at::kLong && targets.is_contiguous(), "targets must be contiguous int64");
  TORCH_CHECK(logits.size(1) % 8 == 0, "vocab must be a multiple of 8");
  c10::cuda::CUDAGuard guard(logits.device());
  check(lbi_ce_fwd_bwd(logits.data_ptr(), targets.data_ptr<int64_t>(), loss_sum.data_ptr<float>(), logits.size(0),
                       (int)logits.size(1), (float)scale, cur_stream()),
        "ce_fwd_bwd");
}

Tensor suffix_scan(const Tensor& mats) {
  TORCH_CHECK(mats.is_cuda() && mats.dim() == 4 && mats.size(2) == mats.size(3), "mats must be [B, K, R, R] on CUDA");
  c10::cuda::CUDAGuard guard(mats.device());
  Tensor m = mats.to(at::kFloat).contiguous();
  const int b = (int)m.size(0), k = (int)m.size(1), r = (int)m.size(2);
  Tensor out = torch::empty({b, k + 1, r, r}, m.options());
  check(lbi_suffix_scan(m.data_ptr<float>(), out.data_ptr<float>(), b, k, r, cur_stream()), "suffix_scan");
  return out;
}

// mats [..., R, R] fp32 -> (spectral norms, Frobenius norms), each shaped like the leading dimensions.
std::tuple<Tensor, Tensor> matrix_norms(const Tensor& mats, int64_t iters) {
  CHECK_F32(mats);
  c10::cuda::CUDAGuard guard(mats.device());
  TORCH_CHECK(mats.dim() >= 2 && mats.size(-1) == mats.size(-2), "matrix_norms: expected [..., R, R]");
  const int64_t r = mats.size(-1);
  const int64_t count = mats.numel() / (r * r);
  auto lead = mats.sizes().vec();
  lead.resize(lead.size() - 2);
  Tensor spec = torch::empty(lead, mats.options()), frob = torch::empty(lead, mats.options());
  check(lbi_matrix_norms(mats.data_ptr<float>(), spec.data_ptr<float>(), frob.data_ptr<float>(), (int)count, (int)r, (int)iters,
                         cur_stream()),
        "matrix_norms");
  return {spec, frob};
}

// Gated / grouped RMSNorm.  x, z [rows, dim] bf16 or fp32 (same dtype), weight fp32 [dim] -> (y, rstd [rows, dim / group]).
std::tuple<Tensor, Tensor> gated_rmsnorm_fwd(const Tensor& x, const c10::optional<Tensor>& z, const Tensor& weight, double eps,
                                             int64_t group_size, bool gate_first) {
  CHECK_F32(weight);
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.dim() == 2 && (x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kFloat),
              "gated_rmsnorm: x must be a contiguous CUDA [rows, dim] bf16 / fp32 tensor");
  TORCH_CHECK(!z || (z->is_contiguous() && z->sizes() == x.sizes() && z->scalar_type() == x.scalar_type()), "gated_rmsnorm: z must match x");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = x.size(0), dim = x.size(1);
  TORCH_CHECK(weight.numel() == dim && group_size > 0 && dim % group_size == 0, "gated_rmsnorm: bad weight / group size");
  Tensor y = torch::empty_like(x);
  Tensor rstd = torch::empty({rows, dim / group_size}, x.options().dtype(at::kFloat));
  check(lbi_gated_rmsnorm_fwd(x.data_ptr(), z ? z->data_ptr() : nullptr, weight.data_ptr<float>(), y.data_ptr(), rstd.data_ptr<float>(),
                              rows, (int)dim, (int)group_size, (float)eps, gate_first ? 1 : 0, x.scalar_type() == at::kBFloat16 ? 1 : 0,
                              cur_stream()),
        "gated_rmsnorm_fwd");
  return {y, rstd};
}

// -> (dx, dz (empty when z is none), dw [dim] fp32)
// dy [P * rows, dim]; x, z [rows, dim] and rstd shared by the P stacked directions -> (dx, dz [P * rows, dim], dweight [dim] or empty).
std::tuple<Tensor, Tensor, Tensor> gated_rmsnorm_bwd(const Tensor& dy, const Tensor& x, const c10::optional<Tensor>& z, const Tensor& weight,
                                                     const Tensor& rstd, int64_t group_size, bool gate_first, bool want_dweight) {
  CHECK_F32(weight);
  CHECK_F32(rstd);
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && dy.is_contiguous() && dy.dim() == 2 && x.dim() == 2 && dy.size(1) == x.size(1) &&
                  x.size(0) > 0 && dy.size(0) % x.size(0) == 0 && dy.scalar_type() == x.scalar_type(),
              "gated_rmsnorm_bwd: dy must hold a whole number of copies of x's rows");
  TORCH_CHECK(!z || (z->is_contiguous() && z->sizes() == x.sizes() && z->scalar_type() == x.scalar_type()), "gated_rmsnorm_bwd: z must match x");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = dy.size(0), frows = x.size(0), dim = x.size(1);
  const int slots = lbi_gated_rmsnorm_slots(rows, (int)dim, (int)group_size, x.scalar_type() == at::kBFloat16 ? 1 : 0);
  TORCH_CHECK(slots > 0, "gated_rmsnorm_bwd: bad shape");
  Tensor dx = torch::empty_like(dy);
  Tensor dz = z ? torch::empty_like(dy) : torch::empty({0}, x.options());
  Tensor partials = want_dweight ? torch::empty({slots, dim}, x.options().dtype(at::kFloat)) : torch::empty({0}, x.options().dtype(at::kFloat));
  check(lbi_gated_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), z ? z->data_ptr() : nullptr, weight.data_ptr<float>(), rstd.data_ptr<float>(),
                              dx.data_ptr(), z ? dz.data_ptr() : nullptr, want_dweight ? partials.data_ptr<float>() : nullptr, rows, frows,
                              (int)dim, (int)group_size, gate_first ? 1 : 0, x.scalar_type() == at::kBFloat16 ? 1 : 0, cur_stream()),
        "gated_rmsnorm_bwd");
  return {dx, dz, want_dweight ? partials.sum(0) : partials};
}

// SISO preprocessing.  q, k [B, L, G, 128] bf16 / fp32; biases [H, 128]; theta [B, L, H, S]; gamma, scale [B, L, H] (all fp32)
// -> (qr, kr [B, L, H, 128] bf16, qk_dot [B, L, H] fp32).
std::tuple<Tensor, Tensor, Tensor> siso_prep_fwd(const Tensor& q, const Tensor& k, const Tensor& q_bias, const Tensor& k_bias,
                                                 const Tensor& theta, const Tensor& gamma, const Tensor& scale) {
  CHECK_F32(q_bias);
  CHECK_F32(k_bias);
  CHECK_F32(theta);
  CHECK_F32(gamma);
  CHECK_F32(scale);
  TORCH_CHECK(q.is_cuda() && q.is_contiguous() && k.is_contiguous() && k.sizes() == q.sizes() && k.scalar_type() == q.scalar_type() &&
                  (q.scalar_type() == at::kBFloat16 || q.scalar_type() == at::kFloat) && q.dim() == 4 && q.size(3) == 128,
              "siso_prep: q, k must be contiguous [B, L, G, 128] bf16 / fp32");
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t batch = q.size(0), seq = q.size(1), groups = q.size(2), heads = q_bias.size(0), na = theta.size(3);
  TORCH_CHECK(theta.dim() == 4 && theta.size(0) == batch && theta.size(1) == seq && theta.size(2) == heads && gamma.numel() == batch * seq * heads &&
                  scale.numel() == gamma.numel() && k_bias.sizes() == q_bias.sizes() && q_bias.size(1) == 128,
              "siso_prep: shape mismatch");
  Tensor qr = torch::empty({batch, seq, heads, 128}, q.options().dtype(at::kBFloat16)), kr = torch::empty_like(qr);
  Tensor qk = torch::empty({batch, seq, heads}, gamma.options());
  check(lbi_siso_prep_fwd(q.data_ptr(), k.data_ptr(), q_bias.data_ptr<float>(), k_bias.data_ptr<float>(), theta.data_ptr<float>(),
                          gamma.data_ptr<float>(), scale.data_ptr<float>(), qr.data_ptr(), kr.data_ptr(), qk.data_ptr<float>(), batch * seq,
                          (int)groups, (int)heads, 128, (int)na, q.scalar_type() == at::kBFloat16 ? 1 : 0, cur_stream()),
        "siso_prep_fwd");
  return {qr, kr, qk};
}

// q, k, theta, gamma, scale: forward tensors of Bf sequences; dqr, dkr (fp32 or bf16), dqk: cotangents of B = P * Bf sequences.
// -> (dq, dk [B, L, G, 128] fp32, dq_bias, dk_bias [H, 128] (empty when !want_bias), dtheta [B, L, H, S], dgamma, dscale [B, L, H])
std::vector<Tensor> siso_prep_bwd(const Tensor& q, const Tensor& k, const Tensor& q_bias, const Tensor& k_bias, const Tensor& theta,
                                  const Tensor& gamma, const Tensor& scale, const Tensor& dqr, const Tensor& dkr, const Tensor& dqk,
                                  bool dkr_reversed, bool want_bias) {
  CHECK_F32(q_bias);
  CHECK_F32(k_bias);
  CHECK_F32(theta);
  CHECK_F32(gamma);
  CHECK_F32(scale);
  CHECK_F32(dqk);
  TORCH_CHECK(q.is_cuda() && q.is_contiguous() && k.is_contiguous() && k.sizes() == q.sizes() && k.scalar_type() == q.scalar_type() &&
                  (q.scalar_type() == at::kBFloat16 || q.scalar_type() == at::kFloat) && q.dim() == 4 && q.size(3) == 128,
              "siso_prep_bwd: q, k must be contiguous [B, L, G, 128] bf16 / fp32");
  TORCH_CHECK(dqr.is_cuda() && dqr.is_contiguous() && dkr.is_contiguous() && dkr.scalar_type() == dqr.scalar_type() &&
                  (dqr.scalar_type() == at::kBFloat16 || dqr.scalar_type() == at::kFloat) && dqr.dim() == 4,
              "siso_prep_bwd: dqr, dkr must be contiguous [B, L, H, 128] fp32 / bf16");
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t fbatch = q.size(0), batch = dqr.size(0), seq = q.size(1), groups = q.size(2), heads = q_bias.size(0), na = theta.size(3);
  TORCH_CHECK(batch % fbatch == 0 && dqr.numel() == batch * seq * heads * 128 && dqk.numel() == batch * seq * heads &&
                  theta.numel() == fbatch * seq * heads * na && gamma.numel() == fbatch * seq * heads && scale.numel() == gamma.numel(),
              "siso_prep_bwd: shape mismatch");
  int64_t dkr_pad = 0;
  if (dkr_reversed) {
    TORCH_CHECK(dkr.dim() == 4 && dkr.size(0) == batch && dkr.size(1) >= seq && dkr.size(2) == heads && dkr.size(3) == 128,
                "siso_prep_bwd: reversed dkr must be [B, Lp >= L, H, 128]");
    dkr_pad = dkr.size(1);
  } else {
    TORCH_CHECK(dkr.numel() == dqr.numel(), "siso_prep_bwd: dkr must match dqr");
  }
  auto f32 = gamma.options();
  Tensor dq = torch::empty({batch, seq, groups, 128}, f32), dk = torch::empty_like(dq);
  Tensor dtheta = torch::empty({batch, seq, heads, na}, f32);
  Tensor dgamma = torch::empty({batch, seq, heads}, f32), dscale = torch::empty_like(dgamma);
  const int blocks = lbi_siso_prep_blocks(batch * seq * groups);
  Tensor partials = want_bias ? torch::empty({blocks, 2, heads, 128}, f32) : torch::empty({0}, f32);
  check(lbi_siso_prep_bwd(q.data_ptr(), k.data_ptr(), q_bias.data_ptr<float>(), k_bias.data_ptr<float>(), theta.data_ptr<float>(),
                          gamma.data_ptr<float>(), scale.data_ptr<float>(), dqr.data_ptr(), dkr.data_ptr(), dqk.data_ptr<float>(),
                          dq.data_ptr<float>(), dk.data_ptr<float>(), dtheta.data_ptr<float>(), dgamma.data_ptr<float>(),
                          dscale.data_ptr<float>(), want_bias ? partials.data_ptr<float>() : nullptr, batch * seq, fbatch * seq, (int)seq,
                          (int)dkr_pad, (int)groups, (int)heads, 128, (int)na, q.scalar_type() == at::kBFloat16 ? 1 : 0,
                          dqr.scalar_type() == at::kBFloat16 ? 1 : 0, cur_stream()),
        "siso_prep_bwd");
  if (!want_bias) return {dq, dk, partials, partials, dtheta, dgamma, dscale};
  Tensor bias = partials.sum(0);
  return {dq, dk, bias.select(0, 0), bias.select(0, 1), dtheta, dgamma, dscale};
}

// ---- Mamba block glue (mamba_small.cu)
Tensor gate_silu_fwd(const Tensor& y, const Tensor& z) {
  CHECK_BF16(y);
  CHECK_BF16(z);
  TORCH_CHECK(z.sizes() == y.sizes() && y.numel() % 8 == 0, "gate_silu_fwd: y, z must have the same shape, numel % 8 == 0");
  c10::cuda::CUDAGuard guard(y.device());
  Tensor out = torch::empty_like(y);
  check(lbi_gate_silu_fwd(y.data_ptr(), z.data_ptr(), out.data_ptr(), y.numel(), cur_stream()), "gate_silu_fwd");
  return out;
}

// dz_out: optional [reps * rows, cols] bf16 view with unit column stride and any row stride (a column range of a wider
// cotangent matrix); dz is written there instead of into a fresh tensor.
std::tuple<Tensor, Tensor> gate_silu_bwd(const Tensor& dyg, const Tensor& y, const Tensor& z, const c10::optional<Tensor>& dz_out) {
  CHECK_BF16(dyg);
  CHECK_BF16(y);
  CHECK_BF16(z);
  TORCH_CHECK(z.sizes() == y.sizes() && y.dim() == 2 && y.size(1) % 8 == 0 && y.numel() > 0 && dyg.numel() % y.numel() == 0,
              "gate_silu_bwd: y, z [rows, cols] with cols % 8 == 0; dyg must hold a whole number of copies of y's shape");
  c10::cuda::CUDAGuard guard(y.device());
  const int64_t reps = dyg.numel() / y.numel(), cols = y.size(1);
  Tensor dy = torch::empty_like(dyg);
  Tensor dz;
  int64_t ld = cols;
  if (dz_out.has_value() && dz_out->defined()) {
    dz = *dz_out;
    TORCH_CHECK(dz.is_cuda() && dz.scalar_type() == at::kBFloat16 && dz.dim() == 2 && dz.size(0) == reps * y.size(0) && dz.size(1) == cols &&
                    dz.stride(1) == 1 && dz.stride(0) % 8 == 0 && dz.stride(0) >= cols && dz.storage_offset() % 8 == 0,
                "gate_silu_bwd: dz_out must be [reps * rows, cols] bf16, unit column stride, row stride and offset multiples of 8");
    ld = dz.stride(0);
  } else {
    dz = torch::empty_like(dyg);
  }
  check(lbi_gate_silu_bwd(dyg.data_ptr(), y.data_ptr(), z.data_ptr(), dy.data_ptr(), dz.data_ptr(), y.numel(), (int)reps, (int)cols, ld,
                          cur_stream()),
        "gate_silu_bwd");
  return {dy, dz};
}

// -> (dt, a, sig, adt, gamma, scale, tanh_angle, theta, sp_dt, sp_a, a_live)
std::vector<Tensor> siso_small_fwd(const Tensor& dd_dt, const Tensor& dd_a, const Tensor& trap, const Tensor& angles,
                                   const Tensor& dt_bias, double a_floor, int64_t batch, int64_t seq_len) {
  CHECK_F32(dd_dt);
  CHECK_F32(dd_a);
  CHECK_F32(trap);
  CHECK_F32(angles);
  CHECK_F32(dt_bias);
  c10::cuda::CUDAGuard guard(dd_dt.device());
  const int64_t heads = dt_bias.numel(), na = angles.size(-1);
  TORCH_CHECK(dd_dt.numel() == batch * seq_len * heads && dd_a.numel() == dd_dt.numel() && trap.numel() == dd_dt.numel() &&
                  angles.numel() == batch * seq_len * na && na <= 64,
              "siso_small_fwd: shape mismatch");
  auto f32 = dd_dt.options();
  std::vector<Tensor> out;
  for (int i = 0; i < 6; ++i) out.push_back(torch::empty({batch, seq_len, heads}, f32));
  out.push_back(torch::empty({batch, seq_len, na}, f32));
  out.push_back(torch::empty({batch, seq_len, heads, na}, f32));
  for (int i = 0; i < 3; ++i) out.push_back(torch::empty({batch, seq_len, heads}, f32));
  TORCH_CHECK(heads <= 32, "siso_small_fwd: at most 32 heads");
  Tensor seg_inc = torch::empty({batch, (int64_t)lbi_siso_small_fwd_segments((int)seq_len), heads, 64}, f32);
  check(lbi_siso_small_fwd(dd_dt.data_ptr<float>(), dd_a.data_ptr<float>(), trap.data_ptr<float>(), angles.data_ptr<float>(),
                           dt_bias.data_ptr<float>(), (float)a_floor, seg_inc.data_ptr<float>(), out[0].data_ptr<float>(), out[1].data_ptr<float>(),
                           out[2].data_ptr<float>(), out[3].data_ptr<float>(), out[4].data_ptr<float>(), out[5].data_ptr<float>(),
                           out[6].data_ptr<float>(), out[7].data_ptr<float>(), out[8].data_ptr<float>(), out[9].data_ptr<float>(),
                           out[10].data_ptr<float>(), (int)batch, (int)seq_len, (int)heads, (int)na, cur_stream()),
        "siso_small_fwd");
  return out;
}

// dt_raw [rows, heads] (bf16 / fp32, unit column stride, any row stride), bias [heads] -> (dt, slope) fp32 [rows, heads]
std::tuple<Tensor, Tensor> softplus_dt(const Tensor& dt_raw, const Tensor& bias, double lo, double hi) {
  CHECK_F32(bias);
  TORCH_CHECK(dt_raw.is_cuda() && dt_raw.dim() == 2 && dt_raw.stride(1) == 1 && dt_raw.stride(0) >= dt_raw.size(1) &&
                  (dt_raw.scalar_type() == at::kBFloat16 || dt_raw.scalar_type() == at::kFloat) && bias.numel() == dt_raw.size(1),
              "softplus_dt: dt_raw [rows, heads] bf16 / fp32 with unit column stride, bias [heads]");
  c10::cuda::CUDAGuard guard(dt_raw.device());
  auto f32 = dt_raw.options().dtype(at::kFloat);
  Tensor dt = torch::empty({dt_raw.size(0), dt_raw.size(1)}, f32), slope = torch::empty_like(dt);
  check(lbi_softplus_dt(dt_raw.data_ptr(), dt_raw.stride(0), dt_raw.scalar_type() == at::kBFloat16 ? 1 : 0, bias.data_ptr<float>(),
                        (float)lo, (float)hi, dt.data_ptr<float>(), slope.data_ptr<float>(), dt_raw.size(0), (int)dt_raw.size(1),
                        cur_stream()),
        "softplus_dt");
  return {dt, slope};
}

// -> (d_dd_dt, d_dd_a, d_trap [P * B * L, H], d_angles [P * B * L, S]) in fp32 or bf16
std::vector<Tensor> siso_small_bwd(const Tensor& dt, const Tensor& a, const Tensor& sig, const Tensor& tanh_a, const Tensor& sp_dt,
                                   const Tensor& sp_a, const Tensor& live, const Tensor& dadt, const Tensor& dtheta,
                                   const Tensor& dgamma, const Tensor& dscale, bool out_bf16) {
  CHECK_F32(dt);
  CHECK_F32(a);
  CHECK_F32(sig);
  CHECK_F32(tanh_a);
  CHECK_F32(sp_dt);
  CHECK_F32(sp_a);
  CHECK_F32(live);
  CHECK_F32(dadt);
  CHECK_F32(dtheta);
  CHECK_F32(dgamma);
  CHECK_F32(dscale);
  c10::cuda::CUDAGuard guard(dt.device());
  TORCH_CHECK(dt.dim() == 3 && tanh_a.dim() == 3, "siso_small_bwd: dt [B, L, H], tanh_angle [B, L, S]");
  const int64_t batch = dt.size(0), seq = dt.size(1), heads = dt.size(2), na = tanh_a.size(2);
  TORCH_CHECK(heads <= 32 && na <= 32, "siso_small_bwd: at most 32 heads and 32 angles");
  TORCH_CHECK(dadt.numel() % dt.numel() == 0 && dgamma.numel() == dadt.numel() && dscale.numel() == dadt.numel() &&
                  dtheta.numel() == dadt.numel() * na,
              "siso_small_bwd: cotangent shapes");
  const int64_t reps = dadt.numel() / dt.numel();
  auto opt = dt.options().dtype(out_bf16 ? at::kBFloat16 : at::kFloat);
  const int64_t rows = reps * batch * seq;
  Tensor d1 = torch::empty({rows, heads}, opt), d2 = torch::empty({rows, heads}, opt), d3 = torch::empty({rows, heads}, opt);
  Tensor d4 = torch::empty({rows, na}, opt);
  Tensor seg_sum = torch::empty({reps * batch, (int64_t)lbi_siso_small_segments((int)seq), heads, 32}, dt.options());
  check(lbi_siso_small_bwd(dt.data_ptr<float>(), a.data_ptr<float>(), sig.data_ptr<float>(), tanh_a.data_ptr<float>(),
                           sp_dt.data_ptr<float>(), sp_a.data_ptr<float>(), live.data_ptr<float>(), dadt.data_ptr<float>(),
                           dtheta.data_ptr<float>(), dgamma.data_ptr<float>(), dscale.data_ptr<float>(), seg_sum.data_ptr<float>(),
                           d1.data_ptr(), d2.data_ptr(),
                           d3.data_ptr(), d4.data_ptr(), (int)batch, (int)reps, (int)seq, (int)heads, (int)na, out_bf16 ? 1 : 0,
                           cur_stream()),
        "siso_small_bwd");
  return {d1, d2, d3, d4};
}

// Skinny fp32 linear maps (interface_jac.cu).  -> (y, pre) with pre empty unless want_pre
std::tuple<Tensor, Tensor> small_linear_fwd(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& bias, int64_t act, bool want_pre) {
  CHECK_F32(x);
  CHECK_F32(w);
  if (bias) CHECK_F32((*bias));
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && w.size(1) == x.size(1), "small_linear_fwd: x [B, din], w [dout, din]");
  Tensor y = torch::empty({x.size(0), w.size(0)}, x.options());
  Tensor pre = want_pre ? torch::empty_like(y) : torch::empty({0}, x.options());
  check(lbi_small_linear_fwd(x.data_ptr<float>(), w.data_ptr<float>(), bias ? bias->data_ptr<float>() : nullptr, y.data_ptr<float>(),
                             want_pre ? pre.data_ptr<float>() : nullptr, (int)x.size(0), (int)x.size(1), (int)w.size(0), (int)act,
                             cur_stream()),
        "small_linear_fwd");
  return {y, pre};
}

Tensor small_linear_dgrad(const Tensor& g, const Tensor& w) {
  CHECK_F32(g);
  CHECK_F32(w);
  c10::cuda::CUDAGuard guard(g.device());
  TORCH_CHECK(g.dim() == 2 && w.dim() == 2 && w.size(0) == g.size(1), "small_linear_dgrad: g [B, dout], w [dout, din]");
  Tensor gx = torch::empty({g.size(0), w.size(1)}, g.options());
  check(lbi_small_linear_dgrad(g.data_ptr<float>(), w.data_ptr<float>(), gx.data_ptr<float>(), (int)g.size(0), (int)w.size(1),
                               (int)w.size(0), cur_stream()),
        "small_linear_dgrad");
  return gx;
}

void small_linear_wgrad_(const Tensor& g, const Tensor& x, Tensor dw, c10::optional<Tensor> db) {
  CHECK_F32(g);
  CHECK_F32(x);
  CHECK_F32(dw);
  if (db) CHECK_F32((*db));
  c10::cuda::CUDAGuard guard(g.device());
  TORCH_CHECK(g.dim() == 2 && x.dim() == 2 && g.size(0) == x.size(0) && dw.numel() == g.size(1) * x.size(1) &&
                  (!db || db->numel() == g.size(1)),
              "small_linear_wgrad: g [B, dout], x [B, din], dw [dout, din], db [dout]");
  check(lbi_small_linear_wgrad(g.data_ptr<float>(), x.data_ptr<float>(), dw.data_ptr<float>(), db ? db->data_ptr<float>() : nullptr,
                               (int)g.size(0), (int)x.size(1), (int)g.size(1), cur_stream()),
        "small_linear_wgrad");
}

// Mamba-2 conv + SiLU.  x [n, C] bf16 -> (pre [n, C], act0 [n, c0], act1 [n, c1], act2 [n, c2]) bf16.
std::vector<Tensor> conv_silu_fwd(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& bias, int64_t seq_len, int64_t c0,
                                  int64_t c1, int64_t c2) {
  CHECK_BF16(x);
  CHECK_F32(w);
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && x.size(1) == c0 + c1 + c2 && w.dim() == 2 && w.size(0) == x.size(1), "conv_silu_fwd: shapes");
  if (bias) CHECK_F32((*bias));
  const int64_t n = x.size(0);
  Tensor pre = torch::empty_like(x);
  Tensor o0 = torch::empty({n, c0}, x.options()), o1 = torch::empty({n, c1}, x.options()), o2 = torch::empty({n, c2}, x.options());
  Tensor wt = w.t().contiguous();   // [W, C]: the kernels read a tap's weights of neighbouring channels with one load
  check(lbi_conv_silu_fwd(x.data_ptr(), wt.data_ptr<float>(), bias ? bias->data_ptr<float>() : nullptr, pre.data_ptr(), o0.data_ptr(),
                          o1.data_ptr(), o2.data_ptr(), (int)c0, (int)c1, (int)c2, n, (int)seq_len, (int)w.size(1), cur_stream()),
        "conv_silu_fwd");
  return {pre, o0, o1, o2};
}

static int is_f32_or_bf16(const Tensor& t, const char* what) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous() && (t.scalar_type() == at::kFloat || t.scalar_type() == at::kBFloat16), what,
              " must be a contiguous CUDA fp32 / bf16 tensor");
  return t.scalar_type() == at::kFloat ? 1 : 0;
}

// d0 [P n, c0], d1 [P n, c1], d2 [P n, c2]; pre [n, C] -> writes the conv-input cotangent into out[:, col0 : col0 + C] (bf16,
// out [P n, width_total]).
void conv_silu_bwd_(const Tensor& d0, const Tensor& d1, const Tensor& d2, const Tensor& pre, const Tensor& w, Tensor out, int64_t col0,
                    int64_t seq_len) {
  CHECK_BF16(pre);
  CHECK_BF16(out);
  CHECK_F32(w);
  c10::cuda::CUDAGuard guard(pre.device());
  const int f0 = is_f32_or_bf16(d0, "d0"), f1 = is_f32_or_bf16(d1, "d1"), f2 = is_f32_or_bf16(d2, "d2");
  TORCH_CHECK(f1 == f2, "conv_silu_bwd: d1, d2 must share a dtype");
  const int64_t tokens = d0.size(0), ftokens = pre.size(0), c0 = d0.size(1), c1 = d1.size(1), c2 = d2.size(1);
  TORCH_CHECK(pre.size(1) == c0 + c1 + c2 && d1.size(0) == tokens && d2.size(0) == tokens && out.dim() == 2 && out.size(0) == tokens &&
                  col0 % 8 == 0 && col0 + c0 + c1 + c2 <= out.size(1),
              "conv_silu_bwd: shapes");
  Tensor wt = w.t().contiguous();
  check(lbi_conv_silu_bwd(d0.data_ptr(), f0, d1.data_ptr(), d2.data_ptr(), f1, pre.data_ptr(), wt.data_ptr<float>(),
                          static_cast<at::BFloat16*>(out.data_ptr()) + col0, out.size(1), (int)c0, (int)c1, (int)c2, tokens, ftokens,
                          (int)seq_len, (int)w.size(1), cur_stream()),
        "conv_silu_bwd");
}

// -> (dw [C, W], db [C]) fp32
std::tuple<Tensor, Tensor> conv_silu_wgrad(const Tensor& d0, const Tensor& d1, const Tensor& d2, const Tensor& pre, const Tensor& x,
                                           int64_t width, int64_t seq_len) {
  CHECK_BF16(pre);
  CHECK_BF16(x);
  c10::cuda::CUDAGuard guard(pre.device());
  const int f0 = is_f32_or_bf16(d0, "d0"), f1 = is_f32_or_bf16(d1, "d1"), f2 = is_f32_or_bf16(d2, "d2");
  TORCH_CHECK(f1 == f2, "conv_silu_wgrad: d1, d2 must share a dtype");
  const int64_t tokens = pre.size(0), c0 = d0.size(1), c1 = d1.size(1), c2 = d2.size(1), ch = pre.size(1);
  TORCH_CHECK(d0.size(0) == tokens && d1.size(0) == tokens && d2.size(0) == tokens && x.sizes() == pre.sizes() && ch == c0 + c1 + c2,
              "conv_silu_wgrad: one direction, shapes must match");
  auto f32 = pre.options().dtype(at::kFloat);
  Tensor dw = torch::zeros({ch, width}, f32), db = torch::zeros({ch}, f32);
  check(lbi_conv_silu_wgrad(d0.data_ptr(), f0, d1.data_ptr(), d2.data_ptr(), f1, pre.data_ptr(), x.data_ptr(), dw.data_ptr<float>(),
                            db.data_ptr<float>(), (int)c0, (int)c1, (int)c2, tokens, (int)seq_len, (int)width, cur_stream()),
        "conv_silu_wgrad");
  return {dw, db};
}

// Weight / bias gradient of the plain depthwise causal conv (no activation): dy, x [tokens, C] bf16 -> (dw [C, W], db [C]) fp32.
// The conv + SiLU weight-gradient kernel with a null pre-activation.
std::tuple<Tensor, Tensor> causal_conv_wgrad(const Tensor& dy, const Tensor& x, int64_t width, int64_t seq_len) {
  CHECK_BF16(dy);
  CHECK_BF16(x);
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(dy.dim() == 2 && dy.sizes() == x.sizes() && dy.size(1) % 8 == 0 && width >= 1 && width <= 8 && seq_len > 0 &&
                  dy.size(0) % seq_len == 0,
              "causal_conv_wgrad: dy, x [tokens, C] with C % 8 == 0, width <= 8, tokens a multiple of seq_len");
  const int64_t tokens = dy.size(0), ch = dy.size(1);
  auto f32 = x.options().dtype(at::kFloat);
  Tensor dw = torch::zeros({ch, width}, f32), db = torch::zeros({ch}, f32);
  check(lbi_conv_silu_wgrad(dy.data_ptr(), 0, dy.data_ptr(), dy.data_ptr(), 0, nullptr, x.data_ptr(), dw.data_ptr<float>(),
                            db.data_ptr<float>(), (int)ch, 0, 0, tokens, (int)seq_len, (int)width, cur_stream()),
        "causal_conv_wgrad");
  return {dw, db};
}

// (((in_scale g) @ wa) o d) @ wb over a basis: g [B, P, din] fp32, wa [din, hidden], d [B, hidden] or none, wb [hidden, dout] or none.
Tensor interface_mlp_jac(const Tensor& g, const Tensor& wa, const c10::optional<Tensor>& d, const c10::optional<Tensor>& wb,
                         double in_scale) {
  CHECK_F32(g);
  CHECK_F32(wa);
  c10::cuda::CUDAGuard guard(g.device());
  TORCH_CHECK(g.dim() == 3 && wa.dim() == 2 && wa.size(0) == g.size(2), "interface_mlp_jac: g [B, P, din], wa [din, hidden]");
  const int64_t batch = g.size(0), p = g.size(1), din = g.size(2), hidden = wa.size(1);
  int64_t dout = hidden;
  if (d) {
    CHECK_F32((*d));
    TORCH_CHECK(d->dim() == 2 && d->size(0) == batch && d->size(1) == hidden, "interface_mlp_jac: d must be [B, hidden]");
  }
  if (wb) {
    CHECK_F32((*wb));
    TORCH_CHECK(wb->dim() == 2 && wb->size(0) == hidden, "interface_mlp_jac: wb must be [hidden, dout]");
    dout = wb->size(1);
  }
  Tensor out = torch::empty({batch, p, dout}, g.options());
  check(lbi_interface_mlp_jac(g.data_ptr<float>(), wa.data_ptr<float>(), d ? d->data_ptr<float>() : nullptr,
                              wb ? wb->data_ptr<float>() : nullptr, out.data_ptr<float>(), (int)batch, (int)p, (int)din, (int)hidden,
                              (int)dout, (float)in_scale, cur_stream()),
        "interface_mlp_jac");
  return out;
}

Tensor layernorm_jac(const Tensor& x, const c10::optional<Tensor>& weight, const Tensor& g, double eps, bool transpose, double out_scale) {
  CHECK_F32(x);
  CHECK_F32(g);
  c10::cuda::CUDAGuard guard(g.device());
  TORCH_CHECK(x.dim() == 2 && g.dim() == 3 && g.size(0) == x.size(0) && g.size(2) == x.size(1), "layernorm_jac: x [B, R], g [B, P, R]");
  if (weight) {
    CHECK_F32((*weight));
    TORCH_CHECK(weight->numel() == x.size(1), "layernorm_jac: weight must be [R]");
  }
  Tensor out = torch::empty_like(g);
  check(lbi_layernorm_jac(x.data_ptr<float>(), weight ? weight->data_ptr<float>() : nullptr, g.data_ptr<float>(), out.data_ptr<float>(),
                          (int)g.size(0), (int)g.size(1), (int)g.size(2), (float)eps, transpose ? 1 : 0, (float)out_scale, cur_stream()),
        "layernorm_jac");
  return out;
}

Tensor affine_suffix_scan(const Tensor& mats, const Tensor& offsets, const c10::optional<Tensor>& seed) {
  CHECK_F32(mats);
  CHECK_F32(offsets);
  c10::cuda::CUDAGuard guard(mats.device());
  const int b = (int)mats.size(0), k = (int)mats.size(1), r = (int)mats.size(2);
  Tensor g = torch::empty({b, k + 1, r}, mats.options());
  const float* sp = (seed.has_value() && seed->defined()) ? seed->data_ptr<float>() : nullptr;
  check(lbi_affine_suffix_scan(mats.data_ptr<float>(), offsets.data_ptr<float>(), sp, g.data_ptr<float>(), b, k, r,
                               cur_stream()),
        "affine_suffix_scan");
  return g;
}

// C = A @ B^T (both K-major by default).  a_t / b_t: the operand is given as its transpose ([K, rows] row-major).
Tensor gemm(const Tensor& a, const Tensor& b, bool a_t, bool b_t, bool out_fp32, const c10::optional<Tensor>& accumulate_into,
            int64_t splits) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16,
              "gemm operands must be CUDA bf16");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1, "gemm operands must be 2-D row-major");
  c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = a_t ? a.size(1) : a.size(0), K = a_t ? a.size(0) : a.size(1);
  const int64_t N = b_t ? b.size(1) : b.size(0), Kb = b_t ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "gemm reduction extents differ: ", K, " vs ", Kb);
  TORCH_CHECK(a.stride(0) % 8 == 0 && b.stride(0) % 8 == 0, "leading dimensions must be multiples of 8");
  TORCH_CHECK(((uintptr_t)a.data_ptr()) % 16 == 0 && ((uintptr_t)b.data_ptr()) % 16 == 0, "operands must be 16-byte aligned");
  TORCH_CHECK(!a_t || M % 64 == 0, "transposed A needs M % 64 == 0");
  TORCH_CHECK(!b_t || N % 64 == 0, "transposed B needs N % 64 == 0");
  Tensor c;
  bool acc = false;
  if (accumulate_into.has_value() && accumulate_into->defined()) {
    c = *accumulate_into;
    TORCH_CHECK(c.scalar_type() == at::kFloat && c.size(0) == M && c.size(1) == N && c.stride(1) == 1, "bad accumulator");
    out_fp32 = true;
    acc = true;
  } else if (splits > 1) {
    c = torch::zeros({M, N}, a.options().dtype(at::kFloat));
    out_fp32 = true;
  } else {
    c = torch::empty({M, N}, a.options().dtype(out_fp32 ? at::kFloat : at::kBFloat16));
  }
  TORCH_CHECK((c.stride(0) * (out_fp32 ? 4 : 2)) % 16 == 0, "C leading dimension must keep rows 16-byte aligned");
  Tensor st = status_word(a);
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  check(lbi_gemm_bf16(a.data_ptr(), b.data_ptr(), c.data_ptr(), (int)M, (int)N, (int)K, a.stride(0), b.stride(0),
                      c.stride(0), a_t ? 1 : 0, b_t ? 1 : 0, out_fp32 ? 1 : 0, acc ? 1 : 0, (int)splits,
                      st.data_ptr<int>(), sms, cur_stream()),
        "gemm_bf16");
  return c;
}

Tensor gemm_tn(const Tensor& a, const Tensor& b, bool out_fp32, const c10::optional<Tensor>& accumulate_into) {
  return gemm(a, b, false, false, out_fp32, accumulate_into, 1);
}

Tensor attn_pullback_packed(const Tensor& d_o, const Tensor& qkv, const Tensor& o, const Tensor& lse, int64_t batch,
                            int64_t seq_len, int64_t heads, int64_t head_dim, double scale,
                            const c10::optional<Tensor>& rope_cos, const c10::optional<Tensor>& rope_sin, bool rope_interleaved) {
  CHECK_LP16(d_o);
  CHECK_LP16(qkv);
  CHECK_LP16(o);
  CHECK_F32(lse);
  TORCH_CHECK(d_o.scalar_type() == qkv.scalar_type() && o.scalar_type() == qkv.scalar_type(), "attn_pullback: d_o, qkv, o must share a dtype");
  c10::cuda::CUDAGuard guard(d_o.device());
  const int64_t n = batch * seq_len;
  TORCH_CHECK(qkv.size(0) == n && qkv.size(1) == 3 * heads * head_dim, "qkv shape mismatch");
  TORCH_CHECK(d_o.size(0) % n == 0 && d_o.size(1) == heads * head_dim, "d_o shape mismatch");
  TORCH_CHECK(o.size(0) == n && o.size(1) == heads * head_dim, "o shape mismatch");
  TORCH_CHECK(lse.numel() == batch * heads * seq_len, "lse shape mismatch");
  const int64_t nbasis = d_o.size(0) / n;
  const float *cos_p = nullptr, *sin_p = nullptr;
  if (rope_cos.has_value()) {
    TORCH_CHECK(rope_sin.has_value(), "rope_sin missing");
    CHECK_F32(*rope_cos);
    CHECK_F32(*rope_sin);
    TORCH_CHECK(rope_cos->size(0) >= seq_len && rope_cos->size(1) == head_dim / 2 && rope_sin->sizes() == rope_cos->sizes(),
                "rope tables must be [seq_len, head_dim / 2]");
    cos_p = rope_cos->data_ptr<float>();
    sin_p = rope_sin->data_ptr<float>();
  }
  Tensor d_qkv = torch::empty({d_o.size(0), qkv.size(1)}, d_o.options());
  Tensor delta = torch::empty({nbasis, batch, heads, seq_len}, lse.options());
  Tensor st = status_word(d_o);
  check(lbi_attn_pullback(qkv.data_ptr(), d_o.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), d_qkv.data_ptr(),
                          delta.data_ptr<float>(), (int)batch, (int)heads, (int)seq_len, (int)head_dim, (int)nbasis,
                          (float)scale, cos_p, sin_p, rope_interleaved ? 1 : 0, qkv.scalar_type() == at::kHalf ? 1 : 0, st.data_ptr<int>(),
                          cur_stream()),
        "attn_pullback");
  return d_qkv;
}

std::tuple<Tensor, Tensor> attn_fwd_packed(const Tensor& qkv, int64_t batch, int64_t seq_len, int64_t heads, int64_t head_dim,
                                           double scale) {
  CHECK_LP16(qkv);
  c10::cuda::CUDAGuard guard(qkv.device());
  const int64_t n = batch * seq_len;
  TORCH_CHECK(qkv.dim() == 2 && qkv.size(0) == n && qkv.size(1) == 3 * heads * head_dim, "qkv shape mismatch");
  Tensor out = torch::empty({n, heads * head_dim}, qkv.options());
  Tensor lse = torch::empty({batch, heads, seq_len}, qkv.options().dtype(at::kFloat));
  Tensor st = status_word(qkv);
  check(lbi_attn_fwd(qkv.data_ptr(), out.data_ptr(), lse.data_ptr<float>(), (int)batch, (int)heads, (int)seq_len, (int)head_dim,
                     (float)scale, qkv.scalar_type() == at::kHalf ? 1 : 0, st.data_ptr<int>(), cur_stream()),
        "attn_fwd");
  return {out, lse};
}

// Mamba-2 SSD chunk scan forward.  x [B, L, H, 64] bf16, dt_raw [B, L, H] fp32, a [H] fp32, bm / cm [B, L, G, N] bf16.
// Returns (y [B, L, H, 64] bf16, final_state [B, H, 64, N] fp32).
std::tuple<Tensor, Tensor, Tensor> ssd_chunk_scan_fwd(const Tensor& x, const Tensor& dt_raw, const Tensor& a, const Tensor& bm, const Tensor& cm,
                                              const c10::optional<Tensor>& d_skip, const c10::optional<Tensor>& dt_bias,
                                              const c10::optional<Tensor>& init_state, bool softplus, double dt_min, double dt_max) {
  CHECK_BF16(x);
  CHECK_BF16(bm);
  CHECK_BF16(cm);
  CHECK_F32(dt_raw);
  CHECK_F32(a);
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 4 && bm.dim() == 4 && cm.dim() == 4 && dt_raw.dim() == 3, "ssd: expected x [B,L,H,P], B/C [B,L,G,N], dt [B,L,H]");
  const int64_t batch = x.size(0), seq = x.size(1), heads = x.size(2), hd = x.size(3), groups = bm.size(2), n = bm.size(3);
  TORCH_CHECK(cm.sizes() == bm.sizes() && dt_raw.size(0) == batch && dt_raw.size(1) == seq && dt_raw.size(2) == heads, "ssd: shape mismatch");
  const int64_t chunks = seq / 128;
  auto f32 = x.options().dtype(at::kFloat);
  Tensor dt = torch::empty({batch, heads, seq}, f32), cum = torch::empty({batch, heads, seq}, f32);
  Tensor states = torch::empty({batch, chunks, heads, hd, n}, f32);
  Tensor prev = torch::empty({batch, chunks, heads, hd, n}, x.options());
  Tensor final_state = torch::empty({batch, heads, hd, n}, f32);
  Tensor y = torch::empty_like(x);
  Tensor st = status_word(x);
  check(lbi_ssd_cumsum(dt_raw.data_ptr<float>(), dt_bias ? dt_bias->data_ptr<float>() : nullptr, a.data_ptr<float>(),
                       dt.data_ptr<float>(), cum.data_ptr<float>(), (int)batch, (int)seq, (int)heads, softplus ? 1 : 0, (float)dt_min,
                       (float)dt_max, cur_stream()),
        "ssd_cumsum");
  check(lbi_ssd_chunk_scan_fwd(x.data_ptr(), bm.data_ptr(), cm.data_ptr(), dt.data_ptr<float>(), cum.data_ptr<float>(),
                               d_skip ? d_skip->data_ptr<float>() : nullptr, init_state ? init_state->data_ptr<float>() : nullptr,
                               states.data_ptr<float>(), prev.data_ptr(), final_state.data_ptr<float>(), y.data_ptr(), (int)batch,
                               (int)seq, (int)heads, (int)groups, (int)hd, (int)n, st.data_ptr<int>(), cur_stream()),
        "ssd_chunk_scan_fwd");
  return {y, final_state, prev};
}

// Mamba-3 SISO chunk scan forward on preprocessed operands.  v [B, L, H, 64] bf16, kr / qr [B, L, H, 128] bf16,
// adt [B, L, H] fp32, skip_tok [B, H, L] fp32, d_skip [H] fp32.  Returns (y [B, L, H, 64] bf16, final_state [B, H, 128, 64]).
std::tuple<Tensor, Tensor, Tensor> siso_chunk_scan_fwd(const Tensor& v, const Tensor& kr, const Tensor& qr, const Tensor& adt,
                                               const c10::optional<Tensor>& d_skip, const c10::optional<Tensor>& skip_tok,
                                               const c10::optional<Tensor>& init_state) {
  CHECK_BF16(v);
  CHECK_BF16(kr);
  CHECK_BF16(qr);
  CHECK_F32(adt);
  c10::cuda::CUDAGuard guard(v.device());
  TORCH_CHECK(v.dim() == 4 && kr.dim() == 4 && qr.sizes() == kr.sizes() && adt.dim() == 3, "siso: expected v [B,L,H,P], kr/qr [B,L,H,N], adt [B,L,H]");
  const int64_t batch = v.size(0), seq = v.size(1), heads = v.size(2), hd = v.size(3), n = kr.size(3);
  TORCH_CHECK(kr.size(2) == heads && adt.size(1) == seq && adt.size(2) == heads, "siso: shape mismatch");
  const int64_t chunks = seq / 128;
  auto f32 = v.options().dtype(at::kFloat);
  Tensor ones = torch::ones({heads}, f32);
  Tensor dt = torch::empty({batch, heads, seq}, f32), cum = torch::empty({batch, heads, seq}, f32);
  Tensor states = torch::empty({batch, chunks, heads, n, hd}, f32);
  Tensor prev = torch::empty({batch, chunks, heads, n, hd}, v.options());
  Tensor final_state = torch::empty({batch, heads, n, hd}, f32);
  Tensor y = torch::empty_like(v);
  Tensor st = status_word(v);
  check(lbi_ssd_cumsum(adt.data_ptr<float>(), nullptr, ones.data_ptr<float>(), dt.data_ptr<float>(), cum.data_ptr<float>(), (int)batch,
                       (int)seq, (int)heads, 0, 0.f, 0.f, cur_stream()),
        "siso_cumsum");
  check(lbi_siso_chunk_scan_fwd(v.data_ptr(), kr.data_ptr(), qr.data_ptr(), cum.data_ptr<float>(),
                                d_skip ? d_skip->data_ptr<float>() : nullptr, skip_tok ? skip_tok->data_ptr<float>() : nullptr,
                                init_state ? init_state->data_ptr<float>() : nullptr, states.data_ptr<float>(), prev.data_ptr(),
                                final_state.data_ptr<float>(), y.data_ptr(), (int)batch, (int)seq, (int)heads, (int)hd, (int)n,
                                st.data_ptr<int>(), cur_stream()),
        "siso_chunk_scan_fwd");
  return {y, final_state, prev};
}

// The chunk scan with free operand roles.  v [B, L, H, 64] bf16; bk / cq [B, L, G, N] bf16 (per_head: G = H, N = 128);
// a [B, L, H] fp32 log-decay per token; weight [B, L, H] fp32 or none; skip_tok [B, H, L]; init [B, H, 64, N] (per_head:
// [B, H, N, 64]).  Returns (y [B, L, H, 64] in bf16 or fp32, final_state).
std::tuple<Tensor, Tensor, Tensor> ssd_scan_generic(const Tensor& v, const Tensor& bk, const Tensor& cq, const Tensor& a,
                                            const c10::optional<Tensor>& weight, const c10::optional<Tensor>& d_skip,
                                            const c10::optional<Tensor>& skip_tok, const c10::optional<Tensor>& init_state,
                                            bool strict, bool per_head, bool out_f32, int64_t v_div, int64_t v_mod) {
  CHECK_BF16(v);
  CHECK_BF16(bk);
  CHECK_BF16(cq);
  CHECK_F32(a);
  c10::cuda::CUDAGuard guard(v.device());
  TORCH_CHECK(v.dim() == 4 && bk.dim() == 4 && cq.sizes() == bk.sizes() && a.dim() == 3, "scan: expected v [B,L,H,64], bk/cq [B,L,G,N], a [B,L,H]");
  const int64_t batch = v.size(0), seq = v.size(1), heads = a.size(2), hd = v.size(3), groups = bk.size(2), n = bk.size(3);
  TORCH_CHECK(hd == 64 && a.size(0) == batch && a.size(1) == seq && bk.size(1) == seq, "scan: shape mismatch");
  TORCH_CHECK(v_div > 0 && v_mod > 0 && v.size(2) == ((heads - 1) / v_div) * v_mod + v_mod, "scan: v has the wrong number of 64-column blocks");
  TORCH_CHECK(!per_head || groups == heads, "scan: per_head wants one bk / cq per head");
  const int64_t chunks = seq / 128;
  auto f32 = v.options().dtype(at::kFloat);
  Tensor ones = torch::ones({heads}, f32);
  Tensor a_t = torch::empty({batch, heads, seq}, f32), cum = torch::empty({batch, heads, seq}, f32);
  Tensor w_t;
  if (weight) {
    CHECK_F32((*weight));
    TORCH_CHECK(weight->sizes() == a.sizes(), "scan: weight must match a");
    w_t = weight->transpose(1, 2).contiguous();
  }
  Tensor states = torch::empty({batch, chunks, heads, hd, n}, f32);
  Tensor prev = torch::empty({batch, chunks, heads, hd, n}, v.options());
  Tensor final_state = per_head ? torch::empty({batch, heads, n, hd}, f32) : torch::empty({batch, heads, hd, n}, f32);
  Tensor y = torch::empty({batch, seq, heads, hd}, out_f32 ? f32 : v.options());
  Tensor st = status_word(v);
  check(lbi_ssd_cumsum(a.data_ptr<float>(), nullptr, ones.data_ptr<float>(), a_t.data_ptr<float>(), cum.data_ptr<float>(), (int)batch,
                       (int)seq, (int)heads, 0, 0.f, 0.f, cur_stream()),
        "scan_cumsum");
  check(lbi_ssd_scan_generic(v.data_ptr(), bk.data_ptr(), cq.data_ptr(), weight ? w_t.data_ptr<float>() : nullptr,
                             cum.data_ptr<float>(), d_skip ? d_skip->data_ptr<float>() : nullptr,
                             skip_tok ? skip_tok->data_ptr<float>() : nullptr, strict ? 1 : 0,
                             init_state ? init_state->data_ptr<float>() : nullptr, states.data_ptr<float>(), prev.data_ptr(),
                             final_state.data_ptr<float>(), out_f32 ? nullptr : y.data_ptr(),
                             out_f32 ? y.data_ptr<float>() : nullptr, (int)batch, (int)seq, (int)heads, (int)groups, (int)n,
                             per_head ? 1 : 0, (int)v_div, (int)v_mod, st.data_ptr<int>(), cur_stream()),
        "ssd_scan_generic");
  return {y, final_state, prev};
}

// Log-decay gradient of the scan (see lbi_ssd_decay_grad).  v, gy [B, L, H, 64] bf16; bk / cq [B, L, G, N] bf16; a, weight
// [B, L, H] fp32; state_in / state_cot_rev: the third result of the forward and of the reversed scan.  Returns da [B, L, H].
Tensor ssd_decay_grad(const Tensor& v, const Tensor& gy, const Tensor& bk, const Tensor& cq, const Tensor& a,
                      const c10::optional<Tensor>& weight, const Tensor& state_in, const Tensor& state_cot_rev, bool per_head) {
  CHECK_BF16(v);
  CHECK_BF16(gy);
  CHECK_BF16(bk);
  CHECK_BF16(cq);
  CHECK_BF16(state_in);
  CHECK_BF16(state_cot_rev);
  CHECK_F32(a);
  c10::cuda::CUDAGuard guard(v.device());
  TORCH_CHECK(v.dim() == 4 && gy.sizes() == v.sizes() && bk.dim() == 4 && cq.sizes() == bk.sizes() && a.dim() == 3, "decay_grad: bad shapes");
  const int64_t batch = v.size(0), seq = v.size(1), heads = v.size(2), hd = v.size(3), groups = bk.size(2), n = bk.size(3);
  TORCH_CHECK(hd == 64 && a.size(0) == batch && a.size(1) == seq && a.size(2) == heads && bk.size(1) == seq, "decay_grad: shape mismatch");
  TORCH_CHECK(!per_head || groups == heads, "decay_grad: per_head wants one bk / cq per head");
  TORCH_CHECK(state_in.numel() == batch * (seq / 128) * heads * hd * n && state_cot_rev.numel() == state_in.numel(),
              "decay_grad: states must be [B, L/128, H, 64, N]");
  auto f32 = v.options().dtype(at::kFloat);
  Tensor ones = torch::ones({heads}, f32);
  Tensor a_t = torch::empty({batch, heads, seq}, f32), cum = torch::empty({batch, heads, seq}, f32);
  Tensor w_t;
  if (weight) {
    CHECK_F32((*weight));
    TORCH_CHECK(weight->sizes() == a.sizes(), "decay_grad: weight must match a");
    w_t = weight->transpose(1, 2).contiguous();
  }
  Tensor da = torch::empty({batch, heads, seq}, f32);
  Tensor st = status_word(v);
  check(lbi_ssd_cumsum(a.data_ptr<float>(), nullptr, ones.data_ptr<float>(), a_t.data_ptr<float>(), cum.data_ptr<float>(), (int)batch,
                       (int)seq, (int)heads, 0, 0.f, 0.f, cur_stream()),
        "decay_grad_cumsum");
  check(lbi_ssd_decay_grad(v.data_ptr(), gy.data_ptr(), bk.data_ptr(), cq.data_ptr(), weight ? w_t.data_ptr<float>() : nullptr,
                           cum.data_ptr<float>(), state_in.data_ptr(), state_cot_rev.data_ptr(), da.data_ptr<float>(), (int)batch,
                           (int)seq, (int)heads, (int)groups, (int)n, per_head ? 1 : 0, st.data_ptr<int>(), cur_stream()),
        "ssd_decay_grad");
  return da.transpose(1, 2);
}

// Fused chunk backward (lbi_ssd_chunk_bwd).  v [Bf, L, H, 64], bk / cq [Bf, L, G, N], a / weight / skip_tok [Bf, L, H], state_in: the
// third result of the forward scan; gy [P * Bf, L, H, 64].  Returns (dv [B, L, H, 64], dcq, dbk [B, L, H, N] per head, da, dskip
// [B, L, H]); dv in bf16 when `dv_bf16`, dcq and dbk in bf16 when `dn_bf16`, else fp32.
std::vector<Tensor> ssd_chunk_bwd(const Tensor& v, const Tensor& gy, const Tensor& bk, const Tensor& cq, const Tensor& a,
                                  const c10::optional<Tensor>& weight, const c10::optional<Tensor>& skip_tok,
                                  const c10::optional<Tensor>& d_skip, const Tensor& state_in, bool per_head, bool strict,
                                  bool dv_bf16, bool dn_bf16, const c10::optional<Tensor>& dv_out) {
  // dv_out: optional [B * L, H * 64] bf16 view with unit column stride and any row stride (a column range of a wider cotangent
  // matrix); with dv_bf16 the kernel's TMA stores write dv there instead of into a fresh tensor
  CHECK_BF16(v);
  CHECK_BF16(gy);
  CHECK_BF16(bk);
  CHECK_BF16(cq);
  CHECK_BF16(state_in);
  CHECK_F32(a);
  c10::cuda::CUDAGuard guard(v.device());
  TORCH_CHECK(v.dim() == 4 && gy.dim() == 4 && bk.dim() == 4 && cq.sizes() == bk.sizes() && a.dim() == 3, "chunk_bwd: bad shapes");
  const int64_t fbatch = v.size(0), batch = gy.size(0), seq = v.size(1), heads = v.size(2), hd = v.size(3), groups = bk.size(2), n = bk.size(3);
  TORCH_CHECK(hd == 64 && batch % fbatch == 0 && gy.size(1) == seq && gy.size(2) == heads && gy.size(3) == 64 && seq % 128 == 0 &&
                  bk.size(0) == fbatch && bk.size(1) == seq && a.size(0) == fbatch && a.size(1) == seq && a.size(2) == heads,
              "chunk_bwd: shape mismatch");
  TORCH_CHECK(!per_head || groups == heads, "chunk_bwd: per_head wants one bk / cq per head");
  const int64_t chunks = seq / 128;
  TORCH_CHECK(state_in.numel() == fbatch * chunks * heads * hd * n, "chunk_bwd: state_in must be [Bf, L/128, H, 64, N]");
  auto f32 = v.options().dtype(at::kFloat);
  Tensor ones = torch::ones({heads}, f32);
  Tensor a_t = torch::empty({fbatch, heads, seq}, f32), cum = torch::empty({fbatch, heads, seq}, f32);
  Tensor w_t, s_t;
  if (weight) {
    CHECK_F32((*weight));
    TORCH_CHECK(weight->sizes() == a.sizes(), "chunk_bwd: weight must match a");
    w_t = weight->transpose(1, 2).contiguous();
  }
  if (skip_tok) {
    CHECK_F32((*skip_tok));
    TORCH_CHECK(skip_tok->sizes() == a.sizes(), "chunk_bwd: skip_tok must match a");
    s_t = skip_tok->transpose(1, 2).contiguous();
  }
  if (d_skip) CHECK_F32((*d_skip));
  Tensor d_out = torch::empty({batch, chunks, heads, hd * n}, v.options());
  Tensor da = torch::empty({batch, heads, seq}, f32), dskip = torch::empty({batch, heads, seq}, f32);
  Tensor dv;
  int64_t dv_ld = 0;
  if (dv_out.has_value() && dv_out->defined()) {
    dv = *dv_out;
    TORCH_CHECK(dv_bf16 && dv.is_cuda() && dv.scalar_type() == at::kBFloat16 && dv.dim() == 2 && dv.size(0) == batch * seq &&
                    dv.size(1) == heads * hd && dv.stride(1) == 1 && dv.stride(0) % 8 == 0 && dv.stride(0) >= heads * hd &&
                    dv.storage_offset() % 8 == 0,
                "chunk_bwd: dv_out must be [B * L, H * 64] bf16, unit column stride, row stride and offset multiples of 8");
    dv_ld = dv.stride(0);
  } else {
    dv = torch::empty({batch, seq, heads, hd}, dv_bf16 ? v.options() : f32);
  }
  Tensor dcq = torch::empty({batch, seq, heads, n}, dn_bf16 ? v.options() : f32), dbk = torch::empty_like(dcq);
  Tensor st = status_word(v);
  check(lbi_ssd_cumsum(a.data_ptr<float>(), nullptr, ones.data_ptr<float>(), a_t.data_ptr<float>(), cum.data_ptr<float>(), (int)fbatch,
                       (int)seq, (int)heads, 0, 0.f, 0.f, cur_stream()),
        "chunk_bwd_cumsum");
  check(lbi_ssd_chunk_bwd(v.data_ptr(), gy.data_ptr(), bk.data_ptr(), cq.data_ptr(), weight ? w_t.data_ptr<float>() : nullptr,
                          cum.data_ptr<float>(), skip_tok ? s_t.data_ptr<float>() : nullptr,
                          d_skip ? d_skip->data_ptr<float>() : nullptr, state_in.data_ptr(), nullptr, nullptr,
                          d_out.data_ptr(), nullptr, da.data_ptr<float>(), dskip.data_ptr<float>(),
                          dv_bf16 ? nullptr : dv.data_ptr<float>(), dv_bf16 ? dv.data_ptr() : nullptr,
                          dn_bf16 ? nullptr : dcq.data_ptr<float>(), dn_bf16 ? nullptr : dbk.data_ptr<float>(),
                          dn_bf16 ? dcq.data_ptr() : nullptr, dn_bf16 ? dbk.data_ptr() : nullptr, (int)batch, (int)fbatch, (int)seq,
                          (int)heads, (int)groups, (int)n, per_head ? 1 : 0, strict ? 1 : 0, dv_ld, st.data_ptr<int>(), cur_stream()),
        "ssd_chunk_bwd");
  return {dv, dcq, dbk, da.transpose(1, 2), dskip.transpose(1, 2)};
}

// dx_rev [B, Lp, H, 64] fp32 (reversed time), x / gy [B, L, H, 64], dt [B, L, H], da [B, Lp, H] (a transposed view of the
// decay-gradient result), a_param [H], d_skip [H] or none -> (dx like x, ddt [B, L, H], dD [H] or empty).
std::tuple<Tensor, Tensor, Tensor> ssd_bwd_finish(const Tensor& dx_rev, const Tensor& x, const Tensor& gy, const Tensor& dt, const Tensor& da,
                                                  const Tensor& a_param, const c10::optional<Tensor>& d_skip, bool reversed) {
  TORCH_CHECK(dx_rev.is_cuda() && dx_rev.is_contiguous() && (dx_rev.scalar_type() == at::kFloat || dx_rev.scalar_type() == at::kBFloat16),
              "ssd_bwd_finish: dx_rev must be a contiguous CUDA fp32 / bf16 tensor");
  CHECK_F32(dt);
  CHECK_F32(a_param);
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && gy.is_contiguous() && gy.dim() == 4 && gy.scalar_type() == x.scalar_type() &&
                  (x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kFloat) && x.dim() == 4 && x.size(3) == 64 &&
                  gy.size(1) == x.size(1) && gy.size(2) == x.size(2) && gy.size(3) == 64 && gy.size(0) % x.size(0) == 0,
              "ssd_bwd_finish: x [Bf, L, H, 64], gy [P * Bf, L, H, 64], contiguous bf16 / fp32");
  const int64_t batch = gy.size(0), fbatch = x.size(0), seq = x.size(1), heads = x.size(2), seq_pad = dx_rev.size(1);
  TORCH_CHECK(dx_rev.dim() == 4 && dx_rev.size(0) == batch && dx_rev.size(2) == heads && dx_rev.size(3) == 64 && seq_pad >= seq,
              "ssd_bwd_finish: dx_rev must be [B, Lp, H, 64]");
  TORCH_CHECK(dt.sizes() == at::IntArrayRef({fbatch, seq, heads}), "ssd_bwd_finish: dt must be [Bf, L, H]");
  Tensor da_t = da.transpose(1, 2).contiguous();   // [B, H, Lp]; free when da is the transposed view the kernel returned
  TORCH_CHECK(da_t.scalar_type() == at::kFloat && da_t.size(0) == batch && da_t.size(1) == heads && da_t.size(2) == seq_pad,
              "ssd_bwd_finish: da must be [B, Lp, H] fp32");
  Tensor dx = torch::empty_like(gy);
  Tensor ddt = torch::empty({batch, seq, heads}, dt.options());
  Tensor dd = d_skip ? torch::zeros({heads}, dt.options()) : torch::empty({0}, dt.options());
  if (d_skip) CHECK_F32((*d_skip));
  check(lbi_ssd_bwd_finish(dx_rev.data_ptr(), dx_rev.scalar_type() == at::kBFloat16 ? 1 : 0, x.data_ptr(), gy.data_ptr(), dt.data_ptr<float>(), da_t.data_ptr<float>(),
                           a_param.data_ptr<float>(), d_skip ? d_skip->data_ptr<float>() : nullptr, dx.data_ptr(), ddt.data_ptr<float>(),
                           d_skip ? dd.data_ptr<float>() : nullptr, (int)batch, (int)seq, (int)seq_pad, (int)heads,
                           x.scalar_type() == at::kBFloat16 ? 1 : 0, reversed ? 1 : 0, (int)fbatch, cur_stream()),
        "ssd_bwd_finish");
  return {dx, ddt, dd};
}

// y [B, Lp, H, width] bf16 -> out [B, L, G, n] (bf16 or fp32): sum over the heads of each group, optional per-head weight
// w [B, L, H], optional time reversal of y.
Tensor ssd_group_sum(const Tensor& y, const c10::optional<Tensor>& w, int64_t seq_len, int64_t groups, int64_t n, bool reversed,
                     bool out_bf16) {
  CHECK_BF16(y);
  c10::cuda::CUDAGuard guard(y.device());
  TORCH_CHECK(y.dim() == 4, "ssd_group_sum: y must be [B, Lp, H, width]");
  const int64_t batch = y.size(0), seq_pad = y.size(1), heads = y.size(2), width = y.size(3);
  if (w) {
    CHECK_F32((*w));
    TORCH_CHECK(w->sizes() == at::IntArrayRef({batch, seq_len, heads}), "ssd_group_sum: w must be [B, L, H]");
  }
  Tensor out = torch::empty({batch, seq_len, groups, n}, y.options().dtype(out_bf16 ? at::kBFloat16 : at::kFloat));
  check(lbi_ssd_group_sum(y.data_ptr(), w ? w->data_ptr<float>() : nullptr, out.data_ptr(), (int)batch, (int)seq_len, (int)seq_pad,
                          (int)heads, (int)groups, (int)n, (int)width, reversed ? 1 : 0, out_bf16 ? 1 : 0, cur_stream()),
        "ssd_group_sum");
  return out;
}

// ---- peer-memory kernels.  `*_ptrs` are int64 CUDA tensors holding one device pointer per rank.
template <typename T>
T ptr_table(const Tensor& t) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kLong && t.is_contiguous(), "pointer table must be a CUDA int64 tensor");
  return reinterpret_cast<T>(t.data_ptr<int64_t>());
}

void set_peer_wait_limit_ms(int64_t ms) { check(lbi_peer_set_wait_limit_ms((int)ms), "set_peer_wait_limit_ms"); }

void peer_barrier(const Tensor& flag_ptrs, int64_t rank, int64_t world, int64_t slot_base, int64_t seq) {
  c10::cuda::CUDAGuard guard(flag_ptrs.device());
  Tensor st = status_word(flag_ptrs);
  check(lbi_peer_barrier(ptr_table<uint32_t* const*>(flag_ptrs), (int)rank, (int)world, (int)slot_base, (uint32_t)seq,
                         st.data_ptr<int>(), cur_stream()),
        "peer_barrier");
}

void peer_signal_all(const Tensor& flag_ptrs, int64_t rank, int64_t world, int64_t slot_base, int64_t seq) {
  c10::cuda::CUDAGuard guard(flag_ptrs.device());
  check(lbi_peer_signal_all(ptr_table<uint32_t* const*>(flag_ptrs), (int)rank, (int)world, (int)slot_base, (uint32_t)seq,
                            cur_stream()),
        "peer_signal_all");
}

// Returns (delta, pre_norm, state_out).  peer_state_ptr / peer_flag_ptr are raw device addresses (0 = local only).
std::tuple<Tensor, Tensor, Tensor> interface_update_handoff(
    const Tensor& state_in, const Tensor& pooled, const Tensor& w1, const c10::optional<Tensor>& b1,
    const c10::optional<Tensor>& w2, const c10::optional<Tensor>& b2, const Tensor& alpha, const Tensor& ln_w,
    const Tensor& ln_b, double ln_eps, int64_t act, int64_t peer_state_ptr, int64_t peer_flag_ptr, int64_t seq,
    const Tensor& done_counter) {
  CHECK_F32(state_in);
  CHECK_F32(pooled);
  CHECK_F32(w1);
  CHECK_F32(ln_w);
  CHECK_F32(ln_b);
  c10::cuda::CUDAGuard guard(state_in.device());
  const int batch = (int)state_in.size(0), width = (int)state_in.size(1), dim = (int)pooled.size(1);
  const bool two_layer = w2.has_value() && w2->defined();
  const int hidden = two_layer ? (int)w1.size(0) : 0;
  TORCH_CHECK(w1.size(1) == dim && (two_layer ? (w2->size(0) == width && w2->size(1) == hidden) : w1.size(0) == width),
              "interface map shapes do not match");
  Tensor delta = torch::empty_like(state_in), pre = torch::empty_like(state_in), out = torch::empty_like(state_in);
  Tensor hidden_buf = torch::empty({batch, std::max(hidden, 1)}, state_in.options());
  auto opt_ptr = [](const c10::optional<Tensor>& t) -> const float* {
    return (t.has_value() && t->defined()) ? t->data_ptr<float>() : nullptr;
  };
  check(lbi_interface_update_handoff(state_in.data_ptr<float>(), pooled.data_ptr<float>(), w1.data_ptr<float>(), opt_ptr(b1),
                                     opt_ptr(w2), opt_ptr(b2), alpha.data_ptr<float>(), ln_w.data_ptr<float>(),
                                     ln_b.data_ptr<float>(), (float)ln_eps, (int)act, batch, dim, hidden, width,
                                     hidden_buf.data_ptr<float>(), delta.data_ptr<float>(), pre.data_ptr<float>(), out.data_ptr<float>(),
                                     reinterpret_cast<float*>(peer_state_ptr), reinterpret_cast<uint32_t*>(peer_flag_ptr),
                                     (uint32_t)seq, reinterpret_cast<uint32_t*>(done_counter.data_ptr<int>()), cur_stream()),
        "interface_update_handoff");
  return {delta, pre, out};
}

Tensor wait_state(const Tensor& mailbox, const Tensor& flags, int64_t flag_index, int64_t seq) {
  CHECK_F32(mailbox);
  c10::cuda::CUDAGuard guard(mailbox.device());
  Tensor out = torch::empty_like(mailbox);
  Tensor st = status_word(mailbox);
  check(lbi_wait_state(mailbox.data_ptr<float>(), reinterpret_cast<const uint32_t*>(flags.data_ptr<int>()) + flag_index,
                       (uint32_t)seq, out.data_ptr<float>(), (int)mailbox.numel(), st.data_ptr<int>(), cur_stream()),
        "wait_state");
  return out;
}

Tensor affine_scan_peer(const Tensor& mats_ptrs, const Tensor& offs_ptrs, const Tensor& flags, int64_t slot_base, int64_t seq,
                        int64_t batch, int64_t world, int64_t k_local, int64_t r) {
  c10::cuda::CUDAGuard guard(flags.device());
  Tensor g = torch::empty({batch, world * k_local, r}, flags.options().dtype(at::kFloat));
  Tensor st = status_word(flags);
  check(lbi_affine_scan_peer(ptr_table<const float* const*>(mats_ptrs), ptr_table<const float* const*>(offs_ptrs),
                             reinterpret_cast<const uint32_t*>(flags.data_ptr<int>()), (int)slot_base, (uint32_t)seq,
                             g.data_ptr<float>(), (int)batch, (int)world, (int)k_local, (int)r, st.data_ptr<int>(),
                             cur_stream()),
        "affine_scan_peer");
  return g;
}

void peer_publish(const Tensor& src_a, const Tensor& dst_a_ptrs, const Tensor& segs_a, const Tensor& src_b, const Tensor& dst_b_ptrs,
                  const Tensor& segs_b, const Tensor& flag_ptrs, int64_t rank, int64_t world, int64_t slot_base, int64_t seq,
                  Tensor done_counter) {
  CHECK_F32(src_a);
  CHECK_F32(src_b);
  c10::cuda::CUDAGuard guard(src_a.device());
  TORCH_CHECK(segs_a.scalar_type() == at::kLong && segs_b.scalar_type() == at::kLong && segs_a.is_cuda() && segs_b.is_cuda() &&
                  segs_a.is_contiguous() && segs_b.is_contiguous() && done_counter.scalar_type() == at::kInt,
              "peer_publish: segment tables must be contiguous CUDA int64 [n, 2], the counter int32");
  check(lbi_peer_publish(src_a.data_ptr<float>(), ptr_table<float* const*>(dst_a_ptrs), segs_a.data_ptr<int64_t>(), (int)(segs_a.numel() / 2),
                         src_b.data_ptr<float>(), ptr_table<float* const*>(dst_b_ptrs), segs_b.data_ptr<int64_t>(), (int)(segs_b.numel() / 2),
                         ptr_table<uint32_t* const*>(flag_ptrs), (int)rank, (int)world, (int)slot_base, (uint32_t)seq,
                         reinterpret_cast<uint32_t*>(done_counter.data_ptr<int>()), cur_stream()),
        "peer_publish");
}

Tensor affine_scan_peer_sum(const Tensor& rows_ptrs, const Tensor& offs_ptrs, const Tensor& flags, int64_t slot_base, int64_t seq,
                            int64_t batch, int64_t world, int64_t k_total, int64_t r, int64_t flag_world) {
  c10::cuda::CUDAGuard guard(flags.device());
  Tensor g = torch::empty({batch, k_total, r}, flags.options().dtype(at::kFloat));
  Tensor st = status_word(flags);
  check(lbi_affine_scan_peer_sum(ptr_table<const float* const*>(rows_ptrs), ptr_table<const float* const*>(offs_ptrs),
                                 reinterpret_cast<const uint32_t*>(flags.data_ptr<int>()), (int)slot_base, (uint32_t)seq,
                                 g.data_ptr<float>(), (int)batch, (int)world, (int)k_total, (int)r, (int)(flag_world > 0 ? flag_world : world),
                                 st.data_ptr<int>(), cur_stream()),
        "affine_scan_peer_sum");
  return g;
}

void grad_reduce_scatter_(const Tensor& grad_ptrs, int64_t mc_ptr, int64_t rank, int64_t world, int64_t lo, int64_t n,
                          Tensor sumsq) {
  CHECK_F32(sumsq);
  c10::cuda::CUDAGuard guard(sumsq.device());
  check(lbi_grad_reduce_scatter(ptr_table<float* const*>(grad_ptrs), reinterpret_cast<const float*>(mc_ptr), (int)rank,
                                (int)world, lo, n, sumsq.data_ptr<float>(), cur_stream()),
        "grad_reduce_scatter");
}

void exchange_scalar(const Tensor& val_ptrs, const Tensor& flag_ptrs, const Tensor& mine, int64_t rank, int64_t world,
                     int64_t slot_base, int64_t seq) {
  CHECK_F32(mine);
  c10::cuda::CUDAGuard guard(mine.device());
  Tensor st = status_word(mine);
  check(lbi_exchange_scalar(ptr_table<float* const*>(val_ptrs), ptr_table<uint32_t* const*>(flag_ptrs), mine.data_ptr<float>(),
                            (int)rank, (int)world, (int)slot_base, (uint32_t)seq, st.data_ptr<int>(), cur_stream()),
        "exchange_scalar");
}

void adamw_allgather_(Tensor param, const Tensor& reduced_grad, Tensor m, Tensor v, const Tensor& shadow_ptrs, int64_t world,
                      int64_t lo, double lr, double beta1, double beta2, double eps, double weight_decay, int64_t step,
                      const Tensor& sumsq_parts, double clip_norm) {
  CHECK_F32(param);
  CHECK_F32(reduced_grad);
  CHECK_F32(m);
  CHECK_F32(v);
  CHECK_F32(sumsq_parts);
  c10::cuda::CUDAGuard guard(param.device());
  check(lbi_adamw_allgather(param.data_ptr<float>(), reduced_grad.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
                            ptr_table<void* const*>(shadow_ptrs), (int)world, lo, param.numel(), (float)lr, (float)beta1,
                            (float)beta2, (float)eps, (float)weight_decay, (int)step, sumsq_parts.data_ptr<float>(),
                            (float)clip_norm, cur_stream()),
        "adamw_allgather");
}

// Reads the device status word (non-zero: a bounded wait in some kernel ran out; the value names the site) and clears it.
int64_t kernel_status(const Tensor& like) {
  Tensor st = status_word(like);
  const int v = st.item<int>();
  if (v != 0) st.zero_();
  return v;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("add_rmsnorm_fwd", &add_rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("rmsnorm_bwd_lowp", &rmsnorm_bwd_lowp);
  m.def("rmsnorm_wgrad", &rmsnorm_wgrad);
  m.def("rope_qkv_", &rope_qkv_);
  m.def("gqa_expand", &gqa_expand);
  m.def("gqa_reduce", &gqa_reduce);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("add_condition", &add_condition);
  m.def("pool_tokens", &pool_tokens);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_scatter_add_", &embedding_scatter_add_);
  m.def("transpose_bf16", &transpose_bf16);
  m.def("causal_conv_fwd", &causal_conv_fwd);
  m.def("causal_conv_dgrad", &causal_conv_dgrad);
  m.def("sumsq_", &sumsq_);
  m.def("adamw_step_", &adamw_step_);
  m.def("ce_fwd_bwd_", &ce_fwd_bwd_);
  m.def("suffix_scan", &suffix_scan);
  m.def("affine_suffix_scan", &affine_suffix_scan);
  m.def("matrix_norms", &matrix_norms);
  m.def("interface_mlp_jac", &interface_mlp_jac);
  m.def("siso_prep_fwd", &siso_prep_fwd);
  m.def("siso_prep_bwd", &siso_prep_bwd, py::arg("q"), py::arg("k"), py::arg("q_bias"), py::arg("k_bias"), py::arg("theta"),
        py::arg("gamma"), py::arg("scale"), py::arg("dqr"), py::arg("dkr"), py::arg("dqk"), py::arg("dkr_reversed") = false,
        py::arg("want_bias") = true);
  m.def("bounds_violations", []() {
    return std::vector<int>{lbi_bounds_site_elementwise(), lbi_bounds_site_mamba_small()};
  });
#ifdef LBI_BOUNDS_CHECK
  m.attr("BOUNDS_CHECK") = true;
#else
  m.attr("BOUNDS_CHECK") = false;
#endif
  m.def("small_linear_fwd", &small_linear_fwd);
  m.def("small_linear_dgrad", &small_linear_dgrad);
  m.def("small_linear_wgrad_", &small_linear_wgrad_);
  m.def("conv_silu_fwd", &conv_silu_fwd);
  m.def("conv_silu_bwd_", &conv_silu_bwd_);
  m.def("conv_silu_wgrad", &conv_silu_wgrad);
  m.def("causal_conv_wgrad", &causal_conv_wgrad);
  m.def("gate_silu_fwd", &gate_silu_fwd);
  m.def("gate_silu_bwd", &gate_silu_bwd, py::arg("dyg"), py::arg("y"), py::arg("z"), py::arg("dz_out") = py::none());
  m.def("softplus_dt", &softplus_dt);
  m.def("siso_small_fwd", &siso_small_fwd);
  m.def("siso_small_bwd", &siso_small_bwd);
  m.def("gated_rmsnorm_fwd", &gated_rmsnorm_fwd);
  m.def("gated_rmsnorm_bwd", &gated_rmsnorm_bwd, py::arg("dy"), py::arg("x"), py::arg("z"), py::arg("weight"), py::arg("rstd"),
        py::arg("group_size"), py::arg("gate_first"), py::arg("want_dweight") = true);
  m.def("layernorm_jac", &layernorm_jac);
  m.def("gemm", &gemm, "bf16 tcgen05 GEMM", py::arg("a"), py::arg("b"), py::arg("a_t") = false, py::arg("b_t") = false,
        py::arg("out_fp32") = false, py::arg("accumulate_into") = py::none(), py::arg("splits") = 1);
  m.def("gemm_tn", &gemm_tn);
  m.def("attn_pullback_packed", &attn_pullback_packed, py::arg("d_o"), py::arg("qkv"), py::arg("o"), py::arg("lse"), py::arg("batch"),
        py::arg("seq_len"), py::arg("heads"), py::arg("head_dim"), py::arg("scale"), py::arg("rope_cos") = py::none(),
        py::arg("rope_sin") = py::none(), py::arg("rope_interleaved") = false);
  m.def("attn_fwd_packed", &attn_fwd_packed);
  m.def("ssd_chunk_scan_fwd", &ssd_chunk_scan_fwd);
  m.def("siso_chunk_scan_fwd", &siso_chunk_scan_fwd);
  m.def("ssd_scan_generic", &ssd_scan_generic);
  m.def("ssd_decay_grad", &ssd_decay_grad);
  m.def("ssd_bwd_finish", &ssd_bwd_finish, py::arg("dx_rev"), py::arg("x"), py::arg("gy"), py::arg("dt"), py::arg("da"),
        py::arg("a_param"), py::arg("d_skip"), py::arg("reversed") = true);
  m.def("ssd_chunk_bwd", &ssd_chunk_bwd, py::arg("v"), py::arg("gy"), py::arg("bk"), py::arg("cq"), py::arg("a"), py::arg("weight"),
        py::arg("skip_tok"), py::arg("d_skip"), py::arg("state_in"), py::arg("per_head"), py::arg("strict"), py::arg("dv_bf16"),
        py::arg("dn_bf16"), py::arg("dv_out") = py::none());
  m.def("ssd_group_sum", &ssd_group_sum);
  m.def("kernel_status", &kernel_status);
  m.def("set_peer_wait_limit_ms", &set_peer_wait_limit_ms);
  m.def("peer_barrier", &peer_barrier);
  m.def("peer_signal_all", &peer_signal_all);
  m.def("interface_update_handoff", &interface_update_handoff);
  m.def("wait_state", &wait_state);
  m.def("affine_scan_peer", &affine_scan_peer);
  m.def("affine_scan_peer_sum", &affine_scan_peer_sum, py::arg("rows_ptrs"), py::arg("offs_ptrs"), py::arg("flags"), py::arg("slot_base"),
        py::arg("seq"), py::arg("batch"), py::arg("world"), py::arg("k_total"), py::arg("r"), py::arg("flag_world") = 0);
  m.def("peer_publish", &peer_publish);
  m.def("grad_reduce_scatter_", &grad_reduce_scatter_);
  m.def("exchange_scalar", &exchange_scalar);
  m.def("adamw_allgather_", &adamw_allgather_);
}
