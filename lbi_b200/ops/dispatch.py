"""Routing between the sm_100a kernels and their PyTorch statements.

A CUDA tensor in a supported dtype/shape goes to the kernel; anything else
(CPU tensors, fp32 activations on the GPU, odd widths) runs the PyTorch
statement on whatever device the tensor lives on.  ``KERNEL_LAUNCHES`` counts
launches of this package's own kernels (bench.py reports it).
"""
from __future__ import annotations

import os

import torch

from . import reference as ref
from .native import ext, native_available

KERNEL_LAUNCHES = {"count": 0}
_LOWP = (torch.bfloat16, torch.float16)

# Routes that leave the sm_100a kernels for CUDA bf16 tensors (an odd shape, a missing entry point, an environment
# switch) are counted per op, so that a run cannot lose its kernels unnoticed; with LBI_B200_STRICT=1 (or
# ``set_strict(True)``) such a route raises instead.  CPU tensors and fp32 activations are not fallbacks: the PyTorch
# statements are their intended path.
FALLBACKS: dict[str, int] = {}
STRICT = {"enabled": os.environ.get("LBI_B200_STRICT", "0") == "1"}


def set_strict(enabled: bool) -> bool:
    """Turn strict mode on or off; returns the previous setting."""
    prev = STRICT["enabled"]
    STRICT["enabled"] = bool(enabled)
    return prev


def fell_back(op: str, *values, why: str = "") -> None:
    """Record that ``op`` is about to run library / PyTorch code; counts (and in strict mode refuses) CUDA bf16 operands."""
    if not any(isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.bfloat16 for t in values):
        return
    FALLBACKS[op] = FALLBACKS.get(op, 0) + 1
    if STRICT["enabled"]:
        shapes = [tuple(t.shape) for t in values if isinstance(t, torch.Tensor)]
        raise RuntimeError(f"strict mode: {op} would leave the sm_100a kernels for CUDA bf16 operands {shapes}" + (f" ({why})" if why else ""))


def _count(n: int = 1) -> None:
    KERNEL_LAUNCHES["count"] += n


def _native(*tensors) -> bool:
    return native_available() and all(t is None or t.is_cuda for t in tensors)


# ---------------------------------------------------------------- RMSNorm
def add_rmsnorm_fwd(branch, stream, weight, eps, out_dtype):
    if _native(branch, stream, weight) and out_dtype == torch.bfloat16 and branch.shape[-1] % 8 == 0:
        _count()
        return ext().add_rmsnorm_fwd(branch.contiguous(), stream, weight.contiguous(), float(eps))
    fell_back("add_rmsnorm_fwd", branch, stream, weight, eps, out_dtype)
    return ref.add_rmsnorm_fwd(branch, stream, weight, eps, out_dtype)


def rmsnorm_bwd(d_normed, stream, rstd, weight, d_stream=None, lowp_dtype=None):
    """d_stream (+)= J^T d_normed.  With ``lowp_dtype`` also returns the result cast to that dtype (one pass on CUDA)."""
    native = _native(d_normed, stream, rstd, weight, d_stream) and d_normed.dtype == torch.bfloat16 and d_normed.shape[-1] % 8 == 0
    if native and lowp_dtype == torch.bfloat16 and hasattr(ext(), "rmsnorm_bwd_lowp"):
        _count()
        return ext().rmsnorm_bwd_lowp(d_normed.contiguous(), stream, rstd, weight.contiguous(), d_stream)
    if native:
        _count()
        out = ext().rmsnorm_bwd(d_normed.contiguous(), stream, rstd, weight.contiguous(), d_stream)
    else:
        fell_back("rmsnorm_bwd", d_normed)
        out = ref.rmsnorm_bwd(d_normed, stream, rstd, weight, d_stream)
    return out if lowp_dtype is None else (out, out.to(lowp_dtype))


def rmsnorm_wgrad(d_normed, stream, rstd):
    if _native(d_normed, stream, rstd) and d_normed.dtype == torch.bfloat16 and d_normed.shape[-1] % 8 == 0:
        _count(2)
        return ext().rmsnorm_wgrad(d_normed.contiguous(), stream, rstd)
    fell_back("rmsnorm_wgrad", d_normed, stream, rstd)
    return ref.rmsnorm_wgrad(d_normed, stream, rstd)


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        shape = x.shape
        rows = x.reshape(-1, shape[-1])
        normed, stream, rstd = add_rmsnorm_fwd(rows, None, weight, eps, torch.bfloat16 if x.dtype in _LOWP else x.dtype)
        ctx.save_for_backward(stream, rstd, weight)
        ctx.in_dtype = x.dtype
        return normed.to(x.dtype).reshape(shape)

    @staticmethod
    def backward(ctx, grad_out):
        stream, rstd, weight = ctx.saved_tensors
        g = grad_out.reshape(-1, grad_out.shape[-1])
        dx = rmsnorm_bwd(g, stream, rstd, weight).to(ctx.in_dtype).reshape(grad_out.shape)
        dw = rmsnorm_wgrad(g, stream, rstd).to(weight.dtype)
        return dx, dw, None


def rmsnorm(x, weight, eps):
    """Autograd-aware RMSNorm used by ``nn.Module`` code paths."""
    if x.is_cuda and x.dtype == torch.bfloat16 and native_available() and x.shape[-1] % 8 == 0:
        return _RMSNormFn.apply(x, weight, eps)
    xf = x.float()
    rstd = torch.rsqrt(xf.square().mean(dim=-1, keepdim=True) + eps)
    return (xf * rstd).to(dtype=x.dtype) * weight.to(dtype=x.dtype)


# ---------------------------------------------------------------- linear (tcgen05 GEMM)
GEMM_NATIVE = {"enabled": os.environ.get("LBI_B200_LIBRARY_GEMM", "0") != "1"}


def _gemm_ok(a, b) -> bool:
    return (
        GEMM_NATIVE["enabled"]
        and _native(a, b)
        and a.dtype == torch.bfloat16
        and b.dtype == torch.bfloat16
        and a.dim() == 2
        and b.dim() == 2
        and a.shape[1] % 8 == 0
        and a.stride(1) == 1
        and b.stride(1) == 1
        and a.stride(0) % 8 == 0
        and b.stride(0) % 8 == 0
        and a.data_ptr() % 16 == 0
        and b.data_ptr() % 16 == 0
        and hasattr(ext(), "gemm_tn")
    )


def gemm_tn(a, b, out_dtype=torch.bfloat16, accumulate_into=None):
    """C[M, N] = A[M, K] @ B[N, K]^T with fp32 accumulation (both operands K-major)."""
    if _gemm_ok(a, b) and (out_dtype in (torch.bfloat16, torch.float32)):
        _count()
        return ext().gemm_tn(a, b, out_dtype == torch.float32, accumulate_into)
    fell_back("gemm_tn", a, b)
    c = (a.float() @ b.float().t()) if out_dtype == torch.float32 else (a @ b.t().to(a.dtype))
    if accumulate_into is not None:
        accumulate_into.add_(c.to(accumulate_into.dtype))
        return accumulate_into
    return c.to(out_dtype)


def linear_fwd(x, w, bias=None):
    if bias is None and _gemm_ok(x, w):
        return gemm_tn(x, w)
    fell_back("linear_fwd", x, w, bias)
    return ref.linear_fwd(x, w, bias)


# MN-major operand support of the GEMM lets dgrad and wgrad read W, dY and X as stored (no transposed copies).
GEMM_MN_MAJOR = {"enabled": True}


def _mn_ok(t) -> bool:
    return t.dim() == 2 and t.stride(1) == 1 and t.shape[1] % 64 == 0 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0


def linear_dgrad(dy, w, w_t=None):
    """dx = dy @ w with w stored [out, in].  Uses the MN-major B path of the GEMM; ``w_t`` ([in, out]) is an
    optional pre-transposed copy for the K-major path."""
    if GEMM_MN_MAJOR["enabled"] and _gemm_ok(dy, dy) and _native(w) and w.dtype == torch.bfloat16 and _mn_ok(w):
        _count()
        return ext().gemm(dy, w, False, True, False, None, 1)
    if w_t is not None and _gemm_ok(dy, w_t):
        return gemm_tn(dy, w_t)
    fell_back("linear_dgrad", dy, w)
    return ref.linear_dgrad(dy, w)


def linear_wgrad(dy, x, accumulate_into=None):
    """dW[out, in] = dy^T @ x with fp32 accumulation (split-K over the token rows)."""
    if GEMM_NATIVE["enabled"] and _native(dy, x) and dy.dtype == torch.bfloat16 and x.dtype == torch.bfloat16:
        if GEMM_MN_MAJOR["enabled"] and _mn_ok(dy) and _mn_ok(x):
            tiles = max(1, (dy.shape[1] // 128) * max(1, x.shape[1] // 256))
            splits = max(1, min(16, 148 // tiles, dy.shape[0] // 512))
            _count()
            return ext().gemm(dy, x, True, True, True, accumulate_into, splits)
        dy_t = transpose_2d(dy)
        x_t = transpose_2d(x)
        if _gemm_ok(dy_t, x_t):
            return gemm_tn(dy_t, x_t, out_dtype=torch.float32, accumulate_into=accumulate_into)
    fell_back("linear_wgrad", dy, x)
    dw = ref.linear_wgrad(dy, x)
    if accumulate_into is not None:
        accumulate_into.add_(dw)
        return accumulate_into
    return dw


def transpose_2d(x):
    if _native(x) and x.dtype == torch.bfloat16 and x.is_contiguous() and hasattr(ext(), "transpose_bf16"):
        _count()
        return ext().transpose_bf16(x)
    fell_back("transpose_2d", x)
    return x.t().contiguous()


# ---------------------------------------------------------------- RoPE
def rope_qkv(qkv, cos, sin, n_heads, n_kv_heads, head_dim, seq_len, interleaved=False, inverse=False):
    if _native(qkv, cos, sin) and qkv.dtype == torch.bfloat16 and qkv.is_contiguous() and head_dim % 2 == 0:
        _count()
        return ext().rope_qkv_(qkv, cos, sin, n_heads, n_kv_heads, head_dim, seq_len, bool(interleaved), bool(inverse))
    fell_back("rope_qkv", qkv, cos, sin, n_heads, n_kv_heads, head_dim, seq_len, interleaved, inverse)
    return ref.rope_qkv(qkv, cos, sin, n_heads, n_kv_heads, head_dim, seq_len, interleaved, inverse)


# ---------------------------------------------------------------- attention
def attention_fwd(qkv, batch, seq_len, n_heads, n_kv_heads, head_dim, scale):
    if qkv.is_cuda and qkv.dtype in _LOWP:
        from .attention import flash_forward_packed

        return flash_forward_packed(qkv, batch, seq_len, n_heads, n_kv_heads, head_dim, scale)
    fell_back("attention_fwd", qkv, batch, seq_len, n_heads, n_kv_heads, head_dim, scale)
    return ref.attention_fwd(qkv, batch, seq_len, n_heads, n_kv_heads, head_dim, scale)


def attention_pullback_packed(do_rows, qkv, o, lse, batch, seq_len, n_heads, n_kv_heads, head_dim, scale, rope=None):
    """``rope = (cos, sin, interleaved)``: also rotate dq and dk back (fused into the kernel epilogue where possible)."""
    if do_rows.is_cuda and do_rows.dtype in _LOWP:
        from .attention import pullback_packed

        return pullback_packed(do_rows, qkv, o, lse, batch, seq_len, n_heads, n_kv_heads, head_dim, scale, rope=rope)
    fell_back("attention_pullback_packed", do_rows)
    d_qkv = ref.attention_pullback_packed(do_rows, qkv, o, lse, batch, seq_len, n_heads, n_kv_heads, head_dim, scale)
    if rope is not None:
        d_qkv = rope_qkv(d_qkv, rope[0], rope[1], n_heads, n_kv_heads, head_dim, seq_len, rope[2], inverse=True)
    return d_qkv


def attention_bwd_packed(do_rows, qkv, o, lse, batch, seq_len, n_heads, n_kv_heads, head_dim, scale):
    """Single-cotangent backward (P = 1) used by parameter VJPs."""
    return attention_pullback_packed(do_rows, qkv, o, lse, batch, seq_len, n_heads, n_kv_heads, head_dim, scale)


# ---------------------------------------------------------------- SwiGLU
def swiglu_fwd(u):
    if _native(u) and u.dtype == torch.bfloat16 and u.is_contiguous() and (u.shape[-1] // 2) % 8 == 0:
        _count()
        return ext().swiglu_fwd(u)
    fell_back("swiglu_fwd", u)
    return ref.swiglu_fwd(u)


def swiglu_bwd(da, u):
    if _native(da, u) and da.dtype == torch.bfloat16 and u.dtype == torch.bfloat16 and da.is_contiguous() and da.shape[-1] % 8 == 0:
        _count()
        return ext().swiglu_bwd(da, u)
    fell_back("swiglu_bwd", da, u)
    return ref.swiglu_bwd(da, u)


# ---------------------------------------------------------------- conv
def causal_conv_fwd(x, weight, bias, batch, seq_len):
    if _native(x, weight, bias) and x.dtype == torch.bfloat16 and hasattr(ext(), "causal_conv_fwd"):
        _count()
        return ext().causal_conv_fwd(x.contiguous(), weight.float().contiguous(), bias, batch, seq_len)
    fell_back("causal_conv_fwd", x, weight, bias, batch, seq_len)
    return ref.causal_conv_fwd(x, weight, bias, batch, seq_len)


def causal_conv_dgrad(dy, weight, batch, seq_len):
    if _native(dy, weight) and dy.dtype == torch.bfloat16 and hasattr(ext(), "causal_conv_dgrad"):
        _count()
        return ext().causal_conv_dgrad(dy.contiguous(), weight.float().contiguous(), batch, seq_len)
    fell_back("causal_conv_dgrad", dy, weight, batch, seq_len)
    return ref.causal_conv_dgrad(dy, weight, batch, seq_len)


def causal_conv_wgrad(dy, x, width, batch, seq_len):
    if (_native(dy, x) and dy.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and dy.shape == x.shape and dy.shape[-1] % 8 == 0
            and width <= 8 and hasattr(ext(), "causal_conv_wgrad")):
        _count()
        return ext().causal_conv_wgrad(dy.contiguous(), x.contiguous(), int(width), int(seq_len))
    fell_back("causal_conv_wgrad", dy, x, width, batch, seq_len)
    return ref.causal_conv_wgrad(dy, x, width, batch, seq_len)


# ---------------------------------------------------------------- LM head + CE
def lm_head_cross_entropy(normed, weight, targets, loss_scale, want_dweight=True, weight_t=None, dweight_into=None):
    if (GEMM_NATIVE["enabled"] and _native(normed, weight, targets) and normed.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and weight.shape[0] % 64 == 0 and normed.shape[1] % 64 == 0):
        from .cross_entropy import fused_lm_head_ce

        return fused_lm_head_ce(normed, weight, targets, loss_scale, want_dweight, weight_t, dweight_into)
    fell_back("lm_head_cross_entropy", normed, weight, targets, loss_scale, want_dweight, dweight_into)
    return ref.lm_head_cross_entropy(normed, weight, targets, loss_scale, want_dweight, dweight_into)


# ---------------------------------------------------------------- embedding
def embedding_fwd(ids, table, out_dtype):
    if _native(ids, table) and out_dtype == torch.bfloat16 and table.dtype in (torch.bfloat16, torch.float32) and table.shape[1] % 8 == 0:
        _count()
        return ext().embedding_fwd(ids.reshape(-1).contiguous(), table)
    fell_back("embedding_fwd", ids, table, out_dtype)
    return ref.embedding_fwd(ids, table, out_dtype)


def embedding_scatter_add(d_table, ids, d_rows):
    if _native(d_table, ids, d_rows) and d_table.dtype == torch.float32 and d_rows.dtype in (torch.float32, torch.bfloat16):
        _count()
        ext().embedding_scatter_add_(d_table, ids.reshape(-1).contiguous(), d_rows.contiguous())
        return d_table
    fell_back("embedding_scatter_add", d_table, ids, d_rows)
    return ref.embedding_scatter_add(d_table, ids, d_rows)


# ---------------------------------------------------------------- interface glue
def add_condition(canvas_rows, cond, seq_len):
    if _native(canvas_rows, cond) and canvas_rows.dtype == torch.bfloat16 and canvas_rows.shape[-1] % 8 == 0:
        _count()
        return ext().add_condition(canvas_rows.contiguous(), cond.float().contiguous(), seq_len)
    fell_back("add_condition", canvas_rows, cond, seq_len)
    return ref.add_condition(canvas_rows, cond, seq_len)


def mean_pool_tokens(rows, batch, seq_len):
    if _native(rows) and rows.dtype in (torch.float32, torch.bfloat16) and rows.is_contiguous():
        _count()
        return ext().pool_tokens(rows, batch, seq_len, 1.0 / float(seq_len))
    fell_back("mean_pool_tokens", rows, batch, seq_len)
    return ref.mean_pool_tokens(rows, batch, seq_len)


def sum_tokens(rows, groups, seq_len):
    if _native(rows) and rows.dtype in (torch.float32, torch.bfloat16) and rows.is_contiguous():
        _count()
        return ext().pool_tokens(rows, groups, seq_len, 1.0)
    fell_back("sum_tokens", rows, groups, seq_len)
    return ref.sum_tokens(rows, groups, seq_len)


# ---------------------------------------------------------------- scans
def suffix_scan_pullbacks(mats):
    if _native(mats) and mats.dim() == 4 and mats.shape[1] > 0 and mats.shape[-1] <= 256:
        _count()
        return ext().suffix_scan(mats.contiguous())
    fell_back("suffix_scan_pullbacks", mats)
    return ref.suffix_scan_pullbacks(mats)


def affine_suffix_scan(mats, offsets, seed=None):
    if _native(mats, offsets, seed) and mats.shape[1] > 0 and mats.shape[-1] <= 1024:
        _count()
        return ext().affine_suffix_scan(mats.float().contiguous(), offsets.float().contiguous(), None if seed is None else seed.float().contiguous())
    fell_back("affine_suffix_scan", mats, offsets, seed)
    return ref.affine_suffix_scan(mats, offsets, seed)


# ---------------------------------------------------------------- optimizer
def adamw_step(param, grad, exp_avg, exp_avg_sq, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0, shadow=None):
    if _native(param, grad, exp_avg, exp_avg_sq, shadow) and param.dtype == torch.float32:
        _count()
        ext().adamw_step_(param, grad, exp_avg, exp_avg_sq, shadow, float(lr), float(beta1), float(beta2), float(eps),
                          float(weight_decay), int(step), grad_scale)
        return param
    gs = float(grad_scale) if not torch.is_tensor(grad_scale) else grad_scale
    fell_back("adamw_step", param, grad, exp_avg, exp_avg_sq, lr, beta1, beta2, eps, weight_decay, step, gs, shadow)
    return ref.adamw_step(param, grad, exp_avg, exp_avg_sq, lr, beta1, beta2, eps, weight_decay, step, gs, shadow)
