"""Plain PyTorch fp32 statements of every fused op.

These are the oracles the CUDA kernels are tested against, and the code path
that runs on CPU tensors.  Shapes use flattened rows: ``n = B * T`` token rows
for activations and ``P * n`` rows for a basis of P cotangents laid out
basis-major, so cached activations are indexed by ``row % n``.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def _bcast_rows(act: torch.Tensor, rows: int) -> torch.Tensor:
    n = act.shape[0]
    if rows == n:
        return act
    if rows % n != 0:
        raise ValueError(f"cotangent rows ({rows}) must be a multiple of activation rows ({n})")
    return act.unsqueeze(0).expand(rows // n, *act.shape).reshape(rows, *act.shape[1:])


# ---------------------------------------------------------------- RMSNorm (+ residual add)
def add_rmsnorm_fwd(branch, stream, weight, eps, out_dtype):
    new_stream = branch.float() if stream is None else branch.float() + stream.float()
    rstd = torch.rsqrt(new_stream.square().mean(dim=-1) + eps)
    normed = (new_stream * rstd.unsqueeze(-1) * weight.float()).to(out_dtype)
    return normed, new_stream, rstd


def rmsnorm_bwd(d_normed, stream, rstd, weight, d_stream=None):
    """dx of y = x * rstd * w; added onto ``d_stream`` when given.  Returns fp32."""
    rows = d_normed.shape[0]
    x = _bcast_rows(stream, rows).float()
    r = _bcast_rows(rstd, rows).float().unsqueeze(-1)
    gw = d_normed.float() * weight.float()
    xhat = x * r
    dx = r * (gw - xhat * (gw * xhat).mean(dim=-1, keepdim=True))
    return dx if d_stream is None else d_stream.float() + dx


def rmsnorm_wgrad(d_normed, stream, rstd):
    return (d_normed.float() * stream.float() * rstd.float().unsqueeze(-1)).sum(dim=0)


# ---------------------------------------------------------------- linear
def linear_fwd(x, w, bias=None):
    return F.linear(x, w.to(x.dtype), None if bias is None else bias.to(x.dtype))


def linear_dgrad(dy, w):
    return dy @ w.to(dy.dtype)


def linear_wgrad(dy, x):
    return dy.float().t() @ x.float()


# ---------------------------------------------------------------- RoPE on a packed qkv buffer
def rope_qkv(qkv, cos, sin, n_heads, n_kv_heads, head_dim, seq_len, interleaved=False, inverse=False):
    """Rotate the q and k heads of qkv [rows, (H + 2 Hkv) * Dh]; position = row % seq_len.  Returns a new tensor."""
    rows = qkv.shape[0]
    n_rot = n_heads + n_kv_heads
    pos = torch.arange(rows, device=qkv.device) % seq_len
    c = cos[pos].unsqueeze(1).float()
    s = sin[pos].unsqueeze(1).float()
    if inverse:
        s = -s
    rot = qkv[:, : n_rot * head_dim].float().reshape(rows, n_rot, head_dim)
    half = head_dim // 2
    if interleaved:
        pairs = rot.unflatten(-1, (half, 2))
        a, b = pairs[..., 0], pairs[..., 1]
        new = torch.stack((a * c - b * s, a * s + b * c), dim=-1).flatten(-2)
    else:
        a, b = rot[..., :half], rot[..., half:]
        new = torch.cat((a * c - b * s, a * s + b * c), dim=-1)
    out = qkv.clone()
    out[:, : n_rot * head_dim] = new.reshape(rows, n_rot * head_dim).to(qkv.dtype)
    return out


# ---------------------------------------------------------------- causal attention on packed qkv
def _split_qkv(qkv, batch, seq_len, n_heads, n_kv_heads, head_dim):
    q_dim, kv_dim = n_heads * head_dim, n_kv_heads * head_dim
    x = qkv.reshape(batch, seq_len, q_dim + 2 * kv_dim)
    q = x[..., :q_dim].reshape(batch, seq_len, n_heads, head_dim).transpose(1, 2)
    k = x[..., q_dim : q_dim + kv_dim].reshape(batch, seq_len, n_kv_heads, head_dim).transpose(1, 2)
    v = x[..., q_dim + kv_dim :].reshape(batch, seq_len, n_kv_heads, head_dim).transpose(1, 2)
    return q, k, v


def attention_probs(q, k, scale, causal=True):
    """softmax(mask(q k^T * scale)) in fp32 together with its log-sum-exp."""
    s = torch.einsum("bhid,bhjd->bhij", q.float(), k.float()) * scale
    if causal:
        t_q, t_k = s.shape[-2:]
        mask = torch.ones(t_q, t_k, dtype=torch.bool, device=s.device).tril(t_k - t_q)
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    return torch.exp(s - lse.unsqueeze(-1)), lse


def attention_fwd(qkv, batch, seq_len, n_heads, n_kv_heads, head_dim, scale):
    q, k, v = _split_qkv(qkv, batch, seq_len, n_heads, n_kv_heads, head_dim)
    rep = n_heads // n_kv_heads
    p, lse = attention_probs(q, k.repeat_interleave(rep, dim=1), scale)
    o = torch.einsum("bhij,bhjd->bhid", p, v.repeat_interleave(rep, dim=1).float())
    o = o.transpose(1, 2).reshape(batch * seq_len, n_heads * head_dim).to(qkv.dtype)
    return o, lse


def attention_input_pullback_dense(q, k, v, dO_basis, scale, causal=True):
    """Dense formula for the per-basis input pullback.

    q, k, v [B, H, T, Dh]; dO_basis [B, P, H, T, Dh] -> dQ, dK, dV [B, P, H, T, Dh] (fp32).
    P = softmax(mask(QK^T s)); dV = P^T dO; dP = dO V^T; dS = P o (dP - rowsum(dP o P)); dQ = s dS K; dK = s dS^T Q.
    """
    p, _ = attention_probs(q, k, scale, causal)
    do = dO_basis.float()
    dv = torch.einsum("bhij,bphid->bphjd", p, do)
    dp = torch.einsum("bphid,bhjd->bphij", do, v.float())
    ds = p.unsqueeze(1) * (dp - (dp * p.unsqueeze(1)).sum(dim=-1, keepdim=True))
    dq = torch.einsum("bphij,bhjd->bphid", ds, k.float()) * scale
    dk = torch.einsum("bphij,bhid->bphjd", ds, q.float()) * scale
    return dq, dk, dv


def attention_pullback_packed(do_rows, qkv, o, lse, batch, seq_len, n_heads, n_kv_heads, head_dim, scale):
    """Packed-layout pullback: do_rows [P*n, H*Dh] -> d_qkv [P*n, (H + 2Hkv)*Dh] (same dtype as do_rows)."""
    n = batch * seq_len
    nb = do_rows.shape[0] // n
    q, k, v = _split_qkv(qkv, batch, seq_len, n_heads, n_kv_heads, head_dim)
    rep = n_heads // n_kv_heads
    do = do_rows.reshape(nb, batch, seq_len, n_heads, head_dim).permute(1, 0, 3, 2, 4)  # [B, P, H, T, Dh]
    dq, dk, dv = attention_input_pullback_dense(
        q, k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1), do, scale, causal=True
    )
    if rep > 1:
        dk = dk.unflatten(2, (n_kv_heads, rep)).sum(dim=3)
        dv = dv.unflatten(2, (n_kv_heads, rep)).sum(dim=3)

    def pack(x):  # [B, P, h, T, Dh] -> [P*n, h*Dh]
        return x.permute(1, 0, 3, 2, 4).reshape(nb * n, -1)

    return torch.cat((pack(dq), pack(dk), pack(dv)), dim=-1).to(do_rows.dtype)


# ---------------------------------------------------------------- SwiGLU: a = up * silu(gate), u = [up | gate]
def swiglu_fwd(u):
    up, gate = u.chunk(2, dim=-1)
    return (up.float() * F.silu(gate.float())).to(u.dtype)


def swiglu_bwd(da, u):
    rows = da.shape[0]
    up, gate = _bcast_rows(u, rows).float().chunk(2, dim=-1)
    sig = torch.sigmoid(gate)
    g = da.float()
    d_up = g * gate * sig
    d_gate = g * up * sig * (1.0 + gate * (1.0 - sig))
    return torch.cat((d_up, d_gate), dim=-1).to(da.dtype)


# ---------------------------------------------------------------- depthwise causal conv over time
def causal_conv_fwd(x, weight, bias, batch, seq_len):
    """x [n, C]; weight [C, W]; y[t] = sum_w weight[:, w] * x[t - (W-1) + w]."""
    width = weight.shape[1]
    xt = x.reshape(batch, seq_len, -1).transpose(1, 2).float()
    y = F.conv1d(F.pad(xt, (width - 1, 0)), weight.float().unsqueeze(1), None if bias is None else bias.float(), groups=xt.shape[1])
    return y.transpose(1, 2).reshape(batch * seq_len, -1).to(x.dtype)


def causal_conv_dgrad(dy, weight, batch, seq_len):
    """Input cotangent of the causal conv; dy may carry a leading basis factor in its rows."""
    width = weight.shape[1]
    reps = dy.shape[0] // (batch * seq_len)
    g = dy.reshape(reps * batch, seq_len, -1).transpose(1, 2).float()
    dx = F.conv1d(F.pad(g, (0, width - 1)), weight.float().flip(-1).unsqueeze(1), groups=g.shape[1])
    return dx.transpose(1, 2).reshape(dy.shape[0], -1).to(dy.dtype)


def causal_conv_wgrad(dy, x, width, batch, seq_len):
    g = dy.reshape(batch, seq_len, -1).float()
    xp = F.pad(x.reshape(batch, seq_len, -1).float(), (0, 0, width - 1, 0))
    dw = torch.stack([(g * xp[:, w : w + seq_len]).sum(dim=(0, 1)) for w in range(width)], dim=-1)
    return dw, g.sum(dim=(0, 1))


# ---------------------------------------------------------------- LM head + cross-entropy
def lm_head_cross_entropy(normed, weight, targets, loss_scale, want_dweight=True, dweight_into=None):
    """loss = loss_scale * sum_rows CE(normed @ W^T, target); returns (loss_sum fp32 scalar, d_normed, dW or None).

    Rows whose target is negative are ignored."""
    logits = (normed.float() @ weight.float().t())
    valid = targets >= 0
    safe = targets.clamp(min=0)
    lse = torch.logsumexp(logits, dim=-1)
    picked = logits.gather(1, safe.unsqueeze(1)).squeeze(1)
    loss = ((lse - picked) * valid).sum() * loss_scale
    probs = torch.exp(logits - lse.unsqueeze(1))
    probs.scatter_add_(1, safe.unsqueeze(1), -torch.ones_like(picked).unsqueeze(1))
    dlogits = probs * (valid.unsqueeze(1) * loss_scale)
    d_normed = (dlogits @ weight.float()).to(normed.dtype)
    dW = dlogits.t() @ normed.float() if want_dweight else None
    if dW is not None and dweight_into is not None:
        dweight_into.add_(dW)
        dW = dweight_into
    return loss, d_normed, dW


# ---------------------------------------------------------------- embedding
def embedding_fwd(ids, table, out_dtype):
    return table[ids.reshape(-1)].to(out_dtype)


def embedding_scatter_add(d_table, ids, d_rows):
    d_table.index_add_(0, ids.reshape(-1), d_rows.to(d_table.dtype))
    return d_table


# ---------------------------------------------------------------- interface glue
def add_condition(canvas_rows, cond, seq_len):
    """canvas_rows [B*T, D] + cond [B, D] broadcast over the T tokens of each sequence."""
    bsz = cond.shape[0]
    return (canvas_rows.reshape(bsz, seq_len, -1).float() + cond.float().unsqueeze(1)).reshape(bsz * seq_len, -1).to(canvas_rows.dtype)


def mean_pool_tokens(rows, batch, seq_len):
    return rows.reshape(batch, seq_len, -1).float().mean(dim=1)


def sum_tokens(rows, groups, seq_len):
    """[groups*T, D] -> [groups, D] fp32 (cotangent of a broadcast over tokens)."""
    return rows.reshape(groups, seq_len, -1).float().sum(dim=1)


# ---------------------------------------------------------------- suffix scan of interface Jacobians
def suffix_scan_pullbacks(mats):
    """mats [B, K, R, R] -> [B, K+1, R, R] fp32 with out[k] = mats[k] @ mats[k+1] @ ... @ mats[K-1], out[K] = I."""
    bsz, k, r, _ = mats.shape
    out = torch.empty(bsz, k + 1, r, r, dtype=torch.float32, device=mats.device)
    acc = torch.eye(r, dtype=torch.float32, device=mats.device).expand(bsz, r, r).contiguous()
    out[:, k] = acc
    for idx in range(k - 1, -1, -1):
        acc = mats[:, idx].float() @ acc
        out[:, idx] = acc
    return out


def affine_suffix_scan(mats, offsets, seed=None):
    """g_k = offsets_k + mats_k g_{k+1}, g_K = seed (zero by default).

    mats [B, K, R, R] with g_k = mats_k @ g_{k+1}; offsets [B, K, R].  Returns g [B, K+1, R] fp32."""
    bsz, k, r, _ = mats.shape
    g = torch.zeros(bsz, k + 1, r, dtype=torch.float32, device=mats.device)
    if seed is not None:
        g[:, k] = seed.float()
    for idx in range(k - 1, -1, -1):
        g[:, idx] = offsets[:, idx].float() + torch.einsum("bij,bj->bi", mats[:, idx].float(), g[:, idx + 1])
    return g


# ---------------------------------------------------------------- AdamW on flat buffers
def adamw_step(param, grad, exp_avg, exp_avg_sq, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0, shadow=None):
    """Decoupled-weight-decay Adam on flat fp32 buffers, same update rule as torch.optim.AdamW.
    ``shadow`` (bf16 copy of the parameters) is refreshed in the same pass when given."""
    g = grad.float() * grad_scale
    param.mul_(1.0 - lr * weight_decay)
    exp_avg.mul_(beta1).add_(g, alpha=1.0 - beta1)
    exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
    bias1 = 1.0 - beta1 ** step
    bias2 = 1.0 - beta2 ** step
    denom = (exp_avg_sq.sqrt() / math.sqrt(bias2)).add_(eps)
    param.addcdiv_(exp_avg, denom, value=-lr / bias1)
    if shadow is not None:
        shadow.copy_(param)
    return param
