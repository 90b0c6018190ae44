"""Causal attention forward and the input pullback over a basis of output cotangents.

``attention_input_pullback_basis`` keeps the reference's call signature and tensor layout
(cuda/transformer/__init__.py:279-355: q, k, v [B, H, T, Dh]; dO_basis [B, P, H, T, Dh] ->
dQ, dK, dV [B, P, H, T, Dh]).  Kernel modes:

* ``"tcgen05_pblock"``  this package's sm_100a kernel: S and P = softmax(S) are recomputed once per
  (query tile, key tile) and reused by every basis direction; all five products run on tcgen05 with
  accumulators in TMEM (replaces the reference's WMMA kernels and host loop,
  cuda/transformer/attention_pullback_mma.cu:60-515);
* ``"fa2_loop"``        P library flash-attention backward passes (the reference's fallback and the
  baseline the kernel is timed against);
* ``"dense"``           the O(T^2) fp32 formula (oracle).
"""
from __future__ import annotations

import math
import os

import torch

from . import reference as ref
from .native import ext, native_available



def _views(qkv, batch, seq_len, n_heads, n_kv_heads, head_dim):
    """Token-major views [B, T, h, Dh] of the q, k and v parts of a packed buffer (no copies)."""
    q_dim, kv_dim = n_heads * head_dim, n_kv_heads * head_dim
    x = qkv.view(batch, seq_len, q_dim + 2 * kv_dim)
    q = x[..., :q_dim].unflatten(-1, (n_heads, head_dim))
    k = x[..., q_dim : q_dim + kv_dim].unflatten(-1, (n_kv_heads, head_dim))
    v = x[..., q_dim + kv_dim :].unflatten(-1, (n_kv_heads, head_dim))
    return q, k, v


def _flash():
    from flash_attn import flash_attn_interface as fa

    return fa


FORWARD_NATIVE = os.environ.get("LBI_B200_LIBRARY_ATTENTION", "0") != "1"


def _gqa_native(qkv, head_dim, n_heads, n_kv_heads, seq_len) -> bool:
    """Grouped kv heads run on the tcgen05 kernels through an expanded copy of k and v (one head per q head)."""
    return (n_kv_heads < n_heads and n_heads % n_kv_heads == 0 and qkv.is_cuda and hasattr(ext(), "gqa_expand")
            and tcgen05_pullback_supported(qkv.dtype, head_dim, n_heads, n_heads, seq_len))


def _gqa_expand(qkv, n_heads, n_kv_heads, head_dim):
    from .dispatch import KERNEL_LAUNCHES

    KERNEL_LAUNCHES["count"] += 1
    return ext().gqa_expand(qkv.contiguous(), n_heads, n_kv_heads, head_dim)


def flash_forward_packed(qkv, batch, seq_len, n_heads, n_kv_heads, head_dim, scale, kernel_mode=None):
    """Causal attention forward on the packed qkv buffer -> (out [n, H*Dh], lse [B, H, T] fp32).

    ``tcgen05``: the extension's own kernel (bf16 or fp16, head_dim 64, T % 128 == 0; grouped kv heads through an expanded copy);
    ``fa2``: the flash_attn library kernel, kept as the baseline and for every other shape."""
    if kernel_mode in (None, "tcgen05") and FORWARD_NATIVE and _gqa_native(qkv, head_dim, n_heads, n_kv_heads, seq_len):
        return flash_forward_packed(_gqa_expand(qkv, n_heads, n_kv_heads, head_dim), batch, seq_len, n_heads, n_heads, head_dim, scale,
                                    kernel_mode="tcgen05")
    mode = kernel_mode or ("tcgen05" if FORWARD_NATIVE and qkv.is_cuda and qkv.is_contiguous() and hasattr(ext(), "attn_fwd_packed")
                           and tcgen05_pullback_supported(qkv.dtype, head_dim, n_heads, n_kv_heads, seq_len) else "fa2")
    if mode == "tcgen05":
        from .dispatch import KERNEL_LAUNCHES

        KERNEL_LAUNCHES["count"] += 1
        out, lse = ext().attn_fwd_packed(qkv, batch, seq_len, n_heads, head_dim, float(scale))
        return out, lse
    from .dispatch import fell_back

    fell_back("attention_fwd (flash_attn library)", qkv, why=f"head_dim {head_dim}, heads {n_heads}/{n_kv_heads}, seq_len {seq_len}")
    q, k, v = _views(qkv, batch, seq_len, n_heads, n_kv_heads, head_dim)
    out, lse, _, _ = _flash()._flash_attn_forward(q, k, v, 0.0, float(scale), True, -1, -1, 0.0, None, False)
    return out.reshape(batch * seq_len, n_heads * head_dim), lse


def pullback_packed(do_rows, qkv, o, lse, batch, seq_len, n_heads, n_kv_heads, head_dim, scale, kernel_mode=None, rope=None):
    """Packed layout: do_rows [P*n, H*Dh] -> d_qkv [P*n, (H+2Hkv)*Dh].

    ``rope = (cos, sin, interleaved)`` asks for dq and dk rotated back through the rotary embedding (its VJP); the
    tcgen05 kernel does that in its epilogue, the other modes in a separate pass."""
    n = batch * seq_len
    nbasis = do_rows.shape[0] // n
    qkv_dim = (n_heads + 2 * n_kv_heads) * head_dim
    if kernel_mode in (None, "tcgen05_pblock") and _gqa_native(qkv, head_dim, n_heads, n_kv_heads, seq_len):
        # every q head gets its own copy of its group's k / v; the cotangents of the copies are summed afterwards (the
        # inverse rotary turn of the epilogue is the same for all heads of a position, so it commutes with the sum)
        from .dispatch import KERNEL_LAUNCHES

        d_full = pullback_packed(do_rows, _gqa_expand(qkv, n_heads, n_kv_heads, head_dim), o, lse, batch, seq_len, n_heads, n_heads,
                                 head_dim, scale, kernel_mode="tcgen05_pblock", rope=rope)
        KERNEL_LAUNCHES["count"] += 1
        return ext().gqa_reduce(d_full.contiguous(), n_heads, n_kv_heads, head_dim)
    mode = kernel_mode or default_kernel_mode(do_rows, head_dim, n_heads, n_kv_heads, seq_len)
    if mode == "tcgen05_pblock":
        from .dispatch import KERNEL_LAUNCHES

        KERNEL_LAUNCHES["count"] += 3
        if rope is None:
            return ext().attn_pullback_packed(do_rows.contiguous(), qkv, o, lse, batch, seq_len, n_heads, head_dim, float(scale))
        return ext().attn_pullback_packed(do_rows.contiguous(), qkv, o, lse, batch, seq_len, n_heads, head_dim, float(scale),
                                          rope[0], rope[1], bool(rope[2]))
    from .dispatch import fell_back

    fell_back("attention_pullback (flash_attn library loop)", do_rows,
              why=f"head_dim {head_dim}, heads {n_heads}/{n_kv_heads}, seq_len {seq_len}, dtype {do_rows.dtype}")
    q, k, v = _views(qkv, batch, seq_len, n_heads, n_kv_heads, head_dim)
    out4 = o.view(batch, seq_len, n_heads, head_dim)
    d_qkv = torch.empty(nbasis * n, qkv_dim, dtype=do_rows.dtype, device=do_rows.device)
    fa = _flash()
    for p in range(nbasis):
        do = do_rows[p * n : (p + 1) * n].view(batch, seq_len, n_heads, head_dim)
        dq, dk, dv = _views(d_qkv[p * n : (p + 1) * n], batch, seq_len, n_heads, n_kv_heads, head_dim)
        fa._flash_attn_backward(do, q, k, v, out4, lse, dq, dk, dv, 0.0, float(scale), True, -1, -1, 0.0, None, False, None)
    if rope is not None:
        from .dispatch import rope_qkv

        d_qkv = rope_qkv(d_qkv, rope[0], rope[1], n_heads, n_kv_heads, head_dim, seq_len, rope[2], inverse=True)
    return d_qkv


def tcgen05_pullback_supported(dtype, head_dim, n_heads, n_kv_heads, seq_len) -> bool:
    return (
        native_available()
        and hasattr(ext(), "attn_pullback_packed")
        and dtype in (torch.bfloat16, torch.float16)
        and head_dim == 64
        and n_heads == n_kv_heads
        and seq_len % 128 == 0
    )


def default_kernel_mode(t, head_dim, n_heads, n_kv_heads, seq_len) -> str:
    if t.is_cuda and tcgen05_pullback_supported(t.dtype, head_dim, n_heads, n_kv_heads, seq_len):
        return "tcgen05_pblock"
    return "fa2_loop"


# the reference's kernel-mode names (cuda/transformer/__init__.py:279-356) and the mode of this package that serves each
REFERENCE_KERNEL_MODES = {
    "fa2_mma_pblock4": None,   # its tensor-core kernels -> the best kernel for the shape (tcgen05 where supported)
    "fa2_mma_p1": None,
    "fa2_p1": None,
    "fa2_loop": "fa2_loop",
    "simple": "dense",
}


def attention_input_pullback_basis(q, k, v, dO_basis, *, scale=None, causal=True, use_cuda=True, kernel_mode=None,
                                   softmax_scale=None):
    """q, k, v [B, H, T, Dh]; dO_basis [B, P, H, T, Dh] -> (dQ, dK, dV) each [B, P, H, T, Dh].

    ``softmax_scale`` is the reference's keyword for ``scale`` (cuda/transformer/__init__.py:279-289)."""
    scale = softmax_scale if scale is None else scale
    kernel_mode = REFERENCE_KERNEL_MODES.get(kernel_mode, kernel_mode)
    if q.dim() != 4 or dO_basis.dim() != 5:
        raise ValueError("expected q,k,v [B,H,T,Dh] and dO_basis [B,P,H,T,Dh]")
    bsz, heads, seqlen, head_dim = q.shape
    nbasis = dO_basis.shape[1]
    scale = float(scale) if scale else 1.0 / math.sqrt(head_dim)
    if not use_cuda or not q.is_cuda or kernel_mode == "dense" or not causal:
        dq, dk, dv = ref.attention_input_pullback_dense(q, k, v, dO_basis, scale, causal)
        return dq.to(q.dtype), dk.to(q.dtype), dv.to(q.dtype)
    if k.shape[1] != heads:
        raise ValueError("expand grouped kv heads before calling the basis pullback")
    # pack to the token-major layout the kernels use
    qkv = torch.cat([x.transpose(1, 2).reshape(bsz * seqlen, heads * head_dim) for x in (q, k, v)], dim=-1).contiguous()
    o_rows, lse = flash_forward_packed(qkv, bsz, seqlen, heads, heads, head_dim, scale)
    do_rows = dO_basis.permute(1, 0, 3, 2, 4).reshape(nbasis * bsz * seqlen, heads * head_dim).contiguous()
    d_qkv = pullback_packed(do_rows, qkv, o_rows.contiguous(), lse, bsz, seqlen, heads, heads, head_dim, scale, kernel_mode)
    parts = d_qkv.view(nbasis, bsz, seqlen, 3, heads, head_dim).permute(3, 1, 0, 4, 2, 5)  # [3, B, P, H, T, Dh]
    return parts[0], parts[1], parts[2]
