"""LM head fused with softmax cross-entropy, forward and backward in one sweep.

The reference materialises fp32 logits for the whole batch (``F.cross_entropy(logits.float())``,
train/eval.py:12-14).  Here rows are processed in chunks: a tcgen05 GEMM writes bf16 logits for the
chunk, one kernel turns them in place into ``scale * (softmax - onehot)`` while accumulating the loss,
and two more GEMMs produce the cotangent of the normalised features and the head-weight gradient.
Peak extra memory is ``chunk_rows * vocab`` bf16 instead of ``rows * vocab`` fp32 (+ autograd copies).
"""
from __future__ import annotations

import torch

from .native import ext

CHUNK_ROWS = 8192


def fused_lm_head_ce(normed, weight, targets, loss_scale, want_dweight=True, weight_t=None, dweight_into=None):
    """normed [n, D] bf16; weight [V, D] bf16; targets [n] int64 (negative = ignored).

    Returns (loss_sum fp32 scalar tensor, d_normed [n, D] bf16, dW [V, D] fp32 or None)."""
    from .dispatch import KERNEL_LAUNCHES, gemm_tn

    n, dim = normed.shape
    vocab = weight.shape[0]
    weight = weight.contiguous()
    loss = torch.zeros(1, dtype=torch.float32, device=normed.device)
    d_normed = torch.empty_like(normed)
    if not want_dweight:
        d_weight = None
    elif dweight_into is not None:
        d_weight = dweight_into
    else:
        d_weight = torch.zeros(vocab, dim, dtype=torch.float32, device=normed.device)
    targets = targets.reshape(-1).contiguous()
    for r0 in range(0, n, CHUNK_ROWS):
        r1 = min(n, r0 + CHUNK_ROWS)
        x = normed[r0:r1]
        logits = gemm_tn(x, weight)  # [rows, V] bf16
        ext().ce_fwd_bwd_(logits, targets[r0:r1], loss, float(loss_scale))
        KERNEL_LAUNCHES["count"] += 1
        d_normed[r0:r1] = ext().gemm(logits, weight, False, True, False, None, 1)  # dlogits @ W, W read MN-major
        KERNEL_LAUNCHES["count"] += 1
        if want_dweight:
            # dW += dlogits^T @ x : both operands are read with the reduction (row) index outermost
            ext().gemm(logits, x, True, True, True, d_weight, 4)
            KERNEL_LAUNCHES["count"] += 1
    return loss[0], d_normed, d_weight
