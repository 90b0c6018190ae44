"""Mamba-2 SSD chunk scan: CUDA forward (csrc/ssd.cu) behind a differentiable wrapper.

``ssd_chunk_scan_cuda`` runs the four sm_100a kernels (cumsum, chunk state, state passing, fused chunk scan) and, when a
gradient is needed, differentiates by recomputing the chunked PyTorch form (``backbones/mamba2/ssd.py``) under
autograd: the forward is the kernel's, the backward is exact for the same math.  The reference's counterpart is the
Triton pipeline ``mamba_chunk_scan_combined`` (backbones/mamba2/ops/triton/ssd_combined.py:343-513).
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F

from .native import ext, native_available

CHUNK = 128
ENABLED = os.environ.get("LBI_B200_TORCH_SSD", "0") != "1"   # set to use the chunked PyTorch scans everywhere


def ssd_cuda_supported(x: torch.Tensor, B: torch.Tensor) -> bool:
    """bf16 or fp32 CUDA inputs with head_dim 64, d_state 64 / 128 and an even number of heads per group."""
    if not (ENABLED and x.is_cuda and native_available() and hasattr(ext(), "ssd_chunk_scan_fwd")):
        return False
    nheads, headdim = x.shape[2], x.shape[3]
    ngroups, dstate = B.shape[2], B.shape[3]
    return headdim == 64 and dstate in (64, 128) and nheads % ngroups == 0 and (nheads // ngroups) % 2 == 0


def _forward_kernels(x, dt, A, B, C, D, initial_state):
    from .dispatch import KERNEL_LAUNCHES

    bsz, seqlen = x.shape[:2]
    pad = (-seqlen) % CHUNK
    xb, Bb, Cb, dtf = x.to(torch.bfloat16), B.to(torch.bfloat16), C.to(torch.bfloat16), dt.float()
    if pad:  # dt = 0 on the padding: no decay, no contribution
        xb, Bb, Cb = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (xb, Bb, Cb))
        dtf = F.pad(dtf, (0, 0, 0, pad))
    y, final = ext().ssd_chunk_scan_fwd(
        xb.contiguous(), dtf.contiguous(), A.float().contiguous(), Bb.contiguous(), Cb.contiguous(),
        None if D is None else D.float().contiguous(), None, None if initial_state is None else initial_state.float().contiguous(),
        False, 0.0, float("inf"))
    KERNEL_LAUNCHES["count"] += 4
    return y[:, :seqlen], final


class _SSDFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dt, A, B, C, D, initial_state):
        y, final = _forward_kernels(x, dt, A, B, C, D, initial_state)
        ctx.save_for_backward(x, dt, A, B, C, D if D is not None else x.new_empty(0),
                              initial_state if initial_state is not None else x.new_empty(0))
        ctx.has_d, ctx.has_init = D is not None, initial_state is not None
        return y.to(x.dtype), final

    @staticmethod
    def backward(ctx, gy, gfinal):
        from ..backbones.mamba2.ssd import ssd_chunk_scan

        x, dt, A, B, C, D, init = ctx.saved_tensors
        leaves = [t.detach().requires_grad_(t.is_floating_point()) for t in (x, dt, A, B, C)]
        d_leaf = D.detach().requires_grad_(True) if ctx.has_d else None
        i_leaf = init.detach().requires_grad_(True) if ctx.has_init else None
        with torch.enable_grad():
            y, final = ssd_chunk_scan(*leaves, chunk_size=CHUNK, D=d_leaf, initial_state=i_leaf, return_final_state=True)
            wanted = [t for t in (*leaves, d_leaf, i_leaf) if t is not None]
            outs, cots = [y], [gy.to(y.dtype)]
            if gfinal is not None:
                outs.append(final)
                cots.append(gfinal.to(final.dtype))
            grads = list(torch.autograd.grad(outs, wanted, cots, allow_unused=True))
        res = grads[:5]
        rest = grads[5:]
        gd = rest.pop(0) if ctx.has_d else None
        gi = rest.pop(0) if ctx.has_init else None
        return (*res, gd, gi)


def ssd_chunk_scan_cuda(x, dt, A, B, C, D=None, initial_state=None, return_final_state: bool = False):
    """x [b, l, h, 64]; dt [b, l, h] (positive); A [h] (negative); B, C [b, l, g, n]; D [h] or None -> y like x."""
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (x, dt, A, B, C, D, initial_state)):
        y, final = _SSDFunction.apply(x, dt, A, B, C, D, initial_state)
    else:
        y, final = _forward_kernels(x, dt, A, B, C, D, initial_state)
        y = y.to(x.dtype)
    return (y, final) if return_final_state else y


# ------------------------------------------------------------------------------------------------ Mamba-3 SISO
def siso_cuda_supported(V: torch.Tensor, Q: torch.Tensor) -> bool:
    """CUDA inputs with head_dim 64 and d_state 128 (the paper's Mamba-3 shape)."""
    return bool(ENABLED and V.is_cuda and native_available() and hasattr(ext(), "siso_chunk_scan_fwd") and V.shape[3] == 64
                and Q.shape[3] == 128)


def _siso_forward_kernels(Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Angles, D):
    """The rotary / bias / trapezoid preprocessing (elementwise, PyTorch) followed by the chunk-scan kernels.

    After the preprocessing the recurrence is the SSD one with per-head operands, a strictly causal score mask and a
    per-token skip coefficient, which is how ``csrc/ssd.cu`` evaluates it (the reference runs one Triton program per
    (head, batch) that walks all chunks serially, mamba3_siso_fwd.py:360-424)."""
    from ..backbones.mamba3.siso import _prepare
    from .dispatch import KERNEL_LAUNCHES

    seqlen = V.shape[1]
    Qr, Kr, adt, qk_dot = _prepare(Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Angles, torch.float32)
    pad = (-seqlen) % CHUNK
    vb, qb, kb = V.to(torch.bfloat16), Qr.to(torch.bfloat16), Kr.to(torch.bfloat16)
    skip = qk_dot
    if pad:  # adt = 0 and k = 0 on the padding: the state is carried unchanged
        vb, qb, kb = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (vb, qb, kb))
        adt, skip = F.pad(adt, (0, 0, 0, pad)), F.pad(skip, (0, 0, 0, pad))
    y, final = ext().siso_chunk_scan_fwd(vb.contiguous(), kb.contiguous(), qb.contiguous(), adt.float().contiguous(),
                                         None if D is None else D.float().contiguous(),
                                         skip.float().transpose(1, 2).contiguous(), None)
    KERNEL_LAUNCHES["count"] += 4
    return y[:, :seqlen], final


class _SISOFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Angles, D):
        y, _ = _siso_forward_kernels(Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Angles, D)
        ctx.save_for_backward(Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Angles, D)
        return y.to(V.dtype)

    @staticmethod
    def backward(ctx, gy):
        from ..backbones.mamba3.siso import mamba3_siso_chunked

        leaves = [t.detach().requires_grad_(True) for t in ctx.saved_tensors]
        with torch.enable_grad():
            y = mamba3_siso_chunked(*leaves[:9], D=leaves[9], Z=None, chunk_size=CHUNK)
            grads = torch.autograd.grad(y, leaves, gy.to(y.dtype), allow_unused=True)
        return tuple(grads)


def mamba3_siso_cuda(Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Angles, D, Z=None):
    """Same arguments and result as ``mamba3_siso_chunked``; forward on the sm_100a kernels, backward by recompute."""
    tensors = (Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Angles, D)
    if torch.is_grad_enabled() and any(t.requires_grad for t in tensors):
        y = _SISOFunction.apply(*tensors)
    else:
        y = _siso_forward_kernels(*tensors)[0].to(V.dtype)
    if Z is not None:
        y = (y.float() * F.silu(Z.float())).to(V.dtype)
    return y
