"""Mamba-2 SSD chunk scan and Mamba-3 SISO recurrence: CUDA forward and backward (csrc/ssd.cu) behind differentiable wrappers.

``ssd_chunk_scan_cuda`` runs the four sm_100a forward kernels (cumsum, chunk state, state passing, fused chunk scan) of

    y_t = sum_{s <= t} exp(c_t - c_s) (cq_t . bk_s) w_s v_s + exp(c_t) cq_t . init

Two backward forms exist.  ``ssd_backward_fused`` / ``chunk_backward``: one kernel walks the chunks backwards for the
cotangents of the chunk-boundary states and one kernel per (direction, chunk, head) emits every input cotangent; the forward
operands may be shared by P stacked cotangent directions.  It is what the region-parallel engine uses and what the autograd
Functions take when no state enters or leaves the sequence.  ``ssd_backward`` / ``siso_core_backward``: the scan is linear in
v, in bk and in cq, and each of the three pullbacks is again a scan of this form in forward or reversed time, so the forward
kernels run three more times with permuted roles, plus a decay-gradient kernel (the identity ``dc_t = C_t . dC_t - B_t . dB_t``
cancels badly in bf16); it handles an initial state and a cotangent of the final state and serves as a cross-check
(``LBI_B200_SSD_PERMUTED_BACKWARD=1``).  The reference's counterpart is the Triton pipeline ``mamba_chunk_scan_combined``
with its ten backward kernels (backbones/mamba2/ops/triton/ssd_combined.py:343-513).
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F

from .native import ext, native_available

CHUNK = 128
ENABLED = os.environ.get("LBI_B200_TORCH_SSD", "0") != "1"   # set to use the chunked PyTorch scans everywhere
BACKWARD_KERNELS = os.environ.get("LBI_B200_SSD_RECOMPUTE_BACKWARD", "0") != "1"   # set to differentiate the PyTorch form


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
    y, final, states = ext().ssd_chunk_scan_fwd(
        xb.contiguous(), dtf.contiguous(), A.float().contiguous(), Bb.contiguous(), Cb.contiguous(),
        None if D is None else D.float().contiguous(), None, None if initial_state is None else initial_state.float().contiguous(),
        False, 0.0, float("inf"))
    KERNEL_LAUNCHES["count"] += 4
    return y[:, :seqlen], final, states


def scan_generic_torch(v, bk, cq, a, weight=None, init=None, strict=False, per_head=False):
    """fp32 PyTorch statement of the kernels' scan operator (token-by-token), the oracle of ``scan_generic``.

    v [b, l, h, p]; bk, cq [b, l, g, n]; a, weight [b, l, h]; init [b, h, p, n] ([b, h, n, p] when ``per_head``).
    Returns (y [b, l, h, p] fp32, final state in the layout of ``init``)."""
    b, l, h, p = v.shape
    g, n = bk.shape[2], bk.shape[3]
    vf, af = v.float(), a.float()
    bkf = bk.float().repeat_interleave(h // g, dim=2)
    cqf = cq.float().repeat_interleave(h // g, dim=2)
    wf = torch.ones_like(af) if weight is None else weight.float()
    state = vf.new_zeros(b, h, p, n) if init is None else (init.float().transpose(2, 3) if per_head else init.float()).clone()
    ys = []
    for t in range(l):
        decayed = state * torch.exp(af[:, t])[..., None, None]
        new = decayed + (wf[:, t, :, None] * vf[:, t])[..., None] * bkf[:, t, :, None, :]
        ys.append(torch.einsum("bhpn,bhn->bhp", decayed if strict else new, cqf[:, t]))
        state = new
    return torch.stack(ys, dim=1), (state.transpose(2, 3) if per_head else state)


def scan_generic(v, bk, cq, a, weight=None, init=None, strict=False, per_head=False, out_f32=True, v_div=1, v_mod=1):
    """The kernels' scan operator with free operand roles; bf16 operands.  ``seq_len % 128 == 0``.

    The number of heads is that of ``a``; head h reads the 64-column block ``(h // v_div) * v_mod + h % v_mod`` of ``v``
    (several heads can share columns of a narrower v).  Returns (y in fp32 or bf16, final state, bf16 incoming state of
    every chunk [b, l / 128, h, 64, n])."""
    from .dispatch import KERNEL_LAUNCHES

    bf = torch.bfloat16
    out = ext().ssd_scan_generic(v.to(bf).contiguous(), bk.to(bf).contiguous(), cq.to(bf).contiguous(), a.float().contiguous(),
                                 None if weight is None else weight.float().contiguous(), None, None,
                                 None if init is None else init.float().contiguous(), bool(strict), bool(per_head), bool(out_f32),
                                 int(v_div), int(v_mod))
    KERNEL_LAUNCHES["count"] += 4
    return out


def decay_grad(v, gy, bk, cq, a, weight, *, states_in, states_cot_rev, per_head=False, init=None, gfinal=None):
    """da_u = sum over pairs s < u <= t of e^{c_t - c_s} (cq_t . bk_s) w_s (gy_t . v_s) on the kernel (csrc/ssd.cu, part 5).

    ``states_in`` / ``states_cot_rev`` are the third results of the forward scan and of the reversed scan that pulled gy
    back; they carry the pairs that reach before the first token (``init``) or past the last one (``gfinal``)."""
    from .dispatch import KERNEL_LAUNCHES

    bf = torch.bfloat16
    KERNEL_LAUNCHES["count"] += 2
    return ext().ssd_decay_grad(v.to(bf).contiguous(), gy.to(bf).contiguous(), bk.to(bf).contiguous(), cq.to(bf).contiguous(),
                                a.float().contiguous(), None if weight is None else weight.float().contiguous(),
                                states_in, states_cot_rev, bool(per_head))


def decay_grad_torch(v, gy, bk, cq, a, weight, *, states_in=None, states_cot_rev=None, per_head=False, init=None, gfinal=None):
    """The same sum taken from its definition in fp32 (O(l^2) memory), the oracle of ``decay_grad``."""
    b, l, h, _ = v.shape
    g = bk.shape[2]
    vf, gyf, af = v.float(), gy.float(), a.float()
    bkf = bk.float().repeat_interleave(h // g, dim=2)
    cqf = cq.float().repeat_interleave(h // g, dim=2)
    wf = torch.ones_like(af) if weight is None else weight.float()
    c = af.cumsum(1)                                                                      # [b, l, h]
    diff = (c[:, :, None] - c[:, None, :]).permute(0, 3, 1, 2)                            # [b, h, t, s]
    strict = torch.ones(l, l, dtype=torch.bool, device=v.device).tril(-1)
    e = (torch.einsum("bthn,bshn->bhts", cqf, bkf) * torch.einsum("bthp,bshp->bhts", gyf, vf)
         * torch.exp(diff.masked_fill(~strict, float("-inf"))) * wf.permute(0, 2, 1)[:, :, None, :])
    # pairs s < u <= t: prefix over s up to u - 1, suffix over t from u
    pre = F.pad(e.cumsum(-1), (1, 0))[..., :l]                                            # [b, h, t, u] = sum_{s < u} e[t, s]
    da = pre.flip(2).cumsum(2).flip(2).diagonal(dim1=2, dim2=3)                           # [b, h, u] = sum_{t >= u} pre[t, u]
    da = da.permute(0, 2, 1).clone()
    ini = None if init is None else (init.float().transpose(2, 3) if per_head else init.float())      # [b, h, p, n]
    gfi = None if gfinal is None else (gfinal.float().transpose(2, 3) if per_head else gfinal.float())
    if ini is not None:    # s before the first token, t inside: every u <= t
        r = torch.exp(c) * torch.einsum("bthp,bhpn,bthn->bth", gyf, ini, cqf)
        da += r.flip(1).cumsum(1).flip(1)
    if gfi is not None:    # s inside, t past the last token: every u > s
        r = wf * torch.exp(c[:, -1:] - c) * torch.einsum("bshp,bhpn,bshn->bsh", vf, gfi, bkf)
        da += r.cumsum(1) - r
        if ini is not None:
            da += (torch.exp(c[:, -1]) * (ini * gfi).sum((2, 3)))[:, None, :]
    return da


def _finish_torch(dx_rev, x, gy, dt, da, A, D):
    """dx = dt dX + D gy, ddt = da A + dX . x, dD = sum gy . x with dX = dx_rev flipped back in time (PyTorch form)."""
    seqlen = x.shape[1]
    dX = dx_rev.flip(1)[:, :seqlen].float()
    dx = dt[..., None] * dX
    ddt = da[:, :seqlen] * A + (dX * x).sum(-1)
    dD = None
    if D is not None:
        dx = dx + D.float()[None, None, :, None] * gy
        dD = (gy.float() * x).sum((0, 1, 3))
    return dx, ddt, dD


def _group_sum_torch(y, w, seqlen, groups, n, reversed_time):
    """[b, lp, h, width] -> [b, l, g, n]: sum over the heads of a group of w[b, l, h] * y[..., :n] (PyTorch form)."""
    b, _, h, width = y.shape
    yy = (y.flip(1) if reversed_time else y)[:, :seqlen].reshape(b, seqlen, groups, h // groups, width)[..., :n]
    if w is not None:
        yy = yy * w.reshape(b, seqlen, groups, h // groups, 1)
    return yy.sum(3, dtype=torch.float32)


class KernelScans:
    """The sm_100a kernels as the backend of ``ssd_backward`` / ``siso_core_backward``."""
    scan = staticmethod(scan_generic)
    decay_grad = staticmethod(decay_grad)

    @staticmethod
    def finish(dx_rev, x, gy, dt, da, A, D):
        from .dispatch import KERNEL_LAUNCHES

        if x.dtype not in (torch.bfloat16, torch.float32) or not hasattr(ext(), "ssd_bwd_finish"):
            return _finish_torch(dx_rev, x, gy, dt, da, A, D)
        KERNEL_LAUNCHES["count"] += 1
        dx, ddt, dD = ext().ssd_bwd_finish(dx_rev.contiguous(), x.contiguous(), gy.to(x.dtype).contiguous(), dt.contiguous(), da,
                                           A.contiguous(), None if D is None else D.float().contiguous())
        return dx, ddt, (dD if D is not None else None)

    @staticmethod
    def group_sum(y, w, seqlen, groups, n, reversed_time):
        from .dispatch import KERNEL_LAUNCHES

        if y.dtype != torch.bfloat16 or n % 2 or not hasattr(ext(), "ssd_group_sum"):
            return _group_sum_torch(y, w, seqlen, groups, n, reversed_time)
        KERNEL_LAUNCHES["count"] += 1
        return ext().ssd_group_sum(y.contiguous(), None if w is None else w.contiguous(), seqlen, groups, n, bool(reversed_time), False)


class TorchScans:
    """fp32 PyTorch statements of the same operators (CPU-runnable oracle)."""

    @staticmethod
    def scan(v, bk, cq, a, weight=None, init=None, strict=False, per_head=False, out_f32=True, v_div=1, v_mod=1):
        if (v_div, v_mod) != (1, 1):
            heads = torch.arange(a.shape[2], device=v.device)
            v = v[:, :, (heads // v_div) * v_mod + heads % v_mod]
        return (*scan_generic_torch(v, bk, cq, a, weight, init, strict=strict, per_head=per_head), None)

    decay_grad = staticmethod(decay_grad_torch)
    finish = staticmethod(_finish_torch)
    group_sum = staticmethod(_group_sum_torch)


def _shift_reverse(a):
    """Log-decays of the time-reversed recurrence: position tau takes a[T - tau], position 0 takes 0."""
    return torch.cat([torch.zeros_like(a[:, :1]), a.flip(1)[:, :-1]], dim=1)


def _blocks(t, dup):
    """[b, l, h, n] -> [b, l, h * max(n // 64, dup), 64]: the state axis as virtual heads of width 64."""
    b, l, h, n = t.shape
    if n == 64 and dup > 1:
        return t.unsqueeze(3).expand(b, l, h, dup, 64).reshape(b, l, h * dup, 64)
    return t.reshape(b, l, h * (n // 64), 64)


def ssd_backward(x, dt, A, B, C, D, init, final, gy, gfinal, ops=KernelScans, fwd_states=None):
    """Gradients of (y, final) = SSD(x, dt, A, B, C, D, init) from three role-permuted scans and the decay-gradient kernel.

    With X = dt x, c the cumulative log-decay and per-head copies of B, C:
      dX_s   = sum_{t >= s} e^{c_t - c_s} (B_s . C_t) gy_t        reversed time: v = gy, bk = C, cq = B, init = gfinal
      dC_t   = sum_{s <= t} e^{c_t - c_s} (gy_t . X_s) B_s        forward time:  v = B,  bk = x (w = dt), cq = gy, init = init^T
      dB_s/dt_s = sum_{t >= s} e^{c_t - c_s} (x_s . gy_t) C_t     reversed time: v = C,  bk = gy, cq = x, init = gfinal^T
    The state axis (64 or 128 wide) of B and C is cut into virtual heads of width 64 for the last two.  The gradient of
    the log-decays a = dt A comes from ``ops.decay_grad`` (every pair counted once; the identity
    ``dc_t = C_t . dC_t - B_t . dB_t`` is exact but cancels badly in bf16).  Then
      ddt = da A + dX . x,  dA = sum da dt,  dx = dt dX + D gy,  dD = sum gy . x.
    All arguments are un-padded; ``ops`` is ``KernelScans`` or ``TorchScans``; ``fwd_states`` are the incoming chunk states
    of the forward kernels (third result of ``_forward_kernels``)."""
    bsz, seqlen, h, p = x.shape
    g, n = B.shape[2], B.shape[3]
    rep = h // g
    pad = (-seqlen) % CHUNK
    xf, dtf, Bf, Cf, gyf = x, dt.float(), B, C, gy            # operands keep their dtype: the scans take bf16, the glue promotes
    if pad:
        xf, Bf, Cf, gyf = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (xf, Bf, Cf, gyf))
        dtf = F.pad(dtf, (0, 0, 0, pad))
    Af = A.float()
    a = dtf * Af
    a_rev = _shift_reverse(a)
    nv = max(n // 64, 2)                                                               # virtual heads per head (even)
    gfin = None if gfinal is None else gfinal.float()
    gy_r, x_r, B_r, C_r = gyf.flip(1), xf.flip(1), Bf.flip(1), Cf.flip(1)              # time-reversed operands, flipped once

    # 1. dX (before the dt factor), the gradient of the initial state, the state cotangents at the chunk boundaries
    y1, fin1, rev_states = ops.scan(gy_r, C_r, B_r, a_rev, None, gfin)
    d_init = fin1 * torch.exp(a[:, 0])[..., None, None] if init is not None else None
    da = ops.decay_grad(xf, gyf, Bf, Cf, a, dtf, states_in=fwd_states, states_cot_rev=rev_states, init=init, gfinal=gfin)

    def state_blocks(st):   # [b, h, p, n] -> [b, h * nv, 64 (n in block), 64 (p)]
        t = st.float().transpose(2, 3)                                                 # [b, h, n, p]
        if n == 64:
            return t.unsqueeze(2).expand(bsz, h, nv, 64, p).reshape(bsz, h * nv, 64, p)
        return t.reshape(bsz, h * nv, 64, p)

    rep_v = lambda t: t.repeat_interleave(nv, dim=2)  # noqa: E731
    # 2. dC per head (forward time), 3. dB / dt per head (reversed time); the state axis as nv virtual heads of width 64
    # (virtual head h * nv + j reads block j of its group's B / C: no per-head copies of B and C are made)
    as_blocks = lambda t: t.reshape(bsz, seqlen + pad, g * (n // 64), 64)  # noqa: E731
    y2 = ops.scan(as_blocks(Bf), xf, gyf, rep_v(a), rep_v(dtf), None if init is None else state_blocks(init), out_f32=False,
                  v_div=nv * rep, v_mod=n // 64)[0]
    y3 = ops.scan(as_blocks(C_r), gy_r, x_r, rep_v(a_rev), None, None if gfin is None else state_blocks(gfin), out_f32=False,
                  v_div=nv * rep, v_mod=n // 64)[0]

    dt_real = dt.float()
    dx, ddt, dD = ops.finish(y1, x, gy, dt_real, da, Af, D)
    dC = ops.group_sum(y2.reshape(bsz, seqlen + pad, h, nv * 64), None, seqlen, g, n, False)
    dB = ops.group_sum(y3.reshape(bsz, seqlen + pad, h, nv * 64), dt_real, seqlen, g, n, True)
    dA = (da[:, :seqlen] * dt_real).sum((0, 1))
    return dx, ddt, dA, dB, dC, dD, d_init


class _SSDFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dt, A, B, C, D, initial_state):
        y, final, states = _forward_kernels(x, dt, A, B, C, D, initial_state)
        ctx.save_for_backward(x, dt, A, B, C, D if D is not None else x.new_empty(0),
                              initial_state if initial_state is not None else x.new_empty(0), final, states)
        ctx.has_d, ctx.has_init = D is not None, initial_state is not None
        ctx.set_materialize_grads(False)   # an unused final state then arrives as None, not as a tensor of zeros
        return y.to(x.dtype), final

    @staticmethod
    def backward(ctx, gy, gfinal):
        x, dt, A, B, C, D, init, final, states = ctx.saved_tensors
        if BACKWARD_KERNELS and hasattr(ext(), "ssd_decay_grad"):
            if gy is None:
                gy = torch.zeros_like(x)
            if (not ctx.has_init and gfinal is None and chunk_backward_supported(x) and x.dtype == torch.bfloat16
                    and (x.shape[2] // B.shape[2]) % 2 == 0):
                # no state enters or leaves the sequence: the fused chunk backward (one kernel per chunk and head instead of
                # three role-permuted scans, the decay-gradient kernel and their glue)
                dx, ddt, dA, dB, dC, dD = ssd_backward_fused(x, dt, A, B, C, D if ctx.has_d else None, gy, states)
                return (dx.to(x.dtype), ddt.to(dt.dtype), dA.to(A.dtype), dB.to(B.dtype), dC.to(C.dtype),
                        None if dD is None else dD.to(D.dtype), None)
            dx, ddt, dA, dB, dC, dD, d_init = ssd_backward(x, dt, A, B, C, D if ctx.has_d else None, init if ctx.has_init else None,
                                                           final, gy, gfinal, fwd_states=states)
            return (dx.to(x.dtype), ddt.to(dt.dtype), dA.to(A.dtype), dB.to(B.dtype), dC.to(C.dtype),
                    None if dD is None else dD.to(D.dtype), None if d_init is None else d_init.to(init.dtype))
        return _SSDFunction._backward_recompute(ctx, gy, gfinal)

    @staticmethod
    def _backward_recompute(ctx, gy, gfinal):
        from ..backbones.mamba2.ssd import ssd_chunk_scan

        x, dt, A, B, C, D, init, _, _ = ctx.saved_tensors
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
        y, final, _ = _forward_kernels(x, dt, A, B, C, D, initial_state)
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
    Qr, Kr, adt, qk_dot = _prepare(Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Angles, torch.float32, fused=True)
    pad = (-seqlen) % CHUNK
    vb, qb, kb = V.to(torch.bfloat16), Qr.to(torch.bfloat16), Kr.to(torch.bfloat16)
    skip = qk_dot
    if pad:  # adt = 0 and k = 0 on the padding: the state is carried unchanged
        vb, qb, kb = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (vb, qb, kb))
        adt, skip = F.pad(adt, (0, 0, 0, pad)), F.pad(skip, (0, 0, 0, pad))
    y, final, states = ext().siso_chunk_scan_fwd(vb.contiguous(), kb.contiguous(), qb.contiguous(), adt.float().contiguous(),
                                                 None if D is None else D.float().contiguous(),
                                                 skip.float().transpose(1, 2).contiguous(), None)
    KERNEL_LAUNCHES["count"] += 4
    return y[:, :seqlen], final, states


def siso_core_backward(Qr, Kr, adt, skip, V, gy, ops=KernelScans, fwd_states=None, keep_dkr_reversed=False):
    """Gradients of y_t = sum_{s < t} e^{c_t - c_s} (Qr_t . Kr_s) V_s + skip_t V_t with respect to the preprocessed operands.

    Qr, Kr [b, l, h, 128]; adt, skip [b, l, h]; V, gy [b, l, h, 64].  Three strict scans with permuted roles:
      dV_s  = sum_{t > s} e^{c_t - c_s} (Kr_s . Qr_t) gy_t + skip_s gy_s    reversed, per head:  v = gy, bk = Qr, cq = Kr
      dQr_t = sum_{s < t} e^{c_t - c_s} (gy_t . V_s) Kr_s                   forward:  v = Kr (two halves), bk = V,  cq = gy
      dKr_s = sum_{t > s} e^{c_t - c_s} (V_s . gy_t) Qr_t                   reversed: v = Qr (two halves), bk = gy, cq = V
    dadt from ``ops.decay_grad`` (pairs s < u <= t counted once), dskip = gy . V.  Returns (dQr, dKr, dadt, dskip, dV)."""
    bsz, seqlen, h, _ = V.shape
    n = Qr.shape[-1]
    pad = (-seqlen) % CHUNK
    Qf, Kf, Vf, gyf, af = Qr, Kr, V, gy, adt.float()
    if pad:
        Qf, Kf, Vf, gyf = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (Qf, Kf, Vf, gyf))
        af = F.pad(af, (0, 0, 0, pad))
    a_rev = _shift_reverse(af)
    nv = n // 64
    rep_v = lambda t: t.repeat_interleave(nv, dim=2)  # noqa: E731
    gy_r, Q_r, K_r, V_r = gyf.flip(1), Qf.flip(1), Kf.flip(1), Vf.flip(1)                # time-reversed operands, flipped once
    y1, _, rev_states = ops.scan(gy_r, Q_r, K_r, a_rev, None, None, strict=True, per_head=True)
    dV = y1.flip(1)[:, :seqlen] + skip.float()[..., None] * gy.float()
    dadt = ops.decay_grad(Vf, gyf, Kf, Qf, af, None, states_in=fwd_states, states_cot_rev=rev_states, per_head=True)[:, :seqlen]
    y2 = ops.scan(_blocks(Kf, nv), Vf, gyf, rep_v(af), None, None, strict=True)[0]
    dQr = y2.reshape(bsz, seqlen + pad, h, n)
    y3 = ops.scan(_blocks(Q_r, nv), gy_r, V_r, rep_v(a_rev), None, None, strict=True)[0]
    dskip = (gy.float() * V.float()).sum(-1)
    if keep_dkr_reversed:   # the caller reads it backwards (token l of the result is row seqlen + pad - 1 - l)
        return dQr[:, :seqlen], y3.reshape(bsz, seqlen + pad, h, n), dadt, dskip, dV
    dKr = y3.flip(1).reshape(bsz, seqlen + pad, h, n)
    return dQr[:, :seqlen], dKr[:, :seqlen], dadt, dskip, dV


class _SISOFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Angles, D):
        y, _, states = _siso_forward_kernels(Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Angles, D)
        ctx.save_for_backward(Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Angles, D, states)
        return y.to(V.dtype)

    @staticmethod
    def backward(ctx, gy):
        if BACKWARD_KERNELS and hasattr(ext(), "ssd_decay_grad"):
            return _SISOFunction._backward_kernels(ctx, gy)
        return _SISOFunction._backward_recompute(ctx, gy)

    @staticmethod
    def _backward_kernels(ctx, gy):
        """Kernel scans for the recurrence; the preprocessing in front of it is differentiated by its own kernel on the
        wide tensors (csrc/siso_prep.cu) and by autograd on the [b, l, h]-sized ones (trapezoid weights, rotary phase)."""
        from ..backbones.mamba3.siso import _prepare, _prepare_small, _wide_kernels_ok

        Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Angles, D, states = ctx.saved_tensors
        if _wide_kernels_ok(Q) and hasattr(ext(), "siso_prep_bwd"):
            from .dispatch import KERNEL_LAUNCHES

            small = [t.detach().requires_grad_(True) for t in (ADT, DT, Trap, Angles)]
            with torch.enable_grad():
                adt, gamma, scale, theta = _prepare_small(*small, torch.float32)
            wide = (Q.contiguous(), K.to(Q.dtype).contiguous(), Q_bias.float().contiguous(), K_bias.float().contiguous(),
                    theta.detach().contiguous(), gamma.detach().contiguous(), scale.detach().contiguous())
            Qr, Kr, qk_dot = ext().siso_prep_fwd(*wide)
            skip = qk_dot + D.float()[None, None]
            if chunk_backward_supported(V) and V.dtype == torch.bfloat16:
                # the fused chunk backward: every cotangent of the recurrence from one kernel per chunk and head, in natural
                # time order and bf16, as the preprocessing backward reads them
                dV, dQr, dKr, dadt, dskip = chunk_backward(V, gy, Kr, Qr, adt.detach(), None, skip, states, per_head=True, strict=True,
                                                           dv_bf16=True, dn_bf16=True)
                gQ, gK, gQb, gKb, dtheta, dgamma, dscale = ext().siso_prep_bwd(*wide, dQr.contiguous(), dKr.contiguous(),
                                                                                dskip.float().contiguous(), False)
            else:
                dQr, dKr_rev, dadt, dskip, dV = siso_core_backward(Qr, Kr, adt.detach(), skip, V, gy, fwd_states=states,
                                                                   keep_dkr_reversed=True)
                gQ, gK, gQb, gKb, dtheta, dgamma, dscale = ext().siso_prep_bwd(*wide, dQr.float().contiguous(),
                                                                                dKr_rev.float().contiguous(), dskip.float().contiguous(), True)
            KERNEL_LAUNCHES["count"] += 2
            gADT, gDT, gTrap, gAng = torch.autograd.grad([adt, theta, gamma, scale], small, [dadt, dtheta, dgamma, dscale],
                                                         allow_unused=True)
            return (gQ.to(Q.dtype), gK.to(K.dtype), dV.to(V.dtype), gADT, gDT, gTrap, gQb.to(Q_bias.dtype), gKb.to(K_bias.dtype), gAng,
                    dskip.sum((0, 1)).to(D.dtype))
        pre = [t.detach().requires_grad_(True) for t in (Q, K, ADT, DT, Trap, Q_bias, K_bias, Angles)]
        with torch.enable_grad():
            Qr, Kr, adt, qk_dot = _prepare(pre[0], pre[1], V, pre[2], pre[3], pre[4], pre[5], pre[6], pre[7], torch.float32)
        skip = qk_dot.detach() + D.float()[None, None]
        dQr, dKr, dadt, dskip, dV = siso_core_backward(Qr.detach(), Kr.detach(), adt.detach(), skip, V, gy, fwd_states=states)
        grads = torch.autograd.grad([Qr, Kr, adt, qk_dot], pre, [dQr, dKr, dadt, dskip], allow_unused=True)
        gQ, gK, gADT, gDT, gTrap, gQb, gKb, gAng = grads
        return gQ, gK, dV.to(V.dtype), gADT, gDT, gTrap, gQb, gKb, gAng, dskip.sum((0, 1)).to(D.dtype)

    @staticmethod
    def _backward_recompute(ctx, gy):
        from ..backbones.mamba3.siso import mamba3_siso_chunked

        leaves = [t.detach().requires_grad_(True) for t in ctx.saved_tensors[:10]]
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


# ------------------------------------------------------------------------------------------------ fused chunk backward
def chunk_backward_supported(v: torch.Tensor) -> bool:
    return bool(ENABLED and v.is_cuda and native_available() and hasattr(ext(), "ssd_chunk_bwd")
                and os.environ.get("LBI_B200_SSD_PERMUTED_BACKWARD", "0") != "1")


def chunk_backward(v, gy, bk, cq, a, weight, skip, states_in, *, per_head: bool, strict: bool, dv_bf16: bool, dn_bf16: bool,
                   dv_out=None):
    """Every input cotangent of the scan ``y_t = sum_{s <= t} e^{c_t - c_s} (cq_t . bk_s) w_s v_s (+ skip_t v_t)`` from one fused
    kernel per (direction, chunk, head) (csrc/ssd.cu, ``bwd_chunk_kernel``).  The forward operands v [b, l, h, 64], bk, cq
    [b, l, g, n], a, weight, skip [b, l, h] and the forward's incoming chunk states are shared by the P = gy.shape[0] / b stacked
    directions of gy.  Returns (d(w v) [+ skip gy], dcq, dbk per head [P b, l, h, n], da, gy . v [P b, l, h]).  ``dv_out``: a
    [P b l, h 64] bf16 view (a column range of a wider cotangent matrix) the kernel writes the first result into (needs
    ``dv_bf16`` and a sequence length that is a multiple of 128; otherwise the result is copied there)."""
    from .dispatch import KERNEL_LAUNCHES

    bf = torch.bfloat16
    seqlen = v.shape[1]
    pad = (-seqlen) % CHUNK
    vb, gyb, bkb, cqb, af = v.to(bf), gy.to(bf), bk.to(bf), cq.to(bf), a.float()
    wf = None if weight is None else weight.float()
    sf = None if skip is None else skip.float()
    if pad:   # a = 0, operands 0 on the padding: the state is carried unchanged and nothing is added
        vb, gyb, bkb, cqb = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (vb, gyb, bkb, cqb))
        af = F.pad(af, (0, 0, 0, pad))
        wf = None if wf is None else F.pad(wf, (0, 0, 0, pad))
        sf = None if sf is None else F.pad(sf, (0, 0, 0, pad))
    KERNEL_LAUNCHES["count"] += 3   # cumulative sum, reversed state passing with its chunk products, chunk backward
    direct = (dv_out is not None and dv_bf16 and not pad and dv_out.dtype == bf and dv_out.dim() == 2 and dv_out.stride(1) == 1
              and dv_out.stride(0) % 8 == 0 and dv_out.storage_offset() % 8 == 0)
    dv, dcq, dbk, da, dskip = ext().ssd_chunk_bwd(vb.contiguous(), gyb.contiguous(), bkb.contiguous(), cqb.contiguous(), af.contiguous(),
                                                  None if wf is None else wf.contiguous(), None if sf is None else sf.contiguous(),
                                                  None, states_in, bool(per_head), bool(strict), bool(dv_bf16), bool(dn_bf16),
                                                  dv_out if direct else None)
    if pad:
        dv, dcq, dbk, da, dskip = (t[:, :seqlen] for t in (dv, dcq, dbk, da, dskip))
    if dv_out is not None and not direct:
        dv_out.copy_(dv.reshape(dv_out.shape))
        dv = dv_out
    return dv, dcq, dbk, da, dskip


def ssd_backward_fused(x, dt, A, B, C, D, gy, fwd_states):
    """SSD input cotangents through the fused chunk backward; x, dt, B, C and the forward's chunk states [b, ...] are shared by
    the P stacked directions of gy [P b, l, h, 64].  Returns (dx, ddt, dA, dB, dC, dD)."""
    bsz, seqlen, h, p = x.shape
    g, n = B.shape[2], B.shape[3]
    reps = gy.shape[0] // bsz
    dtf, Af = dt.float(), A.float()
    # bf16 results leave the chunk kernel through TMA stores; fp32 ones as 128-byte row pieces from registers
    dX, dC_h, dB_h, da, _ = chunk_backward(x, gy, B, C, dtf * Af, dtf, None, fwd_states, per_head=False, strict=False,
                                           dv_bf16=x.dtype == torch.bfloat16, dn_bf16=True)
    xk = x if x.dtype in (torch.bfloat16, torch.float32) else x.float()
    dx, ddt, dD = ext().ssd_bwd_finish(dX.contiguous(), xk.contiguous(), gy.to(xk.dtype).contiguous(), dtf.contiguous(), da,
                                       Af.contiguous(), None if D is None else D.float().contiguous(), False)
    dC = KernelScans.group_sum(dC_h.contiguous(), None, seqlen, g, n, False)
    dB = KernelScans.group_sum(dB_h.contiguous(), None, seqlen, g, n, False)
    dA = (da.reshape(reps, bsz, seqlen, h) * dtf).sum((0, 1, 2))
    from .dispatch import KERNEL_LAUNCHES

    KERNEL_LAUNCHES["count"] += 1
    return dx, ddt, dA, dB, dC, (dD if D is not None else None)


# ------------------------------------------------------------------------------------------------ dense statements
def _pair_weights(a):
    """a [b, l, h] log-decays -> (c [b, h, l] cumulative, diff [b, h, t, s] = c_t - c_s)."""
    c = a.float().cumsum(1).permute(0, 2, 1)
    return c, c[:, :, :, None] - c[:, :, None, :]


def _decay_cotangent(e):
    """e [b, h, t, s] = dW o W for W[t, s] = exp(c_t - c_s) -> cotangent of the per-token log-decays [b, l, h]."""
    dc = e.sum(3) - e.sum(2)                                    # [b, h, l]
    return dc.flip(2).cumsum(2).flip(2).permute(0, 2, 1)


def siso_core_backward_dense(Qr, Kr, adt, skip, V, gy):
    """The gradients of ``siso_core_backward`` from the O(l^2) definition, in fp32, for any head_dim / d_state / length and
    with the forward operands shared by P stacked directions (gy [P * b, ...], the rest [b, ...])."""
    b, l, h, p = V.shape
    reps = gy.shape[0] // b
    g = gy.float().view(reps, b, l, h, p)
    q, k, v = Qr.float(), Kr.float(), V.float()
    _, diff = _pair_weights(adt)
    strict = torch.ones(l, l, dtype=torch.bool, device=V.device).tril(-1)
    w = torch.exp(diff.masked_fill(~strict, float("-inf")))                      # [b, h, t, s]
    gram = torch.einsum("bthn,bshn->bhts", q, k)
    m = w * gram
    dV = torch.einsum("bhts,rbthp->rbshp", m, g) + skip.float()[None, ..., None] * g
    dM = torch.einsum("rbthp,bshp->rbhts", g, v)
    dG = dM * w
    dQr = torch.einsum("rbhts,bshn->rbthn", dG, k)
    dKr = torch.einsum("rbhts,bthn->rbshn", dG, q)
    dadt = _decay_cotangent((dM * m).reshape(reps * b, h, l, l))
    dskip = (g * v).sum(-1)
    n = q.shape[-1]
    return (dQr.reshape(reps * b, l, h, n), dKr.reshape(reps * b, l, h, n), dadt, dskip.reshape(reps * b, l, h),
            dV.reshape(reps * b, l, h, p))


def ssd_backward_dense(x, dt, A, B, C, D, gy):
    """Gradients of y_t = sum_{s <= t} e^{c_t - c_s} (C_t . B_s) dt_s x_s + D x_t from the O(l^2) definition, in fp32, for any
    shape, with the forward operands shared by P stacked directions.  Returns (dx, ddt, dA, dB, dC, dD)."""
    b, l, h, p = x.shape
    grp, n = B.shape[2], B.shape[3]
    rep = h // grp
    reps = gy.shape[0] // b
    g = gy.float().view(reps, b, l, h, p)
    xf, dtf, Af = x.float(), dt.float(), A.float()
    Bh, Ch = B.float().repeat_interleave(rep, dim=2), C.float().repeat_interleave(rep, dim=2)
    _, diff = _pair_weights(dtf * Af)
    causal = torch.ones(l, l, dtype=torch.bool, device=x.device).tril(0)
    w = torch.exp(diff.masked_fill(~causal, float("-inf")))
    gram = torch.einsum("bthn,bshn->bhts", Ch, Bh)
    nmat = w * gram
    X = dtf.unsqueeze(-1) * xf
    dX = torch.einsum("bhts,rbthp->rbshp", nmat, g)
    dx = dtf[None, ..., None] * dX
    ddt = (dX * xf).sum(-1)
    dN = torch.einsum("rbthp,bshp->rbhts", g, X)
    dG = dN * w
    dCh = torch.einsum("rbhts,bshn->rbthn", dG, Bh)
    dBh = torch.einsum("rbhts,bthn->rbshn", dG, Ch)
    da = _decay_cotangent((dN * nmat).reshape(reps * b, h, l, l)).view(reps, b, l, h)
    ddt = ddt + da * Af
    dA = (da * dtf).sum((0, 1, 2))
    dD = None
    if D is not None:
        dx = dx + D.float()[None, None, None, :, None] * g
        dD = (g * xf).sum((0, 1, 2, 4))
    dB = dBh.view(reps, b, l, grp, rep, n).sum(4).reshape(reps * b, l, grp, n)
    dC = dCh.view(reps, b, l, grp, rep, n).sum(4).reshape(reps * b, l, grp, n)
    return dx.reshape(reps * b, l, h, p), ddt.reshape(reps * b, l, h), dA, dB, dC, dD
