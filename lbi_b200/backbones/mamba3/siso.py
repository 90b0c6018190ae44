"""Mamba-3 single-input single-output (SISO) scan.

Maths (reference Triton kernels backbones/mamba3/ops/triton/mamba3/
mamba3_siso_fwd.py:256-424 and angle_dt.py:83-119; the reference ships no
PyTorch restatement of them):

    theta_t = (sum_{i<=t} pi * tanh(angle_i) * dt_i) mod 2pi           rotary phase, per head
    gamma_t = dt_t * sigmoid(trap_t)                                   trapezoid weight of token t at time t
    scale_t = gamma_t + dt_{t+1} * (1 - sigmoid(trap_{t+1}))           total weight with which token t enters the state
    Qr_t = Rot_theta_t(Q_t + b_Q),  Kr_t = Rot_theta_t(K_t + b_K)      pairwise (2i, 2i+1) rotation of the first pairs
    h_t  = exp(ADT_t) h_{t-1} + scale_t * V_t Kr_t^T
    o_t  = Qr_t . (exp(ADT_t) h_{t-1}) + (D + gamma_t <Q_t + b_Q, K_t + b_K>) V_t
    out_t = o_t * silu(Z_t)

``mamba3_siso_chunked`` evaluates this chunk by chunk with differentiable tensor
ops (CPU or CUDA); ``mamba3_siso_recurrent_reference`` is the fp64 token loop
used as the oracle.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

TWO_PI = 2.0 * math.pi


def angle_dt_cumsum(angles: torch.Tensor, dt: torch.Tensor, init: torch.Tensor | None = None) -> torch.Tensor:
    """angles [b, l, h or 1, s], dt [b, l, h] -> cumulative rotary phase [b, l, h, s] in [0, 2pi); ``init`` [b, h, s] is the
    phase reached before the first token."""
    vals = torch.tanh(angles.float()) * math.pi * dt.float().unsqueeze(-1)
    # the scan runs with the token axis innermost (an outer-axis cumulative sum is several times slower on the GPU)
    theta = torch.cumsum(vals.permute(0, 2, 3, 1).contiguous(), dim=-1).permute(0, 3, 1, 2)
    if init is not None:
        theta = theta + init.to(theta.dtype).unsqueeze(1)
    return theta - TWO_PI * torch.floor(theta / TWO_PI)


def _rotate_pairs(x: torch.Tensor, theta: torch.Tensor) -> torch.Tensor:
    """Rotate pairs (2i, 2i+1) of the last dim by theta[..., i]; pairs beyond theta's width stay fixed."""
    n_angles = theta.shape[-1]
    head, tail = x[..., : 2 * n_angles], x[..., 2 * n_angles :]
    pairs = head.unflatten(-1, (n_angles, 2))
    a, b = pairs[..., 0], pairs[..., 1]
    cos, sin = torch.cos(theta), torch.sin(theta)
    rotated = torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1).flatten(-2)
    return torch.cat((rotated, tail), dim=-1)


class _WidePrepFunction(torch.autograd.Function):
    """Bias, qk dot, rotary turn and trapezoid scale on the [b, l, h, 128] tensors: csrc/siso_prep.cu, both directions."""

    @staticmethod
    def forward(ctx, Q, K, Q_bias, K_bias, theta, gamma, scale):
        from lbi_b200.ops import dispatch, ext

        q, k = Q.contiguous(), K.to(Q.dtype).contiguous()
        qb, kb = Q_bias.float().contiguous(), K_bias.float().contiguous()
        th, gm, sc = theta.float().contiguous(), gamma.float().contiguous(), scale.float().contiguous()
        qr, kr, qk = ext().siso_prep_fwd(q, k, qb, kb, th, gm, sc)
        dispatch.KERNEL_LAUNCHES["count"] += 1
        ctx.save_for_backward(q, k, qb, kb, th, gm, sc)
        ctx.dtypes = (Q.dtype, K.dtype, Q_bias.dtype, K_bias.dtype, theta.dtype, gamma.dtype, scale.dtype)
        return qr, kr, qk

    @staticmethod
    def backward(ctx, dqr, dkr, dqk):
        from lbi_b200.ops import dispatch, ext

        q, k, qb, kb, th, gm, sc = ctx.saved_tensors
        zeros = lambda like, shape: torch.zeros(shape, dtype=torch.float32, device=like.device)  # noqa: E731
        dqr = zeros(q, (*th.shape[:3], 128)) if dqr is None else dqr.float().contiguous()
        dkr = zeros(q, (*th.shape[:3], 128)) if dkr is None else dkr.float().contiguous()
        dqk = zeros(q, th.shape[:3]) if dqk is None else dqk.float().contiguous()
        grads = ext().siso_prep_bwd(q, k, qb, kb, th, gm, sc, dqr, dkr, dqk)
        dispatch.KERNEL_LAUNCHES["count"] += 1
        return tuple(g.to(dt) for g, dt in zip(grads, ctx.dtypes))


def _wide_kernels_ok(Q: torch.Tensor) -> bool:
    if not (Q.is_cuda and Q.shape[-1] == 128 and Q.dtype in (torch.bfloat16, torch.float32)):
        return False
    if torch._C._functorch.maybe_current_level() is not None:
        return False
    from lbi_b200.ops import ext, native_available

    return native_available() and hasattr(ext(), "siso_prep_fwd")


def _prepare_small(ADT, DT, Trap, Angles, compute_dtype, angle_state=None):
    """The [b, l, h]-sized part: log-decay, trapezoid weights gamma / scale, cumulative rotary phase theta [b, l, h, s]."""
    dt = DT.to(compute_dtype).transpose(1, 2)  # [b, l, h]
    adt = ADT.to(compute_dtype).transpose(1, 2)
    sig = torch.sigmoid(Trap.to(compute_dtype).transpose(1, 2))
    gamma = dt * sig
    carry = F.pad((dt * (1.0 - sig))[:, 1:], (0, 0, 0, 1))  # dt_{t+1} (1 - sigma_{t+1}), zero after the last token
    scale = gamma + carry
    theta = angle_dt_cumsum(Angles, dt, angle_state).to(compute_dtype)
    return adt, gamma, scale, theta


def _prepare(Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Angles, compute_dtype, fused: bool = False, angle_state=None):
    """Shared preprocessing: per-head biased/rotated Q, K, trapezoid weights.

    The small tensors ([b, l, h] and [b, l, h, angles]: trapezoid weights, cumulative rotary phase) are PyTorch ops.  With
    ``fused`` (the kernel path of ``ops/ssd.py``) everything on the [b, l, h, d_state] tensors runs in one kernel per
    direction and Qr, Kr come back in bf16, the dtype the scan kernels take."""
    bsz, seqlen, nheads, _ = V.shape
    rep = nheads // Q.shape[2]
    adt, gamma, scale, theta = _prepare_small(ADT, DT, Trap, Angles, compute_dtype, angle_state)
    if fused and compute_dtype == torch.float32 and _wide_kernels_ok(Q):
        Qr, Kr, qk_dot = _WidePrepFunction.apply(Q, K, Q_bias, K_bias, theta, gamma, scale)
        return Qr, Kr, adt, qk_dot
    Qh = Q.to(compute_dtype).repeat_interleave(rep, dim=2) + Q_bias.to(compute_dtype)[None, None]
    Kh = K.to(compute_dtype).repeat_interleave(rep, dim=2) + K_bias.to(compute_dtype)[None, None]
    qk_dot = gamma * (Qh * Kh).sum(dim=-1)
    Qr = _rotate_pairs(Qh, theta)
    Kr = _rotate_pairs(Kh, theta) * scale.unsqueeze(-1)
    return Qr, Kr, adt, qk_dot


def mamba3_siso_recurrent_reference(Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Angles, D=None, Z=None):
    """fp64 token-by-token evaluation.  Q, K [b, l, g, n]; V, Z [b, l, h, p]; ADT, DT, Trap [b, h, l];
    Q_bias, K_bias [h, n]; Angles [b, l, h, s]; D [h]."""
    bsz, seqlen, nheads, headdim = V.shape
    Qr, Kr, adt, qk_dot = _prepare(Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Angles, torch.float64)
    Vd = V.double()
    state = torch.zeros(bsz, nheads, headdim, Qr.shape[-1], dtype=torch.float64, device=V.device)
    outs = []
    for t in range(seqlen):
        state = state * torch.exp(adt[:, t])[..., None, None]
        o = torch.einsum("bhpn,bhn->bhp", state, Qr[:, t])
        skip = qk_dot[:, t] if D is None else qk_dot[:, t] + D.double()[None]
        o = o + skip[..., None] * Vd[:, t]
        state = state + Vd[:, t][..., None] * Kr[:, t][:, :, None, :]
        outs.append(o)
    out = torch.stack(outs, dim=1)
    if Z is not None:
        out = out * F.silu(Z.double())
    return out


def mamba3_siso_chunked(Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Angles, D=None, Z=None, chunk_size: int = 64,
                        initial_states=None, return_final_states: bool = False):
    """Chunked evaluation in fp32 with the same argument layout as the recurrent reference.

    ``initial_states`` = (angle_state [b, h, s], ssm_state [b, h, p, n], k_state [b, h, n], v_state [b, h, p]) continues a
    sequence: the phase starts from ``angle_state``, and the state from ``ssm_state`` plus the look-ahead share
    dt_0 (1 - sigmoid(trap_0)) v_state k_state^T that the previous token is owed under the trapezoid rule.  With
    ``return_final_states`` the same four tensors come back for the last token (``ssm_state`` again without that token's
    look-ahead share), so that calls chain and ``Mamba3.step`` can carry on from them."""
    bsz, seqlen, nheads, headdim = V.shape
    out_dtype = V.dtype
    angle0 = ssm0 = None
    if initial_states is not None:
        angle0, ssm0, k0, v0 = initial_states
        owed = DT[:, :, 0].float() * (1.0 - torch.sigmoid(Trap[:, :, 0].float()))
        ssm0 = ssm0.float() + owed[..., None, None] * v0.float()[..., None] * k0.float()[:, :, None, :]
    Qr, Kr, adt, qk_dot = _prepare(Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Angles, torch.float32, angle_state=angle0)
    Vf = V.float()
    pad = (-seqlen) % chunk_size
    if pad:
        Qr = F.pad(Qr, (0, 0, 0, 0, 0, pad))
        Kr = F.pad(Kr, (0, 0, 0, 0, 0, pad))
        Vf = F.pad(Vf, (0, 0, 0, 0, 0, pad))
        adt = F.pad(adt, (0, 0, 0, pad))
        qk_dot = F.pad(qk_dot, (0, 0, 0, pad))
    nchunks = (seqlen + pad) // chunk_size
    dstate = Qr.shape[-1]
    Qc = Qr.view(bsz, nchunks, chunk_size, nheads, dstate)
    Kc = Kr.view(bsz, nchunks, chunk_size, nheads, dstate)
    Vc = Vf.view(bsz, nchunks, chunk_size, nheads, headdim)
    cum = torch.cumsum(adt.view(bsz, nchunks, chunk_size, nheads), dim=2)
    total = cum[:, :, -1]

    strict = torch.ones(chunk_size, chunk_size, dtype=torch.bool, device=V.device).tril(-1)
    diff = cum[:, :, :, None, :] - cum[:, :, None, :, :]
    decay = torch.exp(diff.masked_fill(~strict[None, None, :, :, None], float("-inf")))
    scores = torch.einsum("bcihn,bcjhn->bcijh", Qc, Kc) * decay
    y = torch.einsum("bcijh,bcjhp->bcihp", scores, Vc)

    to_end = torch.exp(total[:, :, None, :] - cum)
    chunk_states = torch.einsum("bcqhp,bcqh,bcqhn->bchpn", Vc, to_end, Kc)
    state = torch.zeros(bsz, nheads, headdim, dstate, dtype=torch.float32, device=V.device) if ssm0 is None else ssm0
    incoming = []
    for c in range(nchunks):
        incoming.append(state)
        state = state * torch.exp(total[:, c])[..., None, None] + chunk_states[:, c]
    prev = torch.stack(incoming, dim=1)
    y = y + torch.einsum("bcqhn,bchpn,bcqh->bcqhp", Qc, prev, torch.exp(cum))

    skip = qk_dot.view(bsz, nchunks, chunk_size, nheads)
    if D is not None:
        skip = skip + D.float()[None, None, None, :]
    y = y + skip.unsqueeze(-1) * Vc
    y = y.reshape(bsz, nchunks * chunk_size, nheads, headdim)[:, :seqlen]
    if Z is not None:
        y = y * F.silu(Z.float())
    if not return_final_states:
        return y.to(out_dtype)
    # zero decay and zero keys on the padding: ``state`` is the state after the last real token
    theta_last = _prepare_small(ADT, DT, Trap, Angles, torch.float32, angle0)[3][:, -1]  # [b, h, s]
    rep = nheads // K.shape[2]
    k_last = K[:, -1].float().repeat_interleave(rep, dim=1) + K_bias.float()[None]
    return y.to(out_dtype), theta_last, state, _rotate_pairs(k_last, theta_last), V[:, -1]


def _packed_edges(cu_seqlens, batch: int, seqlen: int) -> list[tuple[int, int]]:
    if batch != 1:
        raise ValueError("cu_seqlens describes one packed row: the batch size must be 1")
    edges = [int(v) for v in cu_seqlens.tolist()]
    if edges[0] != 0 or edges[-1] != seqlen or any(b < a for a, b in zip(edges[:-1], edges[1:])):
        raise ValueError("cu_seqlens must rise from 0 to the packed length")
    return list(zip(edges[:-1], edges[1:]))


def mamba3_siso_combined(Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Angles, D=None, Z=None, Input_States=None,
                         chunk_size: int = 64, return_final_states: bool = False, cu_seqlens=None):
    """Entry point with the argument list of the reference's combined op
    (backbones/mamba3/ops/triton/mamba3/mamba3_siso_combined.py:291-307).  Q, K [b, l, g, n]; V, Z [b, l, h, p];
    ADT, DT, Trap [b, h, l]; Q_bias, K_bias [h, n]; Angles [b, l, h or 1, s]; D [h].

    Without states the sm_100a kernels run where the shape allows them (``ops.ssd.mamba3_siso_cuda``: bf16, head_dim 64,
    d_state 128); with ``Input_States`` or ``return_final_states`` the chunked fp32 form runs, which carries the four state
    tensors (see ``mamba3_siso_chunked``).  With ``cu_seqlens`` [num_sequences + 1] the single row holds several sequences end
    to end: each is evaluated on its own, the states have one entry per sequence."""
    if cu_seqlens is not None:
        outs, finals = [], []
        for i, (s, e) in enumerate(_packed_edges(cu_seqlens, V.shape[0], V.shape[1])):
            if e == s:
                raise ValueError("cu_seqlens holds an empty sequence")
            init = None if Input_States is None else tuple(t[i : i + 1] for t in Input_States)
            res = mamba3_siso_chunked(Q[:, s:e], K[:, s:e], V[:, s:e], ADT[..., s:e], DT[..., s:e], Trap[..., s:e], Q_bias, K_bias,
                                      Angles[:, s:e], D, None if Z is None else Z[:, s:e], chunk_size=chunk_size,
                                      initial_states=init, return_final_states=True)
            outs.append(res[0])
            finals.append(res[1:])
        y = torch.cat(outs, dim=1)
        if not return_final_states:
            return y
        return (y, *(torch.cat([f[j] for f in finals], dim=0) for j in range(4)))
    if Input_States is None and not return_final_states:
        from lbi_b200.ops import ssd as ops_ssd

        if ops_ssd.siso_cuda_supported(V, Q) and V.dtype == torch.bfloat16 and D is not None:
            return ops_ssd.mamba3_siso_cuda(Q=Q, K=K, V=V, ADT=ADT, DT=DT, Trap=Trap, Q_bias=Q_bias, K_bias=K_bias,
                                            Angles=Angles, D=D, Z=Z)
    return mamba3_siso_chunked(Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Angles, D, Z, chunk_size=chunk_size,
                               initial_states=Input_States, return_final_states=return_final_states)


def angle_dt(angle: torch.Tensor, dt: torch.Tensor, init_state: torch.Tensor | None = None, chunk_size: int = 64,
             return_output_state: bool = False, cu_seqlens=None):
    """Cumulative rotary phase with the argument layout of the reference's op (angle_dt.py:127-152): angle [b, l, h, s] raw
    rates, dt [b, h, l] -> [b, l, h, s] = (init + cumsum(pi tanh(angle) dt)) mod 2 pi, optionally with the last phase
    ([b, h, s], or one entry per sequence of a packed row when ``cu_seqlens`` is given; ``init_state`` likewise)."""
    if cu_seqlens is None:
        theta = angle_dt_cumsum(angle, dt.transpose(1, 2), init_state)
        return (theta, theta[:, -1]) if return_output_state else theta
    parts = []
    for i, (s, e) in enumerate(_packed_edges(cu_seqlens, angle.shape[0], angle.shape[1])):
        parts.append(angle_dt_cumsum(angle[:, s:e], dt[..., s:e].transpose(1, 2), None if init_state is None else init_state[i : i + 1]))
    theta = torch.cat(parts, dim=1)
    return (theta, torch.cat([p[:, -1] for p in parts], dim=0)) if return_output_state else theta
