"""Ops of the closed-form Mamba-2 / Mamba-3 block chains (``backends/mamba_structured.py``).

Every function has a PyTorch statement (fp32, any device, no autograd needed: forward values and explicit
cotangent formulas) and, for bf16 CUDA tensors, a route to the sm_100a kernels.  Functions that pull cotangents
back accept ``P`` stacked directions: the cotangent rows are ``[P * n, ...]`` (direction-major) while the cached
forward operands keep their ``n`` rows and are shared by all directions.

Reference counterparts: the gated RMSNorm Triton kernels (backbones/mamba2/ops/triton/layernorm_gated.py:45-268),
the angle / dt kernels of Mamba-3 (backbones/mamba3/ops/triton/mamba3/angle_dt.py:26-330) and the dd_dt / trap /
rotary part of its backward (mamba3_siso_bwd.py:811-1418).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .native import ext, native_available

TWO_PI = 2.0 * math.pi


def _count(n: int = 1) -> None:
    from .dispatch import KERNEL_LAUNCHES

    KERNEL_LAUNCHES["count"] += n


def _fell_back(op: str, *values) -> None:
    """Count (strict mode: refuse) a PyTorch route taken by CUDA bf16 operands; see ``ops.dispatch.fell_back``."""
    from .dispatch import fell_back

    fell_back(op, *values)


def _kernel_ok(*tensors, name: str | None = None) -> bool:
    if not native_available() or (name is not None and not hasattr(ext(), name)):
        return False
    return all(t is None or t.is_cuda for t in tensors)


def _tile_rows(t: torch.Tensor, reps: int) -> torch.Tensor:
    """[n, ...] -> [reps * n, ...] with the n rows repeated (direction-major stacking)."""
    if reps == 1:
        return t
    return t.unsqueeze(0).expand(reps, *t.shape).reshape(reps * t.shape[0], *t.shape[1:])


# ---------------------------------------------------------------- SiLU gate  yg = y * silu(z)
def gate_silu_fwd(y: torch.Tensor, z: torch.Tensor) -> torch.Tensor:
    if _kernel_ok(y, z, name="gate_silu_fwd") and y.dtype == torch.bfloat16 and z.dtype == torch.bfloat16 and y.shape[-1] % 8 == 0:
        _count()
        return ext().gate_silu_fwd(y.contiguous(), z.contiguous())
    _fell_back("gate_silu_fwd", y, z)
    return (y.float() * F.silu(z.float())).to(y.dtype)


def gate_silu_bwd(dyg: torch.Tensor, y: torch.Tensor, z: torch.Tensor, dz_out: torch.Tensor | None = None):
    """dyg [P * n, d]; y, z [n, d] -> (dy, dz) [P * n, d] in the dtype of dyg.  ``dz_out``: a [P * n, d] view (a column range of
    a wider cotangent matrix) that receives dz in place of a fresh tensor."""
    if (_kernel_ok(dyg, y, z, name="gate_silu_bwd") and dyg.dtype == torch.bfloat16 and y.dtype == torch.bfloat16
            and z.dtype == torch.bfloat16 and y.dim() == 2 and y.shape[-1] % 8 == 0):
        direct = (dz_out is not None and dz_out.dtype == torch.bfloat16 and dz_out.stride(-1) == 1 and dz_out.stride(0) % 8 == 0
                  and dz_out.storage_offset() % 8 == 0)
        _count()
        dy, dz = ext().gate_silu_bwd(dyg.contiguous(), y.contiguous(), z.contiguous(), dz_out if direct else None)
        if dz_out is not None and not direct:
            dz_out.copy_(dz)
            dz = dz_out
        return dy, dz
    _fell_back("gate_silu_bwd", dyg, y, z)
    reps = dyg.shape[0] // y.shape[0]
    g = dyg.float().view(reps, *y.shape)
    zf, yf = z.float(), y.float()
    sig = torch.sigmoid(zf)
    dy = g * (zf * sig)
    dz = (g * yf * (sig * (1.0 + zf * (1.0 - sig)))).reshape(dyg.shape).to(dyg.dtype)
    if dz_out is not None:
        dz_out.copy_(dz)
        dz = dz_out
    return dy.reshape(dyg.shape).to(dyg.dtype), dz


# ---------------------------------------------------------------- RMSNorm over groups of the last axis, optional SiLU gate
def gated_rmsnorm_fwd(x, z, weight, eps: float, group: int, gate_first: bool):
    """x, z [n, d] -> (y [n, d], rstd [n, d / group] fp32).  ``gate_first``: norm(x * silu(z)) (Mamba-2), else
    norm(x) * silu(z); without z a plain grouped RMSNorm (the B / C norms of Mamba-3)."""
    if (_kernel_ok(x, z, weight, name="gated_rmsnorm_fwd") and x.dtype in (torch.bfloat16, torch.float32) and group % 8 == 0
            and x.shape[-1] <= 12288 and x.shape[-1] % group == 0):
        _count()
        return ext().gated_rmsnorm_fwd(x.contiguous(), None if z is None else z.to(x.dtype).contiguous(), weight.float().contiguous(),
                                       float(eps), int(group), bool(gate_first))
    _fell_back("gated_rmsnorm_fwd", x, z)
    xf = x.float()
    if z is not None and gate_first:
        xf = xf * F.silu(z.float())
    grouped = xf.unflatten(-1, (-1, group))
    rstd = torch.rsqrt(grouped.square().mean(dim=-1) + eps)
    y = (grouped * rstd.unsqueeze(-1)).flatten(-2) * weight.float()
    if z is not None and not gate_first:
        y = y * F.silu(z.float())
    return y.to(x.dtype), rstd


def gated_rmsnorm_bwd(dy, x, z, weight, rstd, group: int, gate_first: bool, want_dweight: bool = False):
    """dy [P * n, d]; x, z [n, d]; rstd [n, d / group] -> (dx, dz or None, dweight or None)."""
    reps = dy.shape[0] // x.shape[0]
    if (_kernel_ok(dy, x, z, weight, rstd, name="gated_rmsnorm_bwd") and x.dtype in (torch.bfloat16, torch.float32)
            and group % 8 == 0 and x.shape[-1] <= 12288):
        _count()
        dx, dz, dw = ext().gated_rmsnorm_bwd(dy.to(x.dtype).contiguous(), x.contiguous(), None if z is None else z.to(x.dtype).contiguous(),
                                             weight.float().contiguous(), rstd.contiguous(), int(group), bool(gate_first),
                                             bool(want_dweight))
        return dx, (dz if z is not None else None), (dw if want_dweight else None)
    _fell_back("gated_rmsnorm_bwd", dy, x, z)
    w = weight.float()
    g = dy.float().view(reps, *x.shape)
    xf = x.float()
    dz = None
    if z is not None:
        zf = z.float()
        sig = torch.sigmoid(zf)
        silu, dsilu = zf * sig, sig * (1.0 + zf * (1.0 - sig))
    u = xf * silu if (z is not None and gate_first) else xf
    uh = (u.unflatten(-1, (-1, group)) * rstd.unsqueeze(-1)).flatten(-2)          # normalised input
    if z is not None and not gate_first:
        dz = g * (uh * w) * dsilu
        g = g * silu
    dw = (g * uh).sum(dim=(0, 1)) if want_dweight else None
    wg = (g * w).unflatten(-1, (-1, group))
    uhg = uh.unflatten(-1, (-1, group))
    du = ((wg - uhg * (wg * uhg).mean(dim=-1, keepdim=True)) * rstd.unsqueeze(-1)).flatten(-2)
    if z is not None and gate_first:
        dz = du * xf * dsilu
        du = du * silu
    out_dtype = x.dtype
    return du.reshape(dy.shape).to(out_dtype), (None if dz is None else dz.reshape(dy.shape).to(out_dtype)), dw


# ---------------------------------------------------------------- Mamba-3: the [b, l, h]-sized preprocessing
@dataclass
class SisoSmall:
    """Per-token, per-head scalars of the SISO mixer (all fp32).  dt, a, sig, adt, gamma, scale [b, l, h];
    tanh_angle [b, l, s]; theta [b, l, h, s] in [0, 2 pi); sp_dt, sp_a: the sigmoids of the softplus arguments;
    a_live: 1 where A is not clamped at -A_floor."""
    dt: torch.Tensor
    a: torch.Tensor
    sig: torch.Tensor
    adt: torch.Tensor
    gamma: torch.Tensor
    scale: torch.Tensor
    tanh_angle: torch.Tensor
    theta: torch.Tensor
    sp_dt: torch.Tensor
    sp_a: torch.Tensor
    a_live: torch.Tensor


def siso_small_fwd(dd_dt, dd_a, trap, angles, dt_bias, a_floor: float, batch: int, seq_len: int) -> SisoSmall:
    """dd_dt, dd_a, trap [n, h]; angles [n, s]; dt_bias [h].  DT = softplus(dd_dt + bias), A = min(-softplus(dd_a), -floor),
    gamma = DT sigmoid(trap), scale_t = gamma_t + DT_{t+1} (1 - sigmoid(trap_{t+1})) (0 past the last token of a sequence),
    theta_t = (sum_{i <= t} pi tanh(angle_i) DT_i) mod 2 pi."""
    h, s = dd_dt.shape[-1], angles.shape[-1]
    if _kernel_ok(dd_dt, dd_a, trap, angles, dt_bias, name="siso_small_fwd") and h <= 32 and s <= 64:
        _count(2)   # segment totals + the walk over the segments
        out = ext().siso_small_fwd(dd_dt.float().contiguous(), dd_a.float().contiguous(), trap.float().contiguous(),
                                   angles.float().contiguous(), dt_bias.float().contiguous(), float(a_floor), int(batch), int(seq_len))
        return SisoSmall(*out)
    _fell_back("siso_small_fwd", dd_dt, dd_a, trap, angles)
    pre = dd_dt.float().view(batch, seq_len, h) + dt_bias.float()
    dt = F.softplus(pre)
    raw_a = -F.softplus(dd_a.float().view(batch, seq_len, h))
    a = torch.clamp(raw_a, max=-a_floor)
    sig = torch.sigmoid(trap.float().view(batch, seq_len, h))
    gamma = dt * sig
    carry = F.pad((dt * (1.0 - sig))[:, 1:], (0, 0, 0, 1))
    tanh_angle = torch.tanh(angles.float().view(batch, seq_len, s))
    vals = (math.pi * tanh_angle).unsqueeze(2) * dt.unsqueeze(-1)                       # [b, l, h, s]
    theta = torch.cumsum(vals, dim=1)
    theta = theta - TWO_PI * torch.floor(theta / TWO_PI)
    return SisoSmall(dt=dt, a=a, sig=sig, adt=a * dt, gamma=gamma, scale=gamma + carry, tanh_angle=tanh_angle, theta=theta,
                     sp_dt=torch.sigmoid(pre), sp_a=torch.sigmoid(dd_a.float().view(batch, seq_len, h)),
                     a_live=(raw_a < -a_floor).float())


def siso_small_bwd(small: SisoSmall, dadt, dtheta, dgamma, dscale, out_dtype=torch.float32):
    """Cotangents [P * b, l, h(, s)] of (adt, theta, gamma, scale) -> cotangents of (dd_dt, dd_a, trap) [P * b * l, h] and of
    the angles [P * b * l, s]."""
    b, l, h = small.dt.shape
    s = small.tanh_angle.shape[-1]
    reps = dadt.shape[0] // b
    if _kernel_ok(dadt, dtheta, dgamma, dscale, small.dt, name="siso_small_bwd") and h <= 32 and s <= 32:
        _count(2)   # segment totals + the walk over the segments
        return ext().siso_small_bwd(small.dt, small.a, small.sig, small.tanh_angle, small.sp_dt, small.sp_a, small.a_live,
                                    dadt.float().contiguous(), dtheta.float().contiguous(), dgamma.float().contiguous(),
                                    dscale.float().contiguous(), out_dtype == torch.bfloat16)
    dadt, dgamma, dscale = (t.float().reshape(reps, b, l, h) for t in (dadt, dgamma, dscale))
    dvals = dtheta.float().reshape(reps, b, l, h, s).flip(2).cumsum(2).flip(2)              # reversed cumulative sum over tokens
    d_tanh = math.pi * (dvals * small.dt.unsqueeze(-1)).sum(3)                             # [P, b, l, s]
    d_angles = d_tanh * (1.0 - small.tanh_angle.square())
    d_scale_prev = F.pad(dscale[:, :, :-1], (0, 0, 1, 0))                                  # token t receives dscale_{t-1}
    d_gamma_all = dgamma + dscale
    d_dt = (dadt * small.a + math.pi * (dvals * small.tanh_angle.unsqueeze(2)).sum(-1) + d_gamma_all * small.sig
            + d_scale_prev * (1.0 - small.sig))
    d_sig = small.dt * (d_gamma_all - d_scale_prev)
    d_trap = d_sig * small.sig * (1.0 - small.sig)
    d_dd_a = -(dadt * small.dt) * small.sp_a * small.a_live
    d_dd_dt = d_dt * small.sp_dt
    n = reps * b * l
    return (d_dd_dt.reshape(n, h).to(out_dtype), d_dd_a.reshape(n, h).to(out_dtype), d_trap.reshape(n, h).to(out_dtype),
            d_angles.reshape(n, s).to(out_dtype))


# ---------------------------------------------------------------- Mamba-3: bias, rotary turn, trapezoid scale on [b, l, h, n]
def _rotate_pairs(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    n_angles = cos.shape[-1]
    head, tail = x[..., : 2 * n_angles], x[..., 2 * n_angles:]
    a, b = head.unflatten(-1, (n_angles, 2)).unbind(-1)
    rotated = torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1).flatten(-2)
    return torch.cat((rotated, tail), dim=-1)


def siso_wide_fwd(q, k, q_bias, k_bias, theta, gamma, scale):
    """q, k [b, l, g, n]; biases [h, n]; theta [b, l, h, s]; gamma, scale [b, l, h] -> (Qr, Kr [b, l, h, n], qk [b, l, h] fp32):
    Qr = Rot(q + bq), Kr = scale Rot(k + bk), qk = gamma <q + bq, k + bk>."""
    if _kernel_ok(q, k, theta, name="siso_prep_fwd") and q.shape[-1] == 128 and q.dtype in (torch.bfloat16, torch.float32):
        _count()
        return ext().siso_prep_fwd(q.contiguous(), k.to(q.dtype).contiguous(), q_bias.float().contiguous(), k_bias.float().contiguous(),
                                   theta.float().contiguous(), gamma.float().contiguous(), scale.float().contiguous())
    _fell_back("siso_wide_fwd", q, k)
    h = q_bias.shape[0]
    rep = h // q.shape[2]
    qh = q.float().repeat_interleave(rep, dim=2) + q_bias.float()
    kh = k.float().repeat_interleave(rep, dim=2) + k_bias.float()
    cos, sin = torch.cos(theta.float()), torch.sin(theta.float())
    return (_rotate_pairs(qh, cos, sin).to(q.dtype), (_rotate_pairs(kh, cos, sin) * scale.float().unsqueeze(-1)).to(q.dtype),
            gamma.float() * (qh * kh).sum(-1))


def siso_wide_bwd(q, k, q_bias, k_bias, theta, gamma, scale, dqr, dkr, dqk, dkr_reversed: bool = False, want_bias: bool = True):
    """Cotangents dqr, dkr [P * b, l(p), h, n] (dkr optionally in reversed token order over a padded length), dqk [P * b, l, h]
    -> (dq, dk [P * b, l, g, n] fp32, dq_bias, dk_bias [h, n] or None, dtheta [P * b, l, h, s], dgamma, dscale [P * b, l, h]).
    The forward tensors q, k, theta, gamma, scale [b, ...] are shared by the P directions."""
    b, l = q.shape[:2]
    reps = dqr.shape[0] // b
    if _kernel_ok(q, k, theta, dqr, dkr, dqk, name="siso_prep_bwd") and q.shape[-1] == 128 and q.dtype in (torch.bfloat16, torch.float32):
        _count()
        cot = dqr.dtype if (dqr.dtype == dkr.dtype and dqr.dtype in (torch.bfloat16, torch.float32)) else torch.float32
        out = ext().siso_prep_bwd(q.contiguous(), k.to(q.dtype).contiguous(), q_bias.float().contiguous(), k_bias.float().contiguous(),
                                  theta.float().contiguous(), gamma.float().contiguous(), scale.float().contiguous(),
                                  dqr.to(cot).contiguous(), dkr.to(cot).contiguous(), dqk.float().contiguous(), bool(dkr_reversed),
                                  bool(want_bias))
        if not want_bias:
            out[2] = out[3] = None
        return tuple(out)
    _fell_back("siso_wide_bwd", q, k, dqr, dkr)
    if dkr_reversed:
        dkr = dkr.flip(1)[:, :l]
    h, n = q_bias.shape
    g = q.shape[2]
    rep = h // g
    qh = q.float().repeat_interleave(rep, dim=2) + q_bias.float()
    kh = k.float().repeat_interleave(rep, dim=2) + k_bias.float()
    cos, sin = torch.cos(theta.float()), torch.sin(theta.float())
    dqr_, dkr_, dqk_ = dqr.float().view(reps, b, l, h, n), dkr.float().view(reps, b, l, h, n), dqk.float().view(reps, b, l, h)
    sc, gm = scale.float().unsqueeze(-1), gamma.float()
    dqh = _rotate_pairs(dqr_, cos, -sin) + (dqk_ * gm).unsqueeze(-1) * kh
    dkh = sc * _rotate_pairs(dkr_, cos, -sin) + (dqk_ * gm).unsqueeze(-1) * qh
    na = theta.shape[-1]
    rq, rk = _rotate_pairs(qh, cos, sin), _rotate_pairs(kh, cos, sin)

    def turn_grad(d, r):   # <d_pair, J r_pair> with J (a, b) = (-b, a)
        da, db = d[..., : 2 * na].unflatten(-1, (na, 2)).unbind(-1)
        ra, rb = r[..., : 2 * na].unflatten(-1, (na, 2)).unbind(-1)
        return -da * rb + db * ra

    dtheta = turn_grad(dqr_, rq) + scale.float().unsqueeze(-1) * turn_grad(dkr_, rk)
    dgamma = dqk_ * (qh * kh).sum(-1)
    dscale = (dkr_ * rk).sum(-1)
    dq = dqh.view(reps, b, l, g, rep, n).sum(4).reshape(reps * b, l, g, n)
    dk = dkh.view(reps, b, l, g, rep, n).sum(4).reshape(reps * b, l, g, n)
    return (dq, dk, dqh.sum((0, 1, 2)) if want_bias else None, dkh.sum((0, 1, 2)) if want_bias else None,
            dtheta.reshape(reps * b, l, h, na), dgamma.reshape(reps * b, l, h), dscale.reshape(reps * b, l, h))


# ---------------------------------------------------------------- Mamba-3: the recurrence itself
def siso_scan_fwd(v, kr, qr, adt, skip, d_skip):
    """v [b, l, h, p]; kr, qr [b, l, h, n]; adt, skip [b, l, h]; d_skip [h] ->
    (y_t = sum_{s < t} e^{c_t - c_s} (qr_t . kr_s) v_s + (skip_t + D) v_t, incoming chunk states or None)."""
    from . import ssd

    b, l, h, p = v.shape
    if ssd.siso_cuda_supported(v, qr) and v.dtype == torch.bfloat16:
        pad = (-l) % ssd.CHUNK
        vb, qb, kb, a, sk = v, qr.to(torch.bfloat16), kr.to(torch.bfloat16), adt.float(), skip.float()
        if pad:
            vb, qb, kb = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (vb, qb, kb))
            a, sk = F.pad(a, (0, 0, 0, pad)), F.pad(sk, (0, 0, 0, pad))
        y, _, states = ext().siso_chunk_scan_fwd(vb.contiguous(), kb.contiguous(), qb.contiguous(), a.contiguous(),
                                                 None if d_skip is None else d_skip.float().contiguous(),
                                                 sk.transpose(1, 2).contiguous(), None)
        _count(4)
        return y[:, :l], states
    _fell_back("siso_scan_fwd", v, kr, qr)
    y, _ = ssd.scan_generic_torch(v, kr, qr, adt, None, None, strict=True, per_head=True)
    total_skip = skip.float() if d_skip is None else skip.float() + d_skip.float()
    return (y + total_skip.unsqueeze(-1) * v.float()).to(v.dtype), None


def siso_scan_bwd(qr, kr, adt, skip_total, v, gy, states, dv_out=None):
    """gy [P * b, l, h, p] with the forward operands shared by the P directions ->
    (dQr, dKr, dadt, dskip, dV, dkr_is_time_reversed).  ``dv_out``: a [P b l, h p] view that receives dV (a column range of the
    in_proj cotangent), written by the kernel itself where it can."""
    from . import ssd

    reps = gy.shape[0] // v.shape[0]
    if ssd.siso_cuda_supported(v, qr) and gy.dtype == torch.bfloat16 and states is not None:
        if ssd.chunk_backward_supported(v):
            dv, dqr, dkr, dadt, dskip = ssd.chunk_backward(v, gy, kr, qr, adt, None, skip_total, states, per_head=True, strict=True,
                                                           dv_bf16=True, dn_bf16=True, dv_out=dv_out)
            return dqr, dkr, dadt, dskip, dv, False
        if hasattr(ext(), "ssd_decay_grad"):
            tile = lambda t: None if t is None else _tile_rows(t, reps)  # noqa: E731
            out = ssd.siso_core_backward(tile(qr), tile(kr), tile(adt), tile(skip_total), tile(v), gy, ops=ssd.KernelScans,
                                         fwd_states=tile(states), keep_dkr_reversed=True)
            return (*_place_dv(out, dv_out), True)
    _fell_back("siso_scan_bwd", v, gy, qr, kr)
    return (*_place_dv(ssd.siso_core_backward_dense(qr, kr, adt, skip_total, v, gy), dv_out), False)


def _place_dv(out, dv_out):
    """(dQr, dKr, dadt, dskip, dV) with dV copied into ``dv_out`` when one is given."""
    if dv_out is None:
        return out
    dv_out.copy_(out[4].reshape(dv_out.shape))
    return (*out[:4], dv_out)


# ---------------------------------------------------------------- Mamba-2: softplus of dt, SiLU of the conv output
def softplus_dt_fwd(dt_raw, dt_bias, lo: float, hi: float):
    """-> (dt fp32 like dt_raw, d dt / d dt_raw fp32).  dt_raw may be a column range of a wider matrix (last stride 1)."""
    if _kernel_ok(dt_raw, dt_bias, name="softplus_dt") and dt_raw.dtype in (torch.bfloat16, torch.float32):
        flat = dt_raw if dt_raw.dim() == 2 else dt_raw.reshape(-1, dt_raw.shape[-1])
        if flat.stride(-1) == 1:
            _count()
            dt, slope = ext().softplus_dt(flat, dt_bias.float().contiguous(), float(lo), float(hi))
            return dt.view(dt_raw.shape), slope.view(dt_raw.shape)
    from .dispatch import fell_back

    fell_back("softplus_dt_fwd", dt_raw)
    pre = dt_raw.float() + dt_bias.float()
    dt = F.softplus(pre)
    slope = torch.sigmoid(pre)
    if (lo, hi) != (0.0, float("inf")):
        inside = (dt >= lo) & (dt <= hi)
        dt, slope = dt.clamp(lo, hi), slope * inside
    return dt, slope


def conv_silu_fwd(x, weight, bias, batch: int, seq_len: int, parts: tuple[int, int, int]):
    """Depthwise causal conv + SiLU over x [n, C]; weight [C, W] fp32 -> (pre-activation [n, C], the three parts of the
    activation as contiguous tensors [n, parts[i]])."""
    from . import reference as ref

    if (_kernel_ok(x, weight, bias, name="conv_silu_fwd") and x.dtype == torch.bfloat16 and all(p % 8 == 0 for p in parts)
            and weight.shape[1] <= 8):
        _count()
        pre, o0, o1, o2 = ext().conv_silu_fwd(x.contiguous(), weight.float().contiguous(), None if bias is None else bias.float().contiguous(),
                                              int(seq_len), *map(int, parts))
        return pre, (o0, o1, o2)
    from .dispatch import fell_back

    fell_back("conv_silu_fwd", x)
    pre = ref.causal_conv_fwd(x, weight, bias, batch, seq_len)
    act = F.silu(pre.float()).to(x.dtype)
    return pre, tuple(t.contiguous() for t in torch.split(act, list(parts), dim=-1))


def conv_silu_bwd(d_parts, pre, weight, batch: int, seq_len: int, out: torch.Tensor, col0: int) -> None:
    """Cotangents of the three activation parts ([P * n, parts[i]]) -> cotangent of the conv input, written into
    ``out[:, col0 : col0 + C]``; pre [n, C] is shared by the P directions."""
    from . import reference as ref

    channels = pre.shape[1]
    if (_kernel_ok(*d_parts, pre, out, name="conv_silu_bwd_") and pre.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
            and all(d.shape[1] % 8 == 0 for d in d_parts) and col0 % 8 == 0 and weight.shape[1] <= 8 and out.is_contiguous()):
        _count()
        d0 = d_parts[0].contiguous()
        d12 = torch.float32 if (d_parts[1].dtype == torch.float32 or d_parts[2].dtype == torch.float32) else torch.bfloat16
        ext().conv_silu_bwd_(d0 if d0.dtype in (torch.float32, torch.bfloat16) else d0.float(), d_parts[1].to(d12).contiguous(),
                             d_parts[2].to(d12).contiguous(), pre.contiguous(), weight.float().contiguous(), out, int(col0), int(seq_len))
        return
    from .dispatch import fell_back

    fell_back("conv_silu_bwd", pre)
    reps = d_parts[0].shape[0] // pre.shape[0]
    d_act = torch.cat([d.float() for d in d_parts], dim=-1)
    d_pre = silu_bwd(d_act, pre)
    out[:, col0 : col0 + channels] = ref.causal_conv_dgrad(d_pre, weight, reps * batch, seq_len).to(out.dtype)


def conv_silu_wgrad(d_parts, pre, x, width: int, batch: int, seq_len: int):
    """-> (dweight [C, W], dbias [C]) fp32 for one direction."""
    from . import reference as ref

    if (_kernel_ok(*d_parts, pre, x, name="conv_silu_wgrad") and pre.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
            and all(d.shape[1] % 8 == 0 for d in d_parts) and width <= 8):
        _count()
        d12 = torch.float32 if (d_parts[1].dtype == torch.float32 or d_parts[2].dtype == torch.float32) else torch.bfloat16
        d0 = d_parts[0].contiguous()
        return ext().conv_silu_wgrad(d0 if d0.dtype in (torch.float32, torch.bfloat16) else d0.float(), d_parts[1].to(d12).contiguous(),
                                     d_parts[2].to(d12).contiguous(), pre.contiguous(), x.contiguous(), int(width), int(seq_len))
    from .dispatch import fell_back

    fell_back("conv_silu_wgrad", pre)
    d_pre = silu_bwd(torch.cat([d.float() for d in d_parts], dim=-1), pre)
    return ref.causal_conv_wgrad(d_pre, x, width, batch, seq_len)


def silu_bwd(dy, x):
    """dy [P * n, c]; x [n, c] (the pre-activation)."""
    reps = dy.shape[0] // x.shape[0]
    xf = x.float()
    sig = torch.sigmoid(xf)
    slope = sig * (1.0 + xf * (1.0 - sig))
    return (dy.float().view(reps, *x.shape) * slope).reshape(dy.shape).to(dy.dtype)
