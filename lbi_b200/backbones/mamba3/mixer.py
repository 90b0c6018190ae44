"""Mamba-3 SISO mixer.

in_proj -> [z, x, B, C, dd_dt, dd_A, trap, angles]; A = -softplus(dd_A) clamped
below -A_floor; DT = softplus(dd_dt + dt_bias); RMSNorm on B and C; SISO scan with
Q = C, K = B, V = x; out_proj.  Parameter names and shapes follow the reference's
``backbones/mamba3/mamba3.py:96-143`` (``B_bias``/``C_bias`` keep their
``[nheads, 1, d_state]`` shape).  MIMO is not part of the reference either
(``mamba3.py:75-76`` raises).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from functools import partial

import torch
import torch.nn.functional as F
from torch import nn

from ...ops import ssd as ops_ssd
from ..norms import RMSNormGated
from .siso import mamba3_siso_chunked


@dataclass
class Mamba3ForwardCache:
    input_u: torch.Tensor
    in_proj: torch.Tensor
    z: torch.Tensor
    x: torch.Tensor
    B: torch.Tensor
    C: torch.Tensor
    dd_dt: torch.Tensor
    dd_A: torch.Tensor
    trap: torch.Tensor
    angles: torch.Tensor
    ADT: torch.Tensor
    DT: torch.Tensor
    B_normed: torch.Tensor
    C_normed: torch.Tensor
    y_inner: torch.Tensor
    output: torch.Tensor


class Mamba3(nn.Module):
    def __init__(
        self,
        d_model: int,
        d_state: int = 128,
        expand: int = 2,
        headdim: int = 64,
        ngroups: int = 1,
        rope_fraction: float = 0.5,
        dt_min: float = 0.001,
        dt_max: float = 0.1,
        dt_init_floor: float = 1e-4,
        A_floor: float = 1e-4,
        is_outproj_norm: bool = False,
        is_mimo: bool = False,
        chunk_size: int = 64,
        layer_idx=None,
        device=None,
        dtype=None,
        **_unused,
    ) -> None:
        super().__init__()
        if is_mimo:
            raise NotImplementedError("Mamba-3 MIMO is not supported; use the SISO form.")
        fk = {"device": device, "dtype": dtype}
        self.d_model, self.d_state, self.expand, self.headdim = d_model, d_state, expand, headdim
        self.chunk_size, self.layer_idx, self.A_floor = chunk_size, layer_idx, A_floor
        self.is_outproj_norm = is_outproj_norm
        self.mimo_rank = 1
        self.d_inner = int(expand * d_model)
        if self.d_inner % headdim != 0:
            raise ValueError("expand * d_model must be divisible by headdim")
        self.nheads = self.d_inner // headdim
        self.num_bc_heads = ngroups
        if rope_fraction not in (0.5, 1.0):
            raise ValueError("rope_fraction must be 0.5 or 1.0")
        self.rotary_dim_divisor = int(2 / rope_fraction)
        rotary_width = int(d_state * rope_fraction)
        rotary_width -= rotary_width % 2
        self.split_tensor_size = rotary_width
        self.num_rope_angles = rotary_width // 2
        if self.num_rope_angles <= 0:
            raise ValueError("d_state too small for rotary angles")

        d_in_proj = 2 * self.d_inner + 2 * d_state * ngroups + 3 * self.nheads + self.num_rope_angles
        self.in_proj = nn.Linear(d_model, d_in_proj, bias=False, **fk)
        dt = torch.exp(
            torch.rand(self.nheads, device=device, dtype=torch.float32) * (math.log(dt_max) - math.log(dt_min))
            + math.log(dt_min)
        ).clamp(min=dt_init_floor)
        self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))
        self.dt_bias._no_weight_decay = True
        self.B_bias = nn.Parameter(torch.ones(self.nheads, 1, d_state, dtype=torch.float32, device=device))
        self.C_bias = nn.Parameter(torch.ones(self.nheads, 1, d_state, dtype=torch.float32, device=device))
        self.B_norm = RMSNormGated(d_state, eps=1e-5, **fk)
        self.C_norm = RMSNormGated(d_state, eps=1e-5, **fk)
        self.D = nn.Parameter(torch.ones(self.nheads, device=device))
        self.D._no_weight_decay = True
        if is_outproj_norm:
            self.norm = RMSNormGated(self.d_inner, eps=1e-5, norm_before_gate=True, group_size=headdim, **fk)
        self.out_proj = nn.Linear(self.d_inner, d_model, bias=False, **fk)

    def _forward_impl(self, u: torch.Tensor, *, return_cache: bool = False):
        bsz, seqlen, _ = u.shape
        proj = self.in_proj(u)
        gn = self.d_state * self.num_bc_heads
        z, x, B, C, dd_dt, dd_A, trap, angles = torch.split(
            proj, [self.d_inner, self.d_inner, gn, gn, self.nheads, self.nheads, self.nheads, self.num_rope_angles], dim=-1
        )
        z = z.reshape(bsz, seqlen, self.nheads, self.headdim)
        x = x.reshape(bsz, seqlen, self.nheads, self.headdim)
        B = self.B_norm(B.reshape(bsz, seqlen, self.num_bc_heads, self.d_state))
        C = self.C_norm(C.reshape(bsz, seqlen, self.num_bc_heads, self.d_state))
        A = torch.clamp(-F.softplus(dd_A.float()), max=-self.A_floor)
        DT = F.softplus(dd_dt.float() + self.dt_bias.float())
        ADT = (A * DT).transpose(1, 2)
        DT = DT.transpose(1, 2)
        trap_t = trap.transpose(1, 2)
        angles_h = angles.unsqueeze(-2).expand(-1, -1, self.nheads, -1)
        use_kernels = ops_ssd.siso_cuda_supported(x, C) and x.dtype == torch.bfloat16 and self.D is not None
        siso = ops_ssd.mamba3_siso_cuda if use_kernels else partial(mamba3_siso_chunked, chunk_size=self.chunk_size)
        y = siso(
            Q=C,
            K=B,
            V=x,
            ADT=ADT,
            DT=DT,
            Trap=trap_t,
            Q_bias=self.C_bias.squeeze(1),
            K_bias=self.B_bias.squeeze(1),
            Angles=angles.unsqueeze(-2),   # [b, l, 1, s]: the same angles for every head, broadcast against dt
            D=self.D,
            Z=None if self.is_outproj_norm else z,
        )
        y = y.reshape(bsz, seqlen, self.d_inner)
        if self.is_outproj_norm:
            y = self.norm(y, z.reshape(bsz, seqlen, self.d_inner))
        out = self.out_proj(y.to(self.out_proj.weight.dtype))
        if not return_cache:
            return out
        return out, Mamba3ForwardCache(
            input_u=u, in_proj=proj, z=z, x=x, B=B, C=C, dd_dt=dd_dt, dd_A=dd_A, trap=trap_t, angles=angles_h,
            ADT=ADT, DT=DT, B_normed=B, C_normed=C, y_inner=y, output=out,
        )

    def forward(self, u: torch.Tensor, seq_idx=None, cu_seqlens=None, inference_params=None) -> torch.Tensor:
        if cu_seqlens is not None or inference_params is not None:
            raise NotImplementedError("only the full-sequence training path is implemented")
        return self._forward_impl(u)

    def forward_with_cache(self, u: torch.Tensor):
        return self._forward_impl(u, return_cache=True)

    def input_pullback_matrix(self, u: torch.Tensor, output_cotangent_basis: torch.Tensor) -> torch.Tensor:
        """Pull a basis of output cotangents [B, P, L, D] back to the mixer input -> [B, P, L, D]."""
        bsz, nbasis = output_cotangent_basis.shape[:2]
        rep = u.detach().repeat_interleave(nbasis, dim=0).requires_grad_(True)
        with torch.enable_grad():
            out = self._forward_impl(rep)
        (g,) = torch.autograd.grad(out, rep, output_cotangent_basis.reshape(bsz * nbasis, *u.shape[1:]).to(out.dtype))
        return g.reshape(bsz, nbasis, *u.shape[1:])
