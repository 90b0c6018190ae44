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
from .siso import _rotate_pairs, mamba3_siso_chunked, mamba3_siso_combined


@dataclass
class Mamba3ForwardCache:
    """Intermediates of one mixer forward under the reference's field names."""

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
    """The Mamba-3 SISO mixer (see the module docstring); ``forward_with_cache`` keeps the intermediates, ``step`` / ``prefill`` decode."""

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

    def _forward_impl(self, u: torch.Tensor, *, return_cache: bool = False, decode_states=None, cu_seqlens=None):
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
        use_kernels = (decode_states is None and cu_seqlens is None and ops_ssd.siso_cuda_supported(x, C)
                       and x.dtype == torch.bfloat16 and self.D is not None)
        if cu_seqlens is not None:  # one packed row of several sequences: the scan runs per sequence, the rest is per token
            siso = partial(mamba3_siso_combined, chunk_size=self.chunk_size, cu_seqlens=cu_seqlens)
        elif decode_states is not None:
            angle_state, ssm_state, k_state, v_state = decode_states
            siso = partial(mamba3_siso_chunked, chunk_size=self.chunk_size, return_final_states=True,
                           initial_states=(angle_state, ssm_state, k_state[:, 0], v_state))
        else:
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
        if decode_states is not None:
            y, angle_last, ssm_last, k_last, v_last = y
            angle_state.copy_(angle_last)
            ssm_state.copy_(ssm_last)
            k_state.copy_(k_last.unsqueeze(1).to(k_state.dtype))
            v_state.copy_(v_last.to(v_state.dtype))
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
        """u [B, L, D] -> [B, L, D].  ``cu_seqlens`` [num_sequences + 1] marks the sequences laid end to end in a single row
        (B = 1); each starts from a zero state and a zero rotary phase.  ``seq_idx`` is accepted and unused, as in the reference."""
        self._full_sequence_only(inference_params)
        return self._forward_impl(u, cu_seqlens=cu_seqlens)

    def forward_with_cache(self, u: torch.Tensor, seq_idx=None, cu_seqlens=None, inference_params=None):
        self._full_sequence_only(inference_params)
        return self._forward_impl(u, return_cache=True, cu_seqlens=cu_seqlens)

    @staticmethod
    def _full_sequence_only(inference_params) -> None:
        if inference_params is not None:
            raise NotImplementedError("decode with allocate_inference_cache() and step(); forward() is the full-sequence path")

    def input_pullback_matrix(self, first=None, output_cotangent_basis: torch.Tensor | None = None, *, cache=None, g_out=None,
                              u=None) -> torch.Tensor:
        """Pull a basis of output cotangents [B, P, L, D] back to the mixer input -> [B, P, L, D].

        ``first`` is the mixer input ``u`` or, as in the reference (backbones/mamba3/mamba3.py:306-325), the
        ``Mamba3ForwardCache`` of a ``forward_with_cache`` call, whose ``input_u`` is then used.  All directions go through
        one recomputed forward on a replicated batch instead of one backward pass per direction over a retained graph."""
        first = next((a for a in (first, cache, u) if a is not None), None)
        output_cotangent_basis = g_out if output_cotangent_basis is None else output_cotangent_basis
        if first is None or output_cotangent_basis is None:
            raise TypeError("input_pullback_matrix needs a mixer input or cache and a cotangent basis")
        u = first.input_u if isinstance(first, Mamba3ForwardCache) else first
        if output_cotangent_basis.dim() != 4:
            raise ValueError("the cotangent basis must have shape [B, P, L, D].")
        bsz, nbasis = output_cotangent_basis.shape[:2]
        if tuple(output_cotangent_basis.shape[2:]) != tuple(u.shape[1:]) or output_cotangent_basis.shape[0] != u.shape[0]:
            raise ValueError("the cotangent basis does not match the mixer output shape.")
        rep = u.detach().repeat_interleave(nbasis, dim=0).requires_grad_(True)
        with torch.enable_grad():
            out = self._forward_impl(rep)
        (g,) = torch.autograd.grad(out, rep, output_cotangent_basis.reshape(bsz * nbasis, *u.shape[1:]).to(out.dtype))
        return g.reshape(bsz, nbasis, *u.shape[1:]).to(output_cotangent_basis.dtype)

    # ------------------------------------------------------------------ token-by-token decode
    def allocate_inference_cache(self, batch_size, max_seqlen=None, device=None, dtype=None, inplace_state=None, **_unused):
        """Zeroed decode state ``(angle_state, ssm_state, k_state, v_state)`` with the reference's shapes
        (backbones/mamba3/mamba3.py:363-403): cumulative rotary phase [B, H, S] fp32, SSM state [B, H, P, N] fp32, the previous
        token's rotated key [B, 1, H, N] and value [B, H, P]."""
        device = self.in_proj.weight.device if device is None else device
        dtype = self.in_proj.weight.dtype if dtype is None else dtype
        angle_state = torch.zeros(batch_size, self.nheads, self.num_rope_angles, device=device, dtype=torch.float32)
        ssm_state = torch.zeros(batch_size, self.nheads, self.headdim, self.d_state, device=device, dtype=torch.float32)
        k_state = torch.zeros(batch_size, 1, self.nheads, self.d_state, device=device, dtype=dtype)
        v_state = torch.zeros(batch_size, self.nheads, self.headdim, device=device, dtype=dtype)
        return angle_state, ssm_state, k_state, v_state

    @torch.no_grad()
    def prefill(self, u: torch.Tensor, angle_state, ssm_state, k_state, v_state) -> torch.Tensor:
        """A whole prompt (or the next piece of one) u [B, L, D] in one chunked pass that starts from the four decode-state
        tensors and leaves them at the last token, ready for ``step`` or another ``prefill``."""
        return self._forward_impl(u, decode_states=(angle_state, ssm_state, k_state, v_state))

    @torch.no_grad()
    def step(self, u: torch.Tensor, angle_state, ssm_state, k_state, v_state, **_unused):
        """One token of the recurrence: u [B, D] (or [B, 1, D]) -> output of the same shape; the four state tensors are
        updated in place.  Feeding a sequence token by token from a zeroed cache reproduces ``forward`` (the reference declares
        this method and leaves it unimplemented, backbones/mamba3/mamba3.py:360-361).

        The trapezoid rule gives token t a second weight dt_{t+1} (1 - sigmoid(trap_{t+1})) that is only known one token later,
        so ``ssm_state`` holds the state without that share of the newest token and ``k_state`` / ``v_state`` keep its rotated key
        and value; the share is added at the start of the next step, before the decay."""
        squeeze = u.dim() == 3
        if squeeze:
            if u.shape[1] != 1:
                raise ValueError("step() takes one token per sequence")
            u = u[:, 0]
        bsz = u.shape[0]
        gn = self.d_state * self.num_bc_heads
        proj = self.in_proj(u)
        z, x, B, C, dd_dt, dd_A, trap, angles = torch.split(
            proj, [self.d_inner, self.d_inner, gn, gn, self.nheads, self.nheads, self.nheads, self.num_rope_angles], dim=-1
        )
        z = z.reshape(bsz, self.nheads, self.headdim)
        x = x.reshape(bsz, self.nheads, self.headdim)
        B = self.B_norm(B.reshape(bsz, self.num_bc_heads, self.d_state)).float()
        C = self.C_norm(C.reshape(bsz, self.num_bc_heads, self.d_state)).float()
        rep = self.nheads // self.num_bc_heads
        A = torch.clamp(-F.softplus(dd_A.float()), max=-self.A_floor)
        dt = F.softplus(dd_dt.float() + self.dt_bias.float())  # [B, H]
        sig = torch.sigmoid(trap.float())
        theta = angle_state + math.pi * torch.tanh(angles.float()).unsqueeze(1) * dt.unsqueeze(-1)
        theta = theta - (2.0 * math.pi) * torch.floor(theta / (2.0 * math.pi))
        angle_state.copy_(theta)
        q = C.repeat_interleave(rep, dim=1) + self.C_bias.float().squeeze(1)[None]
        k = B.repeat_interleave(rep, dim=1) + self.B_bias.float().squeeze(1)[None]
        qr, kr = _rotate_pairs(q, theta), _rotate_pairs(k, theta)
        xf = x.float()
        carry = (dt * (1.0 - sig))[..., None, None] * v_state.float()[..., None] * k_state.float()[:, 0, :, None, :]
        h = (ssm_state + carry) * torch.exp(A * dt)[..., None, None]
        gamma = dt * sig
        skip = gamma * (q * k).sum(dim=-1) + (self.D.float()[None] if self.D is not None else 0.0)
        y = torch.einsum("bhpn,bhn->bhp", h, qr) + skip[..., None] * xf
        ssm_state.copy_(h + gamma[..., None, None] * xf[..., None] * kr[:, :, None, :])
        k_state.copy_(kr.unsqueeze(1).to(k_state.dtype))
        v_state.copy_(x.to(v_state.dtype))
        if self.is_outproj_norm:
            y = self.norm(y.reshape(bsz, self.d_inner).to(x.dtype), z.reshape(bsz, self.d_inner))
        else:
            y = (y * F.silu(z.float())).reshape(bsz, self.d_inner)
        out = self.out_proj(y.to(self.out_proj.weight.dtype))
        return out.unsqueeze(1) if squeeze else out
