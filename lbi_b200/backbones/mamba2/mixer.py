"""Mamba-2 mixer (in_proj -> causal depthwise conv + SiLU -> SSD -> gated RMSNorm -> out_proj).

Parameter names, shapes and initialisation ranges follow the reference's
``backbones/mamba2/mamba2_simple.py:24-122`` so its checkpoints load unchanged.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from ...ops import ssd as ops_ssd
from ..norms import RMSNormGated
from .ssd import ssd_chunk_scan


class Mamba2Simple(nn.Module):
    """The Mamba-2 mixer: in_proj -> [z | x B C | dt], causal depthwise conv + SiLU on x B C, SSD scan, gated RMSNorm, out_proj."""

    def __init__(
        self,
        d_model: int,
        d_state: int = 64,
        d_conv: int = 4,
        conv_init: float | None = None,
        expand: int = 2,
        headdim: int = 128,
        ngroups: int = 1,
        A_init_range=(1, 16),
        dt_min: float = 0.001,
        dt_max: float = 0.1,
        dt_init_floor: float = 1e-4,
        dt_limit=(0.0, float("inf")),
        learnable_init_states: bool = False,
        activation: str = "swish",
        bias: bool = False,
        conv_bias: bool = True,
        chunk_size: int = 256,
        use_mem_eff_path: bool = True,
        layer_idx=None,
        device=None,
        dtype=None,
    ) -> None:
        super().__init__()
        fk = {"device": device, "dtype": dtype}
        self.d_model, self.d_state, self.d_conv, self.expand = d_model, d_state, d_conv, expand
        self.d_inner = expand * d_model
        self.headdim, self.ngroups = headdim, ngroups
        if self.d_inner % headdim != 0:
            raise ValueError("expand * d_model must be divisible by headdim")
        self.nheads = self.d_inner // headdim
        self.dt_limit = dt_limit
        if activation not in ("silu", "swish"):
            raise ValueError("the Mamba-2 mixer supports the silu / swish activation only")
        self.conv_init, self.learnable_init_states, self.activation = conv_init, learnable_init_states, activation
        self.chunk_size = chunk_size
        self.use_mem_eff_path = use_mem_eff_path
        self.layer_idx = layer_idx

        # in_proj output order: [z, x, B, C, dt]
        self.in_proj = nn.Linear(d_model, 2 * self.d_inner + 2 * ngroups * d_state + self.nheads, bias=bias, **fk)
        conv_dim = self.d_inner + 2 * ngroups * d_state
        self.conv1d = nn.Conv1d(conv_dim, conv_dim, kernel_size=d_conv, groups=conv_dim, padding=d_conv - 1, bias=conv_bias, **fk)
        if conv_init is not None:
            nn.init.uniform_(self.conv1d.weight, -conv_init, conv_init)
        if learnable_init_states:
            self.init_states = nn.Parameter(torch.zeros(self.nheads, headdim, d_state, **fk))
            self.init_states._no_weight_decay = True

        dt = torch.exp(torch.rand(self.nheads, **fk) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min))
        dt = torch.clamp(dt, min=dt_init_floor)
        self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))  # inverse softplus
        self.dt_bias._no_weight_decay = True
        A = torch.empty(self.nheads, dtype=torch.float32, device=device).uniform_(*A_init_range)
        self.A_log = nn.Parameter(torch.log(A).to(dtype=dtype))
        self.A_log._no_weight_decay = True
        self.D = nn.Parameter(torch.ones(self.nheads, device=device))
        self.D._no_weight_decay = True
        self.norm = RMSNormGated(self.d_inner, eps=1e-5, norm_before_gate=False, **fk)
        self.out_proj = nn.Linear(self.d_inner, d_model, bias=bias, **fk)

    def forward(self, u: torch.Tensor, seq_idx=None) -> torch.Tensor:
        """u [B, L, D] -> [B, L, D].  ``seq_idx`` [B, L] (non-decreasing ids of the sequences packed into each row, as in the
        reference's kernels: mamba2_simple.py:124-147) makes the convolution window and the state start afresh wherever the id
        changes; the learnable initial state, when there is one, belongs to the first sequence of each row."""
        if seq_idx is not None:
            return self._forward_packed(u, seq_idx)
        return self._forward_tokens(u, first_segment=True)

    def _forward_packed(self, u: torch.Tensor, seq_idx: torch.Tensor) -> torch.Tensor:
        if seq_idx.shape != u.shape[:2]:
            raise ValueError("seq_idx must have shape [B, L]")
        rows = []
        for b in range(u.shape[0]):
            cuts = (torch.nonzero(seq_idx[b, 1:] != seq_idx[b, :-1]).flatten() + 1).tolist()
            edges = [0, *cuts, u.shape[1]]
            rows.append(torch.cat([self._forward_tokens(u[b : b + 1, s:e], first_segment=(s == 0))
                                   for s, e in zip(edges[:-1], edges[1:])], dim=1))
        return torch.cat(rows, dim=0)

    def _forward_tokens(self, u: torch.Tensor, *, first_segment: bool) -> torch.Tensor:
        bsz, seqlen, _ = u.shape
        init = None
        if self.learnable_init_states and first_segment:
            init = self.init_states.unsqueeze(0).expand(bsz, -1, -1, -1)
        zxbcdt = self.in_proj(u)
        gn = self.ngroups * self.d_state
        z, xBC, dt = torch.split(zxbcdt, [self.d_inner, self.d_inner + 2 * gn, self.nheads], dim=-1)
        dt = F.softplus(dt.float() + self.dt_bias.float())
        if self.dt_limit != (0.0, float("inf")):
            dt = dt.clamp(self.dt_limit[0], self.dt_limit[1])
        xBC = F.silu(self.conv1d(xBC.transpose(1, 2))[..., :seqlen].transpose(1, 2))
        x, B, C = torch.split(xBC, [self.d_inner, gn, gn], dim=-1)
        x4 = x.reshape(bsz, seqlen, self.nheads, self.headdim)
        B4 = B.reshape(bsz, seqlen, self.ngroups, self.d_state)
        C4 = C.reshape(bsz, seqlen, self.ngroups, self.d_state)
        A = -torch.exp(self.A_log.float())
        if ops_ssd.ssd_cuda_supported(x4, B4) and x4.dtype == torch.bfloat16:
            # sm_100a kernels (chunk 128 inside); the chunk size does not change the result, only the blocking
            y = ops_ssd.ssd_chunk_scan_cuda(x4, dt, A, B4, C4, D=self.D, initial_state=init)
        else:
            y = ssd_chunk_scan(x4, dt, A, B4, C4, chunk_size=self.chunk_size, D=self.D, initial_state=init)
        y = self.norm(y.reshape(bsz, seqlen, self.d_inner), z)
        return self.out_proj(y.to(self.out_proj.weight.dtype))

    # ------------------------------------------------------------------ token-by-token decoding
    def allocate_inference_cache(self, batch_size: int, max_seqlen=None, device=None, dtype=None, **_unused):
        """(conv_state [B, conv_dim, d_conv - 1], ssm_state [B, H, P, N] fp32): the last pre-convolution rows and the scan state,
        which starts from the learnable initial state when the mixer has one."""
        device = self.in_proj.weight.device if device is None else device
        dtype = self.in_proj.weight.dtype if dtype is None else dtype
        conv_dim = self.d_inner + 2 * self.ngroups * self.d_state
        conv_state = torch.zeros(batch_size, conv_dim, self.d_conv - 1, device=device, dtype=dtype)
        ssm_state = torch.zeros(batch_size, self.nheads, self.headdim, self.d_state, device=device, dtype=torch.float32)
        if self.learnable_init_states:
            ssm_state += self.init_states.detach().float().unsqueeze(0)
        return conv_state, ssm_state

    @torch.no_grad()
    def step(self, u: torch.Tensor, conv_state: torch.Tensor, ssm_state: torch.Tensor) -> torch.Tensor:
        """One token u [B, D] -> [B, D]; both state tensors are updated in place.  Token-by-token evaluation from a fresh cache
        reproduces ``forward``."""
        bsz = u.shape[0]
        gn = self.ngroups * self.d_state
        z, xBC, dt = torch.split(self.in_proj(u), [self.d_inner, self.d_inner + 2 * gn, self.nheads], dim=-1)
        window = torch.cat([conv_state, xBC.unsqueeze(-1).to(conv_state.dtype)], dim=-1)  # oldest ... newest
        conv_state.copy_(window[..., 1:])
        xBC = (window * self.conv1d.weight[:, 0].to(window.dtype)).sum(dim=-1)
        if self.conv1d.bias is not None:
            xBC = xBC + self.conv1d.bias
        x, B, C = torch.split(F.silu(xBC), [self.d_inner, gn, gn], dim=-1)
        dt = F.softplus(dt.float() + self.dt_bias.float())
        if self.dt_limit != (0.0, float("inf")):
            dt = dt.clamp(self.dt_limit[0], self.dt_limit[1])
        rep = self.nheads // self.ngroups
        xh = x.float().reshape(bsz, self.nheads, self.headdim)
        Bh = B.float().reshape(bsz, self.ngroups, self.d_state).repeat_interleave(rep, dim=1)
        Ch = C.float().reshape(bsz, self.ngroups, self.d_state).repeat_interleave(rep, dim=1)
        decay = torch.exp(dt * (-torch.exp(self.A_log.float())))
        ssm_state.copy_(ssm_state * decay[..., None, None] + (dt[..., None] * xh)[..., None] * Bh[:, :, None, :])
        y = torch.einsum("bhpn,bhn->bhp", ssm_state, Ch) + self.D.float()[None, :, None] * xh
        y = self.norm(y.reshape(bsz, self.d_inner).to(x.dtype), z)
        return self.out_proj(y.to(self.out_proj.weight.dtype))
