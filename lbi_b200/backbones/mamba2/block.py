"""Add -> RMSNorm -> Mamba-2 mixer block (reference backbones/mamba2/block.py:14-64)."""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from ..norms import RMSNorm
from .mixer import Mamba2Simple


class Mamba2Block(nn.Module):
    """Add -> RMSNorm -> Mamba-2 mixer on the (branch, stream) residual contract of the stacks."""

    def __init__(
        self,
        dim: int,
        *,
        d_state: int = 64,
        d_conv: int = 4,
        expand: int = 2,
        headdim: int = 128,
        ngroups: int = 1,
        chunk_size: int = 256,
        use_mem_eff_path: bool = True,
        bias: bool = False,
        conv_bias: bool = True,
        device=None,
        dtype=None,
    ) -> None:
        super().__init__()
        self.norm = RMSNorm(dim, eps=1e-5, device=device, dtype=dtype)
        self.mixer = Mamba2Simple(
            d_model=dim,
            d_state=d_state,
            d_conv=d_conv,
            expand=expand,
            headdim=headdim,
            ngroups=ngroups,
            chunk_size=chunk_size,
            use_mem_eff_path=use_mem_eff_path,
            bias=bias,
            conv_bias=conv_bias,
            device=device,
            dtype=dtype,
        )

    def forward(self, hidden_states: torch.Tensor, residual: Optional[torch.Tensor] = None, seq_idx=None):
        residual = hidden_states if residual is None else hidden_states + residual
        hidden_states = self.mixer(self.norm(residual.to(dtype=self.norm.weight.dtype)), seq_idx=seq_idx)
        return hidden_states, residual

    def allocate_decode_state(self, batch_size: int, max_len: int, device=None, dtype=None):
        return self.mixer.allocate_inference_cache(batch_size, max_len, device=device, dtype=dtype)

    @torch.no_grad()
    def decode_step(self, hidden_states: torch.Tensor, residual: Optional[torch.Tensor], state):
        """One token: (branch [B, D], stream [B, D] or None) -> (branch, stream), the same contract as ``forward``."""
        residual = hidden_states if residual is None else hidden_states + residual
        return self.mixer.step(self.norm(residual.to(dtype=self.norm.weight.dtype)), *state), residual
