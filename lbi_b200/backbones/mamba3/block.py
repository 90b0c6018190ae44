"""Add -> RMSNorm -> Mamba-3 mixer block (reference backbones/mamba3/block.py:23-123)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
from torch import nn

from ..norms import RMSNorm
from .mixer import Mamba3, Mamba3ForwardCache


@dataclass
class Mamba3BlockCache:
    residual_out: torch.Tensor
    normed: torch.Tensor
    mixer: Mamba3ForwardCache


Mamba3BlockForwardCache = Mamba3BlockCache  # the reference's name for the same record (backbones/mamba3/block.py)


class Mamba3Block(nn.Module):
    def __init__(
        self,
        dim: int,
        *,
        d_state: int = 128,
        expand: int = 2,
        headdim: int = 64,
        ngroups: int = 1,
        chunk_size: int = 64,
        device=None,
        dtype=None,
    ) -> None:
        super().__init__()
        self.norm = RMSNorm(dim, eps=1e-5, device=device, dtype=dtype)
        self.mixer = Mamba3(
            d_model=dim, d_state=d_state, expand=expand, headdim=headdim, ngroups=ngroups, chunk_size=chunk_size,
            device=device, dtype=dtype,
        )

    def forward(self, hidden_states: torch.Tensor, residual: Optional[torch.Tensor] = None, seq_idx=None):
        residual = hidden_states if residual is None else hidden_states + residual
        hidden_states = self.mixer(self.norm(residual.to(dtype=self.norm.weight.dtype)))
        return hidden_states, residual

    def forward_with_cache(self, hidden_states: torch.Tensor, residual: Optional[torch.Tensor] = None):
        residual = hidden_states if residual is None else hidden_states + residual
        normed = self.norm(residual.to(dtype=self.norm.weight.dtype))
        out, mixer_cache = self.mixer.forward_with_cache(normed)
        return out, residual, Mamba3BlockCache(residual_out=residual, normed=normed, mixer=mixer_cache)

    def input_pullback_matrix(self, hidden_states: torch.Tensor, output_cotangent_basis: torch.Tensor) -> torch.Tensor:
        """Pullback of a basis [B, P, L, D] through ``x -> mixer(norm(x)) + x`` (first block of a range)."""
        bsz, nbasis = output_cotangent_basis.shape[:2]
        rep = hidden_states.detach().repeat_interleave(nbasis, dim=0).requires_grad_(True)
        with torch.enable_grad():
            branch, stream = self.forward(rep, None)
            out = branch + stream
        (g,) = torch.autograd.grad(out, rep, output_cotangent_basis.reshape(bsz * nbasis, *hidden_states.shape[1:]).to(out.dtype))
        return g.reshape(bsz, nbasis, *hidden_states.shape[1:])
