"""Pre-norm Transformer block with an fp32 residual stream.

``forward(branch, residual) -> (branch, residual)``: the block adds the incoming
branch to the stream, normalises, runs attention, adds, normalises, runs the MLP
and hands back the MLP branch plus the stream (reference
``backbones/transformer/block.py:25-87``).
"""
from __future__ import annotations

import torch
from torch import nn

from ..norms import RMSNorm
from .attention import CausalSelfAttention
from .mlp import GatedMLP


class TransformerBlock(nn.Module):
    """Pre-norm block on an fp32 residual stream: add -> RMSNorm -> attention, add -> RMSNorm -> SwiGLU MLP."""

    def __init__(
        self,
        dim: int,
        *,
        n_heads: int,
        n_kv_heads: int,
        head_dim: int,
        d_intermediate: int = 0,
        mlp_ratio: float = 4.0,
        rope_base: float = 10000.0,
        rope_interleaved: bool = False,
        softmax_scale: float | None = None,
        d_conv: int = 0,
        use_flash_attn: bool = True,
        residual_in_fp32: bool = True,
        fused_add_norm: bool = True,
        bias: bool = False,
    ) -> None:
        super().__init__()
        self.residual_in_fp32 = residual_in_fp32
        self.fused_add_norm = fused_add_norm
        self.norm = RMSNorm(dim, eps=1e-5)
        self.attn = CausalSelfAttention(
            dim,
            n_heads=n_heads,
            n_kv_heads=n_kv_heads,
            head_dim=head_dim,
            rope_base=rope_base,
            rope_interleaved=rope_interleaved,
            softmax_scale=softmax_scale,
            d_conv=d_conv,
            use_flash_attn=use_flash_attn,
            bias=bias,
        )
        self.norm2 = RMSNorm(dim, eps=1e-5)
        hidden = d_intermediate if d_intermediate > 0 else (max(1, int(dim * mlp_ratio)) if mlp_ratio > 0.0 else None)
        self.mlp = GatedMLP(dim, hidden_features=hidden, out_features=dim, bias=bias)

    def add_norm(self, branch: torch.Tensor, stream: torch.Tensor | None, norm: RMSNorm):
        stream = branch if stream is None else branch + stream
        normed = norm(stream.to(dtype=norm.weight.dtype))
        if self.residual_in_fp32:
            stream = stream.to(torch.float32)
        return normed, stream

    _prenorm = add_norm  # the reference's name for the same step (backbones/transformer/block.py:66-76)

    def forward(self, hidden_states: torch.Tensor, residual: torch.Tensor | None = None):
        hidden_states, residual = self.add_norm(hidden_states, residual, self.norm)
        hidden_states = self.attn(hidden_states)
        hidden_states, residual = self.add_norm(hidden_states, residual, self.norm2)
        hidden_states = self.mlp(hidden_states)
        return hidden_states, residual

    def allocate_decode_state(self, batch_size: int, max_len: int, device=None, dtype=None) -> dict:
        return self.attn.allocate_decode_state(batch_size, max_len, device=device, dtype=dtype)

    @torch.no_grad()
    def decode_step(self, hidden_states: torch.Tensor, residual: torch.Tensor | None, state: dict):
        """One token: (branch [B, D], stream [B, D] or None) -> (branch, stream), the same contract as ``forward``."""
        normed, residual = self.add_norm(hidden_states, residual, self.norm)
        branch = self.attn.step(normed, state)
        normed, residual = self.add_norm(branch, residual, self.norm2)
        return self.mlp(normed), residual
