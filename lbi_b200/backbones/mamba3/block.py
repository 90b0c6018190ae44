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
    """One block forward: the outgoing stream, the normed mixer input, the mixer cache and the block's inputs / output."""

    residual_out: torch.Tensor
    normed: torch.Tensor
    mixer: Mamba3ForwardCache
    hidden_input: Optional[torch.Tensor] = None
    residual_input: Optional[torch.Tensor] = None
    hidden_output: Optional[torch.Tensor] = None

    # the reference's field names for the first three (backbones/mamba3/block.py:12-19)
    @property
    def residual_output(self) -> torch.Tensor:
        return self.residual_out

    @property
    def norm_input(self) -> torch.Tensor:
        return self.normed

    @property
    def mixer_cache(self) -> Mamba3ForwardCache:
        return self.mixer


Mamba3BlockForwardCache = Mamba3BlockCache  # the reference's name for the same record


class Mamba3Block(nn.Module):
    """Add -> RMSNorm -> Mamba-3 mixer on the (branch, stream) residual contract of the stacks."""

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

    def forward(self, hidden_states: torch.Tensor, residual: Optional[torch.Tensor] = None, seq_idx=None, **kwargs):
        residual = hidden_states if residual is None else hidden_states + residual
        hidden_states = self.mixer(self.norm(residual.to(dtype=self.norm.weight.dtype)), seq_idx=seq_idx, **kwargs)
        return hidden_states, residual

    def forward_with_cache(self, hidden_states: torch.Tensor, residual: Optional[torch.Tensor] = None, **kwargs):
        residual_out = hidden_states if residual is None else hidden_states + residual
        normed = self.norm(residual_out.to(dtype=self.norm.weight.dtype))
        out, mixer_cache = self.mixer.forward_with_cache(normed, **kwargs)
        return out, residual_out, Mamba3BlockCache(residual_out=residual_out, normed=normed, mixer=mixer_cache,
                                                   hidden_input=hidden_states, residual_input=residual, hidden_output=out)

    @staticmethod
    def _module_input_pullback_matrix_autograd(module: nn.Module, x: torch.Tensor, g_out: torch.Tensor) -> torch.Tensor:
        """J^T of a module on [B, L, D] inputs for a basis g_out [B, P, L, D]: one backward pass over a replicated batch
        (reference backbones/mamba3/block.py:50-78)."""
        if x.dim() != 3 or g_out.dim() != 4:
            raise ValueError("block pullback expects x [B, L, D] and g_out [B, P, L, D].")
        bsz, nbasis = g_out.shape[:2]
        rep = x.detach().repeat_interleave(nbasis, dim=0).requires_grad_(True)
        with torch.enable_grad():
            y = module(rep)
        (g,) = torch.autograd.grad(y, rep, g_out.to(device=y.device, dtype=y.dtype).reshape_as(y))
        return g.reshape(bsz, nbasis, *x.shape[1:]).to(device=g_out.device, dtype=g_out.dtype)

    def input_pullback_matrix(self, first=None, output_cotangent_basis: Optional[torch.Tensor] = None,
                              g_residual_out: Optional[torch.Tensor] = None, *, cache=None, g_hidden_out=None, hidden_states=None):
        """Two call forms.

        ``(hidden_states [B, L, D], basis [B, P, L, D]) -> [B, P, L, D]``: the pullback through
        ``x -> mixer(norm(x)) + x`` (a block that opens a range, output = branch + stream).

        ``(cache, g_hidden_out, g_residual_out=None) -> (g_hidden_in, g_residual_in)``: the reference's form
        (backbones/mamba3/block.py:104-123) on a ``forward_with_cache`` record: the cotangent of the branch output goes
        through the mixer and the norm, the cotangent of the outgoing stream is added, and both inputs (branch and
        incoming stream, which are summed on entry) receive the total; ``g_residual_in`` is None for a block that had no
        incoming stream."""
        first = next((a for a in (first, cache, hidden_states) if a is not None), None)
        output_cotangent_basis = g_hidden_out if output_cotangent_basis is None else output_cotangent_basis
        if first is None or output_cotangent_basis is None:
            raise TypeError("input_pullback_matrix needs a block input or cache and a cotangent basis")
        if isinstance(first, Mamba3BlockCache):
            cache, g_hidden_out = first, output_cotangent_basis
            if g_hidden_out.dim() != 4:
                raise ValueError("g_hidden_out must have shape [B, P, L, D].")
            bsz, nbasis = g_hidden_out.shape[:2]
            stream = cache.residual_out.detach()
            rep = stream.repeat_interleave(nbasis, dim=0).requires_grad_(True)
            with torch.enable_grad():
                out = self.mixer(self.norm(rep.to(dtype=self.norm.weight.dtype)))
            (g,) = torch.autograd.grad(out, rep, g_hidden_out.reshape(bsz * nbasis, *stream.shape[1:]).to(out.dtype))
            total = g.reshape(bsz, nbasis, *stream.shape[1:])
            if g_residual_out is not None:
                total = total + g_residual_out.to(device=total.device, dtype=total.dtype)
            total = total.to(device=g_hidden_out.device, dtype=g_hidden_out.dtype)
            return total, (None if cache.residual_input is None else total.clone())
        hidden_states = first
        bsz, nbasis = output_cotangent_basis.shape[:2]
        rep = hidden_states.detach().repeat_interleave(nbasis, dim=0).requires_grad_(True)
        with torch.enable_grad():
            branch, stream = self.forward(rep, None)
            out = branch + stream
        (g,) = torch.autograd.grad(out, rep, output_cotangent_basis.reshape(bsz * nbasis, *hidden_states.shape[1:]).to(out.dtype))
        return g.reshape(bsz, nbasis, *hidden_states.shape[1:])

    def allocate_decode_state(self, batch_size: int, max_len: int, device=None, dtype=None):
        return self.mixer.allocate_inference_cache(batch_size, max_len, device=device, dtype=dtype)

    @torch.no_grad()
    def decode_step(self, hidden_states: torch.Tensor, residual: Optional[torch.Tensor], state):
        """One token: (branch [B, D], stream [B, D] or None) -> (branch, stream), the same contract as ``forward``."""
        residual = hidden_states if residual is None else hidden_states + residual
        return self.mixer.step(self.norm(residual.to(dtype=self.norm.weight.dtype)), *state), residual
