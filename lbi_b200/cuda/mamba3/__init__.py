"""Mamba-3 state-mixer pullback.  The reference reserves this entry point and raises NotImplementedError
(cuda/mamba3/__init__.py:4-11); here it is the mixer's basis pullback."""
from __future__ import annotations

import torch


def state_mixer_input_pullback_basis(mixer, mixer_input_or_cache, output_cotangent_basis: torch.Tensor) -> torch.Tensor:
    """Cotangent basis [B, P, L, D] of a ``Mamba3`` mixer's output -> cotangents of its input, same shape.
    ``mixer_input_or_cache`` is the mixer input [B, L, D] or the cache of ``forward_with_cache``.  For whole regions of
    Mamba blocks the engine uses ``backends.mamba_structured.StructuredMambaRegion.input_pullback`` (kernels, no autograd)."""
    return mixer.input_pullback_matrix(mixer_input_or_cache, output_cotangent_basis)


__all__ = ["state_mixer_input_pullback_basis"]
