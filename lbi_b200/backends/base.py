"""Region backend protocol (reference backends/base.py:10-50)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Protocol

import torch
from torch import nn


def current_autocast(device: torch.device) -> tuple[str, torch.dtype] | None:
    """(device type, dtype) of the autocast region the caller runs in, or None: recorded at forward time so that every
    later recompute of the same computation (Jacobian providers, pullbacks, parameter VJPs) runs at the same precision
    and reaches the same kernels."""
    kind = device.type
    if torch.is_autocast_enabled(kind):
        return kind, torch.get_autocast_dtype(kind)
    return None


def autocast_as(state: tuple[str, torch.dtype] | None):
    """Context manager that restores a state recorded by ``current_autocast`` (a no-op context for None)."""
    import contextlib

    return torch.autocast(state[0], dtype=state[1]) if state else contextlib.nullcontext()


@dataclass
class RegionForwardCache:
    """What a backend keeps from a region forward: index, layer range, the input, the structured cache (built lazily), autocast state."""

    region_index: int
    layer_range: tuple[int, int]
    region_input: torch.Tensor | None = None
    structured: Any | None = None
    extras: dict = field(default_factory=dict)
    autocast: tuple | None = None


class RegionBackend(Protocol):
    """Runs one region (``forward_region``), lists its parameters, and differentiates it: a basis of output cotangents pulled back to
    the input (``input_pullback_basis``) and the parameter VJP of one cotangent (``parameter_vjp``)."""

    name: str

    def forward_region(self, *, region_input: torch.Tensor, region_index: int) -> tuple[torch.Tensor, RegionForwardCache]: ...

    def parameters_for_region(self, region_index: int) -> list[nn.Parameter]: ...

    def count_parameters(self) -> int: ...

    def initialize_parameters(self, *, backbone_spec: Any) -> None: ...

    def input_pullback_basis(self, *, cache: RegionForwardCache, output_cotangent_basis: torch.Tensor) -> torch.Tensor: ...

    def parameter_vjp(self, *, cache: RegionForwardCache, output_cotangent: torch.Tensor) -> dict[str, torch.Tensor]: ...
