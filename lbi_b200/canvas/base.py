"""Canvas protocol: maps token ids to the static features every region reads (reference canvas/base.py:10-32)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Protocol, runtime_checkable

import torch
from torch import nn


@dataclass
class CanvasCache:
    """Token ids and the features they were mapped to."""

    input_ids: torch.Tensor
    features: torch.Tensor


@runtime_checkable
class CanvasModule(Protocol):
    """Token ids -> features; ``output_weight`` for tied readouts, ``vjp_parameters`` for the shared-parameter VJP."""

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor: ...

    def forward_with_cache(self, input_ids: torch.Tensor) -> tuple[torch.Tensor, CanvasCache]: ...

    def output_weight(self) -> torch.Tensor: ...

    def vjp_parameters(self) -> list[nn.Parameter]: ...
