"""Readout protocol: region features -> vocabulary logits (reference readouts/base.py:12-28)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Protocol, runtime_checkable

import torch
from torch import nn


@dataclass
class ReadoutCache:
    """Input features, normed features and logits of one readout call."""

    features: torch.Tensor
    normed_features: torch.Tensor
    logits: torch.Tensor


@runtime_checkable
class ReadoutModule(Protocol):
    """Region features -> vocabulary logits; ``vjp_parameters`` lists what the head VJP differentiates."""

    def forward(self, features: torch.Tensor, *, canvas) -> torch.Tensor: ...

    def forward_with_cache(self, features: torch.Tensor, *, canvas) -> tuple[torch.Tensor, ReadoutCache]: ...

    def vjp_parameters(self) -> list[nn.Parameter]: ...
