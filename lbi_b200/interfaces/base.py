"""Abstract bounded interface: the small state that is the only thing consecutive regions exchange.

Mirrors the contract of the reference's ``interfaces/base.py:11-106``:
``initialize`` -> s_0, ``decode(s_k, k)`` -> region condition, ``update(s_k, region_out, k)`` -> s_{k+1},
parameter groupings for local VJPs, and structured Jacobian-transpose hooks over a basis of cotangents.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from typing import Any

import torch
from torch import nn


@dataclass(frozen=True)
class InterfaceSpec:
    """Name and state width of an interface."""

    state_shape: tuple[int, ...]
    state_flat_dim: int
    region_condition_dim: int


@dataclass
class InterfaceStep:
    """Result of one state update: the new state plus diagnostics (pooled features, delta, scale, pre-norm state)."""

    state: torch.Tensor
    diagnostics: dict[str, torch.Tensor] = field(default_factory=dict)
    cache: Any | None = None


class InterfaceModule(nn.Module, ABC):
    """Base class of interfaces: ``initialize``, ``decode``, ``update``, the parameter groups of the local VJPs and the optional
    closed-form Jacobian-transpose hooks the structured engines call."""

    spec: InterfaceSpec

    @abstractmethod
    def validate_region_count(self, num_regions: int) -> None: ...

    @abstractmethod
    def initialize(self, canvas_features: torch.Tensor) -> torch.Tensor: ...

    @abstractmethod
    def decode(self, state: torch.Tensor, region_index: int) -> torch.Tensor: ...

    @abstractmethod
    def update(self, state: torch.Tensor, region_features: torch.Tensor, region_index: int) -> InterfaceStep: ...

    def initial_vjp_parameters(self) -> list[nn.Parameter]:
        return []

    def region_vjp_parameters(self, region_index: int) -> list[nn.Parameter]:
        return []

    def shared_vjp_parameters(self) -> list[nn.Parameter]:
        return []

    def apply_update_jacobian_t_to_region_output(self, *, region_cache: Any, state_out_cotangent_basis: torch.Tensor):
        raise NotImplementedError(f"{type(self).__name__} has no structured update pullback")

    def apply_decode_jacobian_t_to_state_input(self, *, region_cache: Any, region_input_cotangent_basis: torch.Tensor):
        raise NotImplementedError(f"{type(self).__name__} has no structured decode pullback")

    def apply_region_transition_jacobian_t(
        self, *, region_cache: Any, state_out_cotangent_basis: torch.Tensor, region_input_cotangent_basis: torch.Tensor
    ) -> dict[str, torch.Tensor]:
        """Full transition J^T for one region: skip path through the residual update plus the decode path."""
        upd = self.apply_update_jacobian_t_to_region_output(
            region_cache=region_cache, state_out_cotangent_basis=state_out_cotangent_basis
        )
        dec = self.apply_decode_jacobian_t_to_state_input(
            region_cache=region_cache, region_input_cotangent_basis=region_input_cotangent_basis
        )
        return {**upd, **dec, "g_state_input_total": upd["g_state_skip"] + dec["g_state_input"]}
