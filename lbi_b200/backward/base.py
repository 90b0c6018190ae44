"""Shared types of the backward engines (reference backward/base.py:10-90)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Protocol

import torch
from torch import nn

GradMap = dict[str, "torch.Tensor | None"]


@dataclass
class ADResult:
    """Named gradients plus engine diagnostics."""

    grad_map: GradMap
    diagnostics: dict[str, Any] = field(default_factory=dict)


@dataclass
class LBIBackwardResult:
    """Named gradients, the scan-vs-chain residual, optional Jacobian statistics and the state cotangents of a scan backward."""

    grad_map: GradMap
    interface_scan_rms: float
    interface_jacobian_stats: dict[str, float] | None = None
    state_cotangents: list[torch.Tensor] | None = None


class ScanBackpropModel(Protocol):
    """What scan-based backprop needs from a model."""

    num_regions: int
    region_ranges: list[tuple[int, int]]
    interface: Any
    region_backend: Any

    def named_parameters(self, *args: Any, **kwargs: Any) -> Any: ...

    def zero_grad(self, *args: Any, **kwargs: Any) -> None: ...

    def output_head_vjp_parameters(self) -> list[nn.Parameter]: ...

    def canvas_vjp_parameters(self) -> list[nn.Parameter]: ...

    def shared_local_vjp_parameters(self) -> list[nn.Parameter]: ...


_SCAN_MODEL_ATTRS = (
    "num_regions", "region_ranges", "interface", "region_backend", "named_parameters", "zero_grad",
    "output_head_vjp_parameters", "canvas_vjp_parameters", "shared_local_vjp_parameters",
)


def is_scan_backprop_model(model: Any) -> bool:
    """Structural check by attribute lookup.

    ``isinstance`` against a runtime-checkable Protocol with data members does not see ``nn.Module``
    sub-modules on Python >= 3.12 (they live in ``_modules``), which is why the reference's check
    (backward/scan.py:145-146) raises TypeError there."""
    return all(hasattr(model, attr) for attr in _SCAN_MODEL_ATTRS)


class ADEngine(Protocol):
    """What the runners call: ``backward(model=, loss=, cache=) -> ADResult``."""

    name: str

    def backward(self, *, model: nn.Module, loss: torch.Tensor, cache: Any | None = None) -> ADResult: ...


def collect_named_grads(model: nn.Module) -> GradMap:
    return {
        name: (None if p.grad is None else p.grad.detach().clone())
        for name, p in model.named_parameters()
        if p.requires_grad
    }


def assign_grad_map(model: nn.Module, grad_map: GradMap) -> None:
    for name, p in model.named_parameters():
        if p.requires_grad:
            g = grad_map.get(name)
            p.grad = None if g is None else g.detach().to(dtype=p.dtype).clone()


def parameter_name_map(model: nn.Module) -> dict[int, str]:
    return {id(p): name for name, p in model.named_parameters()}


def store_named_grads(grad_map: GradMap, param_name_map: dict[int, str], params, grads, *, accumulate: bool = True) -> None:
    for p, g in zip(params, grads):
        if g is None:
            continue
        name = param_name_map[id(p)]
        prev = grad_map.get(name)
        grad_map[name] = g if (prev is None or not accumulate) else prev + g
