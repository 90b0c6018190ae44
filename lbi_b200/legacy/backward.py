"""Backward step for the LBI-1 model: interface Jacobians (graph or recompute mode) + suffix scan + one surrogate backward
(the reference's ``legacy/backward.py:71-212`` ``_native_backward_step``, both of its Jacobian modes)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from ..backward.pullbacks import build_interface_pullback_provider
from ..backward.scan import lbi_scan_backward_step


class _LegacyRecomputeProvider:
    """Recompute-mode Jacobians through the model's own message map (its caches carry the LBI-1 field names)."""
    name = "recompute"

    def __init__(self, basis_chunk: int) -> None:
        self.basis_chunk = int(basis_chunk)

    def materialize_state_jacobian_t(self, *, model, cache, regions=None):
        mats = model.materialize_interface_pullback_mats(cache, mode="recompute", basis_chunk=self.basis_chunk)
        return mats if regions is None else [mats[k] for k in regions]


@dataclass
class NativeBackwardResult:
    """What the reference's ``_native_backward_step`` returns (legacy/backward.py:13-17)."""
    grad_map: dict[str, torch.Tensor | None]
    interface_scan_rms: float
    interface_jacobian_stats: dict[str, float] | None = None


def _provider(interface_jacobian_mode: str, jacobian_basis_chunk: int):
    if interface_jacobian_mode == "graph":
        return build_interface_pullback_provider("graph", basis_chunk=jacobian_basis_chunk)
    if interface_jacobian_mode == "recompute":
        return _LegacyRecomputeProvider(jacobian_basis_chunk)
    raise ValueError("interface Jacobian mode must be one of: graph, recompute")


def _native_backward_step(model, *, ce_loss: torch.Tensor, cache: dict[str, Any], interface_jacobian_mode: str = "graph",
                          jacobian_basis_chunk: int = 1, interface_recompute_context: Any | None = None,
                          compute_interface_jacobian_stats: bool = False,
                          include_interface_jacobian_suffix: bool = False) -> NativeBackwardResult:
    """The reference's entry point with its keyword names (legacy/backward.py:71-81): interface Jacobians in graph or recompute
    mode, suffix scan, local gradients; optional Frobenius / spectral statistics of the local Jacobians and of their suffix
    products.  Returns the named gradients without touching ``.grad``.  ``interface_recompute_context``: a context manager
    (autocast, say) entered around the Jacobian recomputation."""
    from contextlib import nullcontext

    provider = _provider(interface_jacobian_mode, jacobian_basis_chunk)
    with (interface_recompute_context if interface_recompute_context is not None else nullcontext()):
        result = lbi_scan_backward_step(model=model, loss=ce_loss, cache=cache, pullback_provider=provider,
                                        compute_interface_jacobian_stats=compute_interface_jacobian_stats,
                                        include_interface_jacobian_suffix=include_interface_jacobian_suffix)
    grad_map = {name: (None if result.grad_map.get(name) is None else result.grad_map[name].detach().clone())
                for name, p in model.named_parameters() if p.requires_grad}
    return NativeBackwardResult(grad_map=grad_map, interface_scan_rms=float(result.interface_scan_rms),
                                interface_jacobian_stats=result.interface_jacobian_stats)


def native_backward_step(model, loss: torch.Tensor, cache: dict[str, Any], *, interface_jacobian_mode: str = "graph",
                         jacobian_basis_chunk: int = 1) -> dict[str, Any]:
    """Needs a cache from ``forward_with_cache(..., detach_states=True)``; sets ``.grad`` and returns diagnostics."""
    model.zero_grad(set_to_none=True)
    result = _native_backward_step(model, ce_loss=loss, cache=cache, interface_jacobian_mode=interface_jacobian_mode,
                                   jacobian_basis_chunk=jacobian_basis_chunk)
    for name, p in model.named_parameters():
        g = result.grad_map.get(name)
        p.grad = None if g is None else g
    return {"interface_scan_rms": result.interface_scan_rms}


