"""Backward step for the LBI-1 model: interface Jacobians (graph or recompute mode) + suffix scan + one surrogate backward
(the reference's ``legacy/backward.py:71-212`` ``_native_backward_step``, both of its Jacobian modes)."""
from __future__ import annotations

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


def native_backward_step(model, loss: torch.Tensor, cache: dict[str, Any], *, interface_jacobian_mode: str = "graph",
                         jacobian_basis_chunk: int = 1) -> dict[str, Any]:
    """Needs a cache from ``forward_with_cache(..., detach_states=True)``; sets ``.grad`` and returns diagnostics."""
    if interface_jacobian_mode == "graph":
        provider = build_interface_pullback_provider("graph", basis_chunk=jacobian_basis_chunk)
    elif interface_jacobian_mode == "recompute":
        provider = _LegacyRecomputeProvider(jacobian_basis_chunk)
    else:
        raise ValueError("interface Jacobian mode must be one of: graph, recompute")
    model.zero_grad(set_to_none=True)
    result = lbi_scan_backward_step(model=model, loss=loss, cache=cache, pullback_provider=provider)
    for name, p in model.named_parameters():
        g = result.grad_map.get(name)
        p.grad = None if g is None else g.detach().clone()
    return {"interface_scan_rms": result.interface_scan_rms}


_native_backward_step = native_backward_step
