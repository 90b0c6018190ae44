"""Backward step for the LBI-1 model: graph Jacobians + suffix scan + one surrogate backward
(the reference's ``legacy/backward.py:71-212`` ``_native_backward_step``)."""
from __future__ import annotations

from typing import Any

import torch

from ..backward.pullbacks import build_interface_pullback_provider
from ..backward.scan import lbi_scan_backward_step


def native_backward_step(model, loss: torch.Tensor, cache: dict[str, Any], *, interface_jacobian_mode: str = "graph",
                         jacobian_basis_chunk: int = 1) -> dict[str, Any]:
    """Needs a cache from ``forward_with_cache(..., detach_states=True)``; sets ``.grad`` and returns diagnostics."""
    if interface_jacobian_mode != "graph":
        raise ValueError("the LBI-1 model supports graph-mode Jacobians only; migrate the checkpoint for the other modes")
    provider = build_interface_pullback_provider("graph", basis_chunk=jacobian_basis_chunk)
    model.zero_grad(set_to_none=True)
    result = lbi_scan_backward_step(model=model, loss=loss, cache=cache, pullback_provider=provider)
    for name, p in model.named_parameters():
        g = result.grad_map.get(name)
        p.grad = None if g is None else g.detach().clone()
    return {"interface_scan_rms": result.interface_scan_rms}


_native_backward_step = native_backward_step
