"""Sequential reference for the scan engine: the state cotangents are propagated by a chain of one-step
VJPs through the forward graph instead of materialised Jacobians (reference backward/reference_scan.py:12-34,
backward/suffix_scan.py:82-102).  Slower than dense autograd, but independent of the Jacobian providers."""
from __future__ import annotations

from typing import Any

import torch
from torch import nn

from .base import ADResult, LBIBackwardResult, assign_grad_map, is_scan_backprop_model
from .local_vjp import TorchAutogradLocalVJPProvider, surrogate_backward


def lbi_reference_scan_backward_step(model: Any = None, *, loss: torch.Tensor | None = None, cache: dict,
                                     ce_loss: torch.Tensor | None = None, state_jacobian_mode: str | None = None,
                                     state_jacobian_basis_chunk: int = 1, compute_interface_jacobian_stats: bool = False,
                                     include_interface_jacobian_suffix: bool = False) -> LBIBackwardResult:
    """With ``state_jacobian_mode`` left at None the state cotangents go down the forward graph one VJP at a time; with a
    provider name ("graph", "recompute", ...) the call is the Jacobian scan with that provider, which is what the reference's
    function of this name runs (backward/reference_scan.py:12-34).  ``ce_loss`` is the reference's keyword for ``loss``."""
    loss = ce_loss if loss is None else loss
    if model is None or loss is None:
        raise TypeError("lbi_reference_scan_backward_step needs a model and a loss")
    if state_jacobian_mode is not None:
        from .pullbacks import build_interface_pullback_provider
        from .scan import lbi_scan_backward_step

        provider = build_interface_pullback_provider(state_jacobian_mode, basis_chunk=state_jacobian_basis_chunk)
        return lbi_scan_backward_step(model, loss=loss, cache=cache, pullback_provider=provider,
                                      compute_interface_jacobian_stats=compute_interface_jacobian_stats,
                                      include_interface_jacobian_suffix=include_interface_jacobian_suffix)
    k_regions = model.num_regions
    if cache.get("detached_states", False):
        leaves = cache["state_inputs"]
        direct = torch.autograd.grad(loss, leaves, retain_graph=True, allow_unused=True)
        g = [None] * k_regions
        cur = torch.zeros_like(leaves[-1]) if direct[-1] is None else direct[-1]
        g[k_regions - 1] = cur
        for k in range(k_regions - 2, -1, -1):
            s_next = cache["states"][k + 1]
            (through,) = torch.autograd.grad(s_next, leaves[k], cur.to(s_next.dtype), retain_graph=True)
            cur = through if direct[k] is None else through + direct[k]
            g[k] = cur
        grad_map = surrogate_backward(model=model, loss=loss, cache=cache, state_cotangents=g)
        return LBIBackwardResult(grad_map=grad_map, interface_scan_rms=0.0, state_cotangents=g)

    if getattr(model, "region_axis", "depth") != "depth":
        raise ValueError("sequence-axis regions need a cache built with detach_states=True")
    vjp = TorchAutogradLocalVJPProvider()
    grad_map = vjp.initialize_grad_map(model)
    vjp.output_head_grads(model=model, loss=loss, grad_map=grad_map)
    states = cache["states"]
    g = [None] * k_regions
    cur = vjp.state_adjoint_from_loss(loss=loss, state=states[k_regions - 1])
    g[k_regions - 1] = cur
    for k in range(k_regions - 2, -1, -1):
        (cur,) = torch.autograd.grad(states[k + 1], states[k], cur.to(states[k + 1].dtype), retain_graph=True)
        g[k] = cur
    vjp.initial_state_grads(model=model, cache=cache, state_cotangent=g[0], grad_map=grad_map)
    for k in range(k_regions):
        vjp.region_grads(model=model, cache=cache, region_index=k, loss=loss,
                         next_state_cotangent=None if k == k_regions - 1 else g[k + 1], grad_map=grad_map)
    vjp.shared_grads(model=model, loss=loss, grad_map=grad_map)
    return LBIBackwardResult(grad_map=grad_map, interface_scan_rms=0.0, state_cotangents=g)


class ReferenceScanEngine:
    """The same gradients with the state cotangents pulled through the forward graph one region at a time (no Jacobians)."""

    name = "reference_scan"
    requires_detached_states = True

    def backward(self, *, model: nn.Module, loss: torch.Tensor, cache: Any | None = None) -> ADResult:
        if not is_scan_backprop_model(model):
            raise TypeError("reference scan needs a model with regions, an interface and local-VJP parameter groups")
        if cache is None:
            raise ValueError("reference scan needs the forward cache")
        model.zero_grad(set_to_none=True)
        result = lbi_reference_scan_backward_step(model=model, loss=loss, cache=cache)
        assign_grad_map(model, result.grad_map)
        return ADResult(grad_map=result.grad_map, diagnostics={"interface_scan_rms": 0.0})


def __getattr__(name: str):
    """``ScanADEngine``, ``lbi_scan_backward_step`` and ``build_interface_pullback_provider`` are importable from this module as
    in the reference (backward/reference_scan.py:9, :37-42); resolved on first use because ``scan`` imports this module."""
    if name in ("ScanADEngine", "lbi_scan_backward_step"):
        from . import scan

        return getattr(scan, name)
    if name == "build_interface_pullback_provider":
        from .pullbacks import build_interface_pullback_provider

        return build_interface_pullback_provider
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
