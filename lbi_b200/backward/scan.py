"""Exact region-local backward by suffix scan.

Given the cache of ``LBILanguageModel.forward_with_cache``:

1. b_k  = direct loss cotangent of region k's input state (zero for regions without loss terms),
2. A_k^T = (d s_{k+1} / d s_k)^T for k = 0..K-2 from an ``InterfacePullbackProvider``,
3. g_k  = b_k + A_k^T g_{k+1}, g_K = 0, by a suffix scan (pure product scan when only the last region has loss),
4. parameter gradients from local VJPs with the state cotangents g_k.

With a cache built with ``detach_states=True`` every region's graph is local, so step 4 is one surrogate
backward and both region axes are supported.  With a connected graph (depth axis only) the engine follows
the reference's hook sequence (backward/scan.py:18-97).  ``interface_scan_rms`` is the RMS difference
between the scanned cotangents and a sequential mat-vec chain over the same Jacobians.
"""
from __future__ import annotations

import inspect
from typing import Any

import torch
from torch import nn

from .base import ADResult, LBIBackwardResult, assign_grad_map, is_scan_backprop_model
from .local_vjp import LocalVJPProvider, TorchAutogradLocalVJPProvider, adapt_local_vjp_provider, surrogate_backward
from .pullbacks import InterfacePullbackProvider, build_interface_pullback_provider
from .reference_scan import ReferenceScanEngine  # noqa: F401  (importable from here as in the reference, backward/scan.py:171)
from .suffix_scan import (
    apply_jacobian_t,
    interface_state_jacobian_t_stats,
    propagate_state_adjoint_affine,
    propagate_state_adjoint_by_chain,
    propagate_state_adjoint_from_last_region_input,
)


def _materialize(provider, model, cache, regions) -> list:
    """Jacobians of the listed regions; a provider written to the reference's protocol (no ``regions`` keyword,
    backward/pullbacks.py:9-18) computes all of them and the list is cut here."""
    fn = provider.materialize_state_jacobian_t
    params = inspect.signature(fn).parameters
    if "regions" in params or any(p.kind is inspect.Parameter.VAR_KEYWORD for p in params.values()):
        return fn(model=model, cache=cache, regions=regions)
    every = fn(model=model, cache=cache)
    return [every[k] for k in regions]


def _rms_between(a_list, b_list) -> float:
    num = sum(float((a.detach().float() - b.detach().float()).square().sum()) for a, b in zip(a_list, b_list))
    den = sum(a.numel() for a in a_list)
    return (num / max(1, den)) ** 0.5


def lbi_scan_backward_step(
    model: Any = None,
    *,
    loss: torch.Tensor | None = None,
    cache: dict,
    pullback_provider: InterfacePullbackProvider,
    local_vjp_provider: LocalVJPProvider | None = None,
    compute_interface_jacobian_stats: bool = False,
    include_interface_jacobian_suffix: bool = False,
    compute_scan_diagnostic: bool = True,
    ce_loss: torch.Tensor | None = None,
) -> LBIBackwardResult:
    """Exact region-local backward of one step.  With a cache whose graph was cut at every state (``detach_states=True``): loss
    cotangents per region, Jacobians of regions 0..K-2 from ``pullback_provider``, affine suffix scan, one surrogate backward for
    all parameters.  With a connected graph (depth regions): the reference's sequence of local VJPs through ``local_vjp_provider``.
    Returns the named gradients, the scan-vs-chain residual, optional Jacobian statistics and the state cotangents."""
    loss = ce_loss if loss is None else loss  # ``ce_loss`` is the reference's keyword (backward/scan.py:18-27)
    if model is None or loss is None:
        raise TypeError("lbi_scan_backward_step needs a model and a loss")
    k_regions = model.num_regions
    stats = None
    if cache.get("detached_states", False):
        leaves = cache["state_inputs"]
        direct = torch.autograd.grad(loss, leaves, retain_graph=True, allow_unused=True)
        offsets = [torch.zeros_like(s, dtype=torch.float32) if g is None else g.float() for s, g in zip(leaves, direct)]
        jacobians = _materialize(pullback_provider, model, cache, range(k_regions - 1))
        if compute_interface_jacobian_stats and jacobians:
            stats = interface_state_jacobian_t_stats(jacobians, include_suffix=include_interface_jacobian_suffix)
        only_last = all(not model.plan.region_has_loss(k) for k in range(k_regions - 1)) if hasattr(model, "plan") else False
        if only_last and k_regions > 1:
            g = propagate_state_adjoint_from_last_region_input([*jacobians, None], offsets[-1])
        else:
            g = propagate_state_adjoint_affine(jacobians, offsets)
        rms = _rms_between(g, propagate_state_adjoint_by_chain(jacobians, offsets)) if (compute_scan_diagnostic and k_regions > 1) else 0.0
        grad_map = surrogate_backward(model=model, loss=loss, cache=cache, state_cotangents=g)
        return LBIBackwardResult(grad_map=grad_map, interface_scan_rms=rms, interface_jacobian_stats=stats, state_cotangents=g)

    # connected graph: the reference's sequence of local VJPs (loss terms only in the last region)
    if getattr(model, "region_axis", "depth") != "depth":
        raise ValueError("sequence-axis regions need a cache built with detach_states=True")
    vjp = adapt_local_vjp_provider(local_vjp_provider) or TorchAutogradLocalVJPProvider()
    grad_map = vjp.initialize_grad_map(model)
    vjp.output_head_grads(model=model, loss=loss, grad_map=grad_map)
    states = cache["states"]
    rms = 0.0
    if k_regions == 1:
        g = [vjp.state_adjoint_from_loss(loss=loss, state=states[0])]
    else:
        g_last = vjp.state_adjoint_from_loss(loss=loss, state=states[k_regions - 1])
        jacobians = _materialize(pullback_provider, model, cache, range(k_regions - 1))
        if compute_interface_jacobian_stats:
            stats = interface_state_jacobian_t_stats(jacobians, include_suffix=include_interface_jacobian_suffix)
        g = propagate_state_adjoint_from_last_region_input([*jacobians, None], g_last)
        if compute_scan_diagnostic:
            chain, cur = [g_last], g_last
            for idx in range(k_regions - 2, -1, -1):
                cur = apply_jacobian_t(jacobians[idx], cur)
                chain.append(cur)
            rms = _rms_between(g, chain[::-1])
    vjp.initial_state_grads(model=model, cache=cache, state_cotangent=g[0], grad_map=grad_map)
    for k in range(k_regions):
        vjp.region_grads(model=model, cache=cache, region_index=k, loss=loss,
                         next_state_cotangent=None if k == k_regions - 1 else g[k + 1], grad_map=grad_map)
    vjp.shared_grads(model=model, loss=loss, grad_map=grad_map)
    return LBIBackwardResult(grad_map=grad_map, interface_scan_rms=rms, interface_jacobian_stats=stats, state_cotangents=g)


class ScanADEngine:
    """Exact region-local backward: per-region interface Jacobians from a pullback provider, suffix scan of the state cotangents,
    local VJPs per region; assigns ``.grad`` and reports the scan diagnostics."""

    name = "scan"
    requires_detached_states = True

    def __init__(
        self,
        *,
        state_jacobian_mode: str = "graph",
        state_jacobian_basis_chunk: int = 1,
        compute_interface_jacobian_stats: bool = False,
        include_interface_jacobian_suffix: bool = False,
        compute_scan_diagnostic: bool = True,
        pullback_provider: InterfacePullbackProvider | None = None,
        local_vjp_provider: LocalVJPProvider | None = None,
    ) -> None:
        self.state_jacobian_mode = state_jacobian_mode
        self.state_jacobian_basis_chunk = int(state_jacobian_basis_chunk)
        self.compute_interface_jacobian_stats = bool(compute_interface_jacobian_stats)
        self.include_interface_jacobian_suffix = bool(include_interface_jacobian_suffix)
        self.compute_scan_diagnostic = bool(compute_scan_diagnostic)
        self.pullback_provider = pullback_provider or build_interface_pullback_provider(
            state_jacobian_mode, basis_chunk=self.state_jacobian_basis_chunk
        )
        self.local_vjp_provider = local_vjp_provider or TorchAutogradLocalVJPProvider()
        # A caller's own local-VJP provider is driven hook by hook, which needs the connected forward graph (depth-axis
        # regions, as in the reference); without one the graph is cut at every state and one surrogate backward does the VJPs.
        self.requires_detached_states = local_vjp_provider is None

    @classmethod
    def from_config(cls, cfg: Any, *, compute_interface_jacobian_stats: bool = False) -> "ScanADEngine":
        return cls(
            state_jacobian_mode=cfg.interface_jacobian_mode,
            state_jacobian_basis_chunk=cfg.jacobian_basis_chunk,
            compute_interface_jacobian_stats=compute_interface_jacobian_stats,
            include_interface_jacobian_suffix=bool(getattr(cfg, "log_interface_jacobian_suffix", False)),
        )

    def backward(self, *, model: nn.Module, loss: torch.Tensor, cache: Any | None = None) -> ADResult:
        if not is_scan_backprop_model(model):
            raise TypeError("scan backprop needs a model with regions, an interface and local-VJP parameter groups")
        if cache is None:
            raise ValueError("scan backprop needs the forward cache")
        model.zero_grad(set_to_none=True)
        result = lbi_scan_backward_step(
            model=model,
            loss=loss,
            cache=cache,
            pullback_provider=self.pullback_provider,
            local_vjp_provider=self.local_vjp_provider,
            compute_interface_jacobian_stats=self.compute_interface_jacobian_stats,
            include_interface_jacobian_suffix=self.include_interface_jacobian_suffix,
            compute_scan_diagnostic=self.compute_scan_diagnostic,
        )
        assign_grad_map(model, result.grad_map)
        diagnostics: dict[str, Any] = {
            "interface_scan_rms": result.interface_scan_rms,
            "interface_jacobian_mode": self.state_jacobian_mode,
            "jacobian_basis_chunk": self.state_jacobian_basis_chunk,
            # the two keys the reference's engine reports (backward/scan.py:161-165)
            "interface_pullback_provider": getattr(self.pullback_provider, "name", type(self.pullback_provider).__name__),
            "local_vjp_provider": getattr(self.local_vjp_provider, "name", type(self.local_vjp_provider).__name__),
        }
        if result.interface_jacobian_stats is not None:
            diagnostics["interface_jacobian_stats"] = result.interface_jacobian_stats
        return ADResult(grad_map=result.grad_map, diagnostics=diagnostics)
