"""Local vector-Jacobian products through the retained forward graph.

``LocalVJPProvider`` keeps the six hooks of the reference (backward/local_vjp.py:10-185): head gradients,
the loss cotangent of the last region's input state, initial-encoder gradients, per-region gradients and the
shared canvas / update-scale gradients.  ``surrogate_backward`` is the single-pass form used when the graph
was cut at every interface state: all parameter gradients follow from one backward of
``loss + sum_k <s_k, g_k>`` because each region's graph is then local.
"""
from __future__ import annotations

from typing import Any, Protocol, Sequence

import torch
from torch import nn

from .base import GradMap, parameter_name_map, store_named_grads


class LocalVJPProvider(Protocol):
    """The six local steps of the scan backward (see the module docstring)."""

    name: str

    def initialize_grad_map(self, model: Any) -> GradMap: ...

    def output_head_grads(self, *, model: Any, loss: torch.Tensor, grad_map: GradMap) -> None: ...

    def state_adjoint_from_loss(self, *, loss: torch.Tensor, state: torch.Tensor) -> torch.Tensor: ...

    def initial_state_grads(self, *, model: Any, cache: dict, state_cotangent: torch.Tensor, grad_map: GradMap) -> None: ...

    def region_grads(self, *, model: Any, cache: dict, region_index: int, loss: torch.Tensor,
                     next_state_cotangent: torch.Tensor | None, grad_map: GradMap) -> None: ...

    def shared_grads(self, *, model: Any, loss: torch.Tensor, grad_map: GradMap) -> None: ...


class ReferenceHookLocalVJPProvider:
    """Wraps a provider written against the reference's hook names (``new_grad_map``, ``store_output_head_grads``,
    ``store_initial_interface_grads``, ``store_region_grads``, ``store_shared_canvas_grads``; backward/local_vjp.py:10-62)
    so that the scan engine here can drive it."""

    def __init__(self, inner: Any) -> None:
        self.inner = inner
        self.name = getattr(inner, "name", type(inner).__name__)

    def initialize_grad_map(self, model) -> GradMap:
        return self.inner.new_grad_map(model)

    def output_head_grads(self, *, model, loss, grad_map) -> None:
        self.inner.store_output_head_grads(model=model, loss=loss, grad_map=grad_map)

    def state_adjoint_from_loss(self, *, loss, state) -> torch.Tensor:
        return self.inner.state_adjoint_from_loss(loss=loss, state=state)

    def initial_state_grads(self, *, model, cache, state_cotangent, grad_map) -> None:
        s0 = cache["initial_state"] if "initial_state" in cache else cache["states"][0]
        self.inner.store_initial_interface_grads(model=model, state0=s0, state0_adjoint=state_cotangent.to(s0.dtype),
                                                 grad_map=grad_map)

    def region_grads(self, *, model, cache, region_index, loss, next_state_cotangent, grad_map) -> None:
        states = list(cache["states"])
        num_regions = len(states) - 1
        adjoints: list = [None] * (num_regions + 1)
        if next_state_cotangent is not None:
            adjoints[region_index + 1] = next_state_cotangent.to(states[region_index + 1].dtype)
        self.inner.store_region_grads(model=model, loss=loss, states=states, region_index=region_index,
                                      num_regions=num_regions, state_adjoints=adjoints, grad_map=grad_map)

    def shared_grads(self, *, model, loss, grad_map) -> None:
        self.inner.store_shared_canvas_grads(model=model, loss=loss, grad_map=grad_map)


def adapt_local_vjp_provider(provider: Any) -> Any:
    """A provider with this package's hook names as it is; one with only the reference's names behind the adapter."""
    if provider is None or hasattr(provider, "initialize_grad_map"):
        return provider
    if hasattr(provider, "new_grad_map"):
        return ReferenceHookLocalVJPProvider(provider)
    raise TypeError("a local-VJP provider needs initialize_grad_map (or the reference's new_grad_map) and the matching hooks")


def _grad(outputs, inputs: Sequence[nn.Parameter], grad_outputs=None, retain_graph=True):
    if len(inputs) == 0:
        return []
    return torch.autograd.grad(outputs, list(inputs), grad_outputs=grad_outputs, retain_graph=retain_graph, allow_unused=True)


class TorchAutogradLocalVJPProvider:
    """Every local step as a ``torch.autograd.grad`` call on the retained forward graph."""

    name = "torch_autograd"

    def __init__(self) -> None:
        self._names: dict[int, str] = {}

    def initialize_grad_map(self, model) -> GradMap:
        self._names = parameter_name_map(model)
        return {name: None for name, p in model.named_parameters() if p.requires_grad}

    def output_head_grads(self, *, model, loss, grad_map) -> None:
        params = model.output_head_vjp_parameters()
        store_named_grads(grad_map, self._names, params, _grad(loss, params))

    def state_adjoint_from_loss(self, *, loss, state) -> torch.Tensor:
        (g,) = torch.autograd.grad(loss, state, retain_graph=True, allow_unused=True)
        return torch.zeros_like(state) if g is None else g

    def initial_state_grads(self, *, model, cache, state_cotangent, grad_map) -> None:
        params = model.interface.initial_vjp_parameters()
        s0 = cache["initial_state"] if "initial_state" in cache else cache["states"][0]
        if s0.requires_grad:
            store_named_grads(grad_map, self._names, params, _grad(s0, params, state_cotangent.to(s0.dtype)))

    def region_grads(self, *, model, cache, region_index, loss, next_state_cotangent, grad_map) -> None:
        params = [*model.region_backend.parameters_for_region(region_index), *model.interface.region_vjp_parameters(region_index)]
        if next_state_cotangent is None:
            grads = _grad(loss, params)
        else:
            s_next = cache["states"][region_index + 1]
            grads = _grad(s_next, params, next_state_cotangent.to(s_next.dtype))
        store_named_grads(grad_map, self._names, params, grads)

    def shared_grads(self, *, model, loss, grad_map) -> None:
        params = model.shared_local_vjp_parameters()
        store_named_grads(grad_map, self._names, params, _grad(loss, params, retain_graph=False))

    # The same hooks under the reference's names and argument lists (backward/local_vjp.py:65-185).
    def new_grad_map(self, model) -> GradMap:
        return self.initialize_grad_map(model)

    def store_output_head_grads(self, *, model, loss, grad_map) -> None:
        self._ensure_names(model)
        self.output_head_grads(model=model, loss=loss, grad_map=grad_map)

    def store_initial_interface_grads(self, *, model, state0, state0_adjoint, grad_map) -> None:
        self._ensure_names(model)
        self.initial_state_grads(model=model, cache={"initial_state": state0}, state_cotangent=state0_adjoint, grad_map=grad_map)

    def store_region_grads(self, *, model, loss, states, region_index, num_regions, state_adjoints, grad_map) -> None:
        self._ensure_names(model)
        last = region_index >= num_regions - 1
        self.region_grads(model=model, cache={"states": states}, region_index=region_index, loss=loss,
                          next_state_cotangent=None if last else state_adjoints[region_index + 1], grad_map=grad_map)

    def store_shared_canvas_grads(self, *, model, loss, grad_map) -> None:
        self._ensure_names(model)
        self.shared_grads(model=model, loss=loss, grad_map=grad_map)

    def _param_name_map(self, model) -> dict[int, str]:
        return parameter_name_map(model)

    def _store_grads(self, *, model, grad_map, params, grads) -> None:
        store_named_grads(grad_map, self._param_name_map(model), params, grads)

    def _ensure_names(self, model) -> None:
        if not self._names:
            self._names = parameter_name_map(model)


def surrogate_backward(*, model: Any, loss: torch.Tensor, cache: dict, state_cotangents: Sequence[torch.Tensor]) -> GradMap:
    """One backward pass over region-local graphs.

    ``state_cotangents[k]`` is g_k = dL/ds_k for k = 0..K-1.  The outputs differentiated are the loss, the
    initial state (cotangent g_0) and every region's outgoing state s_{k+1} (cotangent g_{k+1}, k < K-1)."""
    names = parameter_name_map(model)
    params = [p for p in model.parameters() if p.requires_grad]
    outputs, cotangents = [loss], [torch.ones_like(loss)]
    s0 = cache["initial_state"]
    if s0.requires_grad:
        outputs.append(s0)
        cotangents.append(state_cotangents[0].to(s0.dtype))
    for k in range(1, len(state_cotangents)):
        s = cache["states"][k]
        if s.requires_grad:
            outputs.append(s)
            cotangents.append(state_cotangents[k].to(s.dtype))
    grads = torch.autograd.grad(outputs, params, grad_outputs=cotangents, allow_unused=True)
    grad_map: GradMap = {name: None for name, p in model.named_parameters() if p.requires_grad}
    store_named_grads(grad_map, names, params, grads)
    return grad_map
