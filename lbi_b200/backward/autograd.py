"""Dense autograd engine: ``loss.backward()`` and collect (reference backward/autograd.py:11-28)."""
from __future__ import annotations

from typing import Any

import torch
from torch import nn

from .base import ADResult, collect_named_grads


def autograd_backward_step(model: nn.Module, loss: torch.Tensor | None = None, *, ce_loss: torch.Tensor | None = None) -> dict:
    """Dense autograd gradients of ``loss`` by parameter name (``.grad`` is cleared first and left set)."""
    loss = ce_loss if loss is None else loss  # ``ce_loss`` is the reference's keyword (backward/autograd.py:27)
    model.zero_grad(set_to_none=True)
    loss.backward()
    return collect_named_grads(model)


class AutogradEngine:
    """Dense autograd: ``loss.backward()`` and the collected named gradients (the oracle of every other engine)."""

    name = "autograd"
    requires_detached_states = False

    def backward(self, *, model: nn.Module, loss: torch.Tensor, cache: Any | None = None) -> ADResult:
        return ADResult(grad_map=autograd_backward_step(model, loss), diagnostics={})
