"""Transformer region backend with cached activations and pluggable derivative lowerings.

Counterpart of the reference's ``backends/transformer.py`` (backend :88-281, autograd lowering :283-355).
``forward_region`` runs the ordinary modules when autograd is recording (so ``loss.backward()`` and the
autograd-based engines work) and the closed-form ``StructuredTransformerRegion`` otherwise; the structured
cache is built lazily when a lowering needs it.
"""
from __future__ import annotations

from typing import Protocol

import torch
from torch import nn

from ..backbones.general import BackboneSpec, build_backbone_stack, init_transformer_module
from .base import RegionForwardCache, autocast_as, current_autocast
from .transformer_structured import StructuredTransformerRegion


class TransformerLowering(Protocol):
    def input_pullback_basis(self, *, backend: "TransformerRegionBackend", cache: RegionForwardCache,
                             output_cotangent_basis: torch.Tensor) -> torch.Tensor: ...

    def parameter_vjp(self, *, backend: "TransformerRegionBackend", cache: RegionForwardCache,
                      output_cotangent: torch.Tensor) -> dict[str, torch.Tensor]: ...


class TorchAutogradTransformerLowering:
    """Oracle lowering: recompute the region on a basis-replicated batch and differentiate with autograd."""

    def input_pullback_basis(self, *, backend, cache, output_cotangent_basis):
        bsz, nbasis = output_cotangent_basis.shape[:2]
        x = cache.region_input.detach()
        rep = x.unsqueeze(1).expand(bsz, nbasis, *x.shape[1:]).reshape(bsz * nbasis, *x.shape[1:]).clone().requires_grad_(True)
        with torch.enable_grad(), autocast_as(cache.autocast):
            out = backend.backbone.forward_range(rep, *cache.layer_range)
        (g,) = torch.autograd.grad(out, rep, output_cotangent_basis.reshape(bsz * nbasis, *x.shape[1:]).to(out.dtype))
        return g.reshape(bsz, nbasis, *x.shape[1:])

    def parameter_vjp(self, *, backend, cache, output_cotangent):
        named = backend.named_parameters_for_region(cache.region_index)
        with torch.enable_grad(), autocast_as(cache.autocast):
            out = backend.backbone.forward_range(cache.region_input.detach(), *cache.layer_range)
        grads = torch.autograd.grad(out, [p for _, p in named], output_cotangent.to(out.dtype), allow_unused=True)
        return {name: g for (name, _), g in zip(named, grads) if g is not None}


class StructuredTransformerLowering:
    """Closed-form lowering over cached activations (fused sm_100a kernels on CUDA)."""

    def _structured(self, backend, cache):
        if cache.structured is None:
            _, cache.structured = backend.structured.forward(cache.region_input.detach(), cache.layer_range)
        return cache.structured

    def input_pullback_basis(self, *, backend, cache, output_cotangent_basis):
        sc = self._structured(backend, cache)
        bsz, nbasis, seqlen, dim = output_cotangent_basis.shape
        rows = output_cotangent_basis.permute(1, 0, 2, 3).reshape(nbasis * bsz * seqlen, dim)
        g = backend.structured.input_pullback(sc, rows)
        return g.reshape(nbasis, bsz, seqlen, dim).permute(1, 0, 2, 3)

    def parameter_vjp(self, *, backend, cache, output_cotangent):
        sc = self._structured(backend, cache)
        grads: dict[str, torch.Tensor] = {}
        backend.structured.backward(sc, output_cotangent.reshape(-1, output_cotangent.shape[-1]), grads)
        return {f"backbone.{name}": g for name, g in grads.items()}


class TransformerRegionBackend(nn.Module):
    def __init__(self, *, backbone_spec: BackboneSpec, region_ranges: list[tuple[int, int]],
                 lowering: TransformerLowering | None = None) -> None:
        super().__init__()
        if backbone_spec.name != "transformer":
            raise ValueError("TransformerRegionBackend requires a transformer backbone spec")
        self.backbone_spec = backbone_spec
        self.region_ranges = [tuple(r) for r in region_ranges]
        self.backbone = build_backbone_stack(backbone_spec)
        self.lowering: TransformerLowering = lowering or StructuredTransformerLowering()
        object.__setattr__(self, "structured", StructuredTransformerRegion(self.backbone.blocks))

    @property
    def blocks(self) -> nn.ModuleList:
        return self.backbone.blocks

    def forward_region(self, *, region_input: torch.Tensor, region_index: int):
        start, end = self.region_ranges[region_index]
        cache = RegionForwardCache(region_index=region_index, layer_range=(start, end), region_input=region_input,
                                   autocast=current_autocast(region_input.device))
        if torch.is_grad_enabled():
            return self.backbone.forward_range(region_input, start, end), cache
        out, cache.structured = self.structured.forward(region_input, (start, end))
        return out, cache

    def parameters_for_region(self, region_index: int) -> list[nn.Parameter]:
        start, end = self.region_ranges[region_index]
        return [p for block in self.backbone.blocks[start:end] for p in block.parameters() if p.requires_grad]

    def named_parameters_for_region(self, region_index: int) -> list[tuple[str, nn.Parameter]]:
        start, end = self.region_ranges[region_index]
        out = []
        for idx in range(start, end):
            out.extend((f"backbone.blocks.{idx}.{n}", p) for n, p in self.backbone.blocks[idx].named_parameters() if p.requires_grad)
        return out

    def count_parameters(self) -> int:
        return int(sum(p.numel() for p in self.backbone.parameters()))

    def initialize_parameters(self, *, backbone_spec: BackboneSpec) -> None:
        init_transformer_module(self.backbone, n_layers=backbone_spec.layers, n_residuals_per_layer=2)

    def input_pullback_basis(self, *, cache: RegionForwardCache, output_cotangent_basis: torch.Tensor) -> torch.Tensor:
        return self.lowering.input_pullback_basis(backend=self, cache=cache, output_cotangent_basis=output_cotangent_basis)

    def parameter_vjp(self, *, cache: RegionForwardCache, output_cotangent: torch.Tensor) -> dict[str, torch.Tensor]:
        return self.lowering.parameter_vjp(backend=self, cache=cache, output_cotangent=output_cotangent)
