"""Generic region backend over any ``BackboneStack`` (Mamba-2, Mamba-3, hybrid).

Same role as the reference's ``backends/backbone_stack.py:12-82``, but the two derivative entry points
are implemented (there they raise NotImplementedError): the input pullback recomputes the region on a
basis-replicated batch and differentiates once, the parameter VJP differentiates a recomputed region.
"""
from __future__ import annotations

import torch
from torch import nn

from ..backbones.general import BackboneSpec, apply_backbone_init, build_backbone_stack
from .base import RegionForwardCache, autocast_as, current_autocast


class BackboneStackRegionBackend(nn.Module):
    """Region backend over any backbone stack (Mamba-2, Mamba-3, hybrid): regions are layer ranges of the stack."""

    name = "backbone_stack"

    def __init__(self, *, backbone_spec: BackboneSpec | None = None, region_ranges: list[tuple[int, int]],
                 backbone: nn.Module | None = None) -> None:
        super().__init__()
        if backbone is None:
            if backbone_spec is None:
                raise ValueError("backbone_spec is required when backbone is not provided")
            backbone = build_backbone_stack(backbone_spec)
        self.backbone_spec = backbone_spec
        self.region_ranges = [tuple(r) for r in region_ranges]
        if not self.region_ranges:
            raise ValueError("region backend requires at least one region")
        self.backbone = backbone
        self._structured = None

    def _region_range(self, region_index: int) -> tuple[int, int]:
        try:
            return self.region_ranges[region_index]
        except IndexError as exc:
            raise IndexError(f"region_index {region_index} out of range for {len(self.region_ranges)} regions") from exc

    @property
    def structured(self):
        """Closed-form lowering of the stack (forward with caches, basis pullback, parameter VJP without autograd); built
        on first use.  Raises NotImplementedError for a block type that has none."""
        if self._structured is None:
            from .mamba_structured import StructuredMambaRegion

            object.__setattr__(self, "_structured", StructuredMambaRegion(self.backbone.blocks))
        return self._structured

    @property
    def blocks(self) -> nn.ModuleList:
        return self.backbone.blocks

    def forward_region(self, *, region_input: torch.Tensor, region_index: int):
        start, end = self._region_range(region_index)
        out = self.backbone.forward_range(region_input, start, end)
        return out, RegionForwardCache(region_index=region_index, layer_range=(start, end), region_input=region_input,
                                       autocast=current_autocast(region_input.device))

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
        apply_backbone_init(self.backbone, backbone_spec, blocks=self.backbone.blocks)

    def input_pullback_basis(self, *, cache: RegionForwardCache, output_cotangent_basis: torch.Tensor) -> torch.Tensor:
        """output_cotangent_basis [B, P, T, D] -> region-input cotangents [B, P, T, D]."""
        if cache.region_input is None:
            raise ValueError("cache has no region_input to recompute from")
        bsz, nbasis = output_cotangent_basis.shape[:2]
        x = cache.region_input.detach()
        rep = x.unsqueeze(1).expand(bsz, nbasis, *x.shape[1:]).reshape(bsz * nbasis, *x.shape[1:]).clone().requires_grad_(True)
        start, end = cache.layer_range
        with torch.enable_grad(), autocast_as(cache.autocast):
            out = self.backbone.forward_range(rep, start, end)
        (g,) = torch.autograd.grad(out, rep, output_cotangent_basis.reshape(bsz * nbasis, *x.shape[1:]).to(out.dtype))
        return g.reshape(bsz, nbasis, *x.shape[1:])

    def parameter_vjp(self, *, cache: RegionForwardCache, output_cotangent: torch.Tensor) -> dict[str, torch.Tensor]:
        if cache.region_input is None:
            raise ValueError("cache has no region_input to recompute from")
        named = self.named_parameters_for_region(cache.region_index)
        start, end = cache.layer_range
        with torch.enable_grad(), autocast_as(cache.autocast):
            out = self.backbone.forward_range(cache.region_input.detach(), start, end)
        grads = torch.autograd.grad(out, [p for _, p in named], output_cotangent.to(out.dtype), allow_unused=True)
        return {name: g for (name, _), g in zip(named, grads) if g is not None}
