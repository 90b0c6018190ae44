"""Transformer region backend with cached activations and pluggable derivative lowerings.

Counterpart of the reference's ``backends/transformer.py`` (backend :88-281, autograd lowering :283-355).
``forward_region`` runs the ordinary modules when autograd is recording (so ``loss.backward()`` and the
autograd-based engines work) and the closed-form ``StructuredTransformerRegion`` otherwise; the structured
cache is built lazily when a lowering needs it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Protocol

import torch
from torch import nn
from torch.nn import functional as F

from ..backbones.general import BackboneSpec, build_backbone_stack, init_transformer_module
from ..backbones.transformer.rope import apply_rope
from .base import RegionForwardCache, autocast_as, current_autocast
from .transformer_structured import StructuredTransformerRegion


# Named per-layer activation records with the reference's field names (backends/transformer.py:17-61).  The engine does not
# keep these (its kernels read the flat ``StructuredRegionCache``); ``TransformerRegionBackend.forward_region_with_layer_caches``
# fills them from the module code for inspection and for code written against the reference's cache.
@dataclass
class TransformerAttentionCache:
    """Attention intermediates of one layer (inspection view)."""

    norm_input: torch.Tensor
    norm_output: torch.Tensor
    qkv: torch.Tensor
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    q_rope: torch.Tensor
    k_rope: torch.Tensor
    k_expanded: torch.Tensor
    v_expanded: torch.Tensor
    attn_output: torch.Tensor
    out_proj_input: torch.Tensor
    out_proj_output: torch.Tensor


@dataclass
class TransformerMLPCache:
    """MLP intermediates of one layer (inspection view)."""

    norm_input: torch.Tensor
    norm_output: torch.Tensor
    fc1_output: torch.Tensor
    up: torch.Tensor
    gate: torch.Tensor
    activation: torch.Tensor
    down_input: torch.Tensor
    down_output: torch.Tensor


@dataclass
class TransformerLayerCache:
    """One layer of ``forward_region_with_layer_caches``: inputs, attention and MLP records, outputs."""

    layer_index: int
    hidden_input: torch.Tensor
    residual_input: torch.Tensor | None
    attention: TransformerAttentionCache
    mlp: TransformerMLPCache
    hidden_output: torch.Tensor
    residual_output: torch.Tensor | None


@dataclass
class TransformerRegionCache(RegionForwardCache):
    """A region forward with the per-layer records attached."""

    layer_caches: list[TransformerLayerCache] = field(default_factory=list)
    region_output: torch.Tensor | None = None


class TransformerLowering(Protocol):
    """How a Transformer region is differentiated: ``input_pullback_basis`` and ``parameter_vjp`` given the backend and a cache."""

    name: str

    def input_pullback_basis(self, *, backend: "TransformerRegionBackend", cache: RegionForwardCache,
                             output_cotangent_basis: torch.Tensor) -> torch.Tensor: ...

    def parameter_vjp(self, *, backend: "TransformerRegionBackend", cache: RegionForwardCache,
                      output_cotangent: torch.Tensor) -> dict[str, torch.Tensor]: ...


class TorchAutogradTransformerLowering:
    """Oracle lowering: recompute the region on a basis-replicated batch and differentiate with autograd."""

    name = "torch_autograd"

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

    name = "structured"

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
    """Region backend of the Transformer stack: module forward while autograd records, the structured kernels otherwise;
    derivatives through a pluggable lowering (structured by default, autograd as the oracle)."""

    name = "transformer"

    def __init__(self, *, backbone_spec: BackboneSpec | None = None, region_ranges: list[tuple[int, int]],
                 backbone: nn.Module | None = None, lowering: TransformerLowering | None = None) -> None:
        super().__init__()
        if backbone is None:
            if backbone_spec is None:
                raise ValueError("backbone_spec is required when backbone is not provided")
            if backbone_spec.name != "transformer":
                raise ValueError("TransformerRegionBackend requires a transformer backbone spec")
            backbone = build_backbone_stack(backbone_spec)
        self.backbone_spec = backbone_spec
        self.region_ranges = [tuple(r) for r in region_ranges]
        if not self.region_ranges:
            raise ValueError("transformer region backend requires at least one region")
        self.backbone = backbone
        self.lowering: TransformerLowering = lowering or StructuredTransformerLowering()
        object.__setattr__(self, "structured", StructuredTransformerRegion(self.backbone.blocks))

    @property
    def blocks(self) -> nn.ModuleList:
        return self.backbone.blocks

    def forward_region(self, *, region_input: torch.Tensor, region_index: int):
        start, end = self._region_range(region_index)
        cache = RegionForwardCache(region_index=region_index, layer_range=(start, end), region_input=region_input,
                                   autocast=current_autocast(region_input.device))
        if torch.is_grad_enabled():
            return self.backbone.forward_range(region_input, start, end), cache
        out, cache.structured = self.structured.forward(region_input, (start, end))
        return out, cache

    def _region_range(self, region_index: int) -> tuple[int, int]:
        try:
            return self.region_ranges[region_index]
        except IndexError as exc:
            raise IndexError(f"region_index {region_index} out of range for {len(self.region_ranges)} regions") from exc

    @staticmethod
    def _attention_with_cache(attn: nn.Module, normed: torch.Tensor, norm_input: torch.Tensor):
        bsz, seqlen, _ = normed.shape
        qkv = attn.in_proj(normed)
        if attn.d_conv > 0:
            qkv = attn.causal_conv(qkv)
        q, k, v = attn.split_heads(qkv)
        q_rope = apply_rope(q, base=attn.rope_base, interleaved=attn.rope_interleaved)
        k_rope = apply_rope(k, base=attn.rope_base, interleaved=attn.rope_interleaved)
        k_exp, v_exp = attn.expand_kv(k_rope), attn.expand_kv(v)
        heads = F.scaled_dot_product_attention(q_rope, k_exp, v_exp, dropout_p=0.0, is_causal=True,
                                               scale=attn.scale).transpose(1, 2)
        flat = heads.contiguous().view(bsz, seqlen, attn.out_dim)
        out = attn.out_proj(flat)
        return out, TransformerAttentionCache(
            norm_input=norm_input, norm_output=normed, qkv=qkv, q=q, k=k, v=v, q_rope=q_rope, k_rope=k_rope,
            k_expanded=k_exp, v_expanded=v_exp, attn_output=heads, out_proj_input=flat, out_proj_output=out)

    @staticmethod
    def _mlp_with_cache(mlp: nn.Module, normed: torch.Tensor, norm_input: torch.Tensor):
        fc1 = mlp.fc1(normed)
        up, gate = fc1.chunk(2, dim=-1)
        act = F.silu(gate)
        down_in = up * act
        out = mlp.fc2(down_in)
        return out, TransformerMLPCache(norm_input=norm_input, norm_output=normed, fc1_output=fc1, up=up, gate=gate,
                                        activation=act, down_input=down_in, down_output=out)

    # the three steps under the reference's method names and argument lists (backends/transformer.py:118-200)
    def _attention_forward_with_cache(self, attn: nn.Module, norm_output: torch.Tensor):
        return self._attention_with_cache(attn, norm_output, norm_output)

    def _mlp_forward_with_cache(self, mlp: nn.Module, norm_output: torch.Tensor):
        return self._mlp_with_cache(mlp, norm_output, norm_output)

    def _block_forward_with_cache(self, *, block: nn.Module, hidden_states: torch.Tensor, residual: torch.Tensor | None):
        """-> (mlp branch output, residual stream, attention cache, mlp cache) of one block."""
        stream1 = hidden_states if residual is None else hidden_states + residual
        normed1, residual = block.add_norm(hidden_states, residual, block.norm)
        attn_out, attn_cache = self._attention_with_cache(block.attn, normed1, stream1)
        stream2 = attn_out + residual
        normed2, residual = block.add_norm(attn_out, residual, block.norm2)
        out, mlp_cache = self._mlp_with_cache(block.mlp, normed2, stream2)
        return out, residual, attn_cache, mlp_cache

    def forward_region_with_layer_caches(self, *, region_input: torch.Tensor,
                                         region_index: int) -> tuple[torch.Tensor, TransformerRegionCache]:
        """The region through the module code, every intermediate kept under the reference's names
        (backends/transformer.py:201-237).  Not on the engine's path: one region of activations is held several times over."""
        start, end = self._region_range(region_index)
        hidden, residual = region_input, None
        layers: list[TransformerLayerCache] = []
        for idx in range(start, end):
            hidden_in, residual_in = hidden, residual
            hidden, residual, attn_cache, mlp_cache = self._block_forward_with_cache(block=self.backbone.blocks[idx],
                                                                                    hidden_states=hidden, residual=residual)
            layers.append(TransformerLayerCache(layer_index=idx, hidden_input=hidden_in, residual_input=residual_in,
                                                attention=attn_cache, mlp=mlp_cache, hidden_output=hidden,
                                                residual_output=residual))
        out = hidden if residual is None else hidden + residual
        return out, TransformerRegionCache(region_index=region_index, layer_range=(start, end), region_input=region_input,
                                           autocast=current_autocast(region_input.device), layer_caches=layers,
                                           region_output=out)

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
