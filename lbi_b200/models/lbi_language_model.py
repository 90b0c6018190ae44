"""Language model composed of canvas, interface, region backend and readout.

Module names (``canvas``, ``region_backend``, ``readout``, ``interface``) and the cache dictionary follow the
reference's ``models/lbi_language_model.py:57-225``.  Additions: a ``RegionPlan`` that also supports
sequence-axis regions, and ``detach_states=True`` which cuts the autograd graph at every interface state so
each region's graph is local (what region-parallel execution needs).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
from torch import nn

from ..backbones.general import BackboneSpec, init_transformer_module, make_final_norm
from ..backends import BackboneStackRegionBackend, RegionForwardCache, TransformerRegionBackend
from ..backends.base import current_autocast
from ..canvas import TokenEmbeddingCanvas
from ..interfaces import InterfaceModule, InterfaceStep
from ..readouts import NormLMHeadReadout
from .region_plan import RegionPlan, build_region_ranges  # noqa: F401  (importable from here as in the reference)

_VALID_STATE_ABLATIONS = {"none", "zero_all", "noise", "mask"}


@dataclass
class LBIRegionCache:
    """One region of a forward pass: ranges, backend cache, canvas features, incoming state, condition, input, output, interface step."""

    region_index: int
    layer_range: tuple[int, int]
    token_range: tuple[int, int]
    backend_cache: RegionForwardCache
    canvas_features: torch.Tensor
    state_in: torch.Tensor
    condition: torch.Tensor
    region_input: torch.Tensor
    region_output: torch.Tensor
    interface_step: InterfaceStep
    state_out: torch.Tensor


@dataclass
class LBICache:
    """Typed view of the dictionary ``forward_with_cache`` returns."""

    canvas_features: torch.Tensor
    states: list[torch.Tensor]
    region_inputs: list[torch.Tensor]
    region_outputs: list[torch.Tensor]
    region_ranges: list[tuple[int, int]]
    region_caches: list[LBIRegionCache]


class LBILanguageModel(nn.Module):
    """canvas -> interface.initialize -> for every region: decode the state into a condition, run the region backend on
    canvas + condition, update the state from the region output -> readout.  Regions are layer ranges (``region_axis="depth"``, the
    reference's cut) or token spans through the whole stack (``"sequence"``); ``forward_with_cache`` returns the states, region
    inputs / outputs and per-region caches the backward engines work from."""

    def __init__(
        self,
        *,
        vocab_size: int,
        layers_per_region: int,
        backbone_spec: BackboneSpec,
        interface: InterfaceModule,
        tie_embeddings: bool = False,
        region_axis: str = "depth",
        num_sequence_regions: int = 0,
    ) -> None:
        super().__init__()
        backbone_spec.validate()
        if interface.spec.region_condition_dim != backbone_spec.dim:
            raise ValueError(
                "interface region_condition_dim must match backbone hidden dimension "
                f"({interface.spec.region_condition_dim} != {backbone_spec.dim})"
            )
        if region_axis not in ("depth", "sequence"):
            raise ValueError("region_axis must be 'depth' or 'sequence'")
        self.hidden_dim = backbone_spec.dim
        self.layers = backbone_spec.layers
        self.vocab_size = int(vocab_size)
        self.interface_width = interface.spec.state_flat_dim
        self.tie_embeddings = bool(tie_embeddings)
        self.backbone_spec = backbone_spec
        if region_axis == "depth":
            self.plan = RegionPlan.depth(backbone_spec.layers, layers_per_region)
        else:
            self.plan = RegionPlan.sequence(backbone_spec.layers, num_sequence_regions)
        self.region_axis = region_axis
        self.region_ranges = [tuple(r) for r in self.plan.layer_ranges]
        self.num_regions = self.plan.num_regions
        interface.validate_region_count(self.num_regions)

        self.canvas = TokenEmbeddingCanvas(vocab_size=vocab_size, feature_dim=self.hidden_dim)
        backend_cls = TransformerRegionBackend if backbone_spec.name == "transformer" else BackboneStackRegionBackend
        self.region_backend = backend_cls(backbone_spec=backbone_spec, region_ranges=self.region_ranges)
        self.readout = NormLMHeadReadout(
            norm=make_final_norm(backbone_spec), feature_dim=self.hidden_dim, vocab_size=vocab_size, tie_embeddings=self.tie_embeddings
        )
        self.interface = interface

        if backbone_spec.name in {"transformer", "hybrid"}:
            init_transformer_module(self.canvas, n_layers=backbone_spec.layers, n_residuals_per_layer=2)
            self.region_backend.initialize_parameters(backbone_spec=backbone_spec)
            init_transformer_module(self.readout, n_layers=backbone_spec.layers, n_residuals_per_layer=2)
        if self.tie_embeddings:
            nn.init.normal_(self.canvas.embedding.weight, std=0.02)

    # ---- parameter groupings used by the local-VJP engines
    def output_head_vjp_parameters(self) -> list[nn.Parameter]:
        return self.readout.vjp_parameters()

    def canvas_vjp_parameters(self) -> list[nn.Parameter]:
        return self.canvas.vjp_parameters()

    def shared_local_vjp_parameters(self) -> list[nn.Parameter]:
        return [*self.canvas_vjp_parameters(), *self.interface.shared_vjp_parameters()]

    def _apply_state_ablation(self, state, *, mode, noise_std, mask_keep_prob, generator):
        if mode not in _VALID_STATE_ABLATIONS:
            raise ValueError(f"unsupported state ablation mode: {mode}")
        if mode == "none":
            return state
        if mode == "zero_all":
            return torch.zeros_like(state)
        if mode == "noise":
            if noise_std < 0.0:
                raise ValueError("message_noise_std must be >= 0")
            if noise_std == 0.0:
                return state
            return state + noise_std * torch.randn(state.shape, device=state.device, dtype=state.dtype, generator=generator)
        if mask_keep_prob <= 0.0 or mask_keep_prob > 1.0:
            raise ValueError("message_mask_keep_prob must be in (0, 1]")
        if mask_keep_prob == 1.0:
            return state
        keep = torch.rand(state.shape, device=state.device, generator=generator) < mask_keep_prob
        return state * keep.to(dtype=state.dtype)

    def forward_with_cache(
        self,
        input_ids: torch.Tensor,
        *,
        message_ablation: str = "none",
        message_noise_std: float = 1.0,
        message_mask_keep_prob: float = 0.5,
        ablation_generator: torch.Generator | None = None,
        detach_states: bool = False,
    ) -> tuple[torch.Tensor, dict[str, Any]]:
        ablate = dict(mode=message_ablation, noise_std=message_noise_std, mask_keep_prob=message_mask_keep_prob,
                      generator=ablation_generator)
        sequence_axis = self.region_axis == "sequence"
        canvas_features = self.canvas(input_ids)
        token_ranges = self.plan.token_ranges(input_ids.shape[1])
        initial_state = self.interface.initialize(canvas_features, causal=True) if sequence_axis else self.interface.initialize(canvas_features)
        state = self._apply_state_ablation(initial_state, **ablate)
        states, state_inputs = [state], []
        region_inputs, region_outputs, region_caches, region_logits = [], [], [], []

        for k, (start, end) in enumerate(self.region_ranges):
            t0, t1 = token_ranges[k]
            state_in = state.detach().requires_grad_(True) if (detach_states and torch.is_grad_enabled()) else state
            state_inputs.append(state_in)
            condition = self.interface.decode(state_in, k)
            region_canvas = canvas_features[:, t0:t1] if sequence_axis else canvas_features
            region_input = region_canvas + condition.unsqueeze(1)
            region_output, backend_cache = self.region_backend.forward_region(region_input=region_input, region_index=k)
            step = self.interface.update(state_in, region_output, k)
            state = self._apply_state_ablation(step.state, **ablate)
            states.append(state)
            region_inputs.append(region_input)
            region_outputs.append(region_output)
            if sequence_axis:
                region_logits.append(self.readout(region_output, canvas=self.canvas))
            region_caches.append(
                LBIRegionCache(
                    region_index=k, layer_range=(start, end), token_range=(t0, t1), backend_cache=backend_cache,
                    canvas_features=region_canvas, state_in=state_in, condition=condition, region_input=region_input,
                    region_output=region_output, interface_step=step, state_out=state,
                )
            )

        if sequence_axis:
            logits = torch.cat(region_logits, dim=1)
        else:
            logits = self.readout(region_outputs[-1], canvas=self.canvas)
        return logits, {
            "canvas_features": canvas_features,
            "states": states,
            "state_inputs": state_inputs,
            "initial_state": initial_state,
            "region_inputs": region_inputs,
            "region_outputs": region_outputs,
            "region_ranges": self.region_ranges,
            "token_ranges": token_ranges,
            "region_caches": region_caches,
            "detached_states": bool(detach_states and torch.is_grad_enabled()),
            "region_axis": self.region_axis,
            "autocast": current_autocast(canvas_features.device),
        }

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        return self.forward_with_cache(input_ids)[0]
