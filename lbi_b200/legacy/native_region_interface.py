"""LBI-1 model: same computation as ``LBILanguageModel`` on depth regions, with the parameter names of the first
release so that its checkpoints load with ``strict=True`` (reference legacy/native_region_interface.py:92-292).

State-dict quirks kept on purpose: ``blocks`` aliases ``backbone.blocks`` (both prefixes are saved) and a tied model
still saves ``lm_head.weight`` (it is the embedding tensor)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
from torch import nn

from ..backbones.general import BackboneSpec, apply_backbone_init, build_backbone_stack, init_transformer_module, make_final_norm
from ..interfaces.vector_mlp import LegacyVectorMLPInterfaceView, VectorMLPHead
from ..models.region_plan import RegionPlan, build_region_ranges

RegionMessageHead = VectorMLPHead
build_region_slices = lambda layers, region_size: build_region_ranges(layers, region_size)  # noqa: E731


@dataclass
class RegionForwardCache:
    region_idx: int
    region_range: tuple[int, int]
    x_static: torch.Tensor
    message_in: torch.Tensor
    hidden_bias: torch.Tensor
    hidden_input: torch.Tensor
    hidden_output: torch.Tensor
    pooled_hidden: torch.Tensor
    delta_message: torch.Tensor
    alpha: torch.Tensor
    pre_norm_message: torch.Tensor
    message_out: torch.Tensor


class NativeRegionInterfaceModel(nn.Module):
    def __init__(self, *, vocab_size: int, region_size: int, message_dim: int, backbone_spec: BackboneSpec,
                 message_hidden_dim: int = 0, message_scale_init: float = 0.5, tie_embeddings: bool = False) -> None:
        super().__init__()
        backbone_spec.validate()
        self.dim, self.layers, self.message_dim = backbone_spec.dim, backbone_spec.layers, message_dim
        self.tie_embeddings = bool(tie_embeddings)
        self.plan = RegionPlan.depth(backbone_spec.layers, region_size)
        self.region_ranges = [tuple(r) for r in self.plan.layer_ranges]
        self.n_regions = self.num_regions = len(self.region_ranges)
        self.region_axis = "depth"
        self.embedding = nn.Embedding(vocab_size, self.dim)
        self.backbone = build_backbone_stack(backbone_spec)
        self.blocks = self.backbone.blocks
        self.norm = make_final_norm(backbone_spec)
        self.lm_head = nn.Linear(self.dim, vocab_size, bias=False)
        h = message_hidden_dim
        self.input_to_message = VectorMLPHead(self.dim, message_dim, hidden_dim=h)
        self.message_to_hidden = nn.ModuleList([VectorMLPHead(message_dim, self.dim, hidden_dim=h) for _ in range(self.n_regions)])
        self.hidden_to_message = nn.ModuleList([VectorMLPHead(self.dim, message_dim, hidden_dim=h) for _ in range(self.n_regions)])
        self.message_norm = nn.ModuleList([nn.LayerNorm(message_dim) for _ in range(self.n_regions)])
        self.message_alpha = nn.Parameter(torch.full((self.n_regions,), float(message_scale_init)))
        self.interface = LegacyVectorMLPInterfaceView(
            interface_width=message_dim, initial_encoder=self.input_to_message, decoders=self.message_to_hidden,
            encoders=self.hidden_to_message, norms=self.message_norm)
        object.__setattr__(self, "region_backend", self.backbone)  # engine hook only; must not add state-dict keys
        if backbone_spec.name in ("transformer", "hybrid"):
            init_transformer_module(self.embedding, n_layers=backbone_spec.layers)
            apply_backbone_init(self.backbone, backbone_spec, blocks=self.blocks)
            init_transformer_module(self.lm_head, n_layers=backbone_spec.layers)
        if self.tie_embeddings:
            nn.init.normal_(self.embedding.weight, std=0.02)
            self.lm_head.weight = self.embedding.weight

    # ---- hooks that let the shared scan engines drive this model
    def output_head_vjp_parameters(self) -> list[nn.Parameter]:
        params = list(self.norm.parameters())
        return params if self.tie_embeddings else [*params, self.lm_head.weight]

    def canvas_vjp_parameters(self) -> list[nn.Parameter]:
        return [self.embedding.weight]

    def shared_local_vjp_parameters(self) -> list[nn.Parameter]:
        return [self.embedding.weight, self.message_alpha]

    def _forward_region_message_map(self, ridx: int, x_static: torch.Tensor, m_in: torch.Tensor) -> torch.Tensor:
        """The local map m_k -> m_{k+1} of region ``ridx``."""
        start, end = self.region_ranges[ridx]
        x_out = self.backbone.forward_range(x_static + self.interface.decode(m_in, ridx).unsqueeze(1), start, end)
        return self.interface.update(x_out, m_in, ridx, self.message_alpha[ridx]).state

    @staticmethod
    def _ablate(m, mode, noise_std, keep_prob, generator):
        if mode == "none":
            return m
        if mode == "zero_all":
            return torch.zeros_like(m)
        if mode == "noise":
            if noise_std < 0.0:
                raise ValueError("message_noise_std must be >= 0")
            return m if noise_std == 0.0 else m + noise_std * torch.randn(m.shape, device=m.device, dtype=m.dtype, generator=generator)
        if mode == "mask":
            if keep_prob <= 0.0 or keep_prob > 1.0:
                raise ValueError("message_mask_keep_prob must be in (0, 1]")
            return m if keep_prob == 1.0 else m * (torch.rand(m.shape, device=m.device, generator=generator) < keep_prob).to(m.dtype)
        raise ValueError(f"unsupported message ablation mode: {mode}")

    def forward_with_cache(self, input_ids: torch.Tensor, *, message_ablation: str = "none", message_noise_std: float = 1.0,
                           message_mask_keep_prob: float = 0.5, ablation_generator: torch.Generator | None = None,
                           detach_states: bool = False) -> tuple[torch.Tensor, dict[str, Any]]:
        ab = (message_ablation, message_noise_std, message_mask_keep_prob, ablation_generator)
        x_static = self.embedding(input_ids)
        initial = self.interface.initial_state(x_static)
        m = self._ablate(initial, *ab)
        boundaries, hidden_inputs, messages, state_inputs, caches = [x_static], [], [m], [], []
        cut = detach_states and torch.is_grad_enabled()
        for ridx, (start, end) in enumerate(self.region_ranges):
            m_in = m.detach().requires_grad_(True) if cut else m
            state_inputs.append(m_in)
            bias = self.interface.decode(m_in, ridx)
            x_in = x_static + bias.unsqueeze(1)
            x_out = self.backbone.forward_range(x_in, start, end)
            upd = self.interface.update(x_out, m_in, ridx, self.message_alpha[ridx])
            m = self._ablate(upd.state, *ab)
            hidden_inputs.append(x_in)
            boundaries.append(x_out)
            messages.append(m)
            caches.append(RegionForwardCache(ridx, (start, end), x_static, m_in, bias, x_in, x_out, upd.pooled_region_output,
                                             upd.delta_state, upd.update_scale, upd.pre_norm_state, m))
        normed = self.norm(x_out)
        logits = self.lm_head(normed.to(self.lm_head.weight.dtype))
        return logits, {
            "boundaries": boundaries, "region_hidden_inputs": hidden_inputs, "region_messages": messages,
            "region_ranges": self.region_ranges, "region_caches": caches,
            # keys of the owned model's cache, so the shared engines work on this model too
            "states": messages, "state_inputs": state_inputs, "initial_state": initial, "detached_states": cut,
            "region_axis": "depth",
        }

    def forward(self, input_ids: torch.Tensor, **kwargs) -> torch.Tensor:
        return self.forward_with_cache(input_ids, **kwargs)[0]
