"""Dense baseline: canvas -> full backbone -> readout (reference models/dense_language_model.py:11-47).

``self.blocks`` aliases ``self.backbone.blocks`` as in the reference, so a state dict carries both
``backbone.blocks.*`` and ``blocks.*`` keys and reference checkpoints load with ``strict=True``.
"""
from __future__ import annotations

import torch
from torch import nn

from ..backbones.general import BackboneSpec, apply_backbone_init, build_backbone_stack, init_transformer_module, make_final_norm
from ..canvas import TokenEmbeddingCanvas
from ..readouts import NormLMHeadReadout


class DenseLanguageModel(nn.Module):
    """canvas -> the whole backbone -> readout: the baseline without regions or interface."""

    def __init__(self, *, vocab_size: int, backbone_spec: BackboneSpec, tie_embeddings: bool = False) -> None:
        super().__init__()
        backbone_spec.validate()
        self.vocab_size = int(vocab_size)
        self.backbone_spec = backbone_spec
        self.tie_embeddings = bool(tie_embeddings)
        self.canvas = TokenEmbeddingCanvas(vocab_size=self.vocab_size, feature_dim=backbone_spec.dim)
        self.backbone = build_backbone_stack(backbone_spec)
        self.blocks = self.backbone.blocks
        self.readout = NormLMHeadReadout(
            norm=make_final_norm(backbone_spec), feature_dim=backbone_spec.dim, vocab_size=self.vocab_size, tie_embeddings=self.tie_embeddings
        )
        if backbone_spec.name in ("transformer", "hybrid"):
            init_transformer_module(self.canvas, n_layers=backbone_spec.layers)
            apply_backbone_init(self.backbone, backbone_spec, blocks=self.blocks)
            init_transformer_module(self.readout, n_layers=backbone_spec.layers)
        if self.tie_embeddings:
            nn.init.normal_(self.canvas.embedding.weight, std=0.02)

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        return self.readout(self.backbone(self.canvas(input_ids)), canvas=self.canvas)
