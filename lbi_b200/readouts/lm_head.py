"""Final norm followed by the LM head, tied to the canvas embedding or owning ``lm_head`` (no bias).

Same contract and key names as the reference's ``readouts/lm_head.py:11-68``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from .base import ReadoutCache


class NormLMHeadReadout(nn.Module):
    """Final norm, then the vocabulary projection with the canvas embedding (tied) or an own bias-free ``lm_head``."""

    def __init__(self, *, norm: nn.Module, feature_dim: int, vocab_size: int, tie_embeddings: bool = True) -> None:
        super().__init__()
        self.norm = norm
        self.feature_dim = int(feature_dim)
        self.vocab_size = int(vocab_size)
        self.tie_embeddings = bool(tie_embeddings)
        self.lm_head = None if self.tie_embeddings else nn.Linear(self.feature_dim, self.vocab_size, bias=False)

    def head_weight(self, canvas) -> torch.Tensor:
        if self.tie_embeddings:
            return canvas.output_weight()
        if self.lm_head is None:
            raise RuntimeError("untied readout is missing lm_head")
        return self.lm_head.weight

    def forward(self, features: torch.Tensor, *, canvas) -> torch.Tensor:
        return self.forward_with_cache(features, canvas=canvas)[0]

    def forward_with_cache(self, features: torch.Tensor, *, canvas) -> tuple[torch.Tensor, ReadoutCache]:
        normed = self.norm(features)
        weight = self.head_weight(canvas)
        logits = F.linear(normed.to(dtype=weight.dtype) if normed.dtype != weight.dtype else normed, weight)
        return logits, ReadoutCache(features=features, normed_features=normed, logits=logits)

    def vjp_parameters(self) -> list[nn.Parameter]:
        params = [p for p in self.norm.parameters() if p.requires_grad]
        if self.lm_head is not None:
            params.extend(p for p in self.lm_head.parameters() if p.requires_grad)
        return params

    def output_head_parameter_count(self) -> int:
        return 0 if self.lm_head is None else int(sum(p.numel() for p in self.lm_head.parameters()))
