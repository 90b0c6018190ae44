"""Loss and evaluation loops (reference train/eval.py:12-88)."""
from __future__ import annotations

from typing import Any

import torch
import torch.nn.functional as F
from torch import nn


def next_token_loss(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean cross-entropy in fp32 over all positions."""
    return F.cross_entropy(logits.float().reshape(-1, logits.size(-1)), targets.reshape(-1), reduction="mean")


def resolve_eval_message_ablation_modes(cfg: Any, *, ablation_modes: tuple[str, ...]) -> list[str]:
    if cfg.eval_all_message_ablations:
        return list(ablation_modes)
    return [] if cfg.eval_message_ablation == "none" else [cfg.eval_message_ablation]


def _evaluate(model: nn.Module, forward, *, cfg, val_corpus, eval_batches, generator, device, sample_batch_fn,
              autocast_context_fn) -> dict[str, float]:
    model.eval()
    total = 0.0
    with torch.no_grad():
        for _ in range(eval_batches):
            xb, yb = sample_batch_fn(cfg=cfg, corpus=val_corpus, batch_size=cfg.batch_size, generator=generator, device=device)
            with autocast_context_fn(cfg, device):
                logits = forward(xb)
            total += float(next_token_loss(logits, yb).item())
    return {"ce_loss": total / max(1, eval_batches)}


def evaluate_reference(*, cfg, model, val_corpus, eval_batches, generator, device, sample_batch_fn, autocast_context_fn):
    """Validation CE of a dense model."""
    return _evaluate(model, model, cfg=cfg, val_corpus=val_corpus, eval_batches=eval_batches, generator=generator,
                     device=device, sample_batch_fn=sample_batch_fn, autocast_context_fn=autocast_context_fn)


def evaluate_native(*, cfg, model, val_corpus, eval_batches, generator, device, sample_batch_fn, autocast_context_fn,
                    message_ablation: str = "none", ablation_generator: torch.Generator | None = None):
    """Validation CE of an LBI model, optionally with the interface state ablated (zero_all / noise / mask)."""

    def forward(xb):
        return model.forward_with_cache(
            xb, message_ablation=message_ablation, message_noise_std=cfg.message_noise_std,
            message_mask_keep_prob=cfg.message_mask_keep_prob, ablation_generator=ablation_generator,
        )[0]

    return _evaluate(model, forward, cfg=cfg, val_corpus=val_corpus, eval_batches=eval_batches, generator=generator,
                     device=device, sample_batch_fn=sample_batch_fn, autocast_context_fn=autocast_context_fn)
