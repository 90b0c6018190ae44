"""Autoregressive decoding for the language models of this package (the reference has no inference path).

A model cut into regions along the sequence only ever needs the tokens of the region it is in plus the bounded interface state
that summarises everything before it, so decoding keeps one region span of activations alive however long the text: the
finished regions are dropped once their state update has been taken.  ``IncrementalLBIDecoder`` does exactly that: it
re-evaluates the current span's prefix through the stack for every new token (cost proportional to the span, not to the
sequence) and moves the state forward at span boundaries.  The spans are those of a sequence of ``total_len`` tokens, fixed
up front, because the cut of the training forward depends on the sequence length.

Depth-axis LBI models and dense models have no such shortcut (the depth-axis initial state pools the whole sequence):
``generate`` re-runs their forward on the growing sequence.
"""
from __future__ import annotations

from typing import Any

import torch


def _sample(logits: torch.Tensor, temperature: float, top_k: int | None, generator: torch.Generator | None) -> torch.Tensor:
    """logits [B, V] -> token ids [B]: arg-max at temperature 0, else a draw from the (top-k) softmax."""
    if temperature <= 0.0:
        return logits.argmax(dim=-1)
    logits = logits.float() / temperature
    if top_k is not None and 0 < top_k < logits.shape[-1]:
        kth = torch.topk(logits, top_k, dim=-1).values[..., -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    return torch.multinomial(torch.softmax(logits, dim=-1), 1, generator=generator).squeeze(-1)


class IncrementalLBIDecoder:
    """Token-by-token evaluation of a sequence-axis ``LBILanguageModel`` that agrees with its full forward on ``total_len`` tokens.

    ``append(tokens [B, n])`` consumes the next n tokens and returns their logits [B, n, V]; ``position`` tokens have been
    consumed so far.  Memory: one interface state plus, for the current span only, either its token ids (recompute mode) or the
    per-block decode states (cache mode: key / value cache of the span, convolution windows, scan states)."""

    def __init__(self, model: Any, total_len: int, use_cache: bool | None = None) -> None:
        """``use_cache``: keep per-block decode state (key / value cache, convolution window, scan state) for the current span
        so that a token costs one step per block instead of a pass over the span prefix; None turns it on when every block
        of the stack has a ``decode_step``."""
        if getattr(model, "region_axis", "depth") != "sequence":
            raise ValueError("incremental decoding needs regions cut along the sequence (region_axis='sequence')")
        self.model = model
        self.spans = model.plan.token_ranges(int(total_len))
        self.total_len = int(total_len)
        self.position = 0
        self.region = 0
        self.state: torch.Tensor | None = None
        self._span_tokens: torch.Tensor | None = None
        blocks = getattr(model.region_backend.backbone, "blocks", [])
        from .backbones.general import ResidualBackboneStack

        cacheable = (isinstance(model.region_backend.backbone, ResidualBackboneStack) and len(blocks) > 0
                     and all(hasattr(b, "decode_step") for b in blocks))
        if use_cache and not cacheable:
            raise ValueError("use_cache needs a residual stack whose blocks all implement decode_step")
        self.use_cache = cacheable if use_cache is None else bool(use_cache)
        self._block_states: list | None = None
        self._feature_sum: torch.Tensor | None = None

    def _cached_token_features(self, tok: torch.Tensor) -> torch.Tensor:
        """Region output [B, D] of the next token of the current span, one decode step per block."""
        model, k = self.model, self.region
        start, end = model.region_ranges[k]
        canvas = model.canvas(tok)  # [B, 1, D]
        if self.state is None:
            self.state = model.interface.initialize(canvas, causal=True)
        blocks = model.region_backend.backbone.blocks
        if self._block_states is None:
            span = self.spans[k][1] - self.spans[k][0]
            self._block_states = [blocks[i].allocate_decode_state(tok.shape[0], span, device=canvas.device, dtype=canvas.dtype)
                                  for i in range(start, end)]
        branch, stream = canvas[:, 0] + model.interface.decode(self.state, k), None
        for i, st in zip(range(start, end), self._block_states):
            branch, stream = blocks[i].decode_step(branch, stream, st)
        features = branch if stream is None else branch + stream
        self._feature_sum = features.float() if self._feature_sum is None else self._feature_sum + features.float()
        return features

    def _region_features(self, tokens: torch.Tensor) -> torch.Tensor:
        """Region output for the span prefix ``tokens`` [B, n] under the current state."""
        model, k = self.model, self.region
        start, end = model.region_ranges[k]
        canvas = model.canvas(tokens)
        if self.state is None:
            self.state = model.interface.initialize(canvas, causal=True)
        region_input = canvas + model.interface.decode(self.state, k).unsqueeze(1)
        return model.region_backend.backbone.forward_range(region_input, start, end)

    @torch.no_grad()
    def append(self, tokens: torch.Tensor) -> torch.Tensor:
        if tokens.dim() != 2:
            raise ValueError("tokens must have shape [B, n]")
        if self.position + tokens.shape[1] > self.total_len:
            raise ValueError(f"the decoder was laid out for {self.total_len} tokens")
        out = []
        t = 0
        while t < tokens.shape[1]:
            start_tok, end_tok = self.spans[self.region]
            span = end_tok - start_tok
            if self.position == start_tok and tokens.shape[1] - t >= span:
                # a whole span at once (prompt processing): one pass as in training, then only the state is kept
                features = self._region_features(tokens[:, t : t + span])
                out.append(self.model.readout(features, canvas=self.model.canvas))
                self.state = self.model.interface.update(self.state, features, self.region).state
                self.position, self.region, t = end_tok, self.region + 1, t + span
                continue
            tok = tokens[:, t : t + 1]
            t += 1
            if self.use_cache:
                last = self._cached_token_features(tok).unsqueeze(1)
            else:
                self._span_tokens = tok if self._span_tokens is None else torch.cat([self._span_tokens, tok], dim=1)
                features = self._region_features(self._span_tokens)
                last = features[:, -1:]
            out.append(self.model.readout(last, canvas=self.model.canvas))
            self.position += 1
            if self.position == end_tok:  # span complete: take the state update, forget the span
                if self.use_cache:
                    pooled = (self._feature_sum / float(end_tok - start_tok)).to(last.dtype)
                    self.state = self.model.interface.update_from_pooled(self.state, pooled, self.region).state
                    self._block_states, self._feature_sum = None, None
                else:
                    self.state = self.model.interface.update(self.state, features, self.region).state
                    self._span_tokens = None
                self.region += 1
        return torch.cat(out, dim=1)


@torch.no_grad()
def generate(model: Any, input_ids: torch.Tensor, max_new_tokens: int, *, total_len: int | None = None, temperature: float = 0.0,
             top_k: int | None = None, generator: torch.Generator | None = None, use_cache: bool | None = None) -> torch.Tensor:
    """Continue ``input_ids`` [B, T0] by ``max_new_tokens`` tokens -> [B, T0 + max_new_tokens].

    Sequence-axis LBI models decode incrementally under the region spans of a ``total_len``-token sequence (default: the final
    length; pass the training sequence length to decode under the cut the model was trained with).  Every other model re-runs
    its forward on the sequence so far."""
    if input_ids.dim() != 2 or input_ids.shape[1] == 0:
        raise ValueError("input_ids must be a non-empty [B, T] tensor")
    was_training = model.training
    model.eval()
    try:
        final_len = input_ids.shape[1] + int(max_new_tokens)
        tokens = input_ids
        if getattr(model, "region_axis", None) == "sequence":
            decoder = IncrementalLBIDecoder(model, final_len if total_len is None else int(total_len), use_cache=use_cache)
            if final_len > decoder.total_len:
                raise ValueError("total_len is shorter than the prompt plus the new tokens")
            logits = decoder.append(tokens)[:, -1]
            for i in range(int(max_new_tokens)):
                nxt = _sample(logits, temperature, top_k, generator).unsqueeze(1)
                tokens = torch.cat([tokens, nxt], dim=1)
                if i + 1 < int(max_new_tokens):
                    logits = decoder.append(nxt)[:, -1]
            return tokens
        for _ in range(int(max_new_tokens)):
            out = model(tokens)
            nxt = _sample(out[:, -1], temperature, top_k, generator).unsqueeze(1)
            tokens = torch.cat([tokens, nxt], dim=1)
        return tokens
    finally:
        model.train(was_training)


__all__ = ["IncrementalLBIDecoder", "generate"]
