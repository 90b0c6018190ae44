"""Autoregressive decoding for the language models of this package (the reference has no inference path).

A model cut into regions along the sequence only ever needs the tokens of the region it is in plus the bounded interface state
that summarises everything before it, so decoding keeps one region span of activations alive however long the text: the
finished regions are dropped once their state update has been taken.  ``IncrementalLBIDecoder`` does exactly that: it
re-evaluates the current span's prefix through the stack for every new token (cost proportional to the span, not to the
sequence) and moves the state forward at span boundaries.  The spans are those of a sequence of ``total_len`` tokens, fixed
up front, because the cut of the training forward depends on the sequence length.

Dense models decode with the same per-block caches held for the whole sequence (``IncrementalDenseDecoder``).  Depth-axis LBI
models have no shortcut (their initial state pools the whole sequence): ``generate`` re-runs their forward on the growing
sequence.
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


class IncrementalDenseDecoder:
    """Token-by-token evaluation of a ``DenseLanguageModel`` with per-block decode state for up to ``max_len`` tokens (key / value
    caches grow with the sequence: there is no interface to bound them); ``append`` returns logits equal to the full forward."""

    def __init__(self, model: Any, max_len: int) -> None:
        from .backbones.general import ResidualBackboneStack

        blocks = getattr(getattr(model, "backbone", None), "blocks", None)
        if not isinstance(getattr(model, "backbone", None), ResidualBackboneStack) or not blocks or \
                not all(hasattr(b, "decode_step") for b in blocks):
            raise ValueError("cached dense decoding needs a residual stack whose blocks all implement decode_step")
        self.model, self.max_len, self.position = model, int(max_len), 0
        self._states: list | None = None

    @torch.no_grad()
    def append(self, tokens: torch.Tensor) -> torch.Tensor:
        if tokens.dim() != 2:
            raise ValueError("tokens must have shape [B, n]")
        if self.position + tokens.shape[1] > self.max_len:
            raise ValueError(f"the decoder was laid out for {self.max_len} tokens")
        model, out = self.model, []
        for t in range(tokens.shape[1]):
            canvas = model.canvas(tokens[:, t : t + 1])
            if self._states is None:
                self._states = [b.allocate_decode_state(tokens.shape[0], self.max_len, device=canvas.device, dtype=canvas.dtype)
                                for b in model.backbone.blocks]
            branch, stream = canvas[:, 0], None
            for block, state in zip(model.backbone.blocks, self._states):
                branch, stream = block.decode_step(branch, stream, state)
            features = branch if stream is None else branch + stream
            out.append(model.readout(features.unsqueeze(1), canvas=model.canvas))
            self.position += 1
        return torch.cat(out, dim=1)


@torch.no_grad()
def generate(model: Any, input_ids: torch.Tensor, max_new_tokens: int, *, total_len: int | None = None, temperature: float = 0.0,
             top_k: int | None = None, generator: torch.Generator | None = None, use_cache: bool | None = None) -> torch.Tensor:
    """Continue ``input_ids`` [B, T0] by ``max_new_tokens`` tokens -> [B, T0 + max_new_tokens].

    Sequence-axis LBI models decode incrementally under the region spans of a ``total_len``-token sequence (default: the final
    length; pass the training sequence length to decode under the cut the model was trained with).  Dense models decode with
    per-block caches over the whole sequence (``use_cache=False``: by re-running the forward); depth-axis LBI models always
    re-run their forward on the sequence so far."""
    if input_ids.dim() != 2 or input_ids.shape[1] == 0:
        raise ValueError("input_ids must be a non-empty [B, T] tensor")
    was_training = model.training
    model.eval()
    try:
        final_len = input_ids.shape[1] + int(max_new_tokens)
        tokens = input_ids
        if getattr(model, "region_axis", None) == "sequence":
            # a sequence cannot be cut into more spans than it has tokens: short requests use the cut of num_regions tokens
            layout = max(final_len, int(model.num_regions)) if total_len is None else int(total_len)
            decoder = IncrementalLBIDecoder(model, layout, use_cache=use_cache)
            if final_len > decoder.total_len:
                raise ValueError("total_len is shorter than the prompt plus the new tokens")
            logits = decoder.append(tokens)[:, -1]
            for i in range(int(max_new_tokens)):
                nxt = _sample(logits, temperature, top_k, generator).unsqueeze(1)
                tokens = torch.cat([tokens, nxt], dim=1)
                if i + 1 < int(max_new_tokens):
                    logits = decoder.append(nxt)[:, -1]
            return tokens
        dense = None
        if use_cache is not False and hasattr(model, "backbone") and hasattr(model, "readout") and not hasattr(model, "interface"):
            try:
                dense = IncrementalDenseDecoder(model, final_len)
            except ValueError:
                if use_cache:
                    raise
        if dense is not None:
            logits = dense.append(tokens)[:, -1]
            for i in range(int(max_new_tokens)):
                nxt = _sample(logits, temperature, top_k, generator).unsqueeze(1)
                tokens = torch.cat([tokens, nxt], dim=1)
                if i + 1 < int(max_new_tokens):
                    logits = dense.append(nxt)[:, -1]
            return tokens
        for _ in range(int(max_new_tokens)):
            out = model(tokens)
            nxt = _sample(out[:, -1], temperature, top_k, generator).unsqueeze(1)
            tokens = torch.cat([tokens, nxt], dim=1)
        return tokens
    finally:
        model.train(was_training)


def load_run(run_dir, *, checkpoint: str = "latest", device: str = "auto"):
    """(model in eval mode, config) of a trained run directory (``<output>/<run name>/<dense|lbi>``)."""
    from dataclasses import replace
    from pathlib import Path

    from .scripts.evaluate_paper_checkpoints import load_run_config
    from .train.checkpointing import checkpoint_path_from_summary, load_checkpoint, load_model_state
    from .train.config import normalize_model_variant
    from .train.model_builders import build_model_for_regime
    from .train.runners import _resolve_device

    run_dir = Path(run_dir)
    cfg = load_run_config(run_dir, eval_batches=1, batch_size=None, seq_len=None, device=device)
    dev = _resolve_device(cfg)
    path = checkpoint_path_from_summary(run_dir / "summary.json", preference=checkpoint)
    if path is None or not Path(path).exists():
        raise FileNotFoundError(f"no {checkpoint} checkpoint recorded for {run_dir}")
    payload = load_checkpoint(Path(path), device=dev)
    variant = normalize_model_variant(cfg.regime if cfg.regime not in ("", "all") else run_dir.name)
    model = build_model_for_regime(replace(cfg, variants=variant, regime=variant), checkpoint=payload).to(dev)
    load_model_state(model, payload["model_state_dict"])
    return model.eval(), cfg


def load_run_tokenizer(cfg):
    """The text tokenizer a run was trained with, or None for the synthetic and byte-level data modes."""
    if cfg.data_mode not in ("text_bpe", "text_bpe_sharded"):
        return None
    from .data.bpe_tokenizer import load_text_tokenizer
    from .train import data as glue

    train_path = glue._shard_train_path(cfg) if cfg.data_mode == "text_bpe_sharded" else glue.resolve_text_paths(cfg)[0]
    return load_text_tokenizer(tokenizer_type=cfg.tokenizer_type, tokenizer_path=glue.resolve_tokenizer_path(cfg, train_path=train_path),
                               train_path=train_path, vocab_size=cfg.vocab_size, train_bytes=cfg.tokenizer_train_bytes)


def main(argv: list[str] | None = None) -> dict:
    """python -m lbi_b200.inference RUN_DIR (--prompt TEXT | --prompt-ids 1,2,3) [--max-new-tokens N] ..."""
    import argparse
    import json

    p = argparse.ArgumentParser(description="Continue a prompt with a trained run.")
    p.add_argument("run_dir", type=str, help="<output dir>/<run name>/<dense|lbi>")
    p.add_argument("--prompt", type=str, default="", help="text (tokenized with the run's tokenizer; bytes in text_byte mode)")
    p.add_argument("--prompt-ids", type=str, default="", help="comma-separated token ids instead of text")
    p.add_argument("--max-new-tokens", type=int, default=32)
    p.add_argument("--total-len", type=int, default=0, help="sequence length whose region cut is used (default: the run's seq_len)")
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--checkpoint", choices=("best", "latest"), default="latest")
    p.add_argument("--device", choices=("auto", "cpu", "cuda"), default="auto")
    ns = p.parse_args(argv)
    model, cfg = load_run(ns.run_dir, checkpoint=ns.checkpoint, device=ns.device)
    tokenizer = load_run_tokenizer(cfg)
    if ns.prompt_ids:
        ids = [int(x) for x in ns.prompt_ids.split(",") if x.strip()]
    elif not ns.prompt:
        p.error("give --prompt or --prompt-ids")
    elif tokenizer is not None:
        ids = tokenizer.encode_bytes(ns.prompt.encode("utf-8"))
    elif cfg.data_mode == "text_byte":
        ids = list(ns.prompt.encode("utf-8"))
    else:
        p.error("a synthetic-data run has no tokenizer: use --prompt-ids")
    device = next(model.parameters()).device
    prompt = torch.tensor([ids], dtype=torch.long, device=device)
    total = ns.total_len or max(int(cfg.seq_len), prompt.shape[1] + ns.max_new_tokens)
    gen = torch.Generator(device=device).manual_seed(ns.seed) if ns.temperature > 0 else None
    out = generate(model, prompt, ns.max_new_tokens, total_len=total, temperature=ns.temperature, top_k=ns.top_k or None, generator=gen)
    new_ids = out[0, prompt.shape[1]:].tolist()
    result = {"prompt_ids": ids, "new_ids": new_ids}
    if tokenizer is not None and hasattr(tokenizer, "decode"):
        result["text"] = tokenizer.decode(new_ids).decode("utf-8", errors="replace")
    elif cfg.data_mode == "text_byte":
        result["text"] = bytes(i % 256 for i in new_ids).decode("utf-8", errors="replace")
    print(json.dumps(result))
    return result


__all__ = ["IncrementalDenseDecoder", "IncrementalLBIDecoder", "generate", "load_run", "load_run_tokenizer", "main"]


if __name__ == "__main__":
    main()
