"""Minimal HTTP front end for ``inference.generate``:  python -m lbi_b200.serve RUN_DIR [--host 127.0.0.1] [--port 8000]

``POST /generate`` with ``{"prompt": "text"}`` or ``{"prompt_ids": [1, 2, 3]}`` and optional ``max_new_tokens``, ``temperature``,
``top_k``, ``seed``, ``total_len`` returns ``{"prompt_ids", "new_ids", "text"}``; ``GET /health`` reports the model.  Requests are
served one at a time (one model, one device); the request logic is ``GenerationService.handle`` and works without the web stack.
"""
from __future__ import annotations

import threading
from typing import Any

import torch

from .inference import generate, load_run, load_run_tokenizer


class GenerationService:
    """One loaded run (model, config, tokenizer) behind a lock; ``handle(request)`` validates, generates and decodes."""

    def __init__(self, model: Any, cfg: Any, tokenizer: Any = None, *, max_new_tokens_limit: int = 1024) -> None:
        self.model, self.cfg, self.tokenizer = model, cfg, tokenizer
        self.limit = int(max_new_tokens_limit)
        self._lock = threading.Lock()

    @classmethod
    def from_run(cls, run_dir, *, checkpoint: str = "latest", device: str = "auto", **kw) -> "GenerationService":
        model, cfg = load_run(run_dir, checkpoint=checkpoint, device=device)
        return cls(model, cfg, load_run_tokenizer(cfg), **kw)

    def health(self) -> dict:
        return {"status": "ok", "model": type(self.model).__name__, "backbone": self.cfg.backbone, "seq_len": int(self.cfg.seq_len),
                "vocab_size": int(self.cfg.vocab_size), "region_axis": getattr(self.model, "region_axis", None),
                "device": str(next(self.model.parameters()).device)}

    def _encode(self, request: dict) -> list[int]:
        if request.get("prompt_ids"):
            ids = [int(i) for i in request["prompt_ids"]]
        elif not request.get("prompt"):
            raise ValueError("give prompt or prompt_ids")
        elif self.tokenizer is not None:
            ids = self.tokenizer.encode_bytes(str(request["prompt"]).encode("utf-8"))
        elif self.cfg.data_mode == "text_byte":
            ids = list(str(request["prompt"]).encode("utf-8"))
        else:
            raise ValueError("this run has no tokenizer: send prompt_ids")
        if not ids or any(i < 0 or i >= int(self.cfg.vocab_size) for i in ids):
            raise ValueError("prompt ids must be non-empty and inside the vocabulary")
        return ids

    def _decode(self, ids: list[int]) -> str | None:
        if self.tokenizer is not None and hasattr(self.tokenizer, "decode"):
            return self.tokenizer.decode(ids).decode("utf-8", errors="replace")
        if self.cfg.data_mode == "text_byte":
            return bytes(i % 256 for i in ids).decode("utf-8", errors="replace")
        return None

    def handle(self, request: dict) -> dict:
        """One generation request -> response dict; raises ValueError for a malformed request."""
        ids = self._encode(request)
        new = int(request.get("max_new_tokens", 32))
        if new <= 0 or new > self.limit:
            raise ValueError(f"max_new_tokens must be in 1..{self.limit}")
        temperature = float(request.get("temperature", 0.0))
        top_k = int(request.get("top_k", 0)) or None
        device = next(self.model.parameters()).device
        prompt = torch.tensor([ids], dtype=torch.long, device=device)
        total = int(request.get("total_len", 0)) or max(int(self.cfg.seq_len), prompt.shape[1] + new)
        gen = torch.Generator(device=device).manual_seed(int(request.get("seed", 0))) if temperature > 0 else None
        with self._lock:
            out = generate(self.model, prompt, new, total_len=total, temperature=temperature, top_k=top_k, generator=gen)
        new_ids = out[0, prompt.shape[1]:].tolist()
        return {"prompt_ids": ids, "new_ids": new_ids, "text": self._decode(new_ids)}


def build_app(service: GenerationService):
    """The FastAPI application around a service (imported here so that the module loads without the web stack)."""
    from fastapi import FastAPI, HTTPException

    app = FastAPI(title="lbi_b200 generation")

    @app.get("/health")
    def health() -> dict:
        return service.health()

    @app.post("/generate")
    def run(request: dict) -> dict:
        try:
            return service.handle(request)
        except ValueError as exc:
            raise HTTPException(status_code=400, detail=str(exc)) from exc

    return app


def main(argv: list[str] | None = None) -> None:
    import argparse

    p = argparse.ArgumentParser(description="Serve a trained run over HTTP.")
    p.add_argument("run_dir", type=str, help="<output dir>/<run name>/<dense|lbi>")
    p.add_argument("--host", type=str, default="127.0.0.1")
    p.add_argument("--port", type=int, default=8000)
    p.add_argument("--checkpoint", choices=("best", "latest"), default="latest")
    p.add_argument("--device", choices=("auto", "cpu", "cuda"), default="auto")
    p.add_argument("--max-new-tokens-limit", type=int, default=1024)
    ns = p.parse_args(argv)
    import uvicorn

    service = GenerationService.from_run(ns.run_dir, checkpoint=ns.checkpoint, device=ns.device,
                                         max_new_tokens_limit=ns.max_new_tokens_limit)
    uvicorn.run(build_app(service), host=ns.host, port=ns.port)


if __name__ == "__main__":
    main()
