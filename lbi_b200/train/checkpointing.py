"""Single-file checkpoints in the reference's format, path resolution, resume / init semantics.

Payload keys (reference train/checkpointing.py:59-75): step, tokens_seen, best_val_ce_loss, best_val_step, config,
model_state_dict, optimizer_state_dict, torch_rng_state, cuda_rng_state_all, train_generator_state,
eval_generator_state, plus whatever the runner passes in ``extra``.  Files live under
``<run_dir>/checkpoints/{best,latest}.pt`` or below ``checkpoint_root``.  ``load_model_state`` also accepts LBI-1
state dicts (migrated on the fly) and drops the redundant ``readout.lm_head.weight`` of tied LBI-1 checkpoints.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any

import torch
from torch import nn

from .config import compatible_output_names_for_variant


def checkpoint_dir(run_dir: Path, cfg: Any) -> Path:
    if cfg.checkpoint_root:
        output_root = Path(cfg.output_dir).expanduser().resolve()
        root = Path(cfg.checkpoint_root).expanduser().resolve()
        try:
            relative = run_dir.resolve().relative_to(output_root.parent)
        except ValueError:
            relative = Path(run_dir.name)
        out = root / relative / "checkpoints"
    else:
        out = run_dir / "checkpoints"
    out.mkdir(parents=True, exist_ok=True)
    return out


def checkpoint_path_from_summary(summary_path: Path, *, preference: str) -> Path | None:
    """The checkpoint file a ``summary.json`` records (latest or best first, by ``preference``), if it still exists."""
    if not summary_path.exists():
        return None
    summary = json.loads(summary_path.read_text(encoding="utf-8"))
    order = ("latest_checkpoint_path", "best_checkpoint_path") if preference == "latest" else ("best_checkpoint_path", "latest_checkpoint_path")
    for key in order:
        candidate = str(summary.get(key, "")).strip()
        if candidate and Path(candidate).expanduser().exists():
            return Path(candidate).expanduser()
    return None


def save_checkpoint(*, run_dir: Path, filename: str, model: nn.Module, optimizer, cfg: Any, device: torch.device,
                    train_generator: torch.Generator, eval_generator: torch.Generator, step: int, tokens_seen: int,
                    best_val_ce_loss: float, best_val_step: int, extra: dict[str, Any] | None = None) -> Path:
    """Write one checkpoint file (payload keys in the module docstring) atomically; returns its path."""
    payload: dict[str, Any] = {
        "step": int(step),
        "tokens_seen": int(tokens_seen),
        "best_val_ce_loss": float(best_val_ce_loss),
        "best_val_step": int(best_val_step),
        "config": cfg.to_dict(),
        "model_state_dict": {k: v.detach().clone() for k, v in model.state_dict().items()},
        "optimizer_state_dict": optimizer.state_dict(),
        "torch_rng_state": torch.get_rng_state(),
        "cuda_rng_state_all": torch.cuda.get_rng_state_all() if device.type == "cuda" else None,
        "train_generator_state": train_generator.get_state(),
        "eval_generator_state": eval_generator.get_state(),
    }
    if extra:
        payload.update(extra)
    path = checkpoint_dir(run_dir, cfg) / filename
    tmp = path.with_suffix(path.suffix + ".tmp")
    torch.save(payload, tmp)
    tmp.replace(path)  # a reader never sees a half-written file
    return path


def load_checkpoint(path: Path, *, device: torch.device) -> dict[str, Any]:
    return torch.load(path, map_location=device, weights_only=False)


def resolve_checkpoint_path(load_from: str, *, regime: str, preference: str) -> Path | None:
    """Accepts a file, a run directory (has metrics.csv), an experiment root, or directories with a summary.json."""
    if not load_from:
        return None
    source = Path(load_from).expanduser()
    if not source.exists():
        raise FileNotFoundError(f"checkpoint source does not exist: {source}")
    if source.is_file():
        return source
    first, second = ("latest.pt", "best.pt") if preference == "latest" else ("best.pt", "latest.pt")
    is_run_dir = (source / "metrics.csv").exists()
    bases = [source] if is_run_dir else [*(source / name for name in compatible_output_names_for_variant(regime)), source]
    for base in bases:
        for name in (first, second):
            candidate = base / "checkpoints" / name
            if candidate.exists():
                return candidate
    for base in bases:
        hit = checkpoint_path_from_summary(base / "summary.json", preference=preference)
        if hit is not None:
            return hit
    return None


def infer_existing_root_dir(load_from: str) -> Path:
    """The experiment root (``<output_dir>/<run_name>``) that a resume source (file, run directory or root) belongs to."""
    source = Path(load_from).expanduser().resolve()
    if not source.exists():
        raise FileNotFoundError(f"checkpoint source does not exist: {source}")
    if source.is_file():
        return source.parent.parent.parent if source.parent.name == "checkpoints" else source.parent
    if (source / "metrics.csv").exists() or (source / "checkpoints").exists():
        return source.parent
    return source


def load_model_state(model: nn.Module, state_dict: dict[str, torch.Tensor]) -> None:
    """Strict load; LBI-1 key names are migrated and a tied model ignores a stored copy of the LM head."""
    from ..legacy.lbi1_checkpoint import is_lbi1_state_dict, migrate_lbi1_state_dict

    own_keys = set(model.state_dict().keys())
    if is_lbi1_state_dict(state_dict) and any(k.startswith("interface.") for k in own_keys):
        state_dict = migrate_lbi1_state_dict(state_dict)
    if getattr(model, "tie_embeddings", False) and "readout.lm_head.weight" in state_dict and "readout.lm_head.weight" not in own_keys:
        state_dict = {k: v for k, v in state_dict.items() if k != "readout.lm_head.weight"}
    with torch.no_grad():
        # copy into the existing storage: parameters may be views of a flat optimizer buffer
        missing = own_keys - set(state_dict.keys())
        unexpected = set(state_dict.keys()) - own_keys
        if missing or unexpected:
            raise RuntimeError(f"state dict mismatch: missing {sorted(missing)[:5]}, unexpected {sorted(unexpected)[:5]}")
        for key, target in model.state_dict().items():
            target.copy_(state_dict[key].to(device=target.device, dtype=target.dtype))


_FRESH = {"checkpoint_path": "", "start_step": 0, "tokens_seen": 0, "best_val_ce_loss": float("inf"), "best_val_step": -1}


def maybe_restore_training_state(*, mode: str, load_from: str, regime: str, model: nn.Module, optimizer, device: torch.device,
                                 train_generator: torch.Generator, eval_generator: torch.Generator) -> dict[str, Any]:
    """``resume`` restores weights, optimizer, RNG streams and counters; ``init`` loads weights only."""
    if mode not in {"resume", "init"}:
        raise ValueError("mode must be one of: resume, init")
    path = resolve_checkpoint_path(load_from, regime=regime, preference="latest" if mode == "resume" else "best")
    if path is None:
        return dict(_FRESH)
    ckpt = load_checkpoint(path, device=device)
    load_model_state(model, ckpt["model_state_dict"])
    if mode == "init":
        return {**_FRESH, "checkpoint_path": str(path)}
    optimizer.load_state_dict(ckpt["optimizer_state_dict"])
    if ckpt.get("torch_rng_state") is not None:
        torch.set_rng_state(ckpt["torch_rng_state"].cpu())
    if device.type == "cuda" and ckpt.get("cuda_rng_state_all"):
        torch.cuda.set_rng_state_all([s.cpu() for s in ckpt["cuda_rng_state_all"]])
    if ckpt.get("train_generator_state") is not None:
        train_generator.set_state(ckpt["train_generator_state"].cpu())
    if ckpt.get("eval_generator_state") is not None:
        eval_generator.set_state(ckpt["eval_generator_state"].cpu())
    return {
        "checkpoint_path": str(path),
        "start_step": int(ckpt.get("step", 0)),
        "tokens_seen": int(ckpt.get("tokens_seen", 0)),
        "best_val_ce_loss": float(ckpt.get("best_val_ce_loss", float("inf"))),
        "best_val_step": int(ckpt.get("best_val_step", -1)),
    }
