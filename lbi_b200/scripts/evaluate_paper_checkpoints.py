"""Post-hoc evaluation of trained runs: cross-entropy, perplexity and evaluation throughput per checkpoint.

Walks a family directory (``<family>/<run_name>/<variant>/`` with ``config.json`` + ``summary.json``), rebuilds each
model from its stored config, loads ``best.pt`` or ``latest.pt`` and evaluates it on freshly sampled validation batches
with a fixed generator seed.  Writes ``lm_eval_summary.csv`` and ``lm_eval_summary.json`` with the columns of
reference scripts/evaluate_paper_checkpoints.py:122-248 (``posthoc_val_ce_loss``, ``posthoc_val_ppl``,
``eval_tokens_per_s``, ...).  Both the current directory names (``dense`` / ``lbi``) and the legacy ones
(``backprop_ref`` / ``native_region_interface``) are recognised.
"""
from __future__ import annotations

import argparse
import csv
import json
import math
import re
import time
from dataclasses import replace
from pathlib import Path
from typing import Any

import torch

from ..train.checkpointing import checkpoint_path_from_summary, load_checkpoint, load_model_state
from ..train.config import DENSE_VARIANT, LBITrainingConfig, normalize_model_variant
from ..train.data import build_corpora, sample_batch_any
from ..train.eval import next_token_loss
from ..train.model_builders import build_model_for_regime
from ..train.runners import _autocast_context, _resolve_device

_RUN_DIR_NAMES = {"dense", "lbi", "backprop_ref", "native_region_interface"}


def _order_key(run_dir: Path) -> tuple:
    """dense runs first (by seed), then LBI runs by rank and seed, then everything else by path."""
    name = run_dir.parent.name
    m = re.fullmatch(r"dense_seed(\d+)", name)
    if m:
        return (0, 0, int(m.group(1)), name)
    m = re.fullmatch(r"lbi_r(\d+)_seed(\d+)", name)
    if m:
        return (1, int(m.group(1)), int(m.group(2)), name)
    return (2, 0, 0, str(run_dir))


def discover_run_dirs(family_dir: Path) -> list[Path]:
    found = [p for p in family_dir.glob("*/*")
             if p.is_dir() and p.name in _RUN_DIR_NAMES and (p / "config.json").exists() and (p / "summary.json").exists()]
    return sorted(found, key=_order_key)


def load_run_config(run_dir: Path, *, eval_batches: int, batch_size: int | None, seq_len: int | None,
                    device: str, tokenizer_path: str = "") -> LBITrainingConfig:
    """The stored config of a run with checkpoint saving off and the evaluation overrides applied."""
    raw = json.loads((run_dir / "config.json").read_text(encoding="utf-8"))
    raw.update(save_checkpoints=False, resume_from="", init_from="")
    if tokenizer_path:  # the tokenizer the corpora are rebuilt with, when the run's own path is not on this machine
        raw["tokenizer_path"] = tokenizer_path
    cfg = LBITrainingConfig.from_dict(raw)
    updates: dict[str, Any] = {"eval_batches": int(eval_batches)}
    if batch_size is not None:
        updates["batch_size"] = int(batch_size)
    if seq_len is not None:
        updates["seq_len"] = int(seq_len)
    if device != "auto":
        updates["device"] = device
    return replace(cfg, **updates)


def evaluate_model(*, cfg: LBITrainingConfig, model: torch.nn.Module, val_corpus: Any, seed: int,
                   device: torch.device) -> dict[str, float]:
    """Mean next-token cross-entropy, perplexity and tokens / s over ``cfg.eval_batches`` freshly sampled validation batches."""
    gen = torch.Generator(device=device if cfg.data_mode == "synthetic" else torch.device("cpu"))
    gen.manual_seed(int(seed))
    model.eval()
    loss_sum, tokens = 0.0, 0
    if device.type == "cuda":
        torch.cuda.synchronize(device)
    t0 = time.perf_counter()
    with torch.no_grad():
        for _ in range(cfg.eval_batches):
            xb, yb = sample_batch_any(cfg=cfg, corpus=val_corpus, batch_size=cfg.batch_size, generator=gen, device=device)
            with _autocast_context(cfg, device):
                out = model.forward_with_cache(xb)[0] if hasattr(model, "forward_with_cache") else model(xb)
            n = int(yb.numel())
            loss_sum += float(next_token_loss(out, yb)) * n
            tokens += n
    if device.type == "cuda":
        torch.cuda.synchronize(device)
    wall = time.perf_counter() - t0
    ce = loss_sum / max(1, tokens)
    try:
        ppl = math.exp(ce)
    except OverflowError:
        ppl = float("inf")
    return {"ce_loss": ce, "ppl": ppl, "eval_tokens": tokens, "wall_time_s": wall,
            "tokens_per_s": tokens / wall if wall > 0 else 0.0}


def _json_or_empty(path: Path) -> dict[str, Any]:
    return json.loads(path.read_text(encoding="utf-8")) if path.exists() else {}


def evaluate_run(run_dir: Path, *, checkpoint: str, eval_batches: int, batch_size: int | None, seq_len: int | None,
                 eval_seed: int, device: str, tokenizer_path: str = "") -> dict[str, Any]:
    """Rebuild a run's model, load the chosen checkpoint, evaluate it; one row of the summary table."""
    cfg = load_run_config(run_dir, eval_batches=eval_batches, batch_size=batch_size, seq_len=seq_len, device=device,
                          tokenizer_path=tokenizer_path)
    dev = _resolve_device(cfg)
    ckpt_path = checkpoint_path_from_summary(run_dir / "summary.json", preference=checkpoint)
    if ckpt_path is None or not Path(ckpt_path).exists():
        raise FileNotFoundError(f"no {checkpoint} checkpoint recorded for {run_dir}")
    payload = load_checkpoint(Path(ckpt_path), device=dev)
    variant = normalize_model_variant(cfg.regime if cfg.regime not in ("", "all") else run_dir.name)
    model = build_model_for_regime(replace(cfg, variants=variant, regime=variant), checkpoint=payload).to(dev)
    load_model_state(model, payload["model_state_dict"])
    _, val_corpus = build_corpora(cfg, device=dev)
    m = evaluate_model(cfg=cfg, model=model, val_corpus=val_corpus, seed=eval_seed, device=dev)
    summary = _json_or_empty(run_dir / "summary.json")
    info = _json_or_empty(run_dir / "model_info.json")
    is_lbi = variant != DENSE_VARIANT
    row = {
        "label": run_dir.parent.name, "run_dir": str(run_dir), "regime": variant, "backbone": cfg.backbone, "seed": cfg.seed,
        "message_dim": cfg.message_dim if is_lbi else "", "region_size": cfg.region_size if is_lbi else "",
        "checkpoint": checkpoint, "checkpoint_path": str(ckpt_path), "checkpoint_step": int(payload.get("step", -1)),
        "checkpoint_best_val_ce_loss": float(payload.get("best_val_ce_loss", float("nan"))),
        "checkpoint_best_val_step": int(payload.get("best_val_step", -1)),
        "summary_best_val_ce_loss": summary.get("best_val_ce_loss", ""), "summary_best_val_step": summary.get("best_val_step", ""),
        "summary_final_val_ce_loss": summary.get("final_val_ce_loss", ""),
        "posthoc_val_ce_loss": m["ce_loss"], "posthoc_val_ppl": m["ppl"], "eval_batches": cfg.eval_batches,
        "eval_batch_size": cfg.batch_size, "eval_seq_len": cfg.seq_len, "eval_tokens": int(m["eval_tokens"]),
        "eval_seed": int(eval_seed), "eval_wall_time_s": m["wall_time_s"], "eval_tokens_per_s": m["tokens_per_s"],
        "total_params": info.get("total_params", ""),
    }
    del model, payload
    if dev.type == "cuda":
        torch.cuda.empty_cache()
    return row


def write_outputs(rows: list[dict[str, Any]], out_dir: Path) -> None:
    out_dir.mkdir(parents=True, exist_ok=True)
    (out_dir / "lm_eval_summary.json").write_text(json.dumps(rows, indent=2, sort_keys=True) + "\n", encoding="utf-8")
    with (out_dir / "lm_eval_summary.csv").open("w", newline="", encoding="utf-8") as fh:
        if rows:
            w = csv.DictWriter(fh, fieldnames=list(rows[0]))
            w.writeheader()
            w.writerows(rows)


def main(argv: list[str] | None = None) -> list[dict[str, Any]]:
    p = argparse.ArgumentParser(description="Evaluate the checkpoints of one run family.")
    p.add_argument("family_dir", type=Path, nargs="?", default=None,
                   help="directory holding <run_name>/<variant>/ run directories, or one run directory")
    p.add_argument("--family", type=Path, default=None, help="the same directory as a flag (the reference's spelling)")
    p.add_argument("--run-dir", action="append", default=[],
                   help="a run directory to evaluate; may be repeated, and then the family only names the default output directory")
    p.add_argument("--tokenizer-path", type=str, default="", help="tokenizer used to rebuild the corpora instead of the run's own")
    p.add_argument("--output-dir", type=str, default="", help="where lm_eval_summary.{csv,json} go (default: <family_dir>/evals)")
    p.add_argument("--checkpoint", choices=("best", "latest"), default="best")
    p.add_argument("--eval-batches", type=int, default=512)
    p.add_argument("--batch-size", type=int, default=None)
    p.add_argument("--seq-len", type=int, default=None)
    p.add_argument("--eval-seed", type=int, default=12345)
    p.add_argument("--device", choices=("auto", "cpu", "cuda"), default="auto")
    p.add_argument("--include-regex", type=str, default="", help="keep only runs whose <run_name> matches")
    p.add_argument("--exclude-regex", type=str, default="", help="drop runs whose <run_name> matches")
    ns = p.parse_args(argv)
    family = ns.family_dir if ns.family_dir is not None else ns.family
    if family is None and not ns.run_dir:
        p.error("give the family directory (positional or --family) or at least one --run-dir")
    if ns.run_dir:
        runs = [Path(r).expanduser() for r in ns.run_dir]
        family = Path(ns.run_dir[0]).expanduser().parent.parent if family is None else family
    elif (family / "config.json").exists() and (family / "summary.json").exists():
        runs = [family]
    else:
        runs = discover_run_dirs(family)
    if not runs:
        raise FileNotFoundError(f"no completed runs found under: {family}")
    ns.family_dir = family
    if ns.include_regex:
        runs = [r for r in runs if re.search(ns.include_regex, r.parent.name)]
    if ns.exclude_regex:
        runs = [r for r in runs if not re.search(ns.exclude_regex, r.parent.name)]
    rows = [evaluate_run(r, checkpoint=ns.checkpoint, eval_batches=ns.eval_batches, batch_size=ns.batch_size,
                         seq_len=ns.seq_len, eval_seed=ns.eval_seed, device=ns.device, tokenizer_path=ns.tokenizer_path)
            for r in runs]
    write_outputs(rows, Path(ns.output_dir) if ns.output_dir else ns.family_dir / "evals")
    print("run\tposthoc_ce\tppl\ttrain_best_ce\tckpt_step\teval_tokens")
    for r in rows:
        print(f"{r['label']}\t{r['posthoc_val_ce_loss']:.6g}\t{r['posthoc_val_ppl']:.6g}\t{r['summary_best_val_ce_loss']}\t"
              f"{r['checkpoint_step']}\t{r['eval_tokens']}")
    return rows


if __name__ == "__main__":
    main()
