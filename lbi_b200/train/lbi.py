"""Entry point:  python -m lbi_b200.train.lbi --variants lbi --backbone transformer ...

Runs the selected variants (dense and/or lbi) into ``<output_dir>/<run_name | variants_timestamp>/{dense,lbi}`` and
writes a per-experiment summary.json (reference train/lbi.py:35-86).
"""
from __future__ import annotations

import json
import time
from dataclasses import replace
from pathlib import Path
from typing import Any, Dict

from .checkpointing import infer_existing_root_dir
from .config import DENSE_VARIANT, LBI_VARIANT, LBITrainingConfig, build_arg_parser, config_from_args, output_name_for_variant, resolve_model_variants
from .data import resolve_runtime_vocab_size
from .runners import run_dense_training, run_lbi_training


def _prepare_run_dir(cfg: LBITrainingConfig, run_root_name: str) -> Path:
    base = cfg.run_name if cfg.run_name else f"{run_root_name}_{time.strftime('%Y%m%d_%H%M%S')}"
    out = Path(cfg.output_dir) / base
    out.mkdir(parents=True, exist_ok=True)
    return out


def run_lbi_experiment(cfg: LBITrainingConfig) -> Dict[str, Any]:
    """Run the configured variants (dense and / or lbi) into one experiment root and write its ``summary.json``."""
    cfg.vocab_size = resolve_runtime_vocab_size(cfg)
    variants = resolve_model_variants(cfg)
    root_dir = infer_existing_root_dir(cfg.resume_from) if cfg.resume_from else _prepare_run_dir(cfg, "_".join(variants) or "lbi")
    root_dir.mkdir(parents=True, exist_ok=True)
    runs = []
    for variant in variants:
        run_cfg = replace(cfg, variants=variant, regime=variant)
        run_dir = root_dir / output_name_for_variant(variant)
        run_dir.mkdir(parents=True, exist_ok=True)
        if variant == DENSE_VARIANT:
            runs.append(run_dense_training(run_cfg, run_dir=run_dir))
        elif variant == LBI_VARIANT:
            runs.append(run_lbi_training(run_cfg, run_dir=run_dir))
        else:
            raise AssertionError(f"unsupported model variant: {variant}")
    summary = {"variants": list(variants), "root_dir": str(root_dir), "runs": runs}
    (root_dir / "summary.json").write_text(json.dumps(summary, indent=2, sort_keys=True), encoding="utf-8")
    return summary


run_training = run_lbi_experiment


def run_with_restarts(cfg: LBITrainingConfig, max_restarts: int) -> Dict[str, Any]:
    """``run_lbi_experiment`` under ``utils.failure.run_with_recovery``: after a step timeout, a bounded kernel wait that ran out,
    a peer failure or an injected fault the run restarts from its newest loadable checkpoint, at most ``max_restarts`` times
    (device errors are never retried in-process).  Single-process runs only: with one process per GPU every rank would have to
    fail and restart in step, so the launcher's own restart policy (``torch.distributed.run --max-restarts``) plus
    ``--resume-from`` is the tool there."""
    import os

    from ..utils.failure import run_with_recovery

    if max_restarts <= 0 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        return run_lbi_experiment(cfg)
    return run_with_recovery(run_lbi_experiment, cfg, max_restarts=max_restarts)


def main() -> None:
    """``LBI_B200_MAX_RESTARTS=N`` (needs ``--run-name``) restarts a failed single-process run from its newest checkpoint."""
    import os

    cfg = config_from_args(build_arg_parser().parse_args())
    summary = run_with_restarts(cfg, int(os.environ.get("LBI_B200_MAX_RESTARTS", "0")))
    print(json.dumps(summary, indent=2, sort_keys=True))


if __name__ == "__main__":
    main()
