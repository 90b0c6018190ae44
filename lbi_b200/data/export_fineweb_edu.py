"""Stream a bounded FineWeb-Edu subset into local train/val text files (needs ``datasets`` and network access).

    python -m lbi_b200.data.export_fineweb_edu --train-bytes 1000000000 --val-bytes 100000000

Same outputs as the reference's exporter (data/export_fineweb_edu.py:48-104): ``fineweb_edu_train.txt`` and
``fineweb_edu_val.txt`` under ``CORPORA_ROOT/<output-subdir>``, one document per line group, the train file
filled to its byte budget before the validation file starts.
"""
from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

from .data_paths import CORPORA_ROOT, DATA_ROOT


def _parse_args() -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Export a byte-bounded FineWeb-Edu subset to text files.")
    p.add_argument("--config", type=str, default="sample-10BT")
    p.add_argument("--output-subdir", type=str, default="fineweb_edu")
    p.add_argument("--output-dir", type=str, default="")
    p.add_argument("--cache-dir", type=str, default=str(DATA_ROOT / "hf_cache"))
    p.add_argument("--train-bytes", type=int, default=1_000_000_000)
    p.add_argument("--val-bytes", type=int, default=100_000_000)
    p.add_argument("--dataset-name", type=str, default="HuggingFaceFW/fineweb-edu")
    p.add_argument("--force-exit-after-export", action="store_true",
                   help="leave with os._exit(0) after the export (for hosts whose datasets/pyarrow teardown crashes)")
    return p.parse_args()


def export(dataset_iter, train_path: Path, val_path: Path, train_bytes: int, val_bytes: int) -> tuple[int, int]:
    """Fill ``train_path`` then ``val_path`` from an iterable of ``{"text": ...}`` records; returns bytes written."""
    budgets = [train_bytes, val_bytes]
    written = [0, 0]
    with train_path.open("wb") as f_train, val_path.open("wb") as f_val:
        files = (f_train, f_val)
        for n_docs, record in enumerate(dataset_iter, start=1):
            text = record.get("text", "")
            blob = (text.strip() + "\n").encode("utf-8", errors="ignore") if text else b""
            if len(blob) <= 1:
                continue
            split = 0 if written[0] < budgets[0] else 1
            if written[split] >= budgets[split]:
                break
            chunk = blob[: budgets[split] - written[split]]
            files[split].write(chunk)
            written[split] += len(chunk)
            if n_docs % 10000 == 0:
                print(f"[fineweb_edu] docs={n_docs} train_bytes={written[0]} val_bytes={written[1]}", flush=True)
    return written[0], written[1]


def main() -> None:
    args = _parse_args()
    try:
        from datasets import load_dataset
    except ImportError as exc:
        raise ImportError("the `datasets` package is required for the FineWeb-Edu export") from exc
    out_dir = Path(args.output_dir).expanduser() if args.output_dir else CORPORA_ROOT / args.output_subdir
    cache_dir = Path(args.cache_dir).expanduser()
    out_dir.mkdir(parents=True, exist_ok=True)
    cache_dir.mkdir(parents=True, exist_ok=True)
    ds = load_dataset(args.dataset_name, args.config, split="train", streaming=True, cache_dir=str(cache_dir))
    train_path, val_path = out_dir / "fineweb_edu_train.txt", out_dir / "fineweb_edu_val.txt"
    wt, wv = export(ds, train_path, val_path, args.train_bytes, args.val_bytes)
    print(f"[fineweb_edu] wrote train={train_path} bytes={wt}\n[fineweb_edu] wrote val={val_path} bytes={wv}", flush=True)
    if args.force_exit_after_export:  # only after a successful export: a failure above must keep its traceback and exit code
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
