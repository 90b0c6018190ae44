"""Message-ablation figures: validation CE with the interface state intact vs zeroed / noised / masked.

Reads the ``val`` and ``val_<mode>`` rows that training writes when ``--eval-message-ablation`` /
``--eval-all-message-ablations`` is on, averages LBI runs of each backbone over seeds and writes
``<backbone>_ablation_ce_vs_tokens`` and ``<backbone>_ablation_final_ce`` figures plus ``ablation_summary.csv``
(reference scripts/plot_message_ablations.py:241-268).
"""
from __future__ import annotations

import argparse
import math
from collections import defaultdict
from pathlib import Path
from typing import Any

from ._charts import Chart, write_csv
from .plot_training_curves import aggregate, load_groups


def _splits(runs: list[dict]) -> list[str]:
    names = {r["split"] for run in runs for r in run["rows"] if str(r["split"]).startswith("val")}
    return ["val"] + sorted(n for n in names if n != "val") if "val" in names else sorted(names)


def main(argv: list[str] | None = None) -> dict[str, Any]:
    p = argparse.ArgumentParser(description="Plot message-ablation curves from one or more LBI run roots.")
    p.add_argument("run_roots", nargs="+", type=Path, help="Run roots or per-regime run directories.")
    p.add_argument("--output-dir", type=Path, default=None, help="default: <first root>/ablation_plots")
    p.add_argument("--dpi", type=int, default=150)
    p.add_argument("--font-scale", type=float, default=1.0)
    p.add_argument("--include-variant-regex", type=str, default="")
    p.add_argument("--exclude-variant-regex", type=str, default="", help="applied after the include filter")
    ns = p.parse_args(argv)
    out_dir = ns.output_dir or (ns.run_roots[0] / "ablation_plots")
    groups = load_groups(ns.run_roots, include=ns.include_variant_regex, exclude=ns.exclude_variant_regex)
    by_backbone: dict[str, list[dict]] = defaultdict(list)
    for label, runs in groups.items():
        if label == "dense":
            continue
        for run in runs:
            by_backbone[str(run["cfg"].get("backbone", "model"))].append(run)
    summary: list[dict[str, Any]] = []
    files: list[Path] = []
    for backbone, runs in sorted(by_backbone.items()):
        curves = Chart(f"{backbone}: validation CE under message ablations", "tokens seen", "val CE")
        bars = []
        for split in _splits(runs):
            s = aggregate(runs, split, "tokens_seen", "ce_loss")
            if s is None:
                continue
            name = "val" if split == "val" else split.replace("val_", "")
            s.label, s.style = name, "--" if split == "val" else "-"
            curves.series.append(s)
            final, spread = s.y[-1], (s.band[-1] if s.band is not None else 0.0)
            bars.append((name, final, spread if math.isfinite(spread) else 0.0))
            summary.append({"backbone": backbone, "split": split, "num_runs": len(runs), "mean_final_ce": final,
                            "std_final_ce": spread, "final_ce_mean": final, "final_ce_std": spread, "final_tokens_seen": s.x[-1]})
        if curves.series:
            files += curves.save(out_dir / f"{backbone}_ablation_ce_vs_tokens", dpi=ns.dpi, font_scale=ns.font_scale)
            files += Chart(f"{backbone}: final validation CE", "", "val CE", bars=bars).save(
                out_dir / f"{backbone}_ablation_final_ce", dpi=ns.dpi, font_scale=ns.font_scale)
    write_csv(out_dir / "ablation_summary.csv", summary)
    return {"output_dir": str(out_dir), "figures": [str(f) for f in files], "summary": summary}


def generate_message_ablation_plots(run_roots, *, output_dir: Path | None = None, dpi: int = 150, include_variant_regex: str = "",
                                    exclude_variant_regex: str = "") -> Path:
    """Function form with the reference's argument list (scripts/plot_message_ablations.py:241-248); returns the output directory."""
    argv = [str(r) for r in run_roots] + ["--dpi", str(dpi), "--include-variant-regex", include_variant_regex,
                                          "--exclude-variant-regex", exclude_variant_regex]
    if output_dir is not None:
        argv += ["--output-dir", str(output_dir)]
    return Path(main(argv)["output_dir"])


if __name__ == "__main__":
    main()
