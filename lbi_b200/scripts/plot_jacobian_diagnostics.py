"""Interface-Jacobian diagnostics: spectral norm of the local region Jacobians over training, per state width.

Reads runs logged with ``--log-interface-jacobian-every`` (columns ``jac_local_spec_mean/max``, ``jac_local_frob_*``,
``jac_suffix_spec_*`` of ``metrics.csv``), groups them by ``message_dim``, averages over seeds and writes
``jacobian_spec_mean_vs_tokens.{png,pdf}`` plus ``jacobian_final_summary.{csv,tex}``
(reference scripts/plot_jacobian_diagnostics.py:271-287).
"""
from __future__ import annotations

import argparse
import re
from collections import defaultdict
from pathlib import Path
from typing import Any

from ._charts import Chart, mean_std, write_csv
from .plot_training_curves import aggregate, discover_runs, read_metrics

_FIELDS = ("jac_local_spec_mean", "jac_local_spec_max", "jac_local_frob_mean", "jac_local_frob_normed_mean",
           "jac_suffix_spec_mean", "jac_suffix_spec_max")


def _tex_pm(mean: Any, std: Any) -> str:
    if mean is None or std is None or mean != mean:
        return "--"
    return f"{float(mean):.3f} $\\pm$ {0.0 if std != std else float(std):.3f}"


def main(argv: list[str] | None = None) -> dict[str, Any]:
    import json

    p = argparse.ArgumentParser(description="Plot interface Jacobian diagnostics of one run family.")
    p.add_argument("run_root", type=Path, help="Jacobian diagnostic family directory.")
    p.add_argument("--output-dir", type=Path, default=None, help="default: <run_root>/jacobian_plots")
    p.add_argument("--min-step", type=int, default=200, help="Minimum step to include in plots/tables.")
    p.add_argument("--dpi", type=int, default=150, help="Output DPI for PNG figures.")
    p.add_argument("--font-scale", type=float, default=1.0, help="Multiplier for paper font sizes.")
    p.add_argument("--include-rank-regex", type=str, default="", help="Optional regex over rank strings, e.g. '^(16|32)$'.")
    ns = p.parse_args(argv)
    out_dir = ns.output_dir or (ns.run_root / "jacobian_plots")
    by_rank: dict[int, list[dict]] = defaultdict(list)
    for run in discover_runs([ns.run_root]):
        cfg = json.loads((run / "config.json").read_text(encoding="utf-8"))
        rank = int(cfg.get("message_dim", 0))
        if ns.include_rank_regex and not re.search(ns.include_rank_regex, str(rank)):
            continue
        rows = [r for r in read_metrics(run) if (r.get("step") or 0) >= ns.min_step]
        if any(r.get("jac_local_spec_mean") is not None for r in rows):
            by_rank[rank].append({"dir": run, "cfg": cfg, "rows": rows})
    if not by_rank:
        raise SystemExit(f"no Jacobian diagnostic metrics found under {ns.run_root}")
    chart = Chart("Local interface Jacobian spectral norm", "tokens seen", "mean spectral norm")
    table: list[dict[str, Any]] = []
    for rank, runs in sorted(by_rank.items()):
        s = aggregate(runs, "train", "tokens_seen", "jac_local_spec_mean")
        if s is not None:
            s.label = f"R = {rank}"
            chart.series.append(s)
        runs = sorted(runs, key=lambda r: (r["cfg"].get("seed", 0), str(r["dir"])))
        row: dict[str, Any] = {"rank": rank, "num_seeds": len(runs), "seeds": ",".join(str(r["cfg"].get("seed", "")) for r in runs),
                               "message_dim": rank, "num_runs": len(runs)}
        for f in _FIELDS:
            finals = []
            for run in runs:
                vals = [r[f] for r in run["rows"] if r["split"] == "train" and r.get(f) is not None]
                if vals:
                    finals.append(vals[-1])
            row[f + "_mean"], row[f + "_std"] = mean_std(finals)
        table.append(row)
    files = chart.save(out_dir / "jacobian_spec_mean_vs_tokens", dpi=ns.dpi, font_scale=ns.font_scale, also_pdf=True)
    write_csv(out_dir / "jacobian_final_summary.csv", table)
    # the table of the paper: rank | local spectral norm | suffix spectral norm | local Frobenius norm / sqrt(r), mean +- std over seeds
    lines = [r"\begin{tabular}{c|c|c|c}", r"Rank $r$ & Local $\|J\|_2$ & Suffix $\|J\|_2$ & Local $\|J\|_F/\sqrt{r}$ \\", r"\hline"]
    for row in table:
        cells = [_tex_pm(row[f + "_mean"], row[f + "_std"]) for f in ("jac_local_spec_mean", "jac_suffix_spec_mean",
                                                                      "jac_local_frob_normed_mean")]
        lines.append(f"{row['rank']} & " + " & ".join(cells) + r" \\")
    lines += [r"\end{tabular}", ""]
    (out_dir / "jacobian_final_summary.tex").write_text("\n".join(lines), encoding="utf-8")
    return {"output_dir": str(out_dir), "figures": [str(f) for f in files], "table": table}


def generate_jacobian_diagnostic_plots(run_root: Path, *, output_dir: Path | None = None, min_step: int = 200, dpi: int = 150,
                                       font_scale: float = 1.0, include_rank_regex: str = "") -> Path:
    """Function form with the reference's argument list (scripts/plot_jacobian_diagnostics.py:271-279); returns the output directory."""
    argv = [str(run_root), "--min-step", str(min_step), "--dpi", str(dpi), "--font-scale", str(font_scale),
            "--include-rank-regex", include_rank_regex]
    if output_dir is not None:
        argv += ["--output-dir", str(output_dir)]
    return Path(main(argv)["output_dir"])


if __name__ == "__main__":
    main()
