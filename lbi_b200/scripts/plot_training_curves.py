"""Training-curve figures and per-group summary tables from ``metrics.csv`` files.

Runs are discovered below the given roots (any directory with ``metrics.csv`` + ``config.json``), grouped by label
(``dense``, ``lbi r<R>`` ... with the seed stripped), averaged over seeds on the union of logged steps, and drawn as
mean +- one standard deviation.  Outputs follow reference scripts/plot_training_curves.py:672-753:
``ce_vs_tokens``, ``ce_vs_step``, ``paper_val_ce_vs_tokens``, ``paper_val_ce_vs_step``, ``paper_ce_vs_tokens``,
``tokens_per_s_vs_step``, ``message_diagnostics``, ``val_summary_bar`` figures and ``group_summary.{csv,json}``.
"""
from __future__ import annotations

import argparse
import csv
import json
import math
import re
from collections import defaultdict
from pathlib import Path
from typing import Any

from ._charts import Chart, Series, mean_std, moving_average, write_csv, write_json


def discover_runs_with_roots(roots: list[Path]) -> list[tuple[Path, Path]]:
    """(experiment root, run directory) for every directory with ``metrics.csv`` + ``config.json`` at or below the roots; a
    root that is itself a run directory counts with its parent as the experiment root."""
    found: list[tuple[Path, Path]] = []
    for root in roots:
        if (root / "metrics.csv").exists():
            found.append((root.parent, root))
        found.extend((root, p.parent) for p in sorted(root.rglob("metrics.csv")) if p.parent != root)
    seen, out = set(), []
    for root, run in found:
        if run.resolve() not in seen and (run / "config.json").exists():
            seen.add(run.resolve())
            out.append((root, run))
    return out


def discover_runs(roots: list[Path]) -> list[Path]:
    return [run for _, run in discover_runs_with_roots(roots)]


def run_variant(root: Path, run_dir: Path, cfg: dict[str, Any]) -> str:
    """The name the include / exclude filters see: the first directory below the experiment root (``lbi_r32_seed7`` for
    ``<root>/lbi_r32_seed7/lbi``), else the run directory's parent, else a name rebuilt from the config
    (reference scripts/plot_training_curves.py:164-176)."""
    try:
        parts = run_dir.resolve().relative_to(root.resolve()).parts
    except ValueError:
        parts = (run_dir.name,)
    variant = parts[0] if len(parts) > 1 else run_dir.parent.name
    if variant and variant != "." and variant != run_dir.name:
        return variant
    if run_dir.name in {"dense", "backprop_ref"}:
        return f"dense_seed{cfg.get('seed', 'unknown')}"
    return f"lbi_r{cfg.get('message_dim', 'unknown')}_seed{cfg.get('seed', 'unknown')}"


def read_metrics(run_dir: Path) -> list[dict[str, Any]]:
    rows = []
    with (run_dir / "metrics.csv").open(newline="", encoding="utf-8") as fh:
        for row in csv.DictReader(fh):
            parsed: dict[str, Any] = {"split": row.get("split", "")}
            for key, value in row.items():
                if key == "split":
                    continue
                try:
                    parsed[key] = float(value) if value not in ("", None) else None
                except ValueError:
                    parsed[key] = None
            rows.append(parsed)
    return rows


_DENSE_NAMES = {"dense", "backprop_ref"}
_REGIME_ALIASES = {"backprop_ref": "dense", "native_region_interface": "lbi"}
LABEL_MODES = ("auto", "full", "variant", "backbone", "regime", "backbone_regime", "region_size", "rank_region")


def run_regime(run_dir: Path) -> str:
    """``dense`` or ``lbi`` from the run directory's name (the first release's names map onto them)."""
    return _REGIME_ALIASES.get(run_dir.name, run_dir.name)


def run_label(run_dir: Path, cfg: dict[str, Any], mode: str = "auto", *, several_region_sizes: bool = True) -> str:
    """The group a run is averaged into.  ``auto``: dense / lbi r<R>; ``full`` adds the region size; ``variant``: the run
    name without its seed; ``backbone`` / ``regime`` / ``backbone_regime`` / ``region_size`` / ``rank_region`` as in the
    reference (scripts/plot_training_curves.py:226-268)."""
    variant = run_dir.name
    is_dense = variant in _DENSE_NAMES
    backbone, regime = str(cfg.get("backbone", "model")), run_regime(run_dir)
    if mode == "variant":
        return re.sub(r"_seed\d+$", "", run_dir.parent.name) or variant
    if mode == "backbone":
        return backbone
    if mode == "regime":
        return regime
    if mode == "backbone_regime":
        return f"{backbone}:{regime}"
    if is_dense:
        return "dense"
    if mode == "region_size":
        return f"region={cfg.get('region_size', '?')}"
    if mode == "rank_region":
        rank = f"lbi r{cfg.get('message_dim', '?')}"
        return f"{rank}, region={cfg.get('region_size', '?')}" if several_region_sizes else rank
    label = f"lbi r{cfg.get('message_dim', '?')}"
    if mode == "full":
        label += f" rs{cfg.get('region_size', '?')}"
    return label


def load_groups(roots: list[Path], *, include: str = "", exclude: str = "", label_mode: str = "auto",
                regimes: set[str] | None = None) -> dict[str, list[dict]]:
    """``regimes`` keeps only runs of the named kinds (``dense``, ``lbi``; the first release's names are understood)."""
    wanted = None if not regimes else {_REGIME_ALIASES.get(r, r) for r in regimes}
    kept: list[tuple[Path, dict]] = []
    for root, run in discover_runs_with_roots(roots):
        cfg = json.loads((run / "config.json").read_text(encoding="utf-8"))
        name = run_variant(root, run, cfg)
        if include and not re.search(include, name):
            continue
        if exclude and re.search(exclude, name):
            continue
        if wanted is not None and run_regime(run) not in wanted:
            continue
        kept.append((run, cfg))
    sizes = {cfg.get("region_size") for run, cfg in kept if run.name not in _DENSE_NAMES}
    groups: dict[str, list[dict]] = defaultdict(list)
    for run, cfg in kept:
        label = run_label(run, cfg, label_mode, several_region_sizes=len(sizes) > 1)
        groups[label].append({"dir": run, "cfg": cfg, "rows": read_metrics(run)})
    return dict(groups)


def _curve(rows: list[dict], split: str, xkey: str, ykey: str) -> dict[float, float]:
    return {r[xkey]: r[ykey] for r in rows if r["split"] == split and r.get(xkey) is not None and r.get(ykey) is not None}


def aggregate(runs: list[dict], split: str, xkey: str, ykey: str, smooth: int = 1) -> Series | None:
    """Mean curve (and standard-deviation band when several runs) of one metric of one split over the union of logged x values."""
    curves = [_curve(r["rows"], split, xkey, ykey) for r in runs]
    curves = [c for c in curves if c]
    if not curves:
        return None
    xs = sorted(set().union(*[set(c) for c in curves]))
    mean, band = [], []
    for x in xs:
        m, s = mean_std([c[x] for c in curves if x in c])
        mean.append(m)
        band.append(s if math.isfinite(s) else 0.0)
    return Series("", xs, moving_average(mean, smooth), band if len(curves) > 1 else None)


def _population(values: list[float]) -> tuple[float, float]:
    vals = [float(v) for v in values if v is not None and math.isfinite(float(v))]
    if not vals:
        return float("nan"), float("nan")
    m = sum(vals) / len(vals)
    return m, (math.sqrt(sum((v - m) ** 2 for v in vals) / len(vals)) if len(vals) > 1 else 0.0)


def summarize(groups: dict[str, list[dict]]) -> list[dict[str, Any]]:
    """One row per group.  The columns of the reference's table (scripts/plot_training_curves.py:615-647: backbones, regimes,
    seeds, variants, region_sizes, lr_models, seq_lens, mean / std of total parameters and of the final / best validation CE, the
    spread being the population standard deviation) plus the sample-deviation columns the figures here use and the throughput."""
    out = []
    for label, runs in sorted(groups.items()):
        finals, bests, tps, params = [], [], [], []
        for r in runs:
            val = [x for x in r["rows"] if x["split"] == "val" and x.get("ce_loss") is not None]
            train = [x for x in r["rows"] if x["split"] == "train" and x.get("tokens_per_s")]
            if val:
                finals.append(val[-1]["ce_loss"])
                bests.append(min(x["ce_loss"] for x in val))
            if train:
                tps.append(sum(x["tokens_per_s"] for x in train) / len(train))
            info = r["dir"] / "model_info.json"
            if info.exists():
                params.append(json.loads(info.read_text(encoding="utf-8")).get("total_params"))
        fm, fs = mean_std(finals)
        bm, bs = mean_std(bests)
        tm, _ = mean_std(tps)
        cfgs = [r["cfg"] for r in runs]
        lbi_cfgs = [r["cfg"] for r in runs if r["dir"].name not in _DENSE_NAMES]
        by_seed = sorted(runs, key=lambda r: (r["cfg"].get("seed", 0), str(r["dir"])))
        out.append({
            "label": label, "num_runs": len(runs),
            "backbones": ",".join(sorted({str(c.get("backbone", "")) for c in cfgs})),
            "regimes": ",".join(sorted({run_regime(r["dir"]) for r in runs})),
            "seeds": ",".join(str(r["cfg"].get("seed", "")) for r in by_seed),
            "variants": ",".join(sorted(r["dir"].parent.name for r in runs)),
            "region_sizes": ",".join(str(v) for v in sorted({c["region_size"] for c in lbi_cfgs if c.get("region_size") is not None})),
            "lr_models": ",".join(f"{v:g}" for v in sorted({float(c["lr_model"]) for c in cfgs if c.get("lr_model") is not None})),
            "seq_lens": ",".join(str(v) for v in sorted({c["seq_len"] for c in cfgs if c.get("seq_len") is not None})),
            "mean_total_params": _population(params)[0], "std_total_params": _population(params)[1],
            "mean_final_val_ce": _population(finals)[0], "std_final_val_ce": _population(finals)[1],
            "mean_best_val_ce": _population(bests)[0], "std_best_val_ce": _population(bests)[1],
            "final_val_ce_mean": fm, "final_val_ce_std": fs, "best_val_ce_mean": bm, "best_val_ce_std": bs,
            "mean_tokens_per_s": tm,
        })
    return out


def make_figures(groups: dict[str, list[dict]], out_dir: Path, *, dpi: int, font_scale: float, smooth: int) -> list[Path]:
    """Write every figure of the training-curve set for the grouped runs; returns the files written."""
    written: list[Path] = []

    def figure(stem: str, title: str, xlabel: str, ylabel: str, parts: list[tuple[str, str, str, str, str]], logy=False) -> None:
        chart = Chart(title, xlabel, ylabel, logy=logy)
        for label, runs in sorted(groups.items()):
            for split, xkey, ykey, suffix, style in parts:
                s = aggregate(runs, split, xkey, ykey, smooth if split == "train" else 1)
                if s is not None:
                    s.label, s.style = f"{label}{suffix}", style
                    chart.series.append(s)
        if chart.series:
            written.extend(chart.save(out_dir / stem, dpi=dpi, font_scale=font_scale, also_pdf=stem.startswith("paper_")))

    both = lambda x: [("train", x, "ce_loss", " train", "--"), ("val", x, "ce_loss", " val", "-")]  # noqa: E731
    figure("ce_vs_tokens", "Cross-entropy vs tokens", "tokens seen", "CE loss", both("tokens_seen"))
    figure("ce_vs_step", "Cross-entropy vs step", "step", "CE loss", both("step"))
    figure("paper_val_ce_vs_tokens", "Validation cross-entropy", "tokens seen", "val CE", [("val", "tokens_seen", "ce_loss", "", "-")])
    figure("paper_val_ce_vs_step", "Validation cross-entropy", "step", "val CE", [("val", "step", "ce_loss", "", "-")])
    figure("paper_ce_vs_tokens", "Training cross-entropy", "tokens seen", "train CE", [("train", "tokens_seen", "ce_loss", "", "-")])
    figure("tokens_per_s_vs_step", "Throughput", "step", "tokens / s", [("train", "step", "tokens_per_s", "", "-")])
    figure("message_diagnostics", "Interface state norm and scan alignment", "step", "value",
           [("train", "step", "message_norm", " |s|", "-"), ("train", "step", "scan_align", " scan align", "--")])
    summary = summarize(groups)
    bars = [(r["label"], r["final_val_ce_mean"], 0.0 if not math.isfinite(r["final_val_ce_std"]) else r["final_val_ce_std"])
            for r in summary if math.isfinite(r["final_val_ce_mean"])]
    if bars:
        written.extend(Chart("Final validation cross-entropy", "", "val CE", bars=bars).save(out_dir / "val_summary_bar", dpi=dpi,
                                                                                              font_scale=font_scale))
    return written


def main(argv: list[str] | None = None) -> dict[str, Any]:
    p = argparse.ArgumentParser(description="Plot training curves of one or more run roots.")
    p.add_argument("run_roots", nargs="+", type=Path, help="Run roots or per-regime run directories.")
    p.add_argument("--output-dir", type=Path, default=None, help="default: <first root>/plots")
    p.add_argument("--include-variant-regex", type=str, default="")
    p.add_argument("--exclude-variant-regex", type=str, default="")
    p.add_argument("--label-mode", choices=LABEL_MODES, default="auto")
    p.add_argument("--regimes", type=str, default="", help="comma-separated filter, e.g. lbi (or native_region_interface)")
    p.add_argument("--smooth-window", type=int, default=1, help="moving-average window for training curves")
    p.add_argument("--dpi", type=int, default=150)
    p.add_argument("--font-scale", type=float, default=1.0)
    ns = p.parse_args(argv)
    out_dir = ns.output_dir or (ns.run_roots[0] / "plots")
    groups = load_groups(ns.run_roots, include=ns.include_variant_regex, exclude=ns.exclude_variant_regex, label_mode=ns.label_mode,
                         regimes={r.strip() for r in ns.regimes.split(",") if r.strip()} or None)
    if not groups:
        raise SystemExit("no runs with metrics.csv found")
    summary = summarize(groups)
    write_csv(out_dir / "group_summary.csv", summary)
    write_json(out_dir / "group_summary.json", summary)
    files = make_figures(groups, out_dir, dpi=ns.dpi, font_scale=ns.font_scale, smooth=ns.smooth_window)
    return {"output_dir": str(out_dir), "figures": [str(f) for f in files], "groups": summary}


def generate_training_plots(run_roots, *, output_dir: Path | None = None, dpi: int = 150, label_mode: str = "auto", regimes=None,
                            smooth_window: int = 25, font_scale: float = 1.0, include_variant_regex: str = "",
                            exclude_variant_regex: str = "") -> Path:
    """Function form with the reference's argument list (scripts/plot_training_curves.py:672-683); returns the output directory."""
    argv = [str(r) for r in run_roots] + ["--dpi", str(dpi), "--label-mode", label_mode, "--smooth-window", str(smooth_window),
                                          "--font-scale", str(font_scale), "--include-variant-regex", include_variant_regex,
                                          "--exclude-variant-regex", exclude_variant_regex]
    if output_dir is not None:
        argv += ["--output-dir", str(output_dir)]
    if regimes:
        argv += ["--regimes", ",".join(r for r in regimes if r)]
    return Path(main(argv)["output_dir"])


if __name__ == "__main__":
    main()
