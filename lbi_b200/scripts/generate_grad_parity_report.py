"""Gradient-parity report: tables (CSV / JSON / Markdown / LaTeX) and an optional CDF figure.

Runs the cases of ``lbi_b200.utils.grad_parity`` and writes, like reference
scripts/generate_grad_parity_report.py:211-333: ``case_summary.{csv,json,md}``, ``trial_summary.csv``,
``per_parameter.csv``, ``report_config.json``, ``summary.{csv,json,md}`` (aliases of the case view),
``paper_table.{csv,tex}`` and, with ``--plot``, ``grad_rel_error_cdf``.  Defaults: recompute Jacobians with basis chunk
32; the ``report`` preset uses seeds 1000-1019 with 5 batches each.
"""
from __future__ import annotations

import argparse
import dataclasses
from pathlib import Path
from typing import Any, Sequence

from ..utils import grad_parity as gp
from ._charts import Chart, Series, write_csv, write_json

ARCHITECTURES = (("mamba2", "Mamba-2"), ("mamba3", "Mamba-3"), ("transformer", "Transformer"), ("hybrid", "Hybrid"))
REPORT_SEEDS = tuple(range(1000, 1020))
REPORT_BATCHES_PER_SEED = 5
_MD_COLUMNS = ["case_name", "backbone", "region_mode", "interface_jacobian_mode", "jacobian_basis_chunk", "device", "dtype", "status",
               "num_trials", "num_trials_passed", "worst_loss_abs_diff", "min_global_grad_cosine", "max_relative_l2_error",
               "worst_max_abs_grad_diff", "worst_max_rel_grad_diff", "median_p95_rel_grad_diff", "worst_interface_scan_rms",
               "skip_reason"]


def _markdown(path: Path, rows: Sequence[dict[str, Any]]) -> None:
    lines = ["| " + " | ".join(_MD_COLUMNS) + " |", "|" + "---|" * len(_MD_COLUMNS)]
    lines += ["| " + " | ".join(str(r.get(c, "")) for c in _MD_COLUMNS) + " |" for r in rows]
    path.write_text("\n".join(lines) + "\n", encoding="utf-8")


def latex_number(value: Any, digits: int = 3) -> str:
    try:
        x = float(value)
    except (TypeError, ValueError):
        return "--"
    if x == 0.0:
        return "$0$"
    if 1e-3 <= abs(x) < 1e3:
        return f"${x:.{digits}g}$"
    mantissa, exponent = f"{x:.{digits - 1}e}".split("e")
    return rf"${mantissa}\times 10^{{{int(exponent)}}}$"


def paper_rows(case_rows: Sequence[dict[str, Any]]) -> list[dict[str, Any]]:
    multi = {r["backbone"]: r for r in case_rows if r.get("region_mode") == "multi_region"}
    out = []
    for key, title in ARCHITECTURES:
        src = multi.get(key, {})
        out.append({"architecture": title, "backbone": key, "case_name": src.get("case_name", ""), "status": src.get("status", "missing"),
                    "num_trials": src.get("num_trials", ""), "num_trials_passed": src.get("num_trials_passed", ""),
                    "max_abs_delta_loss": src.get("worst_loss_abs_diff", ""), "grad_linf": src.get("worst_max_abs_grad_diff", ""),
                    "grad_relative_l2": src.get("max_relative_l2_error", ""), "grad_cosine": src.get("min_global_grad_cosine", ""),
                    "skip_reason": src.get("skip_reason", "")})
    return out


def _paper_tex(path: Path, rows: Sequence[dict[str, Any]]) -> None:
    trials = sorted({str(r["num_trials"]) for r in rows if r["num_trials"] not in ("", None)})
    note = f" Each entry is the worst case over {trials[0]} trials." if len(trials) == 1 else ""
    body = [" & ".join([r["architecture"], latex_number(r["max_abs_delta_loss"]), latex_number(r["grad_linf"]),
                        latex_number(r["grad_relative_l2"]), latex_number(r["grad_cosine"], 5)]) + r" \\" for r in rows]
    text = [r"\begin{table}[h!]", r"\centering", r"\begin{tabular}{c|c|c|c|c}",
            r"Architecture & $\max |\Delta\mathcal{L}|$ & $\|\Delta g\|_\infty$ & $\|\Delta g\|_2 / \|g\|_2$ & $\cos \mathrm{sim}$ \\",
            r"\hline", *body, r"\end{tabular}",
            r"\caption{Gradient parity of the exact region-local backward against autograd over multi-region cases." + note + "}",
            r"\label{tab:gradient-parity}", r"\end{table}", ""]
    path.write_text("\n".join(text), encoding="utf-8")


def _cdf(path_stem: Path, aggregates: Sequence[gp.CaseAggregate]) -> None:
    chart = Chart("Multi-region gradient parity error distribution", "per-parameter max relative gradient error", "CDF", logx=True)
    labels = dict(ARCHITECTURES)
    for agg in aggregates:
        if agg.region_mode != "multi_region" or agg.backbone not in labels:
            continue
        vals = sorted(max(m.max_rel_diff, 1e-12) for t in agg.trial_metrics for m in t.parameter_metrics
                      if m.has_ref_grad and m.has_native_grad)
        if vals:
            chart.series.append(Series(labels[agg.backbone], vals, [(i + 1) / len(vals) for i in range(len(vals))]))
    if chart.series:
        chart.save(path_stem, dpi=200)


def generate_report(*, output_dir: Path, case_names: Sequence[str] | None = None, plot: bool = False, preset: str = "report",
                    seeds: Sequence[int] | None = None, batches_per_seed: int | None = None,
                    interface_jacobian_mode: str = "recompute", jacobian_basis_chunk: int = 32,
                    repo_root: Path | None = None) -> list[dict[str, Any]]:
    """``repo_root`` is accepted and unused: the reference's function loads its test module from that directory by path
    (scripts/generate_grad_parity_report.py:211-223), here the cases are an importable module (``utils.grad_parity``)."""
    if interface_jacobian_mode not in {"graph", "recompute", "structured", "forward"}:
        raise ValueError("interface_jacobian_mode must be one of: graph, recompute, structured, forward")
    if jacobian_basis_chunk <= 0:
        raise ValueError("jacobian_basis_chunk must be > 0")
    if batches_per_seed is not None and batches_per_seed <= 0:
        raise ValueError("batches_per_seed must be > 0")
    output_dir.mkdir(parents=True, exist_ok=True)
    use_seeds = tuple(seeds) if seeds is not None else (REPORT_SEEDS if preset == "report" else None)
    use_batches = batches_per_seed if batches_per_seed is not None else (REPORT_BATCHES_PER_SEED if preset == "report" else None)
    case_rows: list[dict[str, Any]] = []
    trial_rows: list[dict[str, Any]] = []
    param_rows: list[dict[str, Any]] = []
    aggregates: list[gp.CaseAggregate] = []
    for case in gp.get_grad_parity_cases(case_names, preset=preset):
        case = dataclasses.replace(case, seeds=use_seeds or case.seeds, batches_per_seed=use_batches or case.batches_per_seed)
        reason = gp.grad_parity_skip_reason(case)
        if reason is not None:
            case_rows.append({"case_name": case.name, "backbone": case.backbone_name, "region_mode": case.region_mode,
                              "region_axis": case.region_axis, "interface_jacobian_mode": interface_jacobian_mode,
                              "jacobian_basis_chunk": jacobian_basis_chunk, "device": case.device_type, "dtype": case.dtype_name,
                              "num_trials": "", "num_trials_passed": "", "worst_loss_abs_diff": "", "min_global_grad_cosine": "",
                              "max_relative_l2_error": "", "worst_max_abs_grad_diff": "", "worst_max_rel_grad_diff": "",
                              "median_p95_rel_grad_diff": "", "worst_interface_scan_rms": "", "status": "skipped", "skip_reason": reason})
            continue
        agg = gp.compute_grad_parity_case_aggregate(case, interface_jacobian_mode=interface_jacobian_mode,
                                                    jacobian_basis_chunk=jacobian_basis_chunk)
        gp.assert_grad_parity_aggregate(case, agg)
        aggregates.append(agg)
        case_rows.append({**agg.to_summary_row(), "status": "ok", "skip_reason": ""})
        for t in agg.trial_metrics:
            trial_rows.append({**t.to_summary_row(), "status": "ok" if t.trial_passed else "failed"})
            param_rows.extend(t.per_parameter_rows())
    for stem in ("case_summary", "summary"):
        write_csv(output_dir / f"{stem}.csv", case_rows)
        write_json(output_dir / f"{stem}.json", case_rows)
        _markdown(output_dir / f"{stem}.md", case_rows)
    write_csv(output_dir / "trial_summary.csv", trial_rows)
    write_csv(output_dir / "per_parameter.csv", param_rows)
    write_json(output_dir / "report_config.json", {
        "preset": preset, "interface_jacobian_mode": interface_jacobian_mode, "jacobian_basis_chunk": jacobian_basis_chunk,
        "seeds": list(use_seeds) if use_seeds else None, "batches_per_seed": use_batches,
        "cases": list(case_names) if case_names else None})
    table = paper_rows(case_rows)
    write_csv(output_dir / "paper_table.csv", table)
    _paper_tex(output_dir / "paper_table.tex", table)
    if plot and aggregates:
        _cdf(output_dir / "grad_rel_error_cdf", aggregates)
    return case_rows


def main(argv: list[str] | None = None) -> None:
    p = argparse.ArgumentParser(description="Generate grad parity summary tables and optional appendix plots.")
    p.add_argument("--output-dir", type=Path, default=Path("out/grad_parity"))
    p.add_argument("--cases", nargs="*", default=None, help="Optional subset of grad parity case names to run.")
    p.add_argument("--preset", choices=("report", "test"), default="report")
    p.add_argument("--plot", action="store_true", help="also write the CDF figure")
    p.add_argument("--seeds", nargs="*", type=int, default=None)
    p.add_argument("--batches-per-seed", type=int, default=None)
    p.add_argument("--interface-jacobian-mode", choices=("graph", "recompute", "structured", "forward"), default="recompute")
    p.add_argument("--jacobian-basis-chunk", type=int, default=32)
    ns = p.parse_args(argv)
    generate_report(output_dir=ns.output_dir, case_names=ns.cases, plot=ns.plot, preset=ns.preset, seeds=ns.seeds,
                    batches_per_seed=ns.batches_per_seed, interface_jacobian_mode=ns.interface_jacobian_mode,
                    jacobian_basis_chunk=ns.jacobian_basis_chunk)


if __name__ == "__main__":
    main()
