"""Tiny chart layer for the plotting scripts.

With matplotlib installed the figures are PNG (and PDF where asked); without it the same series are drawn by a small
built-in SVG writer and saved under the requested stem with an ``.svg`` suffix, so the plotting scripts work on a
machine that only has the training dependencies.  The table outputs (CSV / JSON / TeX) never depend on matplotlib.
"""
from __future__ import annotations

import csv
import json
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Sequence

_PALETTE = ["#1f77b4", "#d62728", "#2ca02c", "#ff7f0e", "#9467bd", "#8c564b", "#e377c2", "#7f7f7f", "#17becf", "#bcbd22"]


def have_matplotlib() -> bool:
    try:
        import matplotlib  # noqa: F401
    except ImportError:
        return False
    return True


@dataclass
class Series:
    """One curve: label, x, y, optional band, line style."""

    label: str
    x: Sequence[float]
    y: Sequence[float]
    band: Sequence[float] | None = None  # half-width of a shaded band around y (e.g. one standard deviation)
    style: str = "-"


@dataclass
class Chart:
    """A figure (curves or bars) that saves through matplotlib when installed and through a built-in SVG writer otherwise."""

    title: str
    xlabel: str
    ylabel: str
    series: list[Series] = field(default_factory=list)
    logx: bool = False
    logy: bool = False
    bars: list[tuple[str, float, float]] | None = None  # (label, height, error) for bar charts

    def save(self, stem: Path, *, dpi: int = 150, font_scale: float = 1.0, also_pdf: bool = False) -> list[Path]:
        stem.parent.mkdir(parents=True, exist_ok=True)
        if have_matplotlib():
            return _save_matplotlib(self, stem, dpi=dpi, font_scale=font_scale, also_pdf=also_pdf)
        path = stem.with_suffix(".svg")
        path.write_text(_render_svg(self, font_scale=font_scale), encoding="utf-8")
        return [path]


def _save_matplotlib(chart: Chart, stem: Path, *, dpi: int, font_scale: float, also_pdf: bool) -> list[Path]:
    import matplotlib

    matplotlib.use("Agg")
    import matplotlib.pyplot as plt

    plt.rcParams.update({"font.size": 10 * font_scale})
    fig, ax = plt.subplots(figsize=(7.5, 4.5))
    if chart.bars is not None:
        names = [b[0] for b in chart.bars]
        ax.bar(range(len(names)), [b[1] for b in chart.bars], yerr=[b[2] for b in chart.bars], capsize=3,
               color=[_PALETTE[i % len(_PALETTE)] for i in range(len(names))])
        ax.set_xticks(range(len(names)))
        ax.set_xticklabels(names, rotation=30, ha="right")
    for i, s in enumerate(chart.series):
        colour = _PALETTE[i % len(_PALETTE)]
        ax.plot(list(s.x), list(s.y), s.style, label=s.label, color=colour)
        if s.band is not None:
            lo = [a - b for a, b in zip(s.y, s.band)]
            hi = [a + b for a, b in zip(s.y, s.band)]
            ax.fill_between(list(s.x), lo, hi, color=colour, alpha=0.2)
    if chart.logx:
        ax.set_xscale("log")
    if chart.logy:
        ax.set_yscale("log")
    ax.set_title(chart.title)
    ax.set_xlabel(chart.xlabel)
    ax.set_ylabel(chart.ylabel)
    ax.grid(True, alpha=0.3)
    if chart.series:
        ax.legend(fontsize=8 * font_scale)
    fig.tight_layout()
    out = [stem.with_suffix(".png")]
    fig.savefig(out[0], dpi=dpi)
    if also_pdf:
        out.append(stem.with_suffix(".pdf"))
        fig.savefig(out[1])
    plt.close(fig)
    return out


def _nice_ticks(lo: float, hi: float, n: int = 5) -> list[float]:
    if not math.isfinite(lo) or not math.isfinite(hi) or hi <= lo:
        return [lo]
    raw = (hi - lo) / n
    mag = 10 ** math.floor(math.log10(raw))
    step = min((m * mag for m in (1, 2, 5, 10)), key=lambda s: abs(s - raw))
    first = math.ceil(lo / step) * step
    ticks, t = [], first
    while t <= hi + 1e-12 * abs(hi):
        ticks.append(round(t, 12))
        t += step
    return ticks


def _render_svg(chart: Chart, *, font_scale: float) -> str:
    width, height, left, right, top, bottom = 760, 460, 70, 170, 40, 60
    pw, ph = width - left - right, height - top - bottom
    fs = 11 * font_scale

    def tx(v: float) -> float:
        return math.log10(max(v, 1e-300)) if chart.logx else v

    def ty(v: float) -> float:
        return math.log10(max(v, 1e-300)) if chart.logy else v

    xs: list[float] = []
    ys: list[float] = []
    if chart.bars is not None:
        xs = [0.0, float(len(chart.bars))]
        ys = [0.0] + [b[1] + b[2] for b in chart.bars]
    for s in chart.series:
        for i, (a, b) in enumerate(zip(s.x, s.y)):
            if math.isfinite(a) and math.isfinite(b):
                xs.append(tx(a))
                half = s.band[i] if s.band is not None else 0.0
                ys.extend([ty(b - half) if (b - half) > 0 or not chart.logy else ty(b), ty(b + half)])
    if not xs:
        xs, ys = [0.0, 1.0], [0.0, 1.0]
    x0, x1, y0, y1 = min(xs), max(xs), min(ys), max(ys)
    if x1 == x0:
        x1 = x0 + 1.0
    if y1 == y0:
        y1 = y0 + 1.0
    pad = 0.04 * (y1 - y0)
    y0, y1 = y0 - pad, y1 + pad

    def px(v: float) -> float:
        return left + (tx(v) - x0) / (x1 - x0) * pw

    def py(v: float) -> float:
        return top + ph - (ty(v) - y0) / (y1 - y0) * ph

    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-family="sans-serif" font-size="{fs:.1f}">',
           f'<rect width="{width}" height="{height}" fill="white"/>',
           f'<rect x="{left}" y="{top}" width="{pw}" height="{ph}" fill="none" stroke="#444"/>',
           f'<text x="{left + pw / 2}" y="{top - 14}" text-anchor="middle" font-size="{fs * 1.15:.1f}">{_esc(chart.title)}</text>',
           f'<text x="{left + pw / 2}" y="{height - 14}" text-anchor="middle">{_esc(chart.xlabel)}</text>',
           f'<text x="16" y="{top + ph / 2}" text-anchor="middle" transform="rotate(-90 16 {top + ph / 2})">{_esc(chart.ylabel)}</text>']
    for t in _nice_ticks(y0, y1):
        yy = top + ph - (t - y0) / (y1 - y0) * ph
        label = f"1e{t:g}" if chart.logy else f"{t:g}"
        out.append(f'<line x1="{left}" x2="{left + pw}" y1="{yy:.1f}" y2="{yy:.1f}" stroke="#ddd"/>')
        out.append(f'<text x="{left - 6}" y="{yy + 4:.1f}" text-anchor="end">{label}</text>')
    if chart.bars is None:
        for t in _nice_ticks(x0, x1):
            xx = left + (t - x0) / (x1 - x0) * pw
            label = f"1e{t:g}" if chart.logx else f"{t:g}"
            out.append(f'<line y1="{top}" y2="{top + ph}" x1="{xx:.1f}" x2="{xx:.1f}" stroke="#eee"/>')
            out.append(f'<text x="{xx:.1f}" y="{top + ph + 16}" text-anchor="middle">{label}</text>')
    else:
        bw = pw / max(1, len(chart.bars))
        for i, (name, h, err) in enumerate(chart.bars):
            colour = _PALETTE[i % len(_PALETTE)]
            xa = left + i * bw + 0.15 * bw
            ya, yb = py(h), py(0.0 if y0 <= 0 <= y1 else y0)
            out.append(f'<rect x="{xa:.1f}" y="{min(ya, yb):.1f}" width="{0.7 * bw:.1f}" height="{abs(yb - ya):.1f}" fill="{colour}"/>')
            if err:
                xm = xa + 0.35 * bw
                out.append(f'<line x1="{xm:.1f}" x2="{xm:.1f}" y1="{py(h - err):.1f}" y2="{py(h + err):.1f}" stroke="#000"/>')
            out.append(f'<text x="{xa + 0.35 * bw:.1f}" y="{top + ph + 16}" text-anchor="middle" font-size="{fs * 0.8:.1f}">{_esc(name)}</text>')
    for i, s in enumerate(chart.series):
        colour = _PALETTE[i % len(_PALETTE)]
        pts = [(px(a), py(b)) for a, b in zip(s.x, s.y) if math.isfinite(a) and math.isfinite(b) and (b > 0 or not chart.logy)]
        if s.band is not None and len(pts) > 1:
            upper = [(px(a), py(b + h)) for a, b, h in zip(s.x, s.y, s.band)]
            lower = [(px(a), py(max(b - h, 1e-300) if chart.logy else b - h)) for a, b, h in zip(s.x, s.y, s.band)]
            poly = " ".join(f"{x:.1f},{y:.1f}" for x, y in upper + lower[::-1])
            out.append(f'<polygon points="{poly}" fill="{colour}" opacity="0.18"/>')
        if pts:
            dash = ' stroke-dasharray="5,3"' if s.style == "--" else ""
            out.append(f'<polyline fill="none" stroke="{colour}" stroke-width="1.6"{dash} points="' +
                       " ".join(f"{x:.1f},{y:.1f}" for x, y in pts) + '"/>')
        ly = top + 14 + 16 * i
        out.append(f'<line x1="{left + pw + 10}" x2="{left + pw + 34}" y1="{ly}" y2="{ly}" stroke="{colour}" stroke-width="2"/>')
        out.append(f'<text x="{left + pw + 40}" y="{ly + 4}">{_esc(s.label)}</text>')
    out.append("</svg>")
    return "\n".join(out)


def _esc(text: str) -> str:
    return str(text).replace("&", "&amp;").replace("<", "&lt;").replace(">", "&gt;")


# ---------------------------------------------------------------------------------------------- shared table helpers
def write_csv(path: Path, rows: Sequence[dict[str, Any]]) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    with path.open("w", newline="", encoding="utf-8") as fh:
        if rows:
            w = csv.DictWriter(fh, fieldnames=list(rows[0]))
            w.writeheader()
            w.writerows(rows)


def write_json(path: Path, obj: Any) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(json.dumps(obj, indent=2, sort_keys=True) + "\n", encoding="utf-8")


def mean_std(values: Sequence[float]) -> tuple[float, float]:
    vals = [float(v) for v in values if v is not None and math.isfinite(float(v))]
    if not vals:
        return float("nan"), float("nan")
    m = sum(vals) / len(vals)
    var = sum((v - m) ** 2 for v in vals) / (len(vals) - 1) if len(vals) > 1 else 0.0
    return m, math.sqrt(var)


def moving_average(values: Sequence[float], window: int) -> list[float]:
    if window <= 1:
        return [float(v) for v in values]
    out, acc, q = [], 0.0, []
    for v in values:
        q.append(float(v))
        acc += float(v)
        if len(q) > window:
            acc -= q.pop(0)
        out.append(acc / len(q))
    return out
