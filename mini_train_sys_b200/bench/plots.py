"""Plots of operator-benchmark tables without a plotting library.

One SVG per kernel: a row of panels (forward, forward+backward, backward latency and the speed-up over the library back end),
every panel with one curve per provider over the token sizes on a log2 axis.  The reference draws the same views with
matplotlib (``plot_kernel`` / ``plot_kernel_grid``, benchmarks/operators/measurement.py:917-1040); SVG is text, needs no
dependency and opens in a browser.
"""

from __future__ import annotations

import math
from pathlib import Path
from typing import Sequence
from xml.sax.saxutils import escape

PROVIDER_COLOURS = {"torch": "#3b6ea8", "native": "#2e8b57", "reference": "#8a8a8a", "triton": "#e87722", "cuda": "#2e8b57"}
METRICS = (("fwd_ms", "forward (ms)"), ("full_ms", "forward + backward (ms)"), ("bwd_ms", "backward (ms)"),
           ("speedup_full", "speed-up over torch (x)"))
_FONT = "font-family='Helvetica,Arial,sans-serif'"


def _nice(v: float) -> str:
    return f"{v:.3g}"


def panel_svg(rows: Sequence[dict], metric: str, label: str, *, x0: int, y0: int, width: int = 300, height: int = 220) -> str:
    """One metric of one kernel: provider curves over ``tokens`` (log2 x, linear y from 0)."""

    points: dict[str, list[tuple[int, float]]] = {}
    for r in rows:
        v = r.get(metric)
        if v is None or not math.isfinite(float(v)):
            continue
        points.setdefault(str(r["provider"]), []).append((int(r["tokens"]), float(v)))
    left, top, right, bottom = 52, 26, 10, 34
    pw, ph = width - left - right, height - top - bottom
    parts = [f"<rect x='{x0 + left}' y='{y0 + top}' width='{pw}' height='{ph}' fill='#fbfbfd' stroke='#cfcfd6'/>",
             f"<text x='{x0 + left}' y='{y0 + 16}' {_FONT} font-size='12' font-weight='bold'>{escape(label)}</text>"]
    if not points:
        parts.append(f"<text x='{x0 + left + pw // 2}' y='{y0 + top + ph // 2}' {_FONT} font-size='11' text-anchor='middle' fill='#888888'>no data</text>")
        return "\n".join(parts)
    sizes = sorted({t for pts in points.values() for t, _ in pts})
    lo, hi = math.log2(sizes[0]), math.log2(sizes[-1])
    top_value = max(v for pts in points.values() for _, v in pts) * 1.08 or 1.0

    def sx(tokens: int) -> float:
        return x0 + left + (pw / 2 if hi == lo else pw * (math.log2(tokens) - lo) / (hi - lo))

    def sy(v: float) -> float:
        return y0 + top + ph * (1.0 - v / top_value)

    for k in range(5):
        v = top_value * k / 4
        parts.append(f"<line x1='{x0 + left}' y1='{sy(v):.1f}' x2='{x0 + left + pw}' y2='{sy(v):.1f}' stroke='#e6e6ec'/>")
        parts.append(f"<text x='{x0 + left - 6}' y='{sy(v) + 4:.1f}' {_FONT} font-size='10' text-anchor='end'>{_nice(v)}</text>")
    for t in sizes:
        parts.append(f"<text x='{sx(t):.1f}' y='{y0 + top + ph + 14}' {_FONT} font-size='10' text-anchor='middle'>{t}</text>")
    if metric.startswith("speedup"):
        parts.append(f"<line x1='{x0 + left}' y1='{sy(1.0):.1f}' x2='{x0 + left + pw}' y2='{sy(1.0):.1f}' stroke='#999999' stroke-dasharray='4 3'/>")
    for provider, pts in sorted(points.items()):
        pts.sort()
        colour = PROVIDER_COLOURS.get(provider, "#444444")
        path = " ".join(f"{sx(t):.1f},{sy(v):.1f}" for t, v in pts)
        parts.append(f"<polyline points='{path}' fill='none' stroke='{colour}' stroke-width='2'/>")
        parts += [f"<circle cx='{sx(t):.1f}' cy='{sy(v):.1f}' r='2.8' fill='{colour}'><title>{escape(provider)} {t}: {_nice(v)}</title></circle>" for t, v in pts]
    return "\n".join(parts)


def kernel_grid_svg(rows: Sequence[dict], kernel: str, *, metrics=METRICS) -> str:
    """All panels of one kernel side by side with a shared legend."""

    mine = [r for r in rows if r.get("kernel") == kernel]
    width, height = 300, 220
    body = [panel_svg(mine, metric, label, x0=10 + n * (width + 6), y0=58, width=width, height=height) for n, (metric, label) in enumerate(metrics)]
    providers = sorted({str(r["provider"]) for r in mine})
    for n, provider in enumerate(providers):
        x = 20 + 120 * n
        body.append(f"<line x1='{x}' y1='44' x2='{x + 22}' y2='44' stroke='{PROVIDER_COLOURS.get(provider, '#444444')}' stroke-width='3'/>")
        body.append(f"<text x='{x + 28}' y='48' {_FONT} font-size='12'>{escape(provider)}</text>")
    total_w = 20 + len(metrics) * (width + 6)
    profile = next((str(r.get("profile")) for r in mine if r.get("profile")), "")
    title = f"{kernel} ({profile}): latency by tokens" if profile else f"{kernel}: latency by tokens"
    return (f"<svg xmlns='http://www.w3.org/2000/svg' width='{total_w}' height='{height + 70}' viewBox='0 0 {total_w} {height + 70}'>\n"
            f"<rect width='{total_w}' height='{height + 70}' fill='#ffffff'/>\n"
            f"<text x='{total_w // 2}' y='24' {_FONT} font-size='16' font-weight='bold' text-anchor='middle'>{escape(title)}</text>\n"
            + "\n".join(body) + "\n</svg>\n")


def write_kernel_plots(table: Sequence[dict], directory: str | Path) -> list[str]:
    """One ``<kernel>.svg`` per kernel of a headline table (``bench.operators.headline_table``); returns the file names."""

    out = Path(directory)
    out.mkdir(parents=True, exist_ok=True)
    written = []
    for kernel in sorted({str(r["kernel"]) for r in table}):
        (out / f"{kernel}.svg").write_text(kernel_grid_svg(table, kernel), encoding="utf-8")
        written.append(f"{kernel}.svg")
    return written
