"""Figures of the probe comparison without a plotting library.

The study's figures are small annotated grids (accuracy of a probe per attribute and biography position) and one grouped
bar chart.  They are written as SVG (text: labels, values and a colour scale, viewable in any browser and diffable) with
a PNG twin of each grid encoded by ``runtime.logger.encode_png_rgb`` for tools that want a raster.  What the figures
show follows the reference's ``plot_p_heatmaps`` / ``plot_q_table`` / ``plot_overview``
(experiments/synbios_moe/probes/comparison_report.py:389-553): P-probe grids of both conditions side by side per target,
the Q-probe table (condition x attribute) per target, and an overview of the headline end points.
"""

from __future__ import annotations

from pathlib import Path
from typing import Sequence
from xml.sax.saxutils import escape

import torch

from experiments.synbios_moe.artifact_io import write_text
from experiments.synbios_moe.pretraining.dataset import ATTRIBUTES, WHOLE_ATTRIBUTES

CONDITION_LABELS = {"single": "Single biography", "multi5_permute": "5x paraphrase + permutation"}
_FONT = "font-family='Helvetica,Arial,sans-serif'"


def accuracy_colour(value: float) -> tuple[int, int, int]:
    """Sequential white -> deep teal scale over [0, 1]; out-of-range values are clamped."""

    v = min(max(float(value), 0.0), 1.0)
    lo, hi = (247, 251, 255), (8, 88, 110)
    return tuple(int(round(a + (b - a) * v)) for a, b in zip(lo, hi))


def _hex(rgb: tuple[int, int, int]) -> str:
    return "#%02x%02x%02x" % rgb


def grid_svg(matrix: Sequence[Sequence[float]], *, row_labels: Sequence[str], col_labels: Sequence[str], title: str,
             x0: int = 0, y0: int = 0, cell: int = 64, label_width: int = 130, outlined: Sequence[tuple[int, int]] = ()) -> tuple[str, int, int]:
    """One annotated grid as an SVG fragment placed at (x0, y0); returns (fragment, width, height).  Values are fractions,
    printed as percentages; ``outlined`` cells get a dark frame."""

    rows, cols = len(matrix), len(matrix[0]) if matrix else 0
    if len(row_labels) != rows or len(col_labels) != cols:
        raise ValueError("labels do not match the matrix")
    top = 34
    parts = [f"<text x='{x0 + label_width}' y='{y0 + 18}' {_FONT} font-size='15' font-weight='bold'>{escape(title)}</text>"]
    for r in range(rows):
        y = y0 + top + r * cell
        parts.append(f"<text x='{x0 + label_width - 8}' y='{y + cell // 2 + 5}' {_FONT} font-size='13' text-anchor='end'>{escape(row_labels[r])}</text>")
        for c in range(cols):
            x = x0 + label_width + c * cell
            value = float(matrix[r][c])
            rgb = accuracy_colour(value)
            ink = "#ffffff" if value > 0.55 else "#1b1b1b"
            frame = " stroke='#111111' stroke-width='3'" if (r, c) in outlined else " stroke='#ffffff' stroke-width='1'"
            parts.append(f"<rect x='{x}' y='{y}' width='{cell}' height='{cell}' fill='{_hex(rgb)}'{frame}/>")
            parts.append(f"<text x='{x + cell // 2}' y='{y + cell // 2 + 5}' {_FONT} font-size='13' text-anchor='middle' fill='{ink}'>{100 * value:.1f}</text>")
    for c in range(cols):
        x = x0 + label_width + c * cell + cell // 2
        parts.append(f"<text x='{x}' y='{y0 + top + rows * cell + 18}' {_FONT} font-size='13' text-anchor='middle'>{escape(col_labels[c])}</text>")
    return "\n".join(parts), label_width + cols * cell, top + rows * cell + 28


def colour_bar_svg(x0: int, y0: int, height: int) -> tuple[str, int]:
    steps = 50
    parts = []
    for k in range(steps):
        v = 1.0 - k / (steps - 1)
        parts.append(f"<rect x='{x0}' y='{y0 + k * height / steps:.1f}' width='16' height='{height / steps + 0.6:.1f}' fill='{_hex(accuracy_colour(v))}'/>")
    for v in (0.0, 0.5, 1.0):
        parts.append(f"<text x='{x0 + 22}' y='{y0 + (1.0 - v) * height + 4:.1f}' {_FONT} font-size='11'>{100 * v:.0f}</text>")
    parts.append(f"<text x='{x0}' y='{y0 - 8}' {_FONT} font-size='11'>Accuracy (%)</text>")
    return "\n".join(parts), 60


def wrap_svg(body: str, width: int, height: int, title: str) -> str:
    return (f"<svg xmlns='http://www.w3.org/2000/svg' width='{width}' height='{height}' viewBox='0 0 {width} {height}'>\n"
            f"<rect width='{width}' height='{height}' fill='#ffffff'/>\n"
            f"<text x='{width // 2}' y='26' {_FONT} font-size='19' font-weight='bold' text-anchor='middle'>{escape(title)}</text>\n{body}\n</svg>\n")


def grid_png(matrix: Sequence[Sequence[float]], cell: int = 24) -> bytes:
    """The same grid as a bare raster (no text): ``cell`` pixels per entry."""

    from mini_train_sys_b200.runtime.logger import encode_png_rgb

    rows, cols = len(matrix), len(matrix[0])
    pixels = torch.zeros(rows * cell, cols * cell, 3, dtype=torch.uint8)
    for r in range(rows):
        for c in range(cols):
            pixels[r * cell:(r + 1) * cell, c * cell:(c + 1) * cell] = torch.tensor(accuracy_colour(matrix[r][c]), dtype=torch.uint8)
    return encode_png_rgb(pixels)


def _lookup(rows: Sequence[dict], condition: str, kind: str, target: str, attribute: str, position: int) -> float:
    hits = [r["accuracy"] for r in rows if (r["condition"], r["kind"], r["target"], r["attribute"], r["position"], r["split"]) ==
            (condition, kind, target, attribute, position, "person_held_out_validation")]
    if len(hits) != 1:
        raise ValueError(f"expected one held-out accuracy for {condition}/{kind}/{target}/{attribute}/P{position}, found {len(hits)}")
    return float(hits[0])


def probe_matrix(rows: Sequence[dict], condition: str, kind: str, target: str) -> list[list[float]]:
    attributes = ATTRIBUTES if target == "first" else WHOLE_ATTRIBUTES
    positions = range(6) if kind == "p" else range(1)
    return [[_lookup(rows, condition, kind, target, a, p) for p in positions] for a in attributes]


def p_heatmaps_svg(rows: Sequence[dict], target: str) -> str:
    attributes = ATTRIBUTES if target == "first" else WHOLE_ATTRIBUTES
    body, x, height = [], 10, 0
    for condition in ("single", "multi5_permute"):
        # in the single-biography corpus attribute i always sits at position i: those cells are the ones a P probe can read
        outlined = [(i, ATTRIBUTES.index(a)) for i, a in enumerate(attributes)] if condition == "single" and target == "whole" else ()
        frag, w, h = grid_svg(probe_matrix(rows, condition, "p", target), row_labels=[a.replace("_", " ") for a in attributes],
                              col_labels=[f"P{i}" for i in range(6)], title=CONDITION_LABELS[condition], x0=x, y0=40, outlined=outlined)
        body.append(frag)
        x += w + 30
        height = max(height, h)
    bar, bw = colour_bar_svg(x, 90, height - 80)
    body.append(bar)
    label = "first-token" if target == "first" else "whole-attribute"
    return wrap_svg("\n".join(body), x + bw + 10, height + 60, f"P-probe: {label} held-out accuracy by biography position")


def q_table_svg(rows: Sequence[dict], target: str) -> str:
    attributes = ATTRIBUTES if target == "first" else WHOLE_ATTRIBUTES
    matrix = [[_lookup(rows, c, "q", target, a, 0) for a in attributes] for c in ("single", "multi5_permute")]
    frag, w, h = grid_svg(matrix, row_labels=[CONDITION_LABELS[c] for c in ("single", "multi5_permute")],
                          col_labels=[a.replace("_", " ") for a in attributes], title="", x0=10, y0=40, cell=96, label_width=220)
    bar, bw = colour_bar_svg(w + 40, 90, h - 80)
    label = "first-token" if target == "first" else "whole-attribute"
    return wrap_svg(frag + "\n" + bar, w + bw + 60, h + 60, f"Q-probe: {label} held-out accuracy")


def overview_svg(headline: dict) -> str:
    """Grouped bars of the headline end points (single against multi5+permute)."""

    keys = list(headline["single"])
    colours = {"single": "#9b6a50", "multi5_permute": "#138a82"}
    left, base, bar_w, gap, scale = 60, 330, 26, 46, 2.6
    parts = [f"<line x1='{left}' y1='{base}' x2='{left + len(keys) * (2 * bar_w + gap) + 10}' y2='{base}' stroke='#333333'/>"]
    for tick in (0, 25, 50, 75, 100):
        y = base - tick * scale
        parts.append(f"<text x='{left - 8}' y='{y + 4}' {_FONT} font-size='11' text-anchor='end'>{tick}</text>")
        parts.append(f"<line x1='{left}' y1='{y}' x2='{left + len(keys) * (2 * bar_w + gap) + 10}' y2='{y}' stroke='#dddddd'/>")
    for n, key in enumerate(keys):
        x = left + 14 + n * (2 * bar_w + gap)
        for k, condition in enumerate(("single", "multi5_permute")):
            value = 100 * float(headline[condition][key])
            parts.append(f"<rect x='{x + k * bar_w}' y='{base - value * scale:.1f}' width='{bar_w - 2}' height='{value * scale:.1f}' fill='{colours[condition]}'/>")
            parts.append(f"<text x='{x + k * bar_w + bar_w // 2 - 1}' y='{base - value * scale - 4:.1f}' {_FONT} font-size='10' text-anchor='middle'>{value:.1f}</text>")
        words = key.replace("_", " ")
        for line_no, chunk in enumerate([words[i:i + 18] for i in range(0, len(words), 18)][:4]):
            parts.append(f"<text x='{x + bar_w}' y='{base + 16 + 12 * line_no}' {_FONT} font-size='10' text-anchor='middle'>{escape(chunk)}</text>")
    for k, condition in enumerate(("single", "multi5_permute")):
        parts.append(f"<rect x='{left + 10 + 260 * k}' y='44' width='14' height='14' fill='{colours[condition]}'/>")
        parts.append(f"<text x='{left + 30 + 260 * k}' y='56' {_FONT} font-size='12'>{escape(CONDITION_LABELS[condition])}</text>")
    width = left + len(keys) * (2 * bar_w + gap) + 40
    return wrap_svg("\n".join(parts), width, base + 80, "Headline end points (held-out accuracy, %)")


def write_probe_figures(rows: Sequence[dict], headline: dict, output_dir: str | Path) -> list[str]:
    """All figures of one comparison under ``<output_dir>/figures``; returns the file names written."""

    out = Path(output_dir) / "figures"
    out.mkdir(parents=True, exist_ok=True)
    written = []
    for target in ("first", "whole"):
        write_text(out / f"p_{target}_heatmaps.svg", p_heatmaps_svg(rows, target))
        write_text(out / f"q_{target}_table.svg", q_table_svg(rows, target))
        written += [f"p_{target}_heatmaps.svg", f"q_{target}_table.svg"]
        for condition in ("single", "multi5_permute"):
            name = f"p_{target}_{condition}.png"
            (out / name).write_bytes(grid_png(probe_matrix(rows, condition, "p", target)))
            written.append(name)
    write_text(out / "overview.svg", overview_svg(headline))
    written.append("overview.svg")
    return written


_SERIES_COLOURS = ("#138a82", "#9b6a50", "#3b5ba5", "#c0392b", "#7d3c98", "#d68910", "#2e4053", "#1e8449")


def line_chart_svg(series: dict[str, Sequence[float]], *, title: str, x_labels: Sequence[str], y_label: str = "Accuracy (%)",
                   dashed: Sequence[str] = (), percent: bool = True, width: int = 640, height: int = 380) -> str:
    """Curves over a shared categorical x axis (e.g. the six biography positions).  Values are fractions shown as percentages
    when ``percent``; series named in ``dashed`` are drawn dashed (fits, baselines)."""

    if not series or any(len(v) != len(x_labels) for v in series.values()):
        raise ValueError("every series needs one value per x label")
    left, top, right, bottom = 64, 50, 170, 46
    plot_w, plot_h = width - left - right, height - top - bottom
    scale = 100.0 if percent else 1.0
    lo = min(0.0, min(min(v) for v in series.values()) * scale)
    hi = max(max(max(v) for v in series.values()) * scale, lo + 1e-9)
    if percent:
        hi = max(hi, 100.0) if hi > 50.0 else hi * 1.1

    def sx(i: int) -> float:
        return left + (plot_w * i / max(len(x_labels) - 1, 1))

    def sy(v: float) -> float:
        return top + plot_h * (1.0 - (v * scale - lo) / (hi - lo))

    parts = [f"<rect x='{left}' y='{top}' width='{plot_w}' height='{plot_h}' fill='#fbfcfe' stroke='#cccccc'/>"]
    for k in range(5):
        v = lo + (hi - lo) * k / 4
        y = top + plot_h * (1 - k / 4)
        parts.append(f"<line x1='{left}' y1='{y:.1f}' x2='{left + plot_w}' y2='{y:.1f}' stroke='#e4e7ec'/>")
        parts.append(f"<text x='{left - 8}' y='{y + 4:.1f}' {_FONT} font-size='11' text-anchor='end'>{v:.0f}</text>")
    for i, label in enumerate(x_labels):
        parts.append(f"<text x='{sx(i):.1f}' y='{top + plot_h + 18}' {_FONT} font-size='12' text-anchor='middle'>{escape(label)}</text>")
    parts.append(f"<text x='16' y='{top + plot_h / 2:.0f}' {_FONT} font-size='12' transform='rotate(-90 16 {top + plot_h / 2:.0f})' text-anchor='middle'>{escape(y_label)}</text>")
    for n, (name, values) in enumerate(series.items()):
        colour = _SERIES_COLOURS[n % len(_SERIES_COLOURS)]
        points = " ".join(f"{sx(i):.1f},{sy(float(v)):.1f}" for i, v in enumerate(values))
        dash = " stroke-dasharray='6 4'" if name in dashed else ""
        parts.append(f"<polyline points='{points}' fill='none' stroke='{colour}' stroke-width='2'{dash}/>")
        if name not in dashed:
            parts += [f"<circle cx='{sx(i):.1f}' cy='{sy(float(v)):.1f}' r='3' fill='{colour}'/>" for i, v in enumerate(values)]
        ly = top + 14 + 18 * n
        parts.append(f"<line x1='{left + plot_w + 12}' y1='{ly - 4}' x2='{left + plot_w + 36}' y2='{ly - 4}' stroke='{colour}' stroke-width='2'{dash}/>")
        parts.append(f"<text x='{left + plot_w + 42}' y='{ly}' {_FONT} font-size='11'>{escape(name)}</text>")
    return wrap_svg("\n".join(parts), width, height, title)
