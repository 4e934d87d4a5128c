"""Exposure-position curves of the paired attributes (company and company city).

In a permuted biography the company city is determined by the company.  If a P-whole probe at read-out position k can use
whichever of the pair has already been mentioned, its accuracy should grow with the probability that the partner
attribute lies among the k sentences already read: with six sentences in random order that probability is
``1 - C(4, k) / C(6, k)`` for k <= 4 and 1 afterwards.  Each attribute's curve is fitted as ``baseline + gain * exposure``
by least squares, with a leave-one-out error, which separates the paired attributes (large gain) from the independent
ones (reference: experiments/synbios_moe/mechanisms/company_relation.py:54-277).
"""

from __future__ import annotations

import csv
import math
from pathlib import Path
from typing import Mapping, Sequence

import numpy as np

from experiments.synbios_moe.artifact_io import write_csv, write_json
from experiments.synbios_moe.pretraining.dataset import WHOLE_ATTRIBUTES

PAIR = ("company", "company_city")


def paired_exposure(positions: int = 6, partners: int = 1) -> np.ndarray:
    """P(the partner sentence is among the first k) for k = 0..positions-1 when ``positions`` sentences are shuffled and the
    probed one is excluded from the ``k`` already read (the reference counts two fixed slots: name sentence and the probed
    attribute, hence C(4, k) / C(6, k))."""

    total, free = positions, positions - 1 - partners
    return np.asarray([1.0 - math.comb(free, k) / math.comb(total, k) if k <= free else 1.0 for k in range(positions)], dtype=np.float64)


def fit_exposure_curve(y: Sequence[float], x: Sequence[float]) -> dict:
    y, x = np.asarray(y, dtype=np.float64), np.asarray(x, dtype=np.float64)
    if y.shape != x.shape or y.ndim != 1 or y.size < 3:
        raise ValueError("need two equally long curves of at least three points")
    design = np.column_stack([np.ones_like(x), x])
    coef = np.linalg.lstsq(design, y, rcond=None)[0]
    pred = design @ coef
    rss = float(np.sum((y - pred) ** 2))
    tss = float(np.sum((y - y.mean()) ** 2))
    loo = []
    for held in range(y.size):
        keep = np.arange(y.size) != held
        c = np.linalg.lstsq(design[keep], y[keep], rcond=None)[0]
        loo.append(float(y[held] - design[held] @ c))
    return {"baseline": float(coef[0]), "gain": float(coef[1]), "saturation": float(coef.sum()), "prediction": pred.tolist(),
            "rmse": math.sqrt(rss / y.size), "r_squared": 1.0 - rss / tss if tss else None,
            "leave_one_out_rmse": math.sqrt(float(np.mean(np.square(loo))))}


def load_position_curves(path: str | Path, *, condition: str | None = None) -> dict[str, np.ndarray]:
    """P-whole accuracy by position per attribute from a tidy CSV (columns: attribute, kind, target, position, accuracy and
    optionally condition / split) as written by the formal comparison report."""

    curves: dict[str, dict[int, float]] = {}
    with open(path, encoding="utf-8", newline="") as fh:
        for row in csv.DictReader(fh):
            if row.get("kind") != "p" or row.get("target") != "whole":
                continue
            if condition is not None and row.get("condition") not in (None, "", condition):
                continue
            if row.get("split") not in (None, "", "person_held_out_validation", "validation"):
                continue
            curves.setdefault(row["attribute"], {})[int(row["position"])] = float(row["accuracy"])
    missing = [a for a in WHOLE_ATTRIBUTES if set(curves.get(a, {})) != set(range(6))]
    if missing:
        raise ValueError(f"incomplete P-whole curves for: {missing}")
    return {a: np.asarray([curves[a][i] for i in range(6)]) for a in WHOLE_ATTRIBUTES}


def fit_company_pair(curves: Mapping[str, Sequence[float]], output_dir: str | Path | None = None) -> dict:
    """Fit every whole attribute; report the pair's gains against the largest gain of an unpaired attribute."""

    x = paired_exposure()
    fits = {a: fit_exposure_curve(curves[a], x) for a in WHOLE_ATTRIBUTES}
    unpaired = [a for a in WHOLE_ATTRIBUTES if a not in PAIR]
    summary = {"exposure": x.tolist(), "fits": fits, "pair": list(PAIR),
               "pair_mean_gain": float(np.mean([fits[a]["gain"] for a in PAIR])),
               "unpaired_max_gain": float(max(fits[a]["gain"] for a in unpaired)) if unpaired else None}
    if output_dir is not None:
        out = Path(output_dir)
        out.mkdir(parents=True, exist_ok=True)
        rows = [{"attribute": a, **{k: fits[a][k] for k in ("baseline", "gain", "saturation", "rmse", "r_squared", "leave_one_out_rmse")},
                 "observed_p0": float(curves[a][0]), "observed_p5": float(curves[a][5])} for a in WHOLE_ATTRIBUTES]
        write_csv(out / "company_relation_metrics.csv", rows,
                  ["attribute", "baseline", "gain", "saturation", "rmse", "r_squared", "leave_one_out_rmse", "observed_p0", "observed_p5"])
        write_json(out / "company_relation.json", summary)
        from experiments.synbios_moe.artifact_io import write_text
        from experiments.synbios_moe.probes.figures import line_chart_svg

        series, dashed = {}, []
        for a in PAIR:
            series[f"{a}: observed"] = [float(v) for v in curves[a]]
            series[f"{a}: fit"] = [float(v) for v in fits[a]["prediction"]]
            dashed.append(f"{a}: fit")
        series["partner exposure"] = x.tolist()
        dashed.append("partner exposure")
        write_text(out / "company_relation.svg", line_chart_svg(series, title="P-whole accuracy of the paired attributes against partner exposure",
                                                                x_labels=[f"P{i}" for i in range(6)], dashed=dashed))
    return summary
