"""Report of a ground-truth-first whole-probe run against the original P probes.

Inputs: ``<run_dir>/<attribute>.json`` (one record per attribute from ``train_ground_truth_first_whole_probe``) and the
pipeline root with the original ``p-<attribute>-first`` / ``p-<attribute>-whole`` results.  Output: one row per
(attribute, source position) with the original first-token accuracy, the original whole accuracy, the whole accuracy after
the true first token was appended and the gain in points; a CSV, a JSON summary, a Markdown table and a line figure
(reference: experiments/synbios_moe/mechanisms/intervention_report.py:22-424).
"""

from __future__ import annotations

from pathlib import Path

from experiments.synbios_moe.artifact_io import read_json, write_csv, write_json, write_text
from experiments.synbios_moe.pretraining.dataset import WHOLE_ATTRIBUTES
from experiments.synbios_moe.probes.commands import job_name


def _baseline(probe_root: Path, attribute: str, target: str) -> list[float]:
    name = job_name("p", attribute, target)
    for path in (probe_root / "validation" / f"{name}.json", probe_root / "training" / f"{name}.json", probe_root / f"{name}.json"):
        if path.is_file():
            val = read_json(path).get("validation") or {}
            curve = val.get("accuracy_by_position")
            if curve and len(curve) == 6:
                return [float(v) for v in curve]
    raise FileNotFoundError(f"no P {target} result of {attribute!r} with six positions under {probe_root}")


def _mean(values) -> float | None:
    values = [v for v in values if v is not None]
    return sum(values) / len(values) if values else None


def _pct(value: float | None) -> str:
    return "n/a" if value is None else f"{100 * value:.1f}"


def summarize_ground_truth_first_whole(run_dir: str | Path, probe_root: str | Path, output_dir: str | Path | None = None) -> dict:
    run, probes = Path(run_dir), Path(probe_root)
    out = Path(output_dir) if output_dir is not None else run / "report"
    rows, missing = [], []
    for attribute in WHOLE_ATTRIBUTES:
        path = run / f"{attribute}.json"
        if not path.is_file():
            missing.append(attribute)
            continue
        rec = read_json(path)
        after = rec["whole_accuracy_validation_by_source_position"]
        first, whole = _baseline(probes, attribute, "first"), _baseline(probes, attribute, "whole")
        for position in range(6):
            rows.append({"attribute": attribute, "position": position, "first_accuracy": first[position], "whole_accuracy": whole[position],
                         "whole_accuracy_ground_truth_first": float(after[position]),
                         "gain_points": 100 * (float(after[position]) - whole[position]), "steps": rec.get("steps"),
                         "rank": rec.get("reference_rank")})
    by_attribute = []
    for attribute in WHOLE_ATTRIBUTES:
        part = [r for r in rows if r["attribute"] == attribute]
        if part:
            by_attribute.append({"attribute": attribute, "whole_accuracy": _mean(r["whole_accuracy"] for r in part),
                                 "whole_accuracy_ground_truth_first": _mean(r["whole_accuracy_ground_truth_first"] for r in part),
                                 "gain_points": _mean(r["gain_points"] for r in part),
                                 "gain_points_p0": part[0]["gain_points"], "gain_points_p5": part[-1]["gain_points"]})
    summary = {"protocol": "ground_truth_first_whole_report_v1", "run_dir": str(run.resolve()), "probe_root": str(probes.resolve()),
               "attributes_reported": [r["attribute"] for r in by_attribute], "attributes_missing": missing,
               "mean_gain_points": _mean(r["gain_points"] for r in rows), "by_attribute": by_attribute}
    out.mkdir(parents=True, exist_ok=True)
    write_csv(out / "by_position.csv", rows, ["attribute", "position", "first_accuracy", "whole_accuracy",
                                               "whole_accuracy_ground_truth_first", "gain_points", "steps", "rank"])
    write_json(out / "summary.json", summary)
    lines = ["# Whole-value read-out after the true first token", "",
             "| attribute | whole (original) % | whole (+ true first token) % | gain (points) | gain at P0 | gain at P5 |", "|---|---:|---:|---:|---:|---:|"]
    for r in by_attribute:
        lines.append(f"| {r['attribute']} | {_pct(r['whole_accuracy'])} | {_pct(r['whole_accuracy_ground_truth_first'])} | "
                     f"{r['gain_points']:.1f} | {r['gain_points_p0']:.1f} | {r['gain_points_p5']:.1f} |")
    if missing:
        lines += ["", f"Not yet run: {', '.join(missing)}."]
    if rows:
        from experiments.synbios_moe.probes.figures import line_chart_svg

        # one panel per attribute would need a layout engine; the mean over the reported attributes shows the effect, the CSV has the rest
        def curve(key):
            return [_mean(r[key] for r in rows if r["position"] == p) for p in range(6)]

        series = {"whole, + true first token": curve("whole_accuracy_ground_truth_first"), "whole, original P probe": curve("whole_accuracy"),
                  "first token, original P probe": curve("first_accuracy")}
        write_text(out / "by_position.svg", line_chart_svg(series, title="Whole-value read-out by biography position (mean over attributes)",
                                                           x_labels=[f"P{i}" for i in range(6)], dashed=("first token, original P probe",)))
        lines += ["", "Figure: `by_position.svg`."]
    write_text(out / "report.md", "\n".join(lines) + "\n")
    return summary
