"""Collect probe results into tables (reference: experiments/synbios_moe/probes/results.py:1-156)."""

from __future__ import annotations

from pathlib import Path

from experiments.synbios_moe.artifact_io import read_json


def collect_probe_results(root: str | Path) -> list[dict]:
    """One row per finished job under ``root/training`` (validation numbers override when re-validated)."""

    root = Path(root)
    rows = []
    for path in sorted((root / "training").glob("*.json")):
        rec = read_json(path)
        ident = rec.get("identity", {})
        val = rec.get("validation") or {}
        recheck = root / "validation" / path.name
        if recheck.is_file():
            val = read_json(recheck).get("validation", val)
        row = {"job": path.stem, "kind": ident.get("kind"), "attribute": ident.get("attribute"), "target": ident.get("target"),
               "rank": ident.get("rank"), "steps": rec.get("steps"), "final_loss": rec.get("final_loss"), "classes": rec.get("classes"),
               "validation_accuracy": val.get("accuracy"), "validation_examples": val.get("examples")}
        for i, acc in enumerate(val.get("accuracy_by_position", [])):
            row[f"acc_pos{i}"] = acc
        if "train" in rec:
            row["train_accuracy"] = rec["train"].get("accuracy")
        rows.append(row)
    return rows


def summarize_probe_results(root: str | Path) -> dict:
    rows = collect_probe_results(root)
    by_kind: dict[str, list[float]] = {}
    for r in rows:
        if r["validation_accuracy"] is not None:
            by_kind.setdefault(r["kind"], []).append(r["validation_accuracy"])
    return {"jobs": len(rows), "mean_accuracy": {k: sum(v) / len(v) for k, v in by_kind.items()}, "rows": rows,
            "complete": {k: len(v) for k, v in by_kind.items()}}


def comparison_table(roots: dict[str, str | Path]) -> list[dict]:
    """Side-by-side validation accuracy of several studies (e.g. dense vs MoE, single vs multi5+permute)."""

    merged: dict[str, dict] = {}
    for label, root in roots.items():
        for r in collect_probe_results(root):
            merged.setdefault(r["job"], {"job": r["job"], "kind": r["kind"], "attribute": r["attribute"], "target": r["target"]})[label] = \
                r["validation_accuracy"]
    return [merged[k] for k in sorted(merged)]
