"""Formal comparison of two probe studies (``single`` against ``multi5+permute``).

A study directory is a finished probe pipeline: ``pipeline.json`` plus ``training/`` and ``validation/`` results of the
22 heads (11 tasks x {P, Q}).  The comparison is only meaningful when both studies probe the SAME people with the same
hyper-parameters and differ in nothing but the augmentation of the pre-training corpus, so the loader and the matcher
refuse anything else.  Outputs: a tidy table (one row per condition, task, split, position), the headline macro means
with their multi-minus-single deltas, a Markdown summary and the figures of ``probes/figures.py``
(reference: experiments/synbios_moe/probes/comparison_report.py:59-310, 556-643).
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Sequence

from experiments.synbios_moe.artifact_io import read_json, write_csv, write_json, write_text
from experiments.synbios_moe.pretraining.dataset import ATTRIBUTES, WHOLE_ATTRIBUTES
from experiments.synbios_moe.probes.commands import job_name
from experiments.synbios_moe.probes.dataset import probe_tasks

CONDITIONS = ("single", "multi5_permute")
EXPECTED_VARIANT = {"single": "single", "multi5_permute": "multi5+permute"}
EXPECTED_JOBS = tuple(job_name(kind, t.attribute, t.target) for kind in ("p", "q") for t in probe_tasks())
# Q-probe accuracies (%) reported by Allen-Zhu & Li for their bioS models: the external reference point of the study.
PUBLISHED_Q_REFERENCE = {"single": {"first": [33.5, 1.1, 2.6, 12.0, 5.5, 41.8], "whole": [0.6, 1.0, 10.1, 1.7, 13.4]},
                         "multi5_permute": {"first": [99.9, 99.8, 99.8, 99.9, 99.5, 99.8], "whole": [99.7, 99.7, 99.8, 98.9, 99.1]}}


@dataclass(frozen=True)
class FormalRun:
    condition: str
    root: Path
    pipeline: dict
    cache_manifest: dict
    training: dict[str, dict]
    validation: dict[str, dict]

    @property
    def data_manifest(self) -> dict:
        return self.cache_manifest.get("source_manifest", {})

    @property
    def profiles_sha256(self) -> str | None:
        files = self.data_manifest.get("files", {})
        entry = files.get("profiles.jsonl")
        return entry.get("sha256") if isinstance(entry, dict) else self.data_manifest.get("profiles_sha256")


def load_formal_run(condition: str, root: str | Path, probe_cache: str | Path, *, require_all: bool = True) -> FormalRun:
    """Load one finished study and check that it is complete and internally consistent."""

    if condition not in CONDITIONS:
        raise ValueError(f"condition must be one of {CONDITIONS}")
    root = Path(root).resolve()
    pipeline = read_json(root / "pipeline.json")
    jobs = pipeline.get("jobs", {})
    unfinished = sorted(n for n, j in jobs.items() if j.get("status") not in ("done", "skipped"))
    if unfinished:
        raise ValueError(f"{root} has unfinished jobs: {unfinished[:4]}")
    training, validation = {}, {}
    for name in EXPECTED_JOBS:
        t_path, v_path = root / "training" / f"{name}.json", root / "validation" / f"{name}.json"
        if not t_path.is_file():
            if require_all:
                raise ValueError(f"{condition}: no training result for {name}")
            continue
        rec = read_json(t_path)
        ident = rec.get("identity", {})
        if job_name(ident.get("kind"), ident.get("attribute"), ident.get("target")) != name:
            raise ValueError(f"{condition}/{name}: the result belongs to task {ident}")
        val = read_json(v_path) if v_path.is_file() else rec
        positions = 6 if name.startswith("p-") else 1
        curve = (val.get("validation") or {}).get("accuracy_by_position", [])
        if len(curve) != positions:
            raise ValueError(f"{condition}/{name}: expected {positions} validation positions, found {len(curve)}")
        training[name], validation[name] = rec, val
    cache_manifest = read_json(Path(probe_cache) / "manifest.json")
    return FormalRun(condition, root, pipeline, cache_manifest, training, validation)


def validate_matched_runs(single: FormalRun, multi: FormalRun) -> None:
    """Same people, same heads, same hyper-parameters; only the corpus variant may differ."""

    if single.condition != "single" or multi.condition != "multi5_permute":
        raise ValueError("pass the single run first and the multi5+permute run second")
    if single.profiles_sha256 is None or single.profiles_sha256 != multi.profiles_sha256:
        raise ValueError("the two studies do not probe the same person / profile table")
    for run in (single, multi):
        variant = run.data_manifest.get("variant")
        if variant != EXPECTED_VARIANT[run.condition]:
            raise ValueError(f"the {run.condition} study was built from variant {variant!r}")
    if set(single.training) != set(multi.training):
        raise ValueError("the two studies did not train the same heads")
    for name in single.training:
        a, b = single.training[name]["identity"], multi.training[name]["identity"]
        for field in ("rank", "batch_size", "steps", "seed"):
            if a.get(field) != b.get(field):
                raise ValueError(f"{name}: {field} differs between the studies ({a.get(field)} vs {b.get(field)})")
        if single.training[name].get("classes") != multi.training[name].get("classes"):
            raise ValueError(f"{name}: class count differs between the studies")


def tidy_rows(runs: Sequence[FormalRun]) -> list[dict]:
    rows = []
    for run in runs:
        for name in EXPECTED_JOBS:
            if name not in run.training:
                continue
            ident = run.training[name]["identity"]
            sources = [("person_held_out_validation", run.validation[name].get("validation") or {})]
            if run.training[name].get("train"):
                sources.append(("probe_train_recall", run.training[name]["train"]))
            for split, rec in sources:
                for position, acc in enumerate(rec.get("accuracy_by_position", [])):
                    rows.append({"condition": run.condition, "split": split, "task": name, "kind": ident["kind"], "target": ident["target"],
                                 "attribute": ident["attribute"], "position": position, "accuracy": float(acc),
                                 "examples": rec.get("examples"), "classes": run.training[name].get("classes")})
    return rows


def _accuracy(rows, condition, kind, target, attribute, position, split="person_held_out_validation") -> float:
    hits = [r["accuracy"] for r in rows if (r["condition"], r["kind"], r["target"], r["attribute"], r["position"], r["split"]) ==
            (condition, kind, target, attribute, position, split)]
    if len(hits) != 1:
        raise ValueError(f"expected exactly one metric for {condition}/{kind}/{target}/{attribute}/P{position}/{split}, found {len(hits)}")
    return hits[0]


def _mean(values: Sequence[float]) -> float:
    return float(sum(values) / len(values))


def headline_metrics(rows: Sequence[dict]) -> dict:
    """End points of the report; task granularities and splits are never mixed inside one mean."""

    out: dict = {}
    for condition in CONDITIONS:
        out[condition] = {
            "p_first_position0_non_birth_date_mean": _mean([_accuracy(rows, condition, "p", "first", a, 0) for a in ATTRIBUTES[1:]]),
            "p_first_fixed_order_diagonal_mean": _mean([_accuracy(rows, condition, "p", "first", a, i) for i, a in enumerate(ATTRIBUTES)]),
            "q_first_six_attribute_macro_mean": _mean([_accuracy(rows, condition, "q", "first", a, 0) for a in ATTRIBUTES]),
            "p_whole_position0_five_attribute_macro_mean": _mean([_accuracy(rows, condition, "p", "whole", a, 0) for a in WHOLE_ATTRIBUTES]),
            "p_whole_position5_five_attribute_macro_mean": _mean([_accuracy(rows, condition, "p", "whole", a, 5) for a in WHOLE_ATTRIBUTES]),
            "q_whole_five_attribute_macro_mean": _mean([_accuracy(rows, condition, "q", "whole", a, 0) for a in WHOLE_ATTRIBUTES]),
        }
    out["delta_multi_minus_single"] = {k: out["multi5_permute"][k] - out["single"][k] for k in out["single"]}
    out["published_q_reference_macro_means"] = {c: {t: _mean([v / 100 for v in vals]) for t, vals in targets.items()}
                                                for c, targets in PUBLISHED_Q_REFERENCE.items()}
    return out


def build_formal_report_artifacts(single_root, multi_root, output_dir, *, single_cache, multi_cache) -> dict:
    single = load_formal_run("single", single_root, single_cache)
    multi = load_formal_run("multi5_permute", multi_root, multi_cache)
    validate_matched_runs(single, multi)
    rows = tidy_rows([single, multi])
    head = headline_metrics(rows)
    out = Path(output_dir)
    out.mkdir(parents=True, exist_ok=True)
    write_csv(out / "probe_metrics_tidy.csv", rows, ["condition", "split", "task", "kind", "target", "attribute", "position", "accuracy",
                                                      "examples", "classes"])
    write_json(out / "headline_metrics.json", head)
    lines = ["# Probe comparison: single vs multi5+permute", "", "| end point | single % | multi5+permute % | delta (points) |", "|---|---:|---:|---:|"]
    for key in head["single"]:
        lines.append(f"| {key} | {100 * head['single'][key]:.1f} | {100 * head['multi5_permute'][key]:.1f} | "
                     f"{100 * head['delta_multi_minus_single'][key]:+.1f} |")
    from experiments.synbios_moe.probes.figures import write_probe_figures

    figures = write_probe_figures(rows, head, out)
    lines += ["", "Figures: " + ", ".join(f"`figures/{name}`" for name in figures if name.endswith(".svg"))]
    write_text(out / "report.md", "\n".join(lines) + "\n")
    return {"rows": len(rows), "headline": head, "figures": figures, "output": str(out.resolve())}
