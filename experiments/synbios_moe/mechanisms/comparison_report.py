"""Diagnostic evidence of two studies side by side: the oracle first-token intervention and the routing analyses.

For each condition (``single``, ``multi5_permute``) a diagnostics directory holds ``oracle/summary.json`` (from the oracle
first-token validation), ``routes.json`` (from the router analysis) and, optionally, ``bad_case_routes/`` (t1 / t2 route
branching on the Q read-out's bad cases).  The report checks that both sides ran the same protocol, tabulates the oracle
outcome per attribute, forms difference-in-differences of the route statistics per layer (how much more an attribute decides
the expert under augmentation than without it) and reduces the branching tables to per-layer and headline figures
(reference: experiments/synbios_moe/mechanisms/comparison_report.py:98-404, 755-844).
"""

from __future__ import annotations

from pathlib import Path

import csv

from experiments.synbios_moe.artifact_io import read_json, write_csv, write_json, write_text
from experiments.synbios_moe.mechanisms.oracle_first_token import PROTOCOL as ORACLE_PROTOCOL
from experiments.synbios_moe.mechanisms.token_routes import ROUTE_PROTOCOL

CONDITIONS = ("single", "multi5_permute")
ORACLE_FIELDS = ("examples", "accuracy_before", "accuracy_after", "accuracy_delta", "recovery_rate", "harm_rate")


def _assert_close(left: float, right: float, label: str, tolerance: float = 1e-12) -> None:
    if abs(left - right) > tolerance:
        raise ValueError(f"{label}: {left} != {right}")


def load_diagnostic_evidence(roots: dict[str, str | Path]) -> dict[str, dict]:
    if set(roots) != set(CONDITIONS):
        raise ValueError(f"expected diagnostics for exactly {CONDITIONS}")
    evidence = {}
    for condition, root in roots.items():
        root = Path(root)
        oracle = read_json(root / "oracle" / "summary.json")
        if oracle.get("protocol") != ORACLE_PROTOCOL or oracle.get("parameters_updated") is not False:
            raise ValueError(f"{condition}: the oracle summary was not produced by protocol {ORACLE_PROTOCOL}")
        overall = oracle["overall"]
        # the overall row must be the example-weighted mean of the attribute rows: a truncated or edited summary fails here
        n = sum(a["examples"] for a in oracle["attributes"])
        if n != overall["examples"]:
            raise ValueError(f"{condition}: attribute rows cover {n} examples, the overall row {overall['examples']}")
        if n:
            _assert_close(sum(a["accuracy_before"] * a["examples"] for a in oracle["attributes"]) / n, overall["accuracy_before"],
                          f"{condition} accuracy_before", 1e-9)
        routes_path = root / "routes.json"
        evidence[condition] = {"oracle": oracle, "routes": read_json(routes_path) if routes_path.is_file() else None}
    a, b = (evidence[c]["oracle"] for c in CONDITIONS)
    if [r["attribute"] for r in a["attributes"]] != [r["attribute"] for r in b["attributes"]]:
        raise ValueError("the two oracle summaries cover different attributes")
    return evidence


def oracle_rows(evidence: dict[str, dict]) -> list[dict]:
    rows = []
    for condition in CONDITIONS:
        for rec in evidence[condition]["oracle"]["attributes"]:
            rows.append({"condition": condition, "attribute": rec["attribute"], **{k: rec[k] for k in ORACLE_FIELDS}})
    return rows


def route_rows(evidence: dict[str, dict]) -> list[dict]:
    """Per layer: NMI(attribute, expert) of both conditions and their difference; layers present on both sides only."""

    left, right = (evidence[c]["routes"] for c in CONDITIONS)
    if not left or not right:
        return []
    rows = []
    for layer in sorted(set(left) & set(right), key=lambda k: int(k) if str(k).lstrip("-").isdigit() else 0):
        a, b = left[layer], right[layer]
        row = {"layer": layer}
        for key in ("nmi_attribute_expert", "jaccard_same_fact", "jaccard_other_people", "jaccard_did"):
            if a.get(key) is not None and b.get(key) is not None:
                row[f"{key}_single"], row[f"{key}_multi5_permute"] = a[key], b[key]
                row[f"{key}_delta"] = b[key] - a[key]
        # jaccard_did is itself a difference (same fact rendered twice minus other people's facts of the attribute); its delta
        # between the conditions is the difference in differences: what augmentation adds to fact-specific routing
        if "jaccard_did_delta" in row:
            row["route_jaccard_did_of_did"] = row["jaccard_did_delta"]
        rows.append(row)
    return rows


def _read_csv(path: Path) -> list[dict]:
    with open(path, newline="") as fh:
        return list(csv.DictReader(fh))


def branching_evidence(summary: dict, pair_rows: list[dict], nmi_rows: list[dict]) -> tuple[list[dict], list[dict], dict]:
    """Per-layer rows, per-(attribute, layer) rows and headline figures of one bad-case route run.

    The tables must be complete for the topology and the attributes the summary names (every attribute x layer x pair group
    with at least one pair), overlaps must lie in [0, 1] and every branching score must equal t1 overlap minus t2 overlap:
    a truncated or edited run is refused instead of averaged.  ``difference_in_differences`` is the branching score of pairs
    whose second token differs minus that of pairs whose second token agrees, pair-count weighted."""

    if summary.get("protocol") != ROUTE_PROTOCOL or summary.get("parameters_updated") is not False:
        raise ValueError(f"the route summary was not produced by protocol {ROUTE_PROTOCOL}")
    counts = summary.get("attributes")
    if not isinstance(counts, dict) or sum(int(v) for v in counts.values()) != int(summary["examples"]):
        raise ValueError("route bad-case counts do not close")
    layers, attributes = int(summary["layers"]), [a for a, n in counts.items() if int(n) > 0]
    groups = ("same_t2", "different_t2")
    pairs = {(r["attribute"], int(r["layer"]), r["pair_group"]): r for r in pair_rows}
    expected = {(a, layer, g) for a in attributes for layer in range(layers) for g in groups}
    if len(pairs) != len(pair_rows) or not expected <= set(pairs):
        missing = sorted(expected - set(pairs))[:3]
        raise ValueError(f"the pairwise table is not complete for {len(attributes)} attributes x {layers} layers x 2 groups (first gaps: {missing})")
    for r in pair_rows:
        if int(r["pair_count"]) <= 0:
            raise ValueError("the pairwise table contains an empty group")
        t1, t2 = float(r["t1_route_overlap"]), float(r["t2_route_overlap"])
        if not (0.0 <= t1 <= 1.0 and 0.0 <= t2 <= 1.0):
            raise ValueError(f"route overlap outside [0, 1]: {r}")
        _assert_close(float(r["branching_score"]), t1 - t2, "route branching score", 1e-9)
    nmi = {(r["attribute"], int(r["layer"])): r for r in nmi_rows}
    if not {(a, layer) for a in attributes for layer in range(layers)} <= set(nmi):
        raise ValueError("the token NMI table does not cover every attribute and layer")
    for r in nmi_rows:
        for field in ("t1_top1_token_nmi", "t2_top1_token_nmi"):
            if not -1e-9 <= float(r[field]) <= 1.0 + 1e-9:
                raise ValueError(f"route NMI outside [0, 1]: {r}")

    def weighted(rows: list[dict], field: str) -> float:
        total = sum(int(r["pair_count"]) for r in rows)
        return sum(float(r[field]) * int(r["pair_count"]) for r in rows) / total

    detail = []
    for a in attributes:
        for layer in range(layers):
            same, diff = pairs[(a, layer, "same_t2")], pairs[(a, layer, "different_t2")]
            detail.append({"attribute": a, "layer": layer, "same_t2_branching_score": float(same["branching_score"]),
                           "different_t2_branching_score": float(diff["branching_score"]),
                           "difference_in_differences": float(diff["branching_score"]) - float(same["branching_score"]),
                           "same_t2_pair_count": int(same["pair_count"]), "different_t2_pair_count": int(diff["pair_count"]),
                           "t1_top1_token_nmi": float(nmi[(a, layer)]["t1_top1_token_nmi"]),
                           "t2_top1_token_nmi": float(nmi[(a, layer)]["t2_top1_token_nmi"])})
    by_layer = []
    for layer in range(layers):
        row: dict = {"layer": layer}
        for g in groups:
            chosen = [pairs[(a, layer, g)] for a in attributes]
            row[f"{g}_pair_count"] = sum(int(r["pair_count"]) for r in chosen)
            for field in ("t1_route_overlap", "t2_route_overlap", "branching_score"):
                row[f"{g}_{field}"] = weighted(chosen, field)
        row["difference_in_differences"] = row["different_t2_branching_score"] - row["same_t2_branching_score"]
        by_layer.append(row)
    overall = {g: {"pair_count": sum(int(r["pair_count"]) for r in pair_rows if r["pair_group"] == g),
                   **{f: weighted([r for r in pair_rows if r["pair_group"] == g], f)
                      for f in ("t1_route_overlap", "t2_route_overlap", "branching_score")}} for g in groups} if attributes else {}
    headline = {"bad_case_examples": int(summary["examples"]), "groups": overall,
                "difference_in_differences": (overall["different_t2"]["branching_score"] - overall["same_t2"]["branching_score"]) if overall else None,
                "all_layers_positive": bool(by_layer) and all(r["difference_in_differences"] > 0 for r in by_layer),
                "max_t1_nmi_by_attribute": {a: max(float(nmi[(a, layer)]["t1_top1_token_nmi"]) for layer in range(layers)) for a in attributes},
                "max_t2_nmi_by_attribute": {a: max(float(nmi[(a, layer)]["t2_top1_token_nmi"]) for layer in range(layers)) for a in attributes}}
    return by_layer, detail, headline


def load_branching_evidence(root: str | Path) -> tuple[list[dict], list[dict], dict] | None:
    """``<root>/bad_case_routes`` reduced by ``branching_evidence``; ``None`` when the diagnostic was not run."""

    folder = Path(root) / "bad_case_routes"
    if not (folder / "summary.json").is_file():
        return None
    return branching_evidence(read_json(folder / "summary.json"), _read_csv(folder / "pairwise_branching.csv"),
                              _read_csv(folder / "token_route_nmi.csv"))


def build_diagnostic_report_artifacts(roots: dict[str, str | Path], output_dir: str | Path) -> dict:
    evidence = load_diagnostic_evidence(roots)
    o_rows, r_rows = oracle_rows(evidence), route_rows(evidence)
    out = Path(output_dir)
    out.mkdir(parents=True, exist_ok=True)
    write_csv(out / "oracle_by_attribute.csv", o_rows, ["condition", "attribute", *ORACLE_FIELDS])
    if r_rows:
        write_csv(out / "routes_by_layer.csv", r_rows)
    overall = {c: evidence[c]["oracle"]["overall"] for c in CONDITIONS}
    summary = {"protocol": "synbios_diagnostic_report_v1", "oracle_overall": overall,
               "oracle_recovery_delta": overall["multi5_permute"]["recovery_rate"] - overall["single"]["recovery_rate"],
               "route_layers": len(r_rows)}
    branching = {}
    for condition in CONDITIONS:
        reduced = load_branching_evidence(roots[condition])
        if reduced is not None:
            by_layer, detail, headline = reduced
            write_csv(out / f"route_branching_by_layer_{condition}.csv", by_layer)
            write_csv(out / f"route_branching_by_attribute_layer_{condition}.csv", detail)
            branching[condition] = headline
    if branching:
        summary["route_branching"] = branching
    write_json(out / "summary.json", summary)
    lines = ["# Diagnostics: oracle first token and routing", "", "| condition | accuracy before % | after % | recovered errors % | harmed % |",
             "|---|---:|---:|---:|---:|"]
    for c in CONDITIONS:
        o = overall[c]
        lines.append(f"| {c} | {100 * o['accuracy_before']:.1f} | {100 * o['accuracy_after']:.1f} | {100 * o['recovery_rate']:.1f} | {100 * o['harm_rate']:.1f} |")
    write_text(out / "report.md", "\n".join(lines) + "\n")
    return summary
