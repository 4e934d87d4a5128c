"""Diagnostic evidence of two studies side by side: the oracle first-token intervention and the routing analyses.

For each condition (``single``, ``multi5_permute``) a diagnostics directory holds ``oracle/summary.json`` (from the oracle
first-token validation) and ``routes.json`` (from the router analysis).  The report checks that both sides ran the same
protocol, tabulates the oracle outcome per attribute, and forms difference-in-differences of the route statistics per
layer: how much more an attribute decides the expert under augmentation than without it
(reference: experiments/synbios_moe/mechanisms/comparison_report.py:98-404, 755-844).
"""

from __future__ import annotations

from pathlib import Path

from experiments.synbios_moe.artifact_io import read_json, write_csv, write_json, write_text
from experiments.synbios_moe.mechanisms.oracle_first_token import PROTOCOL as ORACLE_PROTOCOL

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
    write_json(out / "summary.json", summary)
    lines = ["# Diagnostics: oracle first token and routing", "", "| condition | accuracy before % | after % | recovered errors % | harmed % |",
             "|---|---:|---:|---:|---:|"]
    for c in CONDITIONS:
        o = overall[c]
        lines.append(f"| {c} | {100 * o['accuracy_before']:.1f} | {100 * o['accuracy_after']:.1f} | {100 * o['recovery_rate']:.1f} | {100 * o['harm_rate']:.1f} |")
    write_text(out / "report.md", "\n".join(lines) + "\n")
    return summary
