#!/usr/bin/env python
"""Audit an exported results tree: every benchmark summary must be reproducible from the raw rows beside it.

Checks: (1) each ``summary.json`` of the distributed harness lists only rows whose raw file exists and carries the same
identity hash; (2) every successful row was device-timed with at least three warm-up steps; (3) weak-scaling
efficiencies recompute from the rows; (4) operator caches contain no row without a parity verdict for a non-library
provider; (5) text files that name a path of the machine they were made on (a home directory, a scratch mount) are listed
as ``non_portable``: a warning, or a failure with ``--strict-paths``.  Same role as the reference's
``scripts/audit_results_export.py``.
"""

from __future__ import annotations

import argparse
import json
import re
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def audit(root: Path) -> list[str]:
    from mini_train_sys_b200.bench.distributed import weak_scaling_table

    problems: list[str] = []
    for summary_path in sorted(root.rglob("summary.json")):
        summary = json.loads(summary_path.read_text())
        raw = summary_path.parent / "raw"
        for row in summary.get("rows", []):
            name = row.get("name")
            path = raw / f"{name}.json"
            if not path.is_file():
                problems.append(f"{summary_path}: raw file of {name} missing")
                continue
            if json.loads(path.read_text()).get("identity") != row.get("identity"):
                problems.append(f"{summary_path}: identity of {name} differs from its raw file")
            if row.get("status") == "ok":
                if "cuda events" not in str(row.get("timing", "")) and row.get("device_memory_mb", 0) > 0:
                    problems.append(f"{summary_path}: {name} was not device-timed")
                if int(row.get("warmup_steps", 0)) < 3:
                    problems.append(f"{summary_path}: {name} ran fewer than 3 warm-up steps")
        if summary.get("suite") == "weak":
            again = {(w["strategy"], w["engine"], w["ops"], w["batch_size"], w["world_size"]): w["efficiency_pct"]
                     for w in weak_scaling_table(summary["rows"])}
            for w in summary.get("weak", []):
                key = (w["strategy"], w["engine"], w["ops"], w["batch_size"], w["world_size"])
                if w["efficiency_pct"] is not None and abs(again.get(key, -1) - w["efficiency_pct"]) > 1e-6:
                    problems.append(f"{summary_path}: efficiency of {key} does not recompute")
    for cache in sorted(root.rglob("sm*-*.json")):
        for key, rec in json.loads(cache.read_text()).items():
            for row in rec.get("rows", []):
                if row["provider"] not in ("torch",) and "correctness" not in row and rec.get("checked", True) is not False:
                    problems.append(f"{cache}: {row['label']} [{row['provider']}] has no parity verdict")
    return problems


_TEXT_SUFFIXES = {".json", ".jsonl", ".md", ".csv", ".txt", ".svg", ".env", ".yaml", ".yml"}
_MACHINE_PATH = re.compile(r"""(?:(?<![\w.:/-])/(?:home|root|Users|mnt|data|scratch|tmp)/[\w.@+-]+|[A-Za-z]:\\+Users\\+[\w.@+-]+)""")


def non_portable_paths(root: Path, *, limit_per_file: int = 3) -> list[str]:
    """``file: match`` for every text file under ``root`` that names a path of the machine it was made on."""

    found = []
    for path in sorted(p for p in root.rglob("*") if p.is_file() and p.suffix.lower() in _TEXT_SUFFIXES):
        try:
            text = path.read_text(encoding="utf-8")
        except (OSError, UnicodeDecodeError):
            continue
        seen = []
        for match in _MACHINE_PATH.finditer(text):
            if match.group(0) not in seen:
                seen.append(match.group(0))
            if len(seen) == limit_per_file:
                break
        found += [f"{path.relative_to(root)}: {m}" for m in seen]
    return found


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("root", nargs="?")
    ap.add_argument("--results", help="the results tree (same as the positional argument; default: results)")
    ap.add_argument("--artifacts", help="accepted for the reference's command lines: the audit reads the results tree only")
    ap.add_argument("--repo-root", help="accepted for the reference's command lines")
    ap.add_argument("--output", help="also write the report as JSON to this file")
    ap.add_argument("--strict-paths", action="store_true", help="machine paths inside exported text files fail the audit")
    args = ap.parse_args(argv)
    root = Path(args.root or args.results or "results")
    problems = audit(root)
    stray = non_portable_paths(root)
    if args.strict_paths:
        problems += [f"machine path in {item}" for item in stray]
    report = json.dumps({"ok": not problems, "problems": problems, "non_portable": stray}, indent=1)
    if args.output:
        Path(args.output).parent.mkdir(parents=True, exist_ok=True)
        Path(args.output).write_text(report + "\n", encoding="utf-8")
    print(report)
    return 0 if not problems else 1


if __name__ == "__main__":
    sys.exit(main())
