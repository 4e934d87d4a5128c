#!/usr/bin/env python
"""Merge cached operator-benchmark scans into the headline table (and, with ``--plots``, one SVG per kernel).

The same step as ``scripts/bench_ops.py summarize``, kept as a script of its own because result-export tooling calls it by
this name (reference: scripts/summarize_operator_bench.py).  ``--output`` additionally writes the table as JSON.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def summarize(directory: str | Path) -> dict:
    from mini_train_sys_b200.bench import operators

    results = _records(directory)
    return {"table": operators.headline_table(results), "quality_gate": operators.quality_gate(results)}


def _records(source) -> list[dict]:
    """Case records of one source: a cache directory, or a single cache / record file."""

    path = Path(source)
    files = sorted(path.glob("*.json")) if path.is_dir() else [path] if path.is_file() else []
    records = []
    for file in files:
        data = json.loads(file.read_text())
        if isinstance(data, dict) and "rows" in data and "status" in data:
            records.append(data)                                    # one case record
        elif isinstance(data, dict):
            records += [v for v in data.values() if isinstance(v, dict) and "rows" in v]
    return records


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("directory", nargs="?", help="cache directory written by `bench_ops.py run --out`")
    # the reference keeps its sweeps in separate places and names each; here they are further sources merged into one table
    for name in ("dense", "moe", "extensions", "capacity"):
        ap.add_argument(f"--{name}", help="a further cache directory or file (the reference's per-sweep option)")
    ap.add_argument("--output", help="write {table, quality_gate} as JSON (a directory gets summary.json)")
    ap.add_argument("--plots", help="directory for one SVG per kernel")
    args = ap.parse_args(argv)
    sources = [s for s in (args.directory, args.dense, args.moe, args.extensions, args.capacity) if s]
    if not sources:
        ap.error("give a cache directory, or --dense / --moe / --extensions / --capacity")
    from mini_train_sys_b200.bench import operators

    results = [record for source in sources for record in _records(source)]
    summary = {"table": operators.headline_table(results), "quality_gate": operators.quality_gate(results)}
    if args.output:
        target = Path(args.output)
        target = target / "summary.json" if target.is_dir() or not target.suffix else target
        target.parent.mkdir(parents=True, exist_ok=True)
        target.write_text(json.dumps(summary, indent=1))
    if args.plots:
        from mini_train_sys_b200.bench.plots import write_kernel_plots

        summary["plots"] = write_kernel_plots(summary["table"], args.plots)
    print(json.dumps({"rows": len(summary["table"]), **summary["quality_gate"], "plots": summary.get("plots")}))
    return 0 if summary["quality_gate"]["quality_gate_passed"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
