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

    results = []
    for path in sorted(Path(directory).glob("*.json")):
        results += list(json.loads(path.read_text()).values())
    return {"table": operators.headline_table(results), "quality_gate": operators.quality_gate(results)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("directory", help="cache directory written by `bench_ops.py run --out`")
    ap.add_argument("--output", help="write {table, quality_gate} as JSON")
    ap.add_argument("--plots", help="directory for one SVG per kernel")
    args = ap.parse_args(argv)
    summary = summarize(args.directory)
    if args.output:
        Path(args.output).parent.mkdir(parents=True, exist_ok=True)
        Path(args.output).write_text(json.dumps(summary, indent=1))
    if args.plots:
        from mini_train_sys_b200.bench.plots import write_kernel_plots

        summary["plots"] = write_kernel_plots(summary["table"], args.plots)
    print(json.dumps({"rows": len(summary["table"]), **summary["quality_gate"], "plots": summary.get("plots")}))
    return 0 if summary["quality_gate"]["quality_gate_passed"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
