#!/usr/bin/env python
"""Catalogue of a results tree: one line per artifact with its kind, key figures and provenance.

Walks ``results/`` (or any directory) and recognises distributed-benchmark summaries, operator-benchmark caches, bench.py
JSON lines, SynBioS reports (recall / cloze / routes / probe tables) and profile summaries; writes ``CATALOG.json`` and a
Markdown table.  Same role as the reference's ``scripts/build_results_catalog.py``.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def describe(path: Path) -> dict | None:
    try:
        text = path.read_text()
    except (OSError, UnicodeDecodeError):
        return None
    entry = {"path": str(path), "bytes": path.stat().st_size}
    if path.suffix == ".json":
        try:
            data = json.loads(text)
        except ValueError:
            return None
        if isinstance(data, dict) and "suite" in data and "rows" in data:
            ok = [r for r in data["rows"] if r.get("status") == "ok"]
            entry.update(kind=f"distributed/{data['suite']}", rows=len(data["rows"]), ok_rows=len(ok),
                         gates=data.get("quality_gates", {}).get("passed"))
        elif isinstance(data, dict) and "metric" in data and "value" in data:
            entry.update(kind="bench", metric=data["metric"], value=data["value"], n_gpus=data.get("n_gpus"))
        elif isinstance(data, dict) and "per_attribute" in data:
            entry.update(kind="synbios/cloze", exact_match=data.get("overall_exact_match"), items=data.get("items"))
        elif isinstance(data, dict) and "overall" in data and "token_accuracy" in data.get("overall", {}):
            entry.update(kind="synbios/recall", token_accuracy=data["overall"]["token_accuracy"])
        elif isinstance(data, dict) and data and all(isinstance(v, dict) and "rows" in v for v in data.values()):
            entry.update(kind="operators/cache", cases=len(data))
        elif isinstance(data, dict) and "jobs" in data and "identity" in data:
            entry.update(kind="synbios/pipeline", jobs=len(data["jobs"]))
        else:
            entry.update(kind="json")
    elif path.suffix in (".txt", ".md") and "profiles" in path.parts:
        entry.update(kind="profile", first_line=text.splitlines()[0][:100] if text else "")
    else:
        return None
    return entry


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("root", nargs="?")
    ap.add_argument("--results", help="the results tree (same as the positional argument; default: results)")
    ap.add_argument("--artifacts", help="accepted for the reference's command lines: what is catalogued here is the results tree only")
    ap.add_argument("--output", default=None)
    args = ap.parse_args(argv)
    root = Path(args.root or args.results or "results")
    entries = [e for p in sorted(root.rglob("*")) if p.is_file() and p.name not in ("CATALOG.json", "CATALOG.md") for e in [describe(p)] if e]
    for entry in entries:      # the catalogue travels with the tree: paths are relative to it, and the root is named, not located
        entry["path"] = Path(entry["path"]).relative_to(root).as_posix()
    out = Path(args.output) if args.output else root / "CATALOG.json"
    out.write_text(json.dumps({"root": root.name, "entries": entries}, indent=1))
    lines = ["| path | kind | bytes | figures |", "|---|---|---|---|"]
    for e in entries:
        figures = ", ".join(f"{k}={v}" for k, v in e.items() if k not in ("path", "kind", "bytes") and v is not None)
        lines.append(f"| `{e['path']}` | {e['kind']} | {e['bytes']} | {figures} |")
    out.with_suffix(".md").write_text("\n".join(lines) + "\n")
    kinds: dict[str, int] = {}
    for e in entries:
        kinds[e["kind"]] = kinds.get(e["kind"], 0) + 1
    print(json.dumps({"catalog": str(out), "entries": len(entries), "kinds": kinds}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
