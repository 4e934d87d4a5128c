#!/usr/bin/env python
"""SHA-256 manifest of an exported results tree, and its check.

    python scripts/build_results_manifest.py results/            # writes results/MANIFEST.sha256.json
    python scripts/build_results_manifest.py results/ --check    # exit 1 when a file was added, removed or changed

Same role as the reference's ``scripts/build_results_manifest.py`` (evidence integrity gate).
"""

from __future__ import annotations

import argparse
import hashlib
import json
import sys
from pathlib import Path

NAME = "MANIFEST.sha256.json"


def digest(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as fh:
        while block := fh.read(1 << 20):
            h.update(block)
    return h.hexdigest()


def build(root: Path) -> dict[str, dict]:
    return {str(p.relative_to(root)): {"sha256": digest(p), "bytes": p.stat().st_size}
            for p in sorted(root.rglob("*")) if p.is_file() and p.name != NAME}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("root", nargs="?")
    ap.add_argument("--results", help="the results tree (same as the positional argument; default: results)")
    ap.add_argument("--check", action="store_true")
    args = ap.parse_args(argv)
    root = Path(args.root or args.results or "results")
    current = build(root)
    path = root / NAME
    if not args.check:
        path.write_text(json.dumps({"files": current}, indent=1, sort_keys=True))
        print(json.dumps({"manifest": str(path), "files": len(current)}))
        return 0
    recorded = json.loads(path.read_text())["files"]
    added = sorted(set(current) - set(recorded))
    removed = sorted(set(recorded) - set(current))
    changed = sorted(k for k in set(current) & set(recorded) if current[k]["sha256"] != recorded[k]["sha256"])
    print(json.dumps({"ok": not (added or removed or changed), "added": added, "removed": removed, "changed": changed}, indent=1))
    return 0 if not (added or removed or changed) else 1


if __name__ == "__main__":
    sys.exit(main())
