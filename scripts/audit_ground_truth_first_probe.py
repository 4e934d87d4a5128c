#!/usr/bin/env python
"""Audit one result of the ground-truth-first whole probe (``synbios_moe.py ground-truth-first-whole``).

Checks the fields that make the result comparable with the original P-whole probe: protocol name, frozen backbone, rank
bound to the reference probe, six source positions whose totals add up to the evaluated examples, finite loss, the weights
file next to the record, the hash of the reference probe, and (optionally) that a resumed run continued from the expected
step.  Exit code 0 = every check passed; 1 = at least one failed (all failures are listed)
(reference: scripts/audit_ground_truth_first_probe.py:1-182).
"""

from __future__ import annotations

import argparse
import hashlib
import json
import math
import sys
from pathlib import Path


def audit(path: Path, *, expect_resumed_from: int | None = None, max_validation_examples: int | None = None,
          reference_probe: Path | None = None) -> list[str]:
    errors: list[str] = []
    try:
        rec = json.loads(path.read_text(encoding="utf-8"))
    except (OSError, ValueError) as exc:
        return [f"unreadable result: {exc}"]

    def check(ok: bool, message: str) -> None:
        if not ok:
            errors.append(message)

    check(rec.get("protocol") == "ground_truth_first_whole_rank_matched_v1", f"protocol is {rec.get('protocol')!r}")
    check(rec.get("ground_truth_first_token") is True, "ground_truth_first_token is not true")
    check(rec.get("backbone_parameters_updated") is False, "the backbone must stay frozen")
    check(rec.get("target") == "whole", "target must be 'whole'")
    ident = rec.get("identity", {})
    check(ident.get("kind") == "p", "the probe must be a P probe")
    check(ident.get("rank") == rec.get("reference_rank"), f"rank {ident.get('rank')} differs from the reference probe's {rec.get('reference_rank')}")
    acc, hit, tot = (rec.get(k, []) for k in ("whole_accuracy_validation_by_source_position", "whole_correct_validation_by_source_position",
                                              "whole_total_validation_by_source_position"))
    check(len(acc) == len(hit) == len(tot) == 6, "expected six source positions")
    if len(acc) == len(hit) == len(tot) == 6:
        for i in range(6):
            check(0 <= hit[i] <= tot[i], f"position {i}: {hit[i]} correct of {tot[i]}")
            check(tot[i] == 0 or abs(acc[i] - hit[i] / tot[i]) < 1e-9, f"position {i}: accuracy does not equal correct / total")
        check(max(tot) - min(tot) <= 1, "source positions were not evaluated equally often")
        if max_validation_examples is not None:
            check(sum(tot) <= max_validation_examples, f"{sum(tot)} examples evaluated, limit {max_validation_examples}")
    check(rec.get("final_loss") is not None and math.isfinite(float(rec["final_loss"])), "final loss is missing or not finite")
    check(rec.get("steps") == ident.get("steps"), f"trained {rec.get('steps')} of {ident.get('steps')} steps")
    check(path.with_suffix(".pt").is_file(), f"weights file {path.with_suffix('.pt').name} is missing")
    if expect_resumed_from is not None:
        check(rec.get("resumed_from_step") == expect_resumed_from, f"resumed from step {rec.get('resumed_from_step')}, expected {expect_resumed_from}")
    ref = reference_probe or (Path(rec["reference_whole_probe_checkpoint"]) if rec.get("reference_whole_probe_checkpoint") else None)
    if ref is not None and ref.is_file():
        digest = hashlib.sha256(ref.read_bytes()).hexdigest()
        check(digest == ident.get("reference_whole_probe_sha256"), "the reference P-whole probe changed since this probe was trained")
    elif reference_probe is not None:
        errors.append(f"reference probe {reference_probe} not found")
    tokens = rec.get("first_token_text", {})
    check(bool(tokens) and all(t.startswith(" ") for t in tokens.values()), "first-token texts must start with the mid-sentence space")
    return errors


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("results", nargs="+", type=Path)
    ap.add_argument("--expect-resumed-from", type=int)
    ap.add_argument("--max-validation-examples", type=int)
    ap.add_argument("--reference-probe", type=Path)
    args = ap.parse_args(argv)
    failed = False
    for path in args.results:
        errors = audit(path, expect_resumed_from=args.expect_resumed_from, max_validation_examples=args.max_validation_examples,
                       reference_probe=args.reference_probe)
        print(json.dumps({"result": str(path), "ok": not errors, "errors": errors}))
        failed = failed or bool(errors)
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
