"""Lineage audit of a study directory: every derived artifact must point at the inputs it was made from.

Checks (reference: experiments/synbios_moe/audit.py:1-289): dataset manifest hashes match the files; the probe cache
embeds the dataset manifest it was built from; probe results carry an identity and sit beside their weights; a
finished pipeline's identity matches its inputs.
"""

from __future__ import annotations

from pathlib import Path

from experiments.synbios_moe.artifact_io import read_json, sha256_file
from experiments.synbios_moe.probes.dataset import validate_probe_cache


def audit_dataset(data_root: str | Path) -> list[str]:
    root = Path(data_root)
    problems = []
    try:
        manifest = read_json(root / "manifest.json")
    except (OSError, ValueError) as exc:
        return [f"{root}: manifest unreadable ({exc})"]
    for name, meta in manifest.get("files", {}).items():
        path = root / name
        if not path.is_file():
            problems.append(f"{root}: {name} missing")
        elif sha256_file(path) != meta["sha256"]:
            problems.append(f"{root}: {name} differs from the manifest")
    return problems


def audit_study(*, data_root: str | Path | None = None, probe_cache: str | Path | None = None,
                pipeline_root: str | Path | None = None) -> dict:
    problems: list[str] = []
    if data_root is not None:
        problems += audit_dataset(data_root)
    if probe_cache is not None:
        verdict = validate_probe_cache(probe_cache, data_root)
        problems += [f"{probe_cache}: {e}" for e in verdict["errors"]]
    if pipeline_root is not None:
        root = Path(pipeline_root)
        for path in sorted((root / "training").glob("*.json")):
            rec = read_json(path)
            if "identity" not in rec:
                problems.append(f"{path}: result without identity")
            if not path.with_suffix(".pt").is_file():
                problems.append(f"{path}: weights missing beside the result")
        state = root / "pipeline.json"
        if state.is_file():
            data = read_json(state)
            unfinished = [n for n, j in data.get("jobs", {}).items() if j.get("status") not in ("done", "skipped")]
            if unfinished:
                problems.append(f"{state}: unfinished jobs {unfinished[:5]}{'...' if len(unfinished) > 5 else ''}")
    return {"ok": not problems, "problems": problems}
