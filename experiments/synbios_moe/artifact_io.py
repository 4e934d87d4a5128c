"""Atomic artifact writers and content hashes (reference: experiments/synbios_moe/artifact_io.py:1-115).

Every result file of the study is written to a temporary sibling and renamed into place, so an interrupted command never
leaves a half-written artifact that a later stage could mistake for a finished one.
"""

from __future__ import annotations

import csv
import hashlib
import json
import os
import tempfile
from pathlib import Path
from typing import Any, Iterable, Mapping, Sequence


def sha256_file(path: str | Path, chunk: int = 1 << 20) -> str:
    digest = hashlib.sha256()
    with open(path, "rb") as fh:
        while block := fh.read(chunk):
            digest.update(block)
    return digest.hexdigest()


def sha256_json(payload: Any) -> str:
    return hashlib.sha256(json.dumps(payload, sort_keys=True, separators=(",", ":"), default=str).encode()).hexdigest()


def _atomic(path: Path, write) -> Path:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    fd, tmp = tempfile.mkstemp(prefix=f".{path.name}.", suffix=".tmp", dir=path.parent)
    try:
        with os.fdopen(fd, "w", encoding="utf-8", newline="") as fh:
            write(fh)
            fh.flush()
            os.fsync(fh.fileno())
        os.replace(tmp, path)
    except BaseException:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise
    return path


def write_json(path: str | Path, payload: Any) -> Path:
    return _atomic(Path(path), lambda fh: json.dump(payload, fh, indent=1, sort_keys=True, default=str))


def write_text(path: str | Path, text: str) -> Path:
    return _atomic(Path(path), lambda fh: fh.write(text))


def write_csv(path: str | Path, rows: Sequence[Mapping[str, Any]], columns: Sequence[str] | None = None) -> Path:
    cols = list(columns) if columns is not None else sorted({k for r in rows for k in r})

    def emit(fh):
        writer = csv.DictWriter(fh, fieldnames=cols, extrasaction="ignore")
        writer.writeheader()
        writer.writerows(rows)

    return _atomic(Path(path), emit)


def write_jsonl(path: str | Path, rows: Iterable[Mapping[str, Any]]) -> Path:
    def emit(fh):
        for row in rows:
            fh.write(json.dumps(row, ensure_ascii=False) + "\n")

    return _atomic(Path(path), emit)


def read_json(path: str | Path) -> Any:
    return json.loads(Path(path).read_text(encoding="utf-8"))


def read_jsonl(path: str | Path) -> list[dict]:
    with open(path, encoding="utf-8") as fh:
        return [json.loads(line) for line in fh if line.strip()]


def manifest_of(directory: str | Path, names: Sequence[str]) -> dict[str, dict[str, Any]]:
    """sha256 and size of the named files of ``directory`` (for lineage checks between stages)."""

    root = Path(directory)
    return {n: {"sha256": sha256_file(root / n), "bytes": (root / n).stat().st_size} for n in names if (root / n).is_file()}
