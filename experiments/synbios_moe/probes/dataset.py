"""Probe tasks and the memory-mapped probe cache (format 2).

A probe task is (attribute, target): ``first`` classifies the first token of the value (the month name for the birth
date), ``whole`` the complete value; the birth date has no ``whole`` task, so there are 6 + 5 = 11 tasks, each run as a
P probe (six positions inside a biography, one before every attribute value, in left-to-right text order) and as a Q
probe (one position: right after the person's name), 22 jobs in total.

Cache layout (reference: experiments/synbios_moe/probes/dataset.py:24,97-234)
    manifest.json            format, codec, tasks with class names, label coverage, the source dataset manifest
    profile_labels.npy       [profiles, 11] <i4   class id of every task
    profile_splits.npy       [profiles]     u1    0 = train, 1 = validation
    p_tokens.bin / q_tokens.bin   ragged <i4 token streams, ``*_offsets.npy`` <i8 with one more entry than examples
    p_positions.npy          [examples, 6] <i4    P0..P5
    p_profile_indices.npy    [examples]    <i4    row of the profile each biography belongs to
The directory is built under a temporary name and renamed into place.
"""

from __future__ import annotations

import os
import shutil
import tempfile
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Sequence

import numpy as np

from experiments.synbios_moe.artifact_io import read_json, read_jsonl, sha256_file, write_json
from experiments.synbios_moe.codec import get_codec, positions_before_chars
from experiments.synbios_moe.pretraining.dataset import ATTRIBUTES, WHOLE_ATTRIBUTES

CACHE_FORMAT = 2
SPLIT_CODES = {"train": 0, "validation": 1}
ARRAY_FILES = ("profile_labels.npy", "profile_splits.npy", "p_tokens.bin", "p_offsets.npy", "p_positions.npy",
               "p_profile_indices.npy", "q_tokens.bin", "q_offsets.npy")


@dataclass(frozen=True)
class ProbeTask:
    attribute: str
    target: str          # "first" | "whole"

    @property
    def key(self) -> str:
        return f"{self.attribute}:{self.target}"


def probe_tasks() -> tuple[ProbeTask, ...]:
    return tuple(ProbeTask(a, "first") for a in ATTRIBUTES) + tuple(ProbeTask(a, "whole") for a in WHOLE_ATTRIBUTES)


def task_label(profile: dict, attribute: str, target: str, codec) -> str:
    value = str(profile[attribute])
    if target == "whole":
        return value
    if attribute == "birth_date":
        return value.split(" ", 1)[0]                     # the month
    return str(codec.encode(" " + value)[0])             # first token as it appears mid-sentence


def ordered_probe_starts(spans: dict) -> list[int]:
    """Character starts of the six values in text order (a permuted biography changes which fact is P0)."""

    items = []
    for attribute in ATTRIBUTES:
        start, end = spans[attribute]
        if not (isinstance(start, int) and isinstance(end, int) and 0 <= start < end):
            raise ValueError(f"invalid span for {attribute!r}: {spans[attribute]!r}")
        items.append((start, end, attribute))
    items.sort()
    for (s0, e0, a0), (s1, _, a1) in zip(items, items[1:]):
        if s1 < e0:
            raise ValueError(f"overlapping spans: {a0!r} and {a1!r}")
    return [s for s, _, _ in items]


def _ragged(path: Path, rows: Sequence[Sequence[int]]) -> np.ndarray:
    offsets = np.zeros(len(rows) + 1, dtype="<i8")
    with open(path, "wb") as fh:
        for i, row in enumerate(rows):
            arr = np.asarray(row, dtype="<i4")
            fh.write(arr.tobytes())
            offsets[i + 1] = offsets[i] + arr.size
    return offsets


def build_probe_cache(data_root: str | Path, output_dir: str | Path, *, codec_name: str = "gpt2", force: bool = False,
                      require_coverage: bool = False, progress: Callable[[int], None] | None = None) -> Path:
    data_root, output = Path(data_root), Path(output_dir)
    source_manifest = data_root / "manifest.json"
    if not source_manifest.is_file():
        raise FileNotFoundError(f"missing dataset manifest: {source_manifest}")
    if output.exists() and not force:
        raise FileExistsError(f"probe cache already exists: {output} (pass force to rebuild)")
    output.parent.mkdir(parents=True, exist_ok=True)
    staging = Path(tempfile.mkdtemp(prefix=f".{output.name}.tmp-", dir=output.parent))
    try:
        codec = get_codec(codec_name)
        profiles = read_jsonl(data_root / "profiles.jsonl")
        if not profiles:
            raise ValueError("profiles.jsonl is empty")
        index_of = {p["person_id"]: i for i, p in enumerate(profiles)}
        if len(index_of) != len(profiles):
            raise ValueError("profiles.jsonl contains duplicate person_id values")
        tasks = probe_tasks()
        classes = {t.key: sorted({task_label(p, t.attribute, t.target, codec) for p in profiles}) for t in tasks}
        lookup = {k: {name: i for i, name in enumerate(v)} for k, v in classes.items()}
        labels = np.empty((len(profiles), len(tasks)), dtype="<i4")
        splits = np.empty(len(profiles), dtype="u1")
        for row, p in enumerate(profiles):
            splits[row] = SPLIT_CODES[p["split"]]
            for col, t in enumerate(tasks):
                labels[row, col] = lookup[t.key][task_label(p, t.attribute, t.target, codec)]
        # label coverage: classes of the validation split that never occur in the training split cannot be learnt
        coverage = {}
        for col, t in enumerate(tasks):
            seen = set(labels[splits == 0, col].tolist())
            held = set(labels[splits == 1, col].tolist())
            coverage[t.key] = {"classes": len(classes[t.key]), "train_classes": len(seen), "validation_only_classes": len(held - seen)}
        if require_coverage and any(c["validation_only_classes"] for c in coverage.values()):
            raise ValueError(f"validation-only classes present: { {k: c for k, c in coverage.items() if c['validation_only_classes']} }")

        p_tokens, p_positions, p_profile = [], [], []
        for n, bio in enumerate(read_jsonl(data_root / "biographies.jsonl")):
            spans = {k: (int(v[0]), int(v[1])) for k, v in bio["attribute_spans"].items()}
            ids, pos = positions_before_chars(codec, bio["text"], ordered_probe_starts(spans))
            p_tokens.append(ids); p_positions.append(pos); p_profile.append(index_of[bio["person_id"]])
            if progress is not None and n % 1000 == 0:
                progress(n)
        q_tokens = [[codec.eos, *codec.encode(p["full_name"]), codec.eos] for p in profiles]
        np.save(staging / "profile_labels.npy", labels)
        np.save(staging / "profile_splits.npy", splits)
        np.save(staging / "p_offsets.npy", _ragged(staging / "p_tokens.bin", p_tokens))
        np.save(staging / "p_positions.npy", np.asarray(p_positions, dtype="<i4").reshape(len(p_tokens), 6))
        np.save(staging / "p_profile_indices.npy", np.asarray(p_profile, dtype="<i4"))
        np.save(staging / "q_offsets.npy", _ragged(staging / "q_tokens.bin", q_tokens))
        write_json(staging / "manifest.json", {
            "format": CACHE_FORMAT, "codec": codec_name, "vocab_size": codec.vocab_size, "eos": codec.eos,
            "tasks": [{"key": t.key, "attribute": t.attribute, "target": t.target, "classes": classes[t.key]} for t in tasks],
            "coverage": coverage, "profiles": len(profiles), "p_examples": len(p_tokens), "q_examples": len(q_tokens),
            "source_manifest": read_json(source_manifest), "source_manifest_sha256": sha256_file(source_manifest),
            "arrays": {n: sha256_file(staging / n) for n in ARRAY_FILES}})
        if output.exists():
            shutil.rmtree(output)
        os.replace(staging, output)
    except BaseException:
        shutil.rmtree(staging, ignore_errors=True)
        raise
    return output


def validate_probe_cache(cache_dir: str | Path, data_root: str | Path | None = None) -> dict:
    """Structural and lineage checks; returns ``{"ok": bool, "errors": [...]}``."""

    root = Path(cache_dir)
    errors: list[str] = []
    try:
        manifest = read_json(root / "manifest.json")
    except (OSError, ValueError) as exc:
        return {"ok": False, "errors": [f"manifest unreadable: {exc}"]}
    if manifest.get("format") != CACHE_FORMAT:
        errors.append(f"format {manifest.get('format')} != {CACHE_FORMAT}")
    for name, digest in manifest.get("arrays", {}).items():
        path = root / name
        if not path.is_file():
            errors.append(f"missing {name}")
        elif sha256_file(path) != digest:
            errors.append(f"{name} does not match its recorded sha256")
    if not errors:
        labels = np.load(root / "profile_labels.npy")
        splits = np.load(root / "profile_splits.npy")
        p_off, q_off = np.load(root / "p_offsets.npy"), np.load(root / "q_offsets.npy")
        p_pos, p_idx = np.load(root / "p_positions.npy"), np.load(root / "p_profile_indices.npy")
        if labels.shape != (manifest["profiles"], len(manifest["tasks"])):
            errors.append("profile_labels shape mismatch")
        if splits.shape[0] != labels.shape[0] or not set(np.unique(splits)).issubset({0, 1}):
            errors.append("profile_splits malformed")
        if p_pos.shape != (len(p_off) - 1, 6) or p_idx.shape[0] != len(p_off) - 1:
            errors.append("P arrays disagree on the number of examples")
        if len(q_off) - 1 != labels.shape[0]:
            errors.append("Q examples != profiles")
        if (np.diff(p_off) <= 0).any() or (np.diff(q_off) <= 0).any():
            errors.append("empty token rows")
        lengths = np.diff(p_off)
        if (p_pos < 0).any() or (p_pos >= lengths[:, None]).any() or (np.diff(p_pos, axis=1) <= 0).any():
            errors.append("P positions out of range or not increasing")
        for col, task in enumerate(manifest["tasks"]):
            if labels[:, col].min() < 0 or labels[:, col].max() >= len(task["classes"]):
                errors.append(f"labels of {task['key']} out of range")
    if data_root is not None and not errors:
        src = Path(data_root) / "manifest.json"
        if not src.is_file() or sha256_file(src) != manifest.get("source_manifest_sha256"):
            errors.append("cache was built from a different dataset manifest")
    return {"ok": not errors, "errors": errors, "format": manifest.get("format"), "p_examples": manifest.get("p_examples"),
            "q_examples": manifest.get("q_examples")}


@dataclass(frozen=True)
class ProbeItem:
    input_ids: np.ndarray
    positions: np.ndarray
    label: int


class CachedProbeDataset:
    """Examples of one (kind, task, split) served from the memory-mapped cache."""

    def __init__(self, cache_dir: str | Path, *, kind: str, attribute: str, target: str, split: str) -> None:
        root = Path(cache_dir)
        self.manifest = read_json(root / "manifest.json")
        if self.manifest.get("format") != CACHE_FORMAT:
            raise ValueError("unsupported probe cache format")
        keys = [t["key"] for t in self.manifest["tasks"]]
        key = f"{attribute}:{target}"
        if key not in keys:
            raise ValueError(f"no probe task {key!r}")
        if kind not in ("p", "q"):
            raise ValueError("kind must be 'p' or 'q'")
        col = keys.index(key)
        self.kind, self.class_names = kind, self.manifest["tasks"][col]["classes"]
        labels = np.load(root / "profile_labels.npy", mmap_mode="r")[:, col]
        splits = np.load(root / "profile_splits.npy", mmap_mode="r")
        self.offsets = np.load(root / f"{kind}_offsets.npy", mmap_mode="r")
        self.tokens = np.memmap(root / f"{kind}_tokens.bin", dtype="<i4", mode="r")
        want = SPLIT_CODES[split]
        if kind == "p":
            owner = np.load(root / "p_profile_indices.npy", mmap_mode="r")
            self.positions = np.load(root / "p_positions.npy", mmap_mode="r")
            self.examples = np.nonzero(np.asarray(splits)[np.asarray(owner)] == want)[0]
            self.labels = np.asarray(labels)[np.asarray(owner)[self.examples]]
        else:
            self.positions = None
            self.examples = np.nonzero(np.asarray(splits) == want)[0]
            self.labels = np.asarray(labels)[self.examples]
        self.eos = int(self.manifest["eos"])

    def __len__(self) -> int:
        return int(self.examples.shape[0])

    def __getitem__(self, i: int) -> ProbeItem:
        ex = int(self.examples[i])
        ids = np.asarray(self.tokens[self.offsets[ex]:self.offsets[ex + 1]])
        pos = np.asarray(self.positions[ex]) if self.kind == "p" else np.asarray([ids.shape[0] - 1], dtype="<i4")
        return ProbeItem(ids, pos, int(self.labels[i]))

    def longest(self, limit: int) -> list[ProbeItem]:
        lengths = np.diff(np.asarray(self.offsets))[self.examples]
        return [self[int(i)] for i in np.argsort(-lengths)[:limit]]
