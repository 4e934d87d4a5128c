"""Raw text stages: readers -> cleaner -> chunker (tokenisation happens later).

Behaviour mirrors minitrain/data/documents.py:22-225: txt/md/jsonl/parquet readers with
stable document ids, an auditable cleaner (NFC, control-character ratio, length, alphabetic
ratio, repeated lines, exact dedup after normalisation) with per-reason counters, and a
non-overlapping chunker that prefers natural boundaries in the second half of the window.
"""

from __future__ import annotations

import hashlib
import json
import re
import unicodedata
from collections import Counter
from collections.abc import Iterable, Iterator
from dataclasses import asdict, dataclass, field
from pathlib import Path

_TEXT_SUFFIXES = {".txt", ".text", ".md"}
_JSONL_SUFFIXES = {".jsonl", ".jsonlines"}


@dataclass(frozen=True)
class Document:
    id: str
    text: str
    source: str
    metadata: dict[str, object] = field(default_factory=dict)


def _read_jsonl(path: Path, source: str, text_field: str) -> Iterator[Document]:
    with path.open("r", encoding="utf-8") as fh:
        for lineno, line in enumerate(fh, start=1):
            if not line.strip():
                continue
            row = json.loads(line)
            text = row.get(text_field)
            if not isinstance(text, str):
                raise ValueError(f"{path}:{lineno} field {text_field!r} must be a string")
            extra = {k: v for k, v in row.items() if k != text_field}
            yield Document(str(row.get("id", f"{source}:{lineno}")), text, source, extra)


def _read_parquet(path: Path, source: str, text_field: str) -> Iterator[Document]:
    try:
        import pyarrow.parquet as pq
    except ImportError as err:
        raise RuntimeError("Parquet input requires pyarrow") from err
    handle = pq.ParquetFile(path)
    base = 0
    for group in range(handle.num_row_groups):
        table = handle.read_row_group(group, columns=[text_field])
        for i, text in enumerate(table.column(text_field).to_pylist()):
            if not isinstance(text, str):
                raise ValueError(f"{path} row {base + i} is not text")
            yield Document(f"{source}:{base + i}", text, source, {"row_group": group})
        base += table.num_rows


def iter_documents(paths: Iterable[str | Path], *, text_field: str = "text") -> Iterator[Document]:
    for raw in paths:
        path = Path(raw)
        source = str(path.resolve())
        suffix = path.suffix.lower()
        if suffix in _TEXT_SUFFIXES:
            yield Document(f"{source}:0", path.read_text("utf-8"), source)
        elif suffix in _JSONL_SUFFIXES:
            yield from _read_jsonl(path, source, text_field)
        elif suffix == ".parquet":
            yield from _read_parquet(path, source, text_field)
        else:
            raise ValueError(f"unsupported document input format: {path}")


@dataclass(frozen=True)
class CleaningConfig:
    enabled: bool = True
    min_chars: int = 32
    min_alpha_ratio: float = 0.05
    max_control_ratio: float = 0.01
    max_repeated_line_fraction: float = 0.5
    exact_dedup: bool = True

    def to_dict(self) -> dict[str, object]:
        return asdict(self)


@dataclass
class CleaningStats:
    seen: int = 0
    accepted: int = 0
    rejected_empty: int = 0
    rejected_short: int = 0
    rejected_alpha_ratio: int = 0
    rejected_control_ratio: int = 0
    rejected_repetition: int = 0
    rejected_duplicate: int = 0

    def to_dict(self) -> dict[str, int]:
        return asdict(self)


def _is_control(ch: str) -> bool:
    return unicodedata.category(ch) == "Cc" and ch not in "\n\t"


class DocumentCleaner:
    _spaces = re.compile(r"[^\S\r\n]+")
    _many_blank = re.compile(r"\n{3,}")

    def __init__(self, config: CleaningConfig | None = None) -> None:
        self.config = config or CleaningConfig()
        self.stats = CleaningStats()
        self._digests: set[str] = set()

    def normalize(self, text: str) -> str:
        text = unicodedata.normalize("NFC", text)
        text = "".join(ch for ch in text if not _is_control(ch))
        text = self._spaces.sub(" ", text)
        text = "\n".join(line.strip() for line in text.splitlines())
        return self._many_blank.sub("\n\n", text).strip()

    def _reject_reason(self, raw: str, text: str) -> str | None:
        cfg = self.config
        # measured on the raw text so that stripping control bytes cannot hide them
        if sum(map(_is_control, raw)) / max(1, len(raw)) > cfg.max_control_ratio:
            return "control_ratio"
        if not text:
            return "empty"
        if len(text) < cfg.min_chars:
            return "short"
        visible = [ch for ch in text if not ch.isspace()]
        if sum(ch.isalpha() for ch in visible) / max(1, len(visible)) < cfg.min_alpha_ratio:
            return "alpha_ratio"
        lines = [ln.casefold() for ln in text.splitlines() if ln.strip()]
        if len(lines) >= 4:
            repeats = sum(c - 1 for c in Counter(lines).values() if c > 1)
            if repeats / len(lines) > cfg.max_repeated_line_fraction:
                return "repetition"
        return None

    def clean(self, document: Document) -> Document | None:
        self.stats.seen += 1
        if not self.config.enabled:
            self.stats.accepted += 1
            return document
        raw = document.text.replace("\r\n", "\n").replace("\r", "\n")
        # the control-ratio gate precedes normalisation; compute the normal form only if it passes
        over = sum(map(_is_control, raw)) / max(1, len(raw)) > self.config.max_control_ratio
        text = "" if over else self.normalize(raw)
        reason = "control_ratio" if over else self._reject_reason(raw, text)
        if reason is None:
            digest = hashlib.sha256(text.encode("utf-8")).hexdigest()
            if self.config.exact_dedup and digest in self._digests:
                reason = "duplicate"
        if reason is not None:
            setattr(self.stats, f"rejected_{reason}", getattr(self.stats, f"rejected_{reason}") + 1)
            return None
        self._digests.add(digest)
        self.stats.accepted += 1
        return Document(document.id, text, document.source, {**document.metadata, "clean_sha256": digest})


def chunk_document(document: Document, *, max_chars: int) -> Iterator[Document]:
    if max_chars <= 0:
        raise ValueError("max_chars must be positive")
    text = document.text
    if len(text) <= max_chars:
        yield document
        return
    begin, index = 0, 0
    while begin < len(text):
        limit = min(begin + max_chars, len(text))
        end = limit
        if limit < len(text):
            window = text[begin:limit]
            cut = max(window.rfind("\n\n"), window.rfind("\n"), window.rfind(" "))
            if cut >= max_chars // 2:
                end = begin + cut + 1
        piece = text[begin:end].strip()
        if piece:
            yield Document(f"{document.id}#chunk-{index:05d}", piece, document.source,
                           {**document.metadata, "parent_id": document.id, "chunk_index": index,
                            "char_start": begin, "char_stop": end})
            index += 1
        begin = end
