"""Documents -> memory-mappable token shards + document index + manifest.

On-disk contract (format version 1, identical to minitrain/data/preprocess.py:31-365)::

    <out>/{train,validation}/shard_{:05d}.bin   little-endian <u2 (vocab <= 65536) or <u4 token ids
    <out>/{train,validation}/documents.idx      <u8 (token_offset, token_length) pairs over the split stream
    <out>/manifest.json                         written last (tmp + rename): dtype, vocab, boundary id,
                                                tokenizer fingerprint, cleaning/splitting policy, per-split
                                                shard list with sha256, document index record

A shard file only appears under its final name once complete (``.bin.tmp`` + fsync + rename).
Ordinary documents are never split across shards; a document longer than a shard is split
and every continuation starts with a fresh boundary token.
"""

from __future__ import annotations

import hashlib
import json
import os
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import BinaryIO

import numpy as np

from mini_train_sys_b200.data.documents import CleaningConfig, DocumentCleaner, chunk_document, iter_documents
from mini_train_sys_b200.data.tokenizer import Tokenizer

TOKEN_MANIFEST = "manifest.json"
TOKEN_MANIFEST_VERSION = 1
SPLITS = ("train", "validation")


def token_storage_dtype(vocab_size: int) -> np.dtype:
    if vocab_size <= 0:
        raise ValueError("vocab_size must be positive")
    if vocab_size <= 1 << 16:
        return np.dtype("<u2")
    if vocab_size <= 1 << 32:
        return np.dtype("<u4")
    raise ValueError("vocab_size exceeds uint32 token storage")


def deterministic_split(document_id: str, *, validation_fraction: float, seed: int) -> str:
    """Order-independent split: the first 8 bytes of sha256("seed:id") as a fraction of 2^64."""

    if not 0.0 <= validation_fraction < 1.0:
        raise ValueError("validation_fraction must be in [0, 1)")
    head = hashlib.sha256(f"{seed}:{document_id}".encode("utf-8")).digest()[:8]
    return "validation" if int.from_bytes(head, "big") / 2.0**64 < validation_fraction else "train"


def file_sha256(path: Path) -> str:
    digest = hashlib.sha256()
    with path.open("rb") as fh:
        while block := fh.read(1 << 20):
            digest.update(block)
    return digest.hexdigest()


@dataclass
class ShardRecord:
    path: str
    num_tokens: int
    num_bytes: int
    sha256: str


@dataclass
class DocumentIndexRecord:
    path: str
    entries: int
    dtype: str
    columns: list[str]
    num_bytes: int
    sha256: str


class TokenShardWriter:
    def __init__(self, output_dir: Path, *, split: str, dtype: np.dtype, max_tokens: int) -> None:
        if max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
        self.output_dir = Path(output_dir)
        self.split = split
        self.dtype = np.dtype(dtype)
        self.max_tokens = max_tokens
        self.split_dir = self.output_dir / split
        self.split_dir.mkdir(parents=True, exist_ok=True)
        self.records: list[ShardRecord] = []
        self.document_spans: list[tuple[int, int]] = []
        self.total_tokens = 0
        self._fh: BinaryIO | None = None
        self._tmp: Path | None = None
        self._fill = 0
        self._id_limit = 1 << (8 * self.dtype.itemsize)

    def _append(self, ids: list[int]) -> None:
        if not ids:
            return
        if len(ids) > self.max_tokens - self._fill:
            raise ValueError("contiguous token sequence does not fit current shard")
        if min(ids) < 0:
            raise ValueError("token ids must be non-negative")
        if max(ids) >= self._id_limit:
            raise ValueError(f"token id does not fit {self.dtype.name}")
        if self._fh is None:
            self._tmp = self.split_dir / f"shard_{len(self.records):05d}.bin.tmp"
            self._fh = self._tmp.open("wb")
            self._fill = 0
        self._fh.write(np.asarray(ids, dtype=self.dtype).tobytes(order="C"))
        self._fill += len(ids)
        self.total_tokens += len(ids)
        if self._fill == self.max_tokens:
            self._publish()

    def _span(self, ids: list[int]) -> None:
        start = self.total_tokens
        self._append(ids)
        self.document_spans.append((start, len(ids)))

    def write_document(self, token_ids: list[int], *, boundary_token_id: int) -> int:
        if not token_ids or token_ids[0] != boundary_token_id:
            raise ValueError("document token sequence must start with boundary_token_id")
        if len(token_ids) <= self.max_tokens:
            if self._fill and len(token_ids) > self.max_tokens - self._fill:
                self._publish()      # close early instead of splitting an ordinary document
            self._span(token_ids)
            return len(token_ids)
        if self._fill:
            self._publish()
        body, written, step = token_ids[1:], 0, self.max_tokens - 1
        for lo in range(0, len(body), step):
            piece = [boundary_token_id, *body[lo:lo + step]]
            self._span(piece)
            written += len(piece)
            if lo + step < len(body) and self._fill:
                self._publish()
        return written

    def _publish(self) -> None:
        if self._fh is None or self._fill == 0:
            return
        self._fh.flush()
        os.fsync(self._fh.fileno())
        self._fh.close()
        final = self._tmp.with_suffix("")   # drop ".tmp" -> shard_XXXXX.bin
        self._tmp.replace(final)
        self.records.append(ShardRecord(final.relative_to(self.output_dir).as_posix(), self._fill,
                                        final.stat().st_size, file_sha256(final)))
        self._fh, self._tmp, self._fill = None, None, 0

    def close(self) -> None:
        self._publish()

    def write_document_index(self) -> DocumentIndexRecord:
        final = self.split_dir / "documents.idx"
        tmp = final.with_suffix(".idx.tmp")
        pairs = np.asarray(self.document_spans, dtype="<u8").reshape(-1, 2)
        with tmp.open("wb") as fh:
            fh.write(pairs.tobytes(order="C"))
            fh.flush()
            os.fsync(fh.fileno())
        tmp.replace(final)
        return DocumentIndexRecord(final.relative_to(self.output_dir).as_posix(), len(self.document_spans), "<u8",
                                   ["token_offset", "token_length"], final.stat().st_size, file_sha256(final))


def tokenizer_training_texts(paths, *, text_field: str, cleaning: CleaningConfig, max_document_chars: int,
                             max_training_chars: int):
    """Cleaned chunks for BPE training, cut off at a character budget."""

    cleaner = DocumentCleaner(cleaning)
    used = 0
    for doc in iter_documents(paths, text_field=text_field):
        cleaned = cleaner.clean(doc)
        if cleaned is None:
            continue
        for chunk in chunk_document(cleaned, max_chars=max_document_chars):
            if used >= max_training_chars:
                return
            text = chunk.text[:max_training_chars - used]
            if text:
                used += len(text)
                yield text


def write_manifest(output_dir: Path, manifest: dict) -> Path:
    target = Path(output_dir) / TOKEN_MANIFEST
    tmp = target.with_suffix(".json.tmp")
    tmp.write_text(json.dumps(manifest, indent=2, sort_keys=True) + "\n", "utf-8")
    tmp.replace(target)
    return target


def build_manifest(*, tokenizer_vocab: int, boundary_token_id: int, fingerprint: str, dtype: np.dtype,
                   writers: dict[str, TokenShardWriter], split_stats: dict[str, dict[str, int]],
                   cleaning: CleaningConfig, cleaning_stats: dict[str, int], max_document_chars: int,
                   split_seed: int, validation_fraction: float) -> dict:
    indices = {s: writers[s].write_document_index() for s in writers}
    return {
        "format_version": TOKEN_MANIFEST_VERSION, "dtype": dtype.str, "bytes_per_token": dtype.itemsize,
        "vocab_size": tokenizer_vocab, "boundary_token_id": boundary_token_id, "tokenizer_fingerprint": fingerprint,
        "document_boundary": "prepend boundary_token_id to every document chunk",
        "chunking": {"max_document_chars": max_document_chars, "overlap_chars": 0},
        "cleaning": cleaning.to_dict(), "cleaning_stats": cleaning_stats,
        "splitting": {"algorithm": "sha256(seed:document_id)", "seed": split_seed,
                      "validation_fraction": validation_fraction},
        "splits": {s: {**split_stats[s], "shards": [asdict(r) for r in writers[s].records],
                       "document_index": asdict(indices[s])} for s in writers},
    }


def prepare_token_shards(paths, *, output_dir: str | Path, tokenizer: Tokenizer, text_field: str = "text",
                         cleaning: CleaningConfig | None = None, max_document_chars: int = 100_000,
                         max_shard_tokens: int = 10_000_000, validation_fraction: float = 0.01,
                         split_seed: int = 42) -> Path:
    out = Path(output_dir)
    out.mkdir(parents=True, exist_ok=True)
    cleaning = cleaning or CleaningConfig()
    cleaner = DocumentCleaner(cleaning)
    dtype = token_storage_dtype(tokenizer.vocab_size)
    writers = {s: TokenShardWriter(out, split=s, dtype=dtype, max_tokens=max_shard_tokens) for s in SPLITS}
    stats = {s: {"documents": 0, "chunks": 0, "tokens": 0} for s in SPLITS}
    bos = tokenizer.boundary_token_id
    for doc in iter_documents(paths, text_field=text_field):
        cleaned = cleaner.clean(doc)
        if cleaned is None:
            continue
        split = deterministic_split(cleaned.id, validation_fraction=validation_fraction, seed=split_seed)
        stats[split]["documents"] += 1
        for chunk in chunk_document(cleaned, max_chars=max_document_chars):
            ids = [bos, *tokenizer.encode(chunk.text)]
            if max(ids) >= tokenizer.vocab_size:
                raise ValueError("tokenizer emitted an id outside its declared vocabulary")
            stats[split]["tokens"] += writers[split].write_document(ids, boundary_token_id=bos)
            stats[split]["chunks"] += 1
    for w in writers.values():
        w.close()
    manifest = build_manifest(tokenizer_vocab=tokenizer.vocab_size, boundary_token_id=bos,
                              fingerprint=tokenizer.fingerprint, dtype=dtype, writers=writers, split_stats=stats,
                              cleaning=cleaning, cleaning_stats=cleaner.stats.to_dict(),
                              max_document_chars=max_document_chars, split_seed=split_seed,
                              validation_fraction=validation_fraction)
    return write_manifest(out, manifest)


def write_random_token_shards(output_dir: str | Path, *, vocab_size: int, num_tokens: int, seed: int = 0,
                              document_tokens: int = 2048, max_shard_tokens: int = 10_000_000,
                              validation_tokens: int = 0) -> Path:
    """Uniform-random token ids as valid shards + index + manifest (synthetic tokenizer identity).

    Needs no corpus, tokenizer download or network: this is what benchmarks train on.
    """

    from mini_train_sys_b200.data.tokenizer import SyntheticTokenizer

    out = Path(output_dir)
    out.mkdir(parents=True, exist_ok=True)
    tok = SyntheticTokenizer(vocab_size)
    tok.save(out / "tokenizer")
    dtype = token_storage_dtype(vocab_size)
    rng = np.random.default_rng(seed)
    writers = {s: TokenShardWriter(out, split=s, dtype=dtype, max_tokens=max_shard_tokens) for s in SPLITS}
    stats = {s: {"documents": 0, "chunks": 0, "tokens": 0} for s in SPLITS}
    for split, budget in (("train", num_tokens), ("validation", validation_tokens)):
        left = budget
        while left > 0:
            n = min(document_tokens, left)
            ids = [tok.boundary_token_id, *rng.integers(0, vocab_size, size=n - 1).tolist()] if n > 1 else [tok.boundary_token_id]
            stats[split]["tokens"] += writers[split].write_document(ids, boundary_token_id=tok.boundary_token_id)
            stats[split]["documents"] += 1
            stats[split]["chunks"] += 1
            left -= n
    for w in writers.values():
        w.close()
    cleaning = CleaningConfig(enabled=False)
    manifest = build_manifest(tokenizer_vocab=vocab_size, boundary_token_id=tok.boundary_token_id,
                              fingerprint=tok.fingerprint, dtype=dtype, writers=writers, split_stats=stats,
                              cleaning=cleaning, cleaning_stats=DocumentCleaner(cleaning).stats.to_dict(),
                              max_document_chars=0, split_seed=seed, validation_fraction=0.0)
    manifest["synthetic"] = {"distribution": "uniform", "seed": seed}
    return write_manifest(out, manifest)


def load_manifest(path: str | Path) -> tuple[Path, dict[str, object]]:
    path = Path(path)
    manifest_path = path if path.is_file() else path / TOKEN_MANIFEST
    manifest = json.loads(manifest_path.read_text("utf-8"))
    if manifest.get("format_version") != TOKEN_MANIFEST_VERSION:
        raise ValueError(f"unsupported token manifest version: {manifest.get('format_version')}")
    return manifest_path, manifest
