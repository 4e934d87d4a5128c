"""Tokenizer adapters with a reproducible identity (fingerprint).

Contract: ``encode``/``decode``, ``vocab_size``, ``boundary_token_id`` (prepended to every
document chunk) and ``fingerprint`` (recorded in shard manifests and checked at load).
Backends: a trained byte-level BPE (Hugging Face ``tokenizers``), a named ``tiktoken``
encoding, and ``SyntheticTokenizer`` - an offline identity for uniform-random shards
(reference: minitrain/data/tokenizer.py:30-246, which has the first two).
"""

from __future__ import annotations

import hashlib
import importlib.metadata
import json
from abc import ABC, abstractmethod
from collections.abc import Iterable
from pathlib import Path
from typing import Any

TOKENIZER_METADATA_FILE = "tokenizer_metadata.json"
CUSTOM_TOKENIZER_FILE = "tokenizer.json"
TOKENIZER_FORMAT_VERSION = 1


def canonical_digest(payload: dict[str, Any]) -> str:
    return hashlib.sha256(json.dumps(payload, sort_keys=True, separators=(",", ":")).encode("utf-8")).hexdigest()


def _write_metadata(output_dir: str | Path, metadata: dict[str, Any]) -> Path:
    out = Path(output_dir)
    out.mkdir(parents=True, exist_ok=True)
    target = out / TOKENIZER_METADATA_FILE
    target.write_text(json.dumps(metadata, indent=2, sort_keys=True) + "\n", encoding="utf-8")
    return target


class Tokenizer(ABC):
    @property
    @abstractmethod
    def vocab_size(self) -> int: ...

    @property
    @abstractmethod
    def boundary_token_id(self) -> int: ...

    @property
    @abstractmethod
    def fingerprint(self) -> str: ...

    @abstractmethod
    def encode(self, text: str) -> list[int]: ...

    @abstractmethod
    def decode(self, tokens: list[int]) -> str: ...

    @abstractmethod
    def save(self, output_dir: str | Path) -> Path: ...


class ByteLevelBPETokenizer(Tokenizer):
    boundary_token = "<|bos|>"

    def __init__(self, backend: Any, *, fingerprint: str | None = None) -> None:
        self._backend = backend
        bos = backend.token_to_id(self.boundary_token)
        if bos is None:
            raise ValueError(f"custom tokenizer is missing {self.boundary_token!r}")
        self._bos = int(bos)
        self._fingerprint = fingerprint or self.compute_fingerprint()

    @classmethod
    def train_from_iterator(cls, text_iterator: Iterable[str], *, vocab_size: int, min_frequency: int = 2
                            ) -> "ByteLevelBPETokenizer":
        if vocab_size < 257:
            raise ValueError("byte-level BPE vocab_size must be at least 257")
        from tokenizers import Tokenizer as HFTokenizer
        from tokenizers import decoders, models, pre_tokenizers, trainers

        # All 256 byte symbols seed the alphabet, so any UTF-8 text encodes without UNK.
        backend = HFTokenizer(models.BPE())
        backend.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
        backend.decoder = decoders.ByteLevel()
        trainer = trainers.BpeTrainer(vocab_size=vocab_size, min_frequency=min_frequency,
                                      special_tokens=[cls.boundary_token],
                                      initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False)
        backend.train_from_iterator(text_iterator, trainer=trainer)
        return cls(backend)

    @property
    def vocab_size(self) -> int:
        return int(self._backend.get_vocab_size(with_added_tokens=True))

    @property
    def boundary_token_id(self) -> int:
        return self._bos

    @property
    def fingerprint(self) -> str:
        return self._fingerprint

    def encode(self, text: str) -> list[int]:
        return list(self._backend.encode(text, add_special_tokens=False).ids)

    def decode(self, tokens: list[int]) -> str:
        return self._backend.decode(tokens, skip_special_tokens=False)

    def compute_fingerprint(self) -> str:
        return canonical_digest({"format_version": TOKENIZER_FORMAT_VERSION, "kind": "byte_bpe",
                                 "boundary_token": self.boundary_token,
                                 "backend_json": json.loads(self._backend.to_str())})

    def save(self, output_dir: str | Path) -> Path:
        Path(output_dir).mkdir(parents=True, exist_ok=True)
        self._backend.save(str(Path(output_dir) / CUSTOM_TOKENIZER_FILE))
        return _write_metadata(output_dir, {
            "format_version": TOKENIZER_FORMAT_VERSION, "kind": "byte_bpe", "vocab_size": self.vocab_size,
            "boundary_token": self.boundary_token, "boundary_token_id": self.boundary_token_id,
            "fingerprint": self.fingerprint})

    @classmethod
    def load(cls, tokenizer_dir: str | Path) -> "ByteLevelBPETokenizer":
        from tokenizers import Tokenizer as HFTokenizer

        root = Path(tokenizer_dir)
        meta = json.loads((root / TOKENIZER_METADATA_FILE).read_text("utf-8"))
        tok = cls(HFTokenizer.from_file(str(root / CUSTOM_TOKENIZER_FILE)), fingerprint=meta["fingerprint"])
        if tok.compute_fingerprint() != tok.fingerprint:
            raise ValueError("custom tokenizer artifact fingerprint does not match metadata")
        return tok


class TiktokenTokenizer(Tokenizer):
    """Named tiktoken encoding; the runtime version is part of the identity."""

    def __init__(self, encoding_name: str) -> None:
        import tiktoken

        self.encoding_name = encoding_name
        self._backend = tiktoken.get_encoding(encoding_name)
        self._eot = int(self._backend.eot_token)
        self._runtime_version = importlib.metadata.version("tiktoken")
        self._fingerprint = canonical_digest({
            "format_version": TOKENIZER_FORMAT_VERSION, "kind": "tiktoken", "encoding_name": encoding_name,
            "tiktoken_version": self._runtime_version, "vocab_size": self.vocab_size,
            "boundary_token_id": self._eot})

    @property
    def vocab_size(self) -> int:
        return int(self._backend.n_vocab)

    @property
    def boundary_token_id(self) -> int:
        return self._eot

    @property
    def fingerprint(self) -> str:
        return self._fingerprint

    def encode(self, text: str) -> list[int]:
        return list(self._backend.encode_ordinary(text))

    def decode(self, tokens: list[int]) -> str:
        return self._backend.decode(tokens)

    def save(self, output_dir: str | Path) -> Path:
        return _write_metadata(output_dir, {
            "format_version": TOKENIZER_FORMAT_VERSION, "kind": "tiktoken", "encoding_name": self.encoding_name,
            "runtime_version": self._runtime_version, "vocab_size": self.vocab_size,
            "boundary_token_id": self.boundary_token_id, "fingerprint": self.fingerprint})


class SyntheticTokenizer(Tokenizer):
    """Identity over whitespace-separated integer ids; lets random shards carry a real fingerprint."""

    def __init__(self, vocab_size: int, boundary_token_id: int = 0) -> None:
        if not 0 <= boundary_token_id < vocab_size:
            raise ValueError("boundary_token_id must be inside the vocabulary")
        self._vocab = int(vocab_size)
        self._bos = int(boundary_token_id)
        self._fingerprint = canonical_digest({"format_version": TOKENIZER_FORMAT_VERSION, "kind": "synthetic",
                                              "vocab_size": self._vocab, "boundary_token_id": self._bos})

    @property
    def vocab_size(self) -> int:
        return self._vocab

    @property
    def boundary_token_id(self) -> int:
        return self._bos

    @property
    def fingerprint(self) -> str:
        return self._fingerprint

    def encode(self, text: str) -> list[int]:
        ids = [int(piece) for piece in text.split()]
        if any(not 0 <= i < self._vocab for i in ids):
            raise ValueError("synthetic token id outside the vocabulary")
        return ids

    def decode(self, tokens: list[int]) -> str:
        return " ".join(str(int(t)) for t in tokens)

    def save(self, output_dir: str | Path) -> Path:
        return _write_metadata(output_dir, {
            "format_version": TOKENIZER_FORMAT_VERSION, "kind": "synthetic", "vocab_size": self._vocab,
            "boundary_token_id": self._bos, "fingerprint": self._fingerprint})


def load_tokenizer(tokenizer_dir: str | Path) -> Tokenizer:
    root = Path(tokenizer_dir)
    meta = json.loads((root / TOKENIZER_METADATA_FILE).read_text("utf-8"))
    kind = meta.get("kind")
    if kind == "byte_bpe":
        return ByteLevelBPETokenizer.load(root)
    if kind == "tiktoken":
        tok = TiktokenTokenizer(meta["encoding_name"])
        if tok.fingerprint != meta["fingerprint"]:
            raise ValueError("tiktoken runtime fingerprint changed; use the recorded runtime version "
                             f"{meta.get('runtime_version')} or rebuild the token shards")
        return tok
    if kind == "synthetic":
        tok = SyntheticTokenizer(int(meta["vocab_size"]), int(meta["boundary_token_id"]))
        if tok.fingerprint != meta["fingerprint"]:
            raise ValueError("synthetic tokenizer fingerprint does not match metadata")
        return tok
    raise ValueError(f"unsupported tokenizer kind: {kind!r}")
