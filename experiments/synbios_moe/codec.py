"""Text codecs of the study: GPT-2 byte-level BPE (the formal setting), a byte-level BPE trained on the corpus itself,
and a plain UTF-8 byte codec.

All expose the byte length of every token, which is what aligns character spans of attribute values with token
positions (reference: experiments/synbios_moe/probes/model.py:41-75).  The byte codec needs no vocabulary file, so
the whole pipeline can be exercised on a machine without the GPT-2 tables; ``bpe:<directory>`` names a tokenizer
directory written by ``scripts/prepare_data.py train-tokenizer`` (or by ``synbios_moe.py prepare``, which trains one on the
biographies when the directory does not exist yet): real multi-byte tokens with leading spaces, without a download.
"""

from __future__ import annotations


class ByteCodec:
    name = "bytes"
    eos = 256
    vocab_size = 257

    def encode(self, text: str) -> list[int]:
        return list(text.encode("utf-8"))

    def token_num_bytes(self, token: int) -> int:
        return 0 if token == self.eos else 1

    def decode(self, tokens) -> str:
        return bytes(t for t in tokens if t < 256).decode("utf-8", errors="replace")


class Gpt2Codec:
    name = "gpt2"

    def __init__(self) -> None:
        try:
            import tiktoken
        except ImportError as exc:   # pragma: no cover
            raise RuntimeError("the gpt2 codec needs the tiktoken package") from exc
        self.encoding = tiktoken.get_encoding("gpt2")
        self.eos = self.encoding.eot_token
        self.vocab_size = self.encoding.n_vocab

    def encode(self, text: str) -> list[int]:
        return self.encoding.encode(text, allowed_special=set())

    def token_num_bytes(self, token: int) -> int:
        return 0 if token == self.eos else len(self.encoding.decode_single_token_bytes(token))

    def decode(self, tokens) -> str:
        return self.encoding.decode([t for t in tokens if t != self.eos])


def byte_level_alphabet() -> dict[str, int]:
    """Character -> byte of the byte-level BPE alphabet: printable bytes stand for themselves, the other 68 are shifted to
    code points from 256 upwards, in byte order (the published GPT-2 convention, which the ``tokenizers`` ByteLevel
    pre-tokenizer follows)."""

    keep = [*range(ord("!"), ord("~") + 1), *range(0xA1, 0xAC + 1), *range(0xAE, 0xFF + 1)]
    table, shifted = {}, 0
    for byte in range(256):
        if byte in keep:
            table[chr(byte)] = byte
        else:
            table[chr(256 + shifted)] = byte
            shifted += 1
    return table


class BpeCodec:
    """A byte-level BPE trained with this repository's data tools (``data/tokenizer.py:ByteLevelBPETokenizer``)."""

    def __init__(self, directory: str) -> None:
        from mini_train_sys_b200.data.tokenizer import ByteLevelBPETokenizer

        self.directory = str(directory)
        self.name = f"bpe:{self.directory}"
        self.tokenizer = ByteLevelBPETokenizer.load(self.directory)
        self.eos = self.tokenizer.boundary_token_id
        self.vocab_size = self.tokenizer.vocab_size
        self.fingerprint = self.tokenizer.fingerprint
        alphabet = byte_level_alphabet()
        backend = self.tokenizer._backend
        self._num_bytes = []
        for token in range(self.vocab_size):
            text = backend.id_to_token(token)
            # a special token (the boundary) is not made of alphabet characters and covers no text
            self._num_bytes.append(0 if token == self.eos or text is None or any(ch not in alphabet for ch in text) else len(text))

    def encode(self, text: str) -> list[int]:
        return self.tokenizer.encode(text)

    def token_num_bytes(self, token: int) -> int:
        return self._num_bytes[token]

    def decode(self, tokens) -> str:
        return self.tokenizer.decode([int(t) for t in tokens if int(t) != self.eos])


def codec_argument(value: str) -> str:
    """``argparse`` type of ``--codec``: ``gpt2``, ``bytes`` or ``bpe:<tokenizer directory>``."""

    if value in ("gpt2", "bytes") or (value.startswith("bpe:") and len(value) > 4):
        return value
    raise ValueError(f"unknown codec {value!r} (expected 'gpt2', 'bytes' or 'bpe:<tokenizer directory>')")


def get_codec(name: str):
    if name == "bytes":
        return ByteCodec()
    if name == "gpt2":
        return Gpt2Codec()
    if name.startswith("bpe:") and len(name) > 4:
        return BpeCodec(name[4:])
    raise ValueError(f"unknown codec {name!r} (expected 'gpt2', 'bytes' or 'bpe:<tokenizer directory>')")


def positions_before_chars(codec, text: str, char_indices: list[int]) -> tuple[list[int], list[int]]:
    """Tokens of ``[EOS] + text`` and, per character index, the position of the last token that ends at or before it.

    Character indices count code points while token boundaries count UTF-8 bytes; both are mapped to byte offsets.
    With the prepended EOS, the number of tokens that end at or before the byte offset IS that position.
    """

    ids = codec.encode(text)
    byte_starts = [len(text[:i].encode("utf-8")) for i in char_indices]
    ends, consumed = [], 0
    for tok in ids:
        consumed += codec.token_num_bytes(tok)
        ends.append(consumed)
    positions = [sum(1 for e in ends if e <= start) for start in byte_starts]
    return [codec.eos, *ids], positions


def token_span_of_chars(codec, text: str, start: int, end: int) -> tuple[list[int], int, int]:
    """Tokens of ``[EOS] + text`` and the half-open range of token indices whose bytes overlap characters ``[start, end)``."""

    ids = codec.encode(text)
    b_lo, b_hi = len(text[:start].encode("utf-8")), len(text[:end].encode("utf-8"))
    lo = hi = None
    consumed = 0
    for idx, tok in enumerate(ids, start=1):          # index 0 is the EOS
        t0, consumed = consumed, consumed + codec.token_num_bytes(tok)
        if consumed > b_lo and t0 < b_hi:
            lo = idx if lo is None else lo
            hi = idx + 1
    if lo is None:
        lo = hi = 1
    return [codec.eos, *ids], lo, hi


class ShardTokenizer:
    """Adapter that lets the shared shard writer tokenise with a study codec (used for the vocabulary-free byte codec)."""

    def __init__(self, codec) -> None:
        import hashlib

        self.codec = codec
        self._fingerprint = hashlib.sha256(f"synbios-codec:{codec.name}:{codec.vocab_size}:{codec.eos}".encode()).hexdigest()

    vocab_size = property(lambda self: self.codec.vocab_size)
    boundary_token_id = property(lambda self: self.codec.eos)
    fingerprint = property(lambda self: self._fingerprint)

    def encode(self, text: str) -> list[int]:
        return self.codec.encode(text)

    def decode(self, tokens) -> str:
        return self.codec.decode(tokens)

    def save(self, output_dir):
        import json
        from pathlib import Path

        path = Path(output_dir) / "tokenizer_metadata.json"
        path.parent.mkdir(parents=True, exist_ok=True)
        path.write_text(json.dumps({"kind": "synbios_codec", "codec": self.codec.name, "vocab_size": self.vocab_size,
                                    "boundary_token_id": self.boundary_token_id, "fingerprint": self.fingerprint}))
        return path
