"""Text codecs of the study: GPT-2 byte-level BPE (the formal setting) and a plain UTF-8 byte codec.

Both expose the byte length of every token, which is what aligns character spans of attribute values with token
positions (reference: experiments/synbios_moe/probes/model.py:41-75).  The byte codec needs no vocabulary file, so
the whole pipeline can be exercised on a machine without the GPT-2 tables.
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


def get_codec(name: str):
    if name == "bytes":
        return ByteCodec()
    if name == "gpt2":
        return Gpt2Codec()
    raise ValueError(f"unknown codec {name!r} (expected 'gpt2' or 'bytes')")


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
