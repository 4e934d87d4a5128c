"""Data preparation CLI: ``train-tokenizer``, ``use-tiktoken``, ``tokenize``, ``inspect``, ``random-shards``.

The first four sub-commands mirror the reference tool (scripts/prepare_data.py:31-156); ``random-shards`` writes
uniform-random token shards with a synthetic tokenizer identity, which needs neither a corpus nor a download.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from mini_train_sys_b200.data.documents import CleaningConfig  # noqa: E402
from mini_train_sys_b200.data.preprocess import (load_manifest, prepare_token_shards, tokenizer_training_texts,  # noqa: E402
                                                 write_random_token_shards)
from mini_train_sys_b200.data.tokenizer import ByteLevelBPETokenizer, TiktokenTokenizer, load_tokenizer  # noqa: E402

SUFFIXES = {".txt", ".text", ".md", ".jsonl", ".jsonlines", ".parquet"}


def resolve_inputs(items: list[str]) -> list[Path]:
    found: list[Path] = []
    for item in items:
        path = Path(item)
        if path.is_dir():
            found.extend(sorted(p for p in path.rglob("*") if p.is_file() and p.suffix.lower() in SUFFIXES))
        elif path.is_file():
            found.append(path)
        else:
            raise FileNotFoundError(f"input does not exist: {path}")
    if not found:
        raise ValueError("no input documents found")
    return found


def cleaning_from(args) -> CleaningConfig:
    return CleaningConfig(enabled=not args.no_clean, min_chars=args.min_chars, min_alpha_ratio=args.min_alpha_ratio,
                          max_control_ratio=args.max_control_ratio, max_repeated_line_fraction=args.max_repeated_line_fraction,
                          exact_dedup=not args.no_dedup)


def add_cleaning_flags(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--text-field", default="text")
    ap.add_argument("--no-clean", action="store_true")
    ap.add_argument("--no-dedup", "--no-exact-dedup", dest="no_dedup", action="store_true")
    ap.add_argument("--min-chars", type=int, default=32)
    ap.add_argument("--min-alpha-ratio", type=float, default=0.05, help="letters among the visible characters")
    ap.add_argument("--max-control-ratio", type=float, default=0.01, help="control characters in the raw text")
    ap.add_argument("--max-repeated-line-fraction", type=float, default=0.5)
    ap.add_argument("--max-document-chars", type=int, default=100_000)


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__)
    sub = ap.add_subparsers(dest="command", required=True)
    tt = sub.add_parser("train-tokenizer", help="train a byte-level BPE on the cleaned corpus")
    tt.add_argument("inputs", nargs="+")
    tt.add_argument("--output", required=True)
    tt.add_argument("--vocab-size", type=int, default=32000)
    tt.add_argument("--min-frequency", type=int, default=2)
    tt.add_argument("--max-training-chars", type=int, default=200_000_000)
    add_cleaning_flags(tt)
    tk = sub.add_parser("use-tiktoken", help="record a named tiktoken encoding as the tokenizer")
    tk.add_argument("--encoding", default="gpt2")
    tk.add_argument("--output", required=True)
    tz = sub.add_parser("tokenize", help="clean, split, chunk and tokenize documents into token shards")
    tz.add_argument("inputs", nargs="+")
    tz.add_argument("--tokenizer", required=True)
    tz.add_argument("--output", required=True)
    tz.add_argument("--max-shard-tokens", type=int, default=10_000_000)
    tz.add_argument("--validation-fraction", type=float, default=0.01)
    tz.add_argument("--split-seed", type=int, default=42)
    add_cleaning_flags(tz)
    ins = sub.add_parser("inspect", help="print a manifest summary")
    ins.add_argument("path")
    rs = sub.add_parser("random-shards", help="uniform-random token shards (synthetic tokenizer)")
    rs.add_argument("--output", required=True)
    rs.add_argument("--vocab-size", type=int, required=True)
    rs.add_argument("--num-tokens", type=int, required=True)
    rs.add_argument("--validation-tokens", type=int, default=0)
    rs.add_argument("--seed", type=int, default=0)
    rs.add_argument("--max-shard-tokens", type=int, default=10_000_000)
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.command == "train-tokenizer":
        texts = tokenizer_training_texts(resolve_inputs(args.inputs), text_field=args.text_field, cleaning=cleaning_from(args),
                                         max_document_chars=args.max_document_chars, max_training_chars=args.max_training_chars)
        tok = ByteLevelBPETokenizer.train_from_iterator(texts, vocab_size=args.vocab_size, min_frequency=args.min_frequency)
        print(json.dumps({"metadata": str(tok.save(args.output)), "vocab_size": tok.vocab_size, "fingerprint": tok.fingerprint}))
    elif args.command == "use-tiktoken":
        tok = TiktokenTokenizer(args.encoding)
        print(json.dumps({"metadata": str(tok.save(args.output)), "vocab_size": tok.vocab_size, "fingerprint": tok.fingerprint}))
    elif args.command == "tokenize":
        manifest = prepare_token_shards(resolve_inputs(args.inputs), output_dir=args.output, tokenizer=load_tokenizer(args.tokenizer),
                                        text_field=args.text_field, cleaning=cleaning_from(args),
                                        max_document_chars=args.max_document_chars, max_shard_tokens=args.max_shard_tokens,
                                        validation_fraction=args.validation_fraction, split_seed=args.split_seed)
        print(json.dumps({"manifest": str(manifest)}))
    elif args.command == "inspect":
        _, manifest = load_manifest(args.path)
        summary = {k: manifest[k] for k in ("format_version", "dtype", "vocab_size", "boundary_token_id", "tokenizer_fingerprint")}
        summary["splits"] = {s: {"documents": v["documents"], "tokens": v["tokens"], "shards": len(v["shards"])}
                             for s, v in manifest["splits"].items()}
        summary["cleaning_stats"] = manifest.get("cleaning_stats")
        print(json.dumps(summary, indent=2))
    else:
        manifest = write_random_token_shards(args.output, vocab_size=args.vocab_size, num_tokens=args.num_tokens, seed=args.seed,
                                             max_shard_tokens=args.max_shard_tokens, validation_tokens=args.validation_tokens)
        print(json.dumps({"manifest": str(manifest)}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
