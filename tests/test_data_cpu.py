"""Documents -> shards -> loaders: format, determinism, rank disjointness, interoperability with the reference loader."""

import json
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from mini_train_sys_b200.data.dataloader import (RandomizedDocumentBlockDataset, RandomizedDocumentSampler, ShardAwareBlockSampler,
                                                 ShardedTokenBlockDataset, TokenBlockDataset, build_training_dataloader,
                                                 load_tokens_from_file, resolve_data_workers)
from mini_train_sys_b200.data.documents import CleaningConfig, Document, DocumentCleaner, chunk_document, iter_documents
from mini_train_sys_b200.data.preprocess import (TokenShardWriter, deterministic_split, load_manifest, prepare_token_shards,
                                                 token_storage_dtype, write_random_token_shards)
from mini_train_sys_b200.data.tokenizer import ByteLevelBPETokenizer, SyntheticTokenizer, load_tokenizer
from mini_train_sys_b200.runtime.config import DataConfig

ROOT = Path(__file__).resolve().parents[1]


def test_cleaner_gates_and_stats():
    cleaner = DocumentCleaner(CleaningConfig(min_chars=10))
    good = cleaner.clean(Document("a", "Hello   world,\r\nthis is  fine.\n\n\n\nEnd", "s"))
    assert good is not None and good.text == "Hello world,\nthis is fine.\n\nEnd" and "clean_sha256" in good.metadata
    assert cleaner.clean(Document("b", "Hello world,\nthis is fine.\n\nEnd", "s")) is None        # duplicate after normalisation
    assert cleaner.clean(Document("c", "short", "s")) is None
    assert cleaner.clean(Document("d", "12345 67890 12345 67890 !!!", "s")) is None               # no letters
    assert cleaner.clean(Document("e", "x" * 20 + "\x00" * 5, "s")) is None                       # control characters
    assert cleaner.clean(Document("f", "\n".join(["same line"] * 6), "s")) is None                # repetition
    assert cleaner.clean(Document("g", "   \n ", "s")) is None
    st = cleaner.stats.to_dict()
    assert st == {"seen": 7, "accepted": 1, "rejected_empty": 1, "rejected_short": 1, "rejected_alpha_ratio": 1,
                  "rejected_control_ratio": 1, "rejected_repetition": 1, "rejected_duplicate": 1}


def test_chunking_is_non_overlapping_and_prefers_boundaries():
    text = " ".join(f"word{i}" for i in range(400))
    chunks = list(chunk_document(Document("d", text, "s"), max_chars=300))
    assert all(len(c.text) <= 300 for c in chunks) and len(chunks) > 5
    assert " ".join(c.text for c in chunks) == text
    assert [c.metadata["chunk_index"] for c in chunks] == list(range(len(chunks)))
    assert chunks[0].id == "d#chunk-00000"


def test_readers(tmp_path):
    (tmp_path / "a.txt").write_text("plain text")
    (tmp_path / "b.jsonl").write_text(json.dumps({"id": "x1", "text": "one", "lang": "en"}) + "\n\n" + json.dumps({"text": "two"}) + "\n")
    docs = list(iter_documents([tmp_path / "a.txt", tmp_path / "b.jsonl"]))
    assert [d.text for d in docs] == ["plain text", "one", "two"]
    assert docs[1].id == "x1" and docs[1].metadata == {"id": "x1", "lang": "en"} and docs[2].id.endswith(":3")
    with pytest.raises(ValueError):
        list(iter_documents([tmp_path / "c.csv"]))


def test_split_and_dtype_rules():
    assert token_storage_dtype(65536) == np.dtype("<u2") and token_storage_dtype(65537) == np.dtype("<u4")
    picks = [deterministic_split(f"doc{i}", validation_fraction=0.2, seed=1) for i in range(2000)]
    assert 0.15 < picks.count("validation") / 2000 < 0.25
    assert picks == [deterministic_split(f"doc{i}", validation_fraction=0.2, seed=1) for i in range(2000)]


def test_shard_writer_never_splits_ordinary_documents(tmp_path):
    w = TokenShardWriter(tmp_path, split="train", dtype=np.dtype("<u2"), max_tokens=10)
    w.write_document([0, 1, 2, 3, 4, 5], boundary_token_id=0)
    w.write_document([0, 7, 8, 9, 10, 11], boundary_token_id=0)          # does not fit the remaining 4: new shard
    w.write_document([0, *range(20, 45)], boundary_token_id=0)           # oversize: split, every piece starts with BOS
    w.close()
    assert [r.num_tokens for r in w.records] == [6, 6, 10, 10, 8]
    data = [np.fromfile(tmp_path / r.path, dtype="<u2") for r in w.records]
    assert all(int(d[0]) == 0 for d in data)
    spans = w.document_spans
    assert spans[0] == (0, 6) and spans[1] == (6, 6) and sum(n for _, n in spans) == w.total_tokens
    assert not list(tmp_path.rglob("*.tmp"))
    with pytest.raises(ValueError):
        w.write_document([5, 1], boundary_token_id=0)


@pytest.fixture()
def shards(tmp_path):
    manifest = write_random_token_shards(tmp_path / "data", vocab_size=500, num_tokens=20_000, seed=3, document_tokens=333,
                                         max_shard_tokens=4_000, validation_tokens=2_000)
    return manifest.parent


def test_random_shards_manifest_and_loaders(shards):
    _, manifest = load_manifest(shards)
    assert manifest["format_version"] == 1 and manifest["dtype"] == "<u2" and manifest["vocab_size"] == 500
    assert manifest["splits"]["train"]["tokens"] == 20_000 and len(manifest["splits"]["train"]["shards"]) >= 5
    tok = load_tokenizer(shards / "tokenizer")
    assert isinstance(tok, SyntheticTokenizer) and tok.fingerprint == manifest["tokenizer_fingerprint"]
    ds = ShardedTokenBlockDataset(shards, split="train", seq_len=64)
    assert len(ds) == (20_000 - 1) // 64
    stream = np.concatenate([np.fromfile(shards / r["path"], dtype="<u2") for r in manifest["splits"]["train"]["shards"]])
    for i in (0, 61, len(ds) - 1):          # block 61 straddles a shard boundary
        ex = ds[i]
        assert torch.equal(ex["input_ids"], torch.from_numpy(stream[i * 64:i * 64 + 64].astype(np.int64)))
        assert torch.equal(ex["targets"], torch.from_numpy(stream[i * 64 + 1:i * 64 + 65].astype(np.int64)))
    rds = RandomizedDocumentBlockDataset(shards, split="train", seq_len=64)
    sampler = RandomizedDocumentSampler(rds, shuffle=True, seed=5)
    sampler.set_epoch(2)
    specs = list(sampler)
    assert len(specs) == len(rds) and all(sum(n for _, n in s.segments) == 65 for s in specs)
    assert rds[specs[0]]["input_ids"].shape == (64,)


def test_document_sampler_cursor_resumes_inside_the_reordered_stream(shards):
    rds = RandomizedDocumentBlockDataset(shards, split="train", seq_len=64)
    for world in (1, 3):
        for rank in range(world):
            sampler = RandomizedDocumentSampler(rds, shuffle=True, seed=5, rank=rank, world_size=world)
            sampler.set_epoch(2)
            full = list(sampler)
            sampler.set_start(7)
            assert list(sampler) == full[7:] and list(sampler) == full           # one iteration only
            sampler.set_start(len(full))
            assert list(sampler) == []


@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_sampler_ranks_are_disjoint_equal_and_deterministic(shards, world):
    ds = ShardedTokenBlockDataset(shards, split="train", seq_len=32)
    per_rank = []
    for rank in range(world):
        s = ShardAwareBlockSampler(ds, shuffle=True, seed=11, rank=rank, world_size=world, shuffle_window=50)
        s.set_epoch(4)
        per_rank.append(list(s))
        assert per_rank[-1] == list(s) and len(per_rank[-1]) == len(ds) // world
    flat = [i for r in per_rank for i in r]
    assert len(set(flat)) == len(flat)
    s0 = ShardAwareBlockSampler(ds, shuffle=True, seed=11, rank=0, world_size=world, shuffle_window=50)
    s0.set_epoch(5)
    assert list(s0) != per_rank[0]


def test_training_loader_guards(shards):
    cfg = DataConfig(source="token_shards", path=str(shards), num_workers=0, persistent_workers=False, pin_memory=False)
    loader = build_training_dataloader(cfg, seq_len=64, batch_size=4, vocab_size=500, seed=0)
    batch = next(iter(loader))
    assert batch["input_ids"].shape == (4, 64) and batch["targets"].dtype == torch.long
    with pytest.raises(ValueError, match="vocab"):
        build_training_dataloader(cfg, seq_len=64, batch_size=4, vocab_size=100, seed=0)
    from dataclasses import replace

    with pytest.raises(ValueError, match="fingerprint"):
        build_training_dataloader(replace(cfg, tokenizer_fingerprint="nope"), seq_len=64, batch_size=4, vocab_size=500, seed=0)
    rnd = DataConfig(source="random", num_tokens=1000, num_workers=0, persistent_workers=False, pin_memory=False)
    a = next(iter(build_training_dataloader(rnd, seq_len=16, batch_size=2, vocab_size=50, seed=7)))
    b = next(iter(build_training_dataloader(rnd, seq_len=16, batch_size=2, vocab_size=50, seed=7)))
    assert torch.equal(a["input_ids"], b["input_ids"])
    assert resolve_data_workers(DataConfig(num_workers=3)) == 3


def test_legacy_token_files(tmp_path):
    toks = torch.arange(100)
    torch.save({"tokens": toks}, tmp_path / "t.pt")
    np.save(tmp_path / "t.npy", toks.numpy())
    toks.numpy().astype(np.uint16).tofile(tmp_path / "t.bin")
    for name in ("t.pt", "t.npy", "t.bin"):
        assert torch.equal(load_tokens_from_file(tmp_path / name), toks)
    assert len(TokenBlockDataset(toks, 9)) == 11


def test_bpe_tokenizer_roundtrip_and_pipeline(tmp_path):
    texts = [f"The quick brown fox number {i} jumps over the lazy dog near the river bank." for i in range(200)]
    tok = ByteLevelBPETokenizer.train_from_iterator(iter(texts), vocab_size=300)
    tok.save(tmp_path / "tok")
    again = load_tokenizer(tmp_path / "tok")
    assert again.fingerprint == tok.fingerprint and again.decode(again.encode(texts[3])) == texts[3]
    meta = json.loads((tmp_path / "tok" / "tokenizer_metadata.json").read_text())
    meta["fingerprint"] = "0" * 64
    (tmp_path / "tok" / "tokenizer_metadata.json").write_text(json.dumps(meta))
    with pytest.raises(ValueError):
        load_tokenizer(tmp_path / "tok")
    src = tmp_path / "docs.jsonl"
    src.write_text("\n".join(json.dumps({"id": f"d{i}", "text": t}) for i, t in enumerate(texts)))
    manifest = prepare_token_shards([src], output_dir=tmp_path / "out", tokenizer=tok, max_shard_tokens=1500, validation_fraction=0.1)
    _, m = load_manifest(manifest)
    assert m["cleaning_stats"]["accepted"] == 200 and m["splits"]["train"]["documents"] + m["splits"]["validation"]["documents"] == 200
    idx = np.fromfile(tmp_path / "out" / "train" / "documents.idx", dtype="<u8").reshape(-1, 2)
    assert int(idx[:, 1].sum()) == m["splits"]["train"]["tokens"] and int(idx[0, 0]) == 0


def test_shards_load_in_the_reference_loader(shards):
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "minitrain").is_dir():
        pytest.skip("reference package not installed")
    sys.path.insert(0, str(ref))
    try:
        from minitrain.data.dataloader import ShardedTokenBlockDataset as RefDataset
    finally:
        sys.path.remove(str(ref))
    theirs, ours = RefDataset(shards, split="train", seq_len=64), ShardedTokenBlockDataset(shards, split="train", seq_len=64)
    assert len(theirs) == len(ours) and theirs.sample_ranges == ours.sample_ranges
    for i in (0, 61, 100):
        assert torch.equal(theirs[i]["input_ids"], ours[i]["input_ids"])
