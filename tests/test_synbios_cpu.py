"""SynBioS layer end to end on CPU with the byte codec and a tiny MoE model."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
CLI = [sys.executable, str(ROOT / "scripts" / "synbios_moe.py")]


@pytest.fixture(scope="module")
def study(tmp_path_factory):
    """dataset (multi2+permute, 24 people) -> shards -> probe cache -> randomly initialised model.pt"""

    root = tmp_path_factory.mktemp("synbios")
    data = root / "data"
    run = lambda *a: subprocess.run([*CLI, *a], capture_output=True, text=True, timeout=600)   # noqa: E731
    out = run("prepare", "--output", str(data), "--variant", "multi2+permute", "--num-people", "24", "--codec", "bytes", "--quiet")
    assert out.returncode == 0, out.stderr[-2000:]
    out = run("cache-probes", "--data", str(data), "--output", str(root / "cache"), "--codec", "bytes")
    assert out.returncode == 0, out.stderr[-2000:]
    cfg = {"model": {"vocab_size": 257, "seq_len": 512, "n_layers": 2, "n_heads": 2, "hidden_size": 32, "intermediate_size": 32,
                     "ffn_type": "moe", "num_experts": 4, "experts_per_token": 2, "dropout": 0.0}}
    (root / "model.yaml").write_text(json.dumps(cfg))      # JSON is YAML
    from mini_train_sys_b200.models import MiniTransformer, ModelConfig, get_ops_backend

    torch.manual_seed(0)
    model = MiniTransformer(ModelConfig(**cfg["model"]), get_ops_backend("torch"), activation_dtype=torch.float32)
    torch.save(model.state_dict(), root / "model.pt")
    return {"root": root, "data": data, "cache": root / "cache", "model_config": root / "model.yaml", "checkpoint": root / "model.pt", "run": run}


def test_profiles_are_identical_across_variants_and_spans_are_exact(tmp_path):
    from experiments.synbios_moe.pretraining.dataset import ATTRIBUTES, VARIANTS, entries_per_person, write_dataset

    a = write_dataset(tmp_path / "a", num_people=30, variant="single", seed=7)
    b = write_dataset(tmp_path / "b", num_people=30, variant="multi5+permute", seed=7)
    assert (a / "profiles.jsonl").read_bytes() == (b / "profiles.jsonl").read_bytes()
    profiles = {json.loads(l)["person_id"]: json.loads(l) for l in (b / "profiles.jsonl").read_text().splitlines()}
    bios = [json.loads(l) for l in (b / "biographies.jsonl").read_text().splitlines()]
    assert len(bios) == 30 * 5 and entries_per_person("single+permute5") == 5 and len(VARIANTS) == 9
    orders = set()
    for bio in bios:
        for attribute in ATTRIBUTES:
            lo, hi = bio["attribute_spans"][attribute]
            assert bio["text"][lo:hi] == profiles[bio["person_id"]][attribute]
        orders.add(tuple(sorted(ATTRIBUTES, key=lambda x: bio["attribute_spans"][x][0])))
        assert bio["text"].count(profiles[bio["person_id"]]["full_name"]) == 1     # the name appears once, in the first sentence
    assert len(orders) > 5                                                            # sentences really are permuted
    assert {p["split"] for p in profiles.values()} == {"train", "validation"}
    # regenerating gives byte-identical files
    c = write_dataset(tmp_path / "c", num_people=30, variant="multi5+permute", seed=7)
    assert (b / "biographies.jsonl").read_bytes() == (c / "biographies.jsonl").read_bytes()


def test_prepare_writes_shards_and_manifest(study):
    manifest = json.loads((study["data"] / "token_shards" / "manifest.json").read_text())
    assert manifest["vocab_size"] == 257 and (study["data"] / "token_shards" / "train" / "shard_00000.bin").is_file()
    assert json.loads((study["data"] / "manifest.json").read_text())["num_biographies"] == 48


def test_probe_cache_layout_and_validation(study):
    from experiments.synbios_moe.probes.dataset import CachedProbeDataset, validate_probe_cache

    cache = study["cache"]
    verdict = validate_probe_cache(cache, study["data"])
    assert verdict["ok"], verdict
    assert np.load(cache / "profile_labels.npy").shape == (24, 11)
    assert np.load(cache / "p_positions.npy").shape == (48, 6)
    ds = CachedProbeDataset(cache, kind="p", attribute="university", target="whole", split="train")
    item = ds[0]
    assert item.positions.shape == (6,) and (np.diff(item.positions) > 0).all() and item.input_ids[0] == 256
    q = CachedProbeDataset(cache, kind="q", attribute="birth_date", target="first", split="validation")
    assert q[0].positions.tolist() == [q[0].input_ids.shape[0] - 1] and set(q.class_names) <= {
        "January", "February", "March", "April", "May", "June", "July", "August", "September", "October", "November", "December"}
    # the byte before every P position ends right before the value: decode and compare
    from experiments.synbios_moe.codec import ByteCodec
    bios = [json.loads(l) for l in (study["data"] / "biographies.jsonl").read_text().splitlines()]
    ids = np.memmap(cache / "p_tokens.bin", dtype="<i4", mode="r")
    off = np.load(cache / "p_offsets.npy"); pos = np.load(cache / "p_positions.npy")
    text0 = ByteCodec().decode(ids[off[0]:off[1]].tolist())
    assert text0 == bios[0]["text"]
    starts = sorted(v[0] for v in bios[0]["attribute_spans"].values())
    assert pos[0].tolist() == starts            # byte codec: position p (EOS at 0) is the token that ends at character p
    # tampering is detected
    (cache / "q_offsets.npy").write_bytes((cache / "q_offsets.npy").read_bytes()[:-8] + b"\0" * 8)
    assert not validate_probe_cache(cache)["ok"]


def test_recall_cloze_and_router_reports(study):
    run = study["run"]
    common = ["--data", str(study["data"]), "--model-config", str(study["model_config"]), "--checkpoint", str(study["checkpoint"]),
              "--codec", "bytes", "--device", "cpu", "--max-items", "6"]
    out = run("evaluate", *common, "--output", str(study["root"] / "recall.json"))
    assert out.returncode == 0, out.stderr[-2000:]
    recall = json.loads((study["root"] / "recall.json").read_text())
    assert recall["overall"]["values"] == 36 and 0.0 <= recall["overall"]["token_accuracy"] <= 1.0
    out = run("cloze-evaluate", *common, "--output", str(study["root"] / "cloze.json"), "--batch-size", "4")
    assert out.returncode == 0, out.stderr[-2000:]
    cloze = json.loads((study["root"] / "cloze.json").read_text())
    assert cloze["items"] == 36 and set(cloze["per_attribute"]) == {"birth_date", "birth_city", "university", "major", "company", "company_city"}
    out = run("cloze-evaluate", *common, "--output", str(study["root"] / "cloze_progressive.json"), "--batch-size", "3", "--protocol",
              "progressive", "--examples", "4", "--max-new-tokens", "6", "--sample-biographies", "2")
    assert out.returncode == 0, out.stderr[-2000:]
    prog = json.loads((study["root"] / "cloze_progressive.json").read_text())
    # --max-items (6, from the common arguments) takes precedence over --examples
    assert prog["protocol"] == "progressive_original_biography_cloze_greedy" and prog["biographies"] == 6 and prog["fields"] == 36
    assert len(prog["samples"]) == 2 and set(prog["samples"][0]["predicted"]) == set(prog["per_attribute"])
    assert sum(prog["biography_correct_field_count_histogram"].values()) == 6 and 0.0 <= prog["mean_character_similarity"] <= 1.0
    out = run("summarize-cloze", str(study["root"] / "cloze.json"), str(study["root"] / "cloze_progressive.json"), "--output",
              str(study["root"] / "cloze_table.csv"))
    assert out.returncode == 0, out.stderr[-2000:]          # both protocols feed the same table
    out = run("analyze", *common, "--output", str(study["root"] / "routes.json"))
    assert out.returncode == 0, out.stderr[-2000:]
    routes = json.loads((study["root"] / "routes.json").read_text())
    assert set(routes) == {"0", "1"} and 0.0 <= routes["0"]["nmi_attribute_expert"] <= 1.0
    assert abs(sum(routes["0"]["value_token_load"]) - 1.0) < 1e-6 and routes["0"]["jaccard_same_fact"] is not None


def test_cloze_of_a_memorising_model_is_exact():
    """A 'model' that already knows the text must score 100 %: checks prompt / answer alignment and the decode loop."""

    from experiments.synbios_moe.codec import ByteCodec
    from experiments.synbios_moe.pretraining.cloze import evaluate_cloze
    from experiments.synbios_moe.pretraining.dataset import generate_profiles, render_biography

    codec = ByteCodec()
    profiles = generate_profiles(3, 5)
    rows = []
    for p in profiles:
        bio = render_biography(p, variant="single", sample=0, seed=5)
        rows.append({"person_id": p.person_id, "text": bio.text, "attribute_spans": bio.attribute_spans})
    texts = [[codec.eos, *codec.encode(r["text"])] for r in rows]

    class Oracle(torch.nn.Module):
        class cfg:  # noqa: N801
            seq_len = 4096

        def hidden_states(self, ids):
            out = torch.zeros(ids.shape[0], ids.shape[1], 257)
            for b in range(ids.shape[0]):
                for t in range(ids.shape[1]):
                    prefix = ids[b, :t + 1].tolist()
                    for full in texts:
                        if full[:t + 1] == prefix and len(full) > t + 1:
                            out[b, t, full[t + 1]] = 1.0
                            break
            return out

        def lm_head(self, h):
            return h

        def forward(self, ids):
            return self.hidden_states(ids)

    report = evaluate_cloze(Oracle(), codec, rows, batch_size=5)
    assert report["overall_exact_match"] == 1.0 and report["items"] == 18
    from experiments.synbios_moe.pretraining.attribute_recall import evaluate_attribute_recall

    recall = evaluate_attribute_recall(Oracle(), codec, rows)
    assert recall["overall"]["token_accuracy"] == 1.0 and recall["company"]["whole_value_accuracy"] == 1.0


def test_probe_training_resumes_with_identical_result(study, tmp_path):
    from experiments.synbios_moe.probes.model import train_probe
    from scripts.synbios_moe import load_backbone

    def backbone():
        return load_backbone(str(study["model_config"]), str(study["checkpoint"]), "cpu")

    kw = dict(kind="q", attribute="company_city", target="whole", steps=6, batch_size=4, seed=3, max_eval_items=8)
    full = train_probe(backbone(), study["cache"], **kw)
    rec = tmp_path / "rec.pt"

    class Stop(Exception):
        pass

    def interrupt(event):
        if event["event"] == "probe_train" and event["step"] == 6:
            raise AssertionError("should not get here in the interrupted run")

    # run 3 steps (checkpoint every 3), then "crash": emulate by asking for steps=6 but stopping via a short first run
    first = train_probe(backbone(), study["cache"], **{**kw}, recovery_checkpoint=rec, checkpoint_interval_steps=3,
                        on_event=lambda e: (_ for _ in ()).throw(Stop()) if e["event"] == "probe_train" and e.get("step") == 10 else None)
    assert rec.is_file()                                 # written at step 3
    resumed = train_probe(backbone(), study["cache"], **kw, recovery_checkpoint=rec, checkpoint_interval_steps=3)
    # the recovery file holds step 3: the resumed run replays steps 4..6 with the same batches and lr
    for k, v in full["probe_state"].items():
        assert torch.allclose(v.float(), resumed["probe_state"][k].float(), atol=1e-6), k
    assert first["final_loss"] == pytest.approx(full["final_loss"])
    with pytest.raises(ValueError):
        train_probe(backbone(), study["cache"], **{**kw, "seed": 4}, recovery_checkpoint=rec)      # another job's checkpoint


def test_probe_pipeline_schedules_validates_and_skips_fresh_jobs(study, tmp_path):
    run = study["run"]
    args = ["probe-pipeline", "--data", str(study["data"]), "--probe-cache", str(study["cache"]), "--model-config", str(study["model_config"]),
            "--checkpoint", str(study["checkpoint"]), "--codec", "bytes", "--device", "cpu", "--devices", "cpu,cpu", "--stage", "smoke",
            "--steps", "3", "--attributes", "major", "--output", str(tmp_path / "pipe"), "--heartbeat-seconds", "1", "--max-eval-items", "8",
            "--quiet"]
    out = run(*args)
    assert out.returncode == 0, (out.stdout[-1500:], out.stderr[-1500:])
    summary = json.loads(out.stdout.strip().splitlines()[-1])
    assert summary["ok"] and set(summary["training"]) == {"p-major-first", "p-major-whole", "q-major-first", "q-major-whole"}
    state = json.loads((tmp_path / "pipe" / "pipeline.json").read_text())
    assert all(j["status"] == "done" for j in state["jobs"].values()) and len(state["jobs"]) == 8
    trained = json.loads((tmp_path / "pipe" / "training" / "q-major-first.json").read_text())
    # 2 layers x 4 experts x (2 * 32 * 32 + 32 * 32) expert weights, two of four active per token
    assert trained["model_parameters"]["total"] - trained["model_parameters"]["active_estimate"] == 2 * 4 * 3 * 32 * 32 // 2
    assert trained["checkpoint_bytes"] > 0 and trained["checkpoint"].endswith("model.pt")
    assert (tmp_path / "pipe" / "training" / "p-major-whole.pt").is_file() and (tmp_path / "pipe" / "validation" / "q-major-first.json").is_file()
    again = json.loads(run(*args).stdout.strip().splitlines()[-1])
    assert set(again["training"].values()) == {"skipped"} and set(again["validation"].values()) == {"skipped"}
    out = run("summarize-probes", str(tmp_path / "pipe"), "--output", str(tmp_path / "table.csv"))
    assert out.returncode == 0 and json.loads(out.stdout.strip().splitlines()[-1])["jobs"] == 4
    audit = run("audit-synbios-repository", "--data", str(study["data"]), "--pipeline", str(tmp_path / "pipe"))
    assert audit.returncode == 0, audit.stdout


def test_nmi_extremes():
    from experiments.synbios_moe.mechanisms.routing import normalized_mutual_information

    labels = torch.tensor([0, 0, 1, 1, 2, 2, -1])
    assert normalized_mutual_information(labels, torch.tensor([0, 0, 1, 1, 2, 2, 3]), 4) == pytest.approx(1.0)
    assert normalized_mutual_information(torch.tensor([0, 1, 0, 1]), torch.tensor([0, 0, 1, 1]), 2) == pytest.approx(0.0, abs=1e-9)


class _ToyBpe:
    """Greedy longest-match tokens over UTF-8 bytes: multi-byte tokens, some with a leading space, like a byte-level BPE."""

    name = "toy"

    def __init__(self) -> None:
        pieces = [" was born", " born", " in", " the", " uni", "vers", "ity", "An", "na", " Zür", "ich", "é", " ", "on ", "19", "90"]
        self.table = [p.encode("utf-8") for p in pieces]
        self.eos = 256 + len(self.table)
        self.vocab_size = self.eos + 1

    def encode(self, text: str) -> list[int]:
        data, out, i = text.encode("utf-8"), [], 0
        while i < len(data):
            best = max((k for k, piece in enumerate(self.table) if data.startswith(piece, i)), key=lambda k: len(self.table[k]), default=None)
            if best is None:
                out.append(data[i]); i += 1
            else:
                out.append(256 + best); i += len(self.table[best])
        return out

    def token_num_bytes(self, token: int) -> int:
        return 0 if token == self.eos else (1 if token < 256 else len(self.table[token - 256]))

    def decode(self, tokens) -> str:
        return b"".join(bytes([t]) if t < 256 else self.table[t - 256] for t in tokens if t != self.eos).decode("utf-8", errors="replace")


def test_character_spans_map_to_token_positions_with_multi_byte_tokens():
    """The span arithmetic behind every probe position: character offsets (code points) against token boundaries (bytes)."""

    from experiments.synbios_moe.codec import positions_before_chars, token_span_of_chars

    codec = _ToyBpe()
    text = "Anna Rée was born in Zürich on 1990."
    ids = codec.encode(text)
    assert codec.decode(ids) == text and any(codec.token_num_bytes(t) > 2 for t in ids)
    starts = [text.index("Zürich"), text.index("1990"), 0]
    tokens, positions = positions_before_chars(codec, text, starts)
    assert tokens[0] == codec.eos and tokens[1:] == ids
    for start, pos in zip(starts, positions):
        # the tokens up to and including position `pos` spell exactly the text before the value (position 0 is the EOS)
        prefix = codec.decode(tokens[1:pos + 1])
        assert text.startswith(prefix) and len(prefix) <= start
        # ... and the next token already reaches into the value: the read-out sits right before it
        longer = codec.decode(tokens[1:pos + 2])
        assert len(longer) > start or pos + 1 == len(tokens)
    # " Zür" carries the leading space: the value's first token starts before the value's first character
    z = text.index("Zürich")
    toks, lo, hi = token_span_of_chars(codec, text, z, z + len("Zürich"))
    assert "Zürich" in codec.decode(toks[lo:hi]) and codec.decode(toks[lo:hi]).strip() == "Zürich"
    toks, lo, hi = token_span_of_chars(codec, text, text.index("é"), text.index("é") + 1)
    assert codec.decode(toks[lo:hi]) == "é"                      # a two-byte character that is one token


def test_gpt2_alignment_when_the_vocabulary_is_available():
    from experiments.synbios_moe.codec import get_codec, positions_before_chars

    try:
        codec = get_codec("gpt2")
    except Exception as exc:       # no network / no cached BPE tables on this machine
        pytest.skip(f"GPT-2 tables unavailable: {type(exc).__name__}")
    text = "Anya Briar Forger was born on October 2, 1996. She spent her early years in Princeton, NJ."
    start = text.index("Princeton")
    tokens, (pos,) = positions_before_chars(codec, text, [start])
    assert codec.decode(tokens[1:pos + 1]) == text[:start].rstrip(" ") or codec.decode(tokens[1:pos + 1]) == text[:start]
    assert codec.decode(tokens[pos + 1:pos + 2]).strip().startswith("Pr")


def test_trained_bpe_codec_aligns_every_attribute_span_and_drives_the_study(tmp_path):
    """``--codec bpe:<dir>``: a byte-level BPE trained on the biographies themselves.  Real merges, tokens with leading
    spaces, values of several tokens: the alignment contract is checked on every attribute of every biography, and the
    commands that consume a codec run with it."""

    pytest.importorskip("tokenizers")
    from experiments.synbios_moe.artifact_io import read_json, read_jsonl
    from experiments.synbios_moe.codec import byte_level_alphabet, get_codec, positions_before_chars, token_span_of_chars
    from experiments.synbios_moe.pretraining.dataset import ATTRIBUTES

    alphabet = byte_level_alphabet()
    assert len(alphabet) == 256 and sorted(alphabet.values()) == list(range(256)) and alphabet["A"] == 65 and alphabet["\u0120"] == 32

    data, tok = tmp_path / "data", tmp_path / "tok"
    run = lambda *a: subprocess.run([*CLI, *a], capture_output=True, text=True, timeout=600)   # noqa: E731
    out = run("prepare", "--output", str(data), "--variant", "multi2+permute", "--num-people", "60", "--codec", f"bpe:{tok}",
              "--bpe-vocab-size", "700", "--quiet")
    assert out.returncode == 0, out.stderr[-2000:]
    codec = get_codec(f"bpe:{tok}")
    assert codec.vocab_size == 700 and codec.token_num_bytes(codec.eos) == 0
    shard_manifest = read_json(data / "token_shards" / "manifest.json")
    assert shard_manifest["tokenizer_fingerprint"] == codec.fingerprint and shard_manifest["vocab_size"] == 700
    multi_token_values = 0
    for bio in read_jsonl(data / "biographies.jsonl"):
        text = bio["text"]
        ids = codec.encode(text)
        assert sum(codec.token_num_bytes(t) for t in ids) == len(text.encode("utf-8")) and codec.decode(ids) == text
        assert len(ids) < 0.6 * len(text)                                  # merges happened: this is not the byte codec
        for attribute in ATTRIBUTES:
            lo_c, hi_c = bio["attribute_spans"][attribute]
            value = text[lo_c:hi_c]
            tokens, lo, hi = token_span_of_chars(codec, text, lo_c, hi_c)
            covered = codec.decode(tokens[lo:hi])
            assert value in covered and codec.decode(tokens[1:lo]) + covered + codec.decode(tokens[hi:]) == text
            # minimal cover: dropping the first or the last token of the range loses part of the value
            assert value not in codec.decode(tokens[lo + 1:hi]) and value not in codec.decode(tokens[lo:hi - 1])
            multi_token_values += hi - lo > 1
            _, (pos,) = positions_before_chars(codec, text, [lo_c])
            before = codec.decode(tokens[1:pos + 1])
            assert text.startswith(before) and len(before) <= lo_c          # the read-out has seen nothing of the value
            assert len(codec.decode(tokens[1:pos + 2])) > lo_c              # ... and the very next token reaches into it
            assert pos + 1 == lo or covered.startswith(" ")                 # the value's first token may carry the space before it
    assert multi_token_values > 100
    # a second prepare with the same directory reuses the tokenizer instead of training another
    before = (tok / "tokenizer.json").read_bytes()
    assert run("prepare", "--output", str(tmp_path / "again"), "--variant", "single", "--num-people", "10", "--codec", f"bpe:{tok}",
               "--quiet").returncode == 0 and (tok / "tokenizer.json").read_bytes() == before
    out = run("cache-probes", "--data", str(data), "--output", str(tmp_path / "cache"), "--codec", f"bpe:{tok}")
    assert out.returncode == 0, out.stderr[-2000:]
    check = run("validate-probe-cache", "--probe-cache", str(tmp_path / "cache"), "--data", str(data))
    assert check.returncode == 0 and json.loads(check.stdout)["ok"], check.stdout + check.stderr[-1000:]
    manifest = read_json(tmp_path / "cache" / "manifest.json")
    assert manifest["codec"] == f"bpe:{tok}" and manifest["vocab_size"] == 700
    stats = run("token-statistics", "--data", str(data), "--output", str(tmp_path / "stats.json"), "--codec", f"bpe:{tok}")
    assert stats.returncode == 0, stats.stderr[-2000:]
    assert run("token-statistics", "--data", str(data), "--output", str(tmp_path / "x.json"), "--codec", "wordpiece").returncode != 0


def test_character_similarity_and_progressive_cloze_with_an_oracle_model(tmp_path):
    """A stand-in model that always continues with the source text reproduces every field: the progressive protocol must then
    score 6 / 6 per biography, terminate every field at the source's full stop and rebuild the original text."""

    import torch

    from experiments.synbios_moe.codec import get_codec
    from experiments.synbios_moe.pretraining.cloze import biography_fields, character_similarity, evaluate_progressive_cloze
    from dataclasses import asdict

    from experiments.synbios_moe.pretraining.dataset import ATTRIBUTES, generate_profiles, iter_biographies

    assert character_similarity("MIT", "mit") == 1.0 and character_similarity("", "") == 1.0
    assert character_similarity("abcd", "abcf") == pytest.approx(0.75) and character_similarity("x", "") == 0.0
    assert character_similarity("New   York", "new york") == 1.0

    codec = get_codec("bytes")
    profiles = generate_profiles(4, seed=5)
    rows = [asdict(b) for b in iter_biographies(profiles, "single", 5)]
    book = {}
    for row in rows:
        ids, fields = biography_fields(codec, row)
        assert sorted(f["attribute"] for f in fields) == sorted(ATTRIBUTES) and [f["lo"] for f in fields] == sorted(f["lo"] for f in fields)
        book[row["person_id"]] = ids

    class Oracle(torch.nn.Module):
        """hidden state = one-hot of the token that follows the prefix in the source biography; lm_head is the identity."""

        class cfg:  # noqa: N801
            seq_len = 4096

        def __init__(self, wrong_for=None):
            super().__init__()
            self.wrong_for = wrong_for

        def hidden_states(self, batch):
            out = torch.zeros(*batch.shape, 257)
            for r in range(batch.shape[0]):
                seq = batch[r].tolist()

                def shared(ids):
                    n = 0
                    while n < min(len(ids), len(seq)) and ids[n] == seq[n]:
                        n += 1
                    return n

                source = max(book.values(), key=shared)           # the biography this row is a prefix of
                for t in range(batch.shape[1]):
                    nxt = source[t + 1] if t + 1 < len(source) else codec.eos
                    out[r, t, nxt] = 1.0
            return out

        def lm_head(self, h):
            return h

    report = evaluate_progressive_cloze(Oracle(), codec, rows, max_biographies=3, start_index=1, batch_size=2, max_new_tokens=64)
    assert report["protocol"] == "progressive_original_biography_cloze_greedy" and report["biographies"] == 3 and report["fields"] == 18
    assert report["micro_field_accuracy"] == 1.0 and report["biography_all_fields_accuracy"] == 1.0 and report["unterminated_fields"] == 0
    assert report["biography_correct_field_count_histogram"]["6"] == 3 and report["overall_exact_match"] == 1.0
    assert set(report["per_attribute"]) == set(ATTRIBUTES)
    for sample in report["samples"]:
        assert sample["filled_text"] == sample["original_text"] and sample["exact_fields"] == 6
    # too few new tokens: (almost) nothing reaches its full stop, predictions are truncated, similarity stays between 0 and 1
    short = evaluate_progressive_cloze(Oracle(), codec, rows, max_biographies=2, batch_size=2, max_new_tokens=2)
    assert short["unterminated_fields"] >= 10 and short["micro_field_accuracy"] < 0.5 and 0.0 < short["mean_character_similarity"] < 1.0
    with pytest.raises(ValueError):
        evaluate_progressive_cloze(Oracle(), codec, rows, max_biographies=0)


def test_attribute_token_distribution_tables(tmp_path):
    from experiments.synbios_moe.codec import get_codec
    from experiments.synbios_moe.pretraining.dataset import ATTRIBUTES
    from experiments.synbios_moe.pretraining.token_statistics import attribute_token_distribution, entropy_bits, percentile

    from collections import Counter

    assert entropy_bits(Counter({1: 2, 2: 2})) == pytest.approx(1.0) and entropy_bits(Counter()) == 0.0
    assert percentile([1, 2, 3, 4, 5], 50) == 3 and percentile([1, 2], 95) == pytest.approx(1.95)
    base = {a: "x" for a in ATTRIBUTES}
    people = [{**base, "university": "MIT"}, {**base, "university": "MIT"}, {**base, "university": "Ohio"}, {**base, "university": "M"}]
    report = attribute_token_distribution(get_codec("bytes"), people, tmp_path / "dist")
    uni = report["attributes"]["university"]
    # byte codec: " MIT" is 4 tokens, " Ohio" 5, " M" 2; every value starts with the space, so one first-token class holds all three
    assert uni["unique_values"] == 3 and uni["token_length"]["minimum"] == 2 and uni["token_length"]["maximum"] == 5
    assert uni["token_length"]["mean_profile_weighted"] == pytest.approx((4 + 4 + 5 + 2) / 4)
    assert uni["first_token"]["unique_tokens_unique_values"] == 1 and uni["first_token"]["whole_classes_per_first_token"]["maximum"] == 3
    assert uni["first_token"]["entropy_bits_profile_weighted"] == 0.0
    assert uni["position_unique_token_counts"]["2"] == 2           # 'M' or 'O' at the second position
    assert uni["position_entropy_bits_profile_weighted"]["2"] == pytest.approx(entropy_bits(Counter({77: 3, 79: 1})))
    assert uni["leading_space_comparison"]["changed_fraction"] == 1.0 and uni["leading_space_comparison"]["bare_first_token_classes"] == 2
    assert report["protocol"] == "synbios_attribute_leading_space_token_distribution_v1"
    rows = (tmp_path / "dist" / "position_token_distribution.csv").read_text().splitlines()
    assert rows[0].startswith("attribute,token_position,token_id,token_text") and any(",2,77,M,3,0.75,0.75,2" in r for r in rows)
    lengths = (tmp_path / "dist" / "length_distribution.csv").read_text().splitlines()
    assert "university,profile_weighted,4,2,0.5" in lengths and "university,unique_values,4,1,0.3333333333333333" in lengths
    assert len((tmp_path / "dist" / "attribute_summary.csv").read_text().splitlines()) == 1 + len(ATTRIBUTES)


def test_token_statistics_command_writes_both_reports(study):
    out = study["run"]("token-statistics", "--data", str(study["data"]), "--codec", "bytes", "--output", str(study["root"] / "tokens.json"),
                       "--distribution-dir", str(study["root"] / "token_distribution"))
    assert out.returncode == 0, out.stderr[-2000:]
    stats = json.loads((study["root"] / "tokens.json").read_text())
    assert stats["biographies"] == 48 and set(stats["attributes"]) == {"birth_date", "birth_city", "university", "major", "company", "company_city"}
    dist = json.loads((study["root"] / "token_distribution" / "summary.json").read_text())
    assert dist["num_people"] == 24 and dist["attributes"]["major"]["profile_count"] == 24
    for name in dist["artifacts"].values():
        assert (study["root"] / "token_distribution" / name).is_file()


def test_phase_duration_estimates_scale_steps_and_devices(tmp_path):
    from experiments.synbios_moe.probes.pipeline import estimate_phase_durations
    from experiments.synbios_moe.probes.spec import JobSpec

    def job(name, phase):
        return JobSpec(name, ("x",), tmp_path / f"{name}.json", tmp_path / f"{name}.log", phase=phase)

    jobs = [job("p-a", "training"), job("q-a", "training"), job("p-a.val", "validation"), job("q-a.val", "validation")]
    previous = {"settings": {"steps": 100}, "jobs": {"p-a": {"phase": "training", "status": "done", "seconds": 10.0},
                                                      "q-a": {"phase": "training", "status": "skipped", "seconds": 30.0},
                                                      "p-a.val": {"phase": "validation", "status": "done", "seconds": 4.0},
                                                      "q-a.val": {"phase": "validation", "status": "done", "seconds": 6.0}}}
    est = estimate_phase_durations(previous, jobs, steps=1000, device_count=2)
    assert est == {"training": pytest.approx((10.0 + 30.0) * 10 / 2), "validation": pytest.approx(5.0)}
    # a different job set, an unfinished job or a missing step count: that phase is not estimated
    assert "training" not in estimate_phase_durations(previous, jobs[1:], steps=1000, device_count=2)
    broken = json.loads(json.dumps(previous)); broken["jobs"]["p-a"]["status"] = "failed"
    assert estimate_phase_durations(broken, jobs, steps=1000, device_count=2) == {"validation": pytest.approx(5.0)}
    nosteps = json.loads(json.dumps(previous)); del nosteps["settings"]
    assert estimate_phase_durations(nosteps, jobs, steps=1000, device_count=2) == {"validation": pytest.approx(5.0)}
    assert estimate_phase_durations(None, jobs, steps=10, device_count=1) == {} and estimate_phase_durations(previous, jobs, steps=10, device_count=0) == {}
    assert estimate_phase_durations(previous, jobs, steps=0, device_count=2) == {"validation": pytest.approx(5.0)}     # a per-task step table


def test_probe_pipeline_cloze_gate_runs_once_and_can_refuse(study, tmp_path):
    """The gate is the progressive cloze; its verdict is cached by checkpoint, data and settings, and a threshold the model
    does not reach stops the stage before any probe job starts."""

    run = study["run"]
    cfg = tmp_path / "pipeline.yaml"
    base = {"stages": {"smoke": {"requires": None, "steps": 2, "tasks": [{"attribute": "major", "kind": "q", "target": "first"}]}}}
    cfg.write_text(json.dumps({**base, "gate": {"batch_size": 4, "examples": 5, "max_new_tokens": 4, "sample_biographies": 2, "threshold": 0.0}}))
    args = ["probe-pipeline", "--data", str(study["data"]), "--probe-cache", str(study["cache"]), "--model-config", str(study["model_config"]),
            "--checkpoint", str(study["checkpoint"]), "--codec", "bytes", "--device", "cpu", "--devices", "cpu", "--stage", "smoke",
            "--config", str(cfg), "--output", str(tmp_path / "pipe"), "--heartbeat-seconds", "1", "--max-eval-items", "4", "--quiet"]
    out = run(*args)
    assert out.returncode == 0, (out.stdout[-1500:], out.stderr[-1500:])
    gate = json.loads((tmp_path / "pipe" / "gate.json").read_text())
    assert gate["protocol"] == "progressive_original_biography_cloze_greedy" and gate["biographies"] == 5 and gate["items"] == 30
    assert gate["passed"] and gate["reused"] is False and len(gate["samples"]) == 2
    out = run(*args)
    assert out.returncode == 0 and json.loads((tmp_path / "pipe" / "gate.json").read_text())["reused"] is True
    cfg.write_text(json.dumps({**base, "gate": {"batch_size": 4, "examples": 5, "max_new_tokens": 4, "threshold": 0.99}}))
    out = run(*[a if a != str(tmp_path / "pipe") else str(tmp_path / "pipe2") for a in args])
    assert out.returncode == 3 and "cloze gate failed" in out.stdout and not (tmp_path / "pipe2" / "pipeline.json").exists()


def test_option_names_of_the_reference_cli_do_what_they_say(study, tmp_path):
    """The reference's spellings: --examples, --probe-checkpoint, --run, --num-gpus-free overrides, --attribute (repeatable),
    --log-interval / --tensorboard; each through the command that accepts it."""

    run = study["run"]
    common = ["--data", str(study["data"]), "--model-config", str(study["model_config"]), "--checkpoint", str(study["checkpoint"]), "--codec", "bytes",
              "--device", "cpu"]
    out = run("evaluate", *common, "--output", str(tmp_path / "recall.json"), "--examples", "6", "--log-interval", "5", "--no-tensorboard")
    assert out.returncode == 0, out.stderr[-2000:]
    assert json.loads((tmp_path / "recall.json").read_text())["overall"]["values"] == 36                 # six biographies x six attributes
    probe_json = tmp_path / "probe" / "q-major-first.json"
    out = run("probe", *common, "--probe-cache", str(study["cache"]), "--attribute", "major", "--target", "first", "--kind", "q", "--steps", "4",
              "--batch-size", "8", "--output", str(probe_json), "--max-eval-items", "8", "--log-dir", str(tmp_path / "events"), "--log-interval", "2",
              "--tensorboard")
    assert out.returncode == 0, out.stderr[-2000:]
    shown = [json.loads(line) for line in out.stdout.splitlines() if line.startswith("{") and '"probe_train"' in line]
    logged = [json.loads(line) for line in (tmp_path / "events" / "events.jsonl").read_text().splitlines() if '"probe_train"' in line]
    assert len(logged) >= len(shown) and all(e["step"] % 2 == 0 or e["step"] == e.get("steps_total") for e in shown)
    assert any(p.name.startswith("events.out.tfevents") for p in (tmp_path / "events").iterdir())
    # the reference's name of the saved head, its batch size option, and the guard against another backbone
    verdict = tmp_path / "verdict.json"
    out = run("validate-probe", *common, "--probe-cache", str(study["cache"]), "--probe-checkpoint", str(probe_json.with_suffix(".pt")), "--batch-size", "4",
              "--output", str(verdict), "--max-eval-items", "8", "--quiet")
    assert out.returncode == 0 and "validation" in json.loads(verdict.read_text()), out.stderr[-2000:]
    other = tmp_path / "other_model.pt"
    state = torch.load(study["checkpoint"], weights_only=False)
    torch.save({k: (v + 1 if v.is_floating_point() else v) for k, v in state.items()}, other)
    mismatch = [a if a != str(study["checkpoint"]) else str(other) for a in common]
    out = run("validate-probe", *mismatch, "--probe-cache", str(study["cache"]), "--probe-checkpoint", str(probe_json.with_suffix(".pt")),
              "--output", str(tmp_path / "v2.json"), "--max-eval-items", "8", "--quiet")
    assert out.returncode == 3 and "another backbone" in out.stdout
    out = run("validate-probe", *mismatch, "--probe-cache", str(study["cache"]), "--probe-checkpoint", str(probe_json.with_suffix(".pt")),
              "--output", str(tmp_path / "v2.json"), "--max-eval-items", "8", "--quiet", "--allow-checkpoint-mismatch")
    assert out.returncode == 0
    # NAME=DIRECTORY runs
    stage = tmp_path / "stage"
    (stage / "training").mkdir(parents=True)
    (stage / "training" / "q-major-first.json").write_text(probe_json.read_text())
    out = run("summarize-probes", "--run", f"mine={stage}", "--run", f"again={stage / 'validation'}", "--output", str(tmp_path / "runs.csv"))
    assert out.returncode == 0 and json.loads(out.stdout)["runs"] == ["mine", "again"], out.stdout + out.stderr[-1000:]
    table = (tmp_path / "runs.csv").read_text().splitlines()
    assert "run" in table[0].split(",") and len(table) == 3
    assert run("summarize-probes", "--run", "broken").returncode == 2
