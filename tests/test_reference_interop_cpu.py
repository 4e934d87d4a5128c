"""Interoperability with the unmodified reference package (installed under ``baseline/_ref``; skipped where it is not):
the same weights give the same numbers, the same seeds the same batches, the same schedule the same learning rates."""

import contextlib
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "baseline" / "_ref"
pytestmark = pytest.mark.skipif(not (REF / "minitrain").is_dir(), reason="reference package not installed")


@contextlib.contextmanager
def reference_on_path():
    sys.path.insert(0, str(REF))
    try:
        yield
    finally:
        sys.path.remove(str(REF))


MODEL_SHAPES = {
    "dense": dict(vocab_size=211, seq_len=24, n_layers=2, n_heads=4, hidden_size=64, intermediate_size=96, ffn_type="dense", dropout=0.0),
    "moe": dict(vocab_size=211, seq_len=24, n_layers=2, n_heads=4, hidden_size=64, intermediate_size=48, ffn_type="moe", num_experts=4,
                experts_per_token=2, dropout=0.0, tie_word_embeddings=True),
}


@pytest.mark.parametrize("kind", sorted(MODEL_SHAPES))
def test_same_weights_give_the_same_loss_gradients_and_metrics(kind):
    from mini_train_sys_b200.models import MiniTransformer, ModelConfig, get_ops_backend

    with reference_on_path():
        from minitrain.model.config import ModelConfig as RefConfig
        from minitrain.model.ops import get_ops_backend as ref_backend
        from minitrain.model.transformer import MiniTransformer as RefTransformer

        torch.manual_seed(3)
        theirs = RefTransformer(RefConfig(**MODEL_SHAPES[kind]), ref_backend("torch"))
    ours = MiniTransformer(ModelConfig(**MODEL_SHAPES[kind]), get_ops_backend("torch"))
    state = theirs.state_dict()
    assert list(state) == list(ours.state_dict())                     # same names in the same order: checkpoints are exchangeable
    ours.load_state_dict(state)
    tokens = torch.randint(0, 211, (3, 25), generator=torch.Generator().manual_seed(4))
    ids, targets = tokens[:, :-1], tokens[:, 1:]
    for fused in (False, True):
        for model in (theirs, ours):
            model.zero_grad(set_to_none=True)
        loss_t, _ = theirs(ids, targets=targets, use_fused_loss=fused)
        loss_o, _ = ours(ids, targets=targets, use_fused_loss=fused)
        assert float(loss_o.detach()) == pytest.approx(float(loss_t.detach()), abs=1e-6)
        loss_t.backward()
        loss_o.backward()
        for (name, pt), (_, po) in zip(theirs.named_parameters(), ours.named_parameters()):
            assert torch.allclose(po.grad, pt.grad, atol=2e-6, rtol=1e-5), (fused, name)
    shared = set(theirs.last_training_metrics) & set(ours.last_training_metrics)
    assert {"loss/lm_cross_entropy", "loss/total"} <= shared
    for key in shared:
        assert torch.allclose(ours.last_training_metrics[key].float(), theirs.last_training_metrics[key].float(), atol=1e-5), key
    assert set(theirs.last_training_metrics) <= set(ours.last_training_metrics)        # every reference metric is published here too
    _, logits_t = theirs(ids)
    _, logits_o = ours(ids)
    assert torch.allclose(logits_o, logits_t, atol=1e-5)


def test_same_seed_gives_the_same_batches(tmp_path):
    from mini_train_sys_b200.data.dataloader import (RandomizedDocumentBlockDataset, RandomizedDocumentSampler, ShardAwareBlockSampler,
                                                     ShardedTokenBlockDataset)
    from mini_train_sys_b200.data.preprocess import write_random_token_shards

    shards = write_random_token_shards(tmp_path / "data", vocab_size=300, num_tokens=12_000, seed=1, document_tokens=211,
                                       max_shard_tokens=2_500).parent
    with reference_on_path():
        from minitrain.data import dataloader as ref

    for world in (1, 3):
        for rank in range(world):
            for epoch in (0, 2):
                mine = ShardAwareBlockSampler(ShardedTokenBlockDataset(shards, split="train", seq_len=32), shuffle=True, seed=9, rank=rank,
                                              world_size=world, shuffle_window=13)
                theirs = ref.ShardAwareBlockSampler(ref.ShardedTokenBlockDataset(shards, split="train", seq_len=32), shuffle=True, seed=9,
                                                    rank=rank, world_size=world, shuffle_window=13)
                mine.set_epoch(epoch)
                theirs.set_epoch(epoch)
                assert list(mine) == list(theirs)
                docs_mine = RandomizedDocumentSampler(RandomizedDocumentBlockDataset(shards, split="train", seq_len=32), shuffle=True, seed=9,
                                                      rank=rank, world_size=world)
                ref_ds = ref.RandomizedDocumentBlockDataset(shards, split="train", seq_len=32)
                docs_theirs = ref.RandomizedDocumentSampler(ref_ds, shuffle=True, seed=9, rank=rank, world_size=world)
                docs_mine.set_epoch(epoch)
                docs_theirs.set_epoch(epoch)
                a, b = list(docs_mine), list(docs_theirs)
                assert [s.segments for s in a] == [tuple(map(tuple, s.segments)) for s in b]
                first = docs_mine.dataset[a[0]]
                assert torch.equal(first["input_ids"], ref_ds[b[0]]["input_ids"])


def test_same_schedule_gives_the_same_learning_rates():
    from mini_train_sys_b200.runtime.config import LRSchedulerConfig
    from mini_train_sys_b200.train.lr_scheduler import LearningRateScheduler

    with reference_on_path():
        from minitrain.runtime.config import LRSchedulerConfig as RefSchedule
        from minitrain.train.lr_scheduler import LearningRateScheduler as RefScheduler

    for options in (dict(schedule="cosine", warmup_steps=7, min_lr_ratio=0.1), dict(schedule="constant", warmup_steps=3),
                    dict(schedule="cosine", warmup_steps=0, decay_steps=20, min_lr_ratio=0.0)):
        rates = []
        for scheduler_type, config_type in ((LearningRateScheduler, LRSchedulerConfig), (RefScheduler, RefSchedule)):
            optimizer = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=2e-3)
            scheduler = scheduler_type(optimizer, config_type(**options), total_steps=40)
            seen = []
            for step in range(45):
                scheduler.step(step)
                seen.append(optimizer.param_groups[0]["lr"])
            rates.append(seen)
        assert rates[0] == pytest.approx(rates[1], rel=1e-12), options


@pytest.mark.parametrize("writer", ["reference", "this repository"])
def test_checkpoints_are_exchangeable_in_both_directions(tmp_path, writer):
    """A checkpoint directory written by one package (weights, AdamW moments, counters) resumes in the other and the next
    optimizer step gives the same loss: same layout (DCP payload, ``runtime.pt``, RNG side car, ``COMMITTED``), same keys."""

    from mini_train_sys_b200.models import MiniTransformer, ModelConfig, get_ops_backend
    from mini_train_sys_b200.train import checkpoint as ours_ckpt
    from mini_train_sys_b200.train.optim import build_optimizer

    with reference_on_path():
        from minitrain.model.config import ModelConfig as RefConfig
        from minitrain.model.ops import get_ops_backend as ref_backend
        from minitrain.model.transformer import MiniTransformer as RefTransformer
        from minitrain.train import checkpoint as ref_ckpt
        from minitrain.train.optim import build_optimizer as ref_build_optimizer

    shape = MODEL_SHAPES["moe"]
    tokens = torch.randint(0, 211, (4, 4, 25), generator=torch.Generator().manual_seed(8))

    def make(side):
        torch.manual_seed(5)
        if side == "reference":
            model = RefTransformer(RefConfig(**shape), ref_backend("torch"))
            return model, ref_build_optimizer(model, lr=1e-2, weight_decay=0.1)
        model = MiniTransformer(ModelConfig(**shape), get_ops_backend("torch"))
        return model, build_optimizer(model, lr=1e-2, weight_decay=0.1)

    def step(model, optimizer, batch):
        optimizer.zero_grad(set_to_none=True)
        loss, _ = model(batch[:, :-1], targets=batch[:, 1:])
        loss.backward()
        optimizer.step()
        return float(loss.detach())

    reader = "this repository" if writer == "reference" else "reference"
    module = {"reference": ref_ckpt, "this repository": ours_ckpt}
    source_model, source_opt = make(writer)
    for i in range(2):
        step(source_model, source_opt, tokens[i])
    path = tmp_path / "run" / "epoch_000001_step_000000002"
    module[writer].save_checkpoint(path, source_model, source_opt, 2, epoch=1, tokens_seen=192, export_model=True)
    assert {p.name for p in path.iterdir()} >= {"distributed", "runtime.pt", "COMMITTED", "model.pt", "rng_rank_00000.pt"}

    target_model, target_opt = make(reader)
    with torch.no_grad():
        for p in target_model.parameters():
            p.add_(1.0)                                   # make sure the restore is what equalises them
    got = module[reader].restore_training_checkpoint(path, target_model, target_opt)
    assert got["step"] == 2 and got["epoch"] == 1 and got["tokens_seen"] == 192
    for (name, a), (_, b) in zip(source_model.named_parameters(), target_model.named_parameters()):
        assert torch.equal(a, b), name
    assert step(target_model, target_opt, tokens[2]) == pytest.approx(step(source_model, source_opt, tokens[2]), abs=1e-7)
    assert step(target_model, target_opt, tokens[3]) == pytest.approx(step(source_model, source_opt, tokens[3]), abs=1e-6)   # moments came along
    exported = module[reader].load_model_state_dict_from_checkpoint(path)
    assert list(exported) == list(target_model.state_dict())


def test_tokenizer_and_shard_writer_produce_the_same_files(tmp_path):
    """One corpus, one tokenizer directory: both packages load it (same fingerprint, same ids) and write byte-identical shards,
    document indices and, apart from nothing, identical manifests."""

    pytest.importorskip("tokenizers")
    import json

    from mini_train_sys_b200.data.documents import CleaningConfig
    from mini_train_sys_b200.data.preprocess import prepare_token_shards
    from mini_train_sys_b200.data.tokenizer import ByteLevelBPETokenizer, load_tokenizer

    with reference_on_path():
        from minitrain.data.documents import CleaningConfig as RefCleaning
        from minitrain.data.preprocess import prepare_token_shards as ref_prepare
        from minitrain.data.tokenizer import load_tokenizer as ref_load_tokenizer

    words = ["alpha", "beta", "gamma", "delta", "epsilon", "zeta", "eta", "theta", "iota", "kappa", "Zürich", "naïve"]
    gen = torch.Generator().manual_seed(2)
    texts = [" ".join(words[int(i)] for i in torch.randint(0, len(words), (int(n),), generator=gen)) + f". Document {d}."
             for d, n in enumerate(torch.randint(20, 400, (120,), generator=gen))]
    texts.append(texts[0])                                                       # an exact duplicate: both cleaners must drop it
    corpus = tmp_path / "docs.jsonl"
    corpus.write_text("\n".join(json.dumps({"id": f"d{i}", "text": t}) for i, t in enumerate(texts)), encoding="utf-8")
    tokenizer = ByteLevelBPETokenizer.train_from_iterator(iter(texts), vocab_size=400)
    tokenizer.save(tmp_path / "tok")
    mine, theirs = load_tokenizer(tmp_path / "tok"), ref_load_tokenizer(tmp_path / "tok")
    assert mine.fingerprint == theirs.fingerprint and mine.vocab_size == theirs.vocab_size and mine.boundary_token_id == theirs.boundary_token_id
    assert all(mine.encode(t) == theirs.encode(t) for t in texts[:10])

    options = dict(max_document_chars=900, max_shard_tokens=3000, validation_fraction=0.1, split_seed=7)
    ours_manifest = prepare_token_shards([corpus], output_dir=tmp_path / "ours", tokenizer=mine, cleaning=CleaningConfig(min_chars=8), **options)
    ref_manifest = ref_prepare([corpus], output_dir=tmp_path / "theirs", tokenizer=theirs, cleaning=RefCleaning(min_chars=8), **options)
    a, b = json.loads(Path(ours_manifest).read_text()), json.loads(Path(ref_manifest).read_text())
    assert a == b                                                                 # dtype, counts, sha256 of every shard and index, cleaning statistics
    assert a["cleaning_stats"]["rejected_duplicate"] == 1 and len(a["splits"]["train"]["shards"]) > 1
    for split in ("train", "validation"):
        for record in [*a["splits"][split]["shards"], a["splits"][split]["document_index"]]:
            assert (tmp_path / "ours" / record["path"]).read_bytes() == (tmp_path / "theirs" / record["path"]).read_bytes(), record["path"]


def test_run_files_resolve_to_the_same_settings_in_both_loaders():
    """Every shipped run file that the reference's loader accepts resolves (``extends`` included) to the same values here, key
    by key, for the keys the reference knows."""

    from dataclasses import asdict

    from mini_train_sys_b200.runtime.config import load_experiment

    with reference_on_path():
        from minitrain.runtime.config import experiment_config_from_dict as ref_from_dict
        from minitrain.runtime.config import load_yaml_dict as ref_yaml

    def ref_load(path):
        return ref_from_dict(ref_yaml(path))

    compared = 0
    for path in sorted((ROOT / "configs").rglob("*.yaml")):
        try:
            theirs = ref_load(path)
        except Exception:                      # model files, fragments, and run files that use this repository's additions
            continue
        ours = load_experiment(path)
        for section, value in asdict(theirs).items():
            mine = getattr(ours, section)
            mine = mine if isinstance(mine, dict) else asdict(mine)
            for key, expected in (value.items() if isinstance(value, dict) else ()):
                if isinstance(expected, dict):                 # parallel.ddp / parallel.fsdp
                    for inner, inner_expected in expected.items():
                        assert mine[key][inner] == inner_expected, (path.name, section, key, inner)
                else:
                    assert mine[key] == expected, (path.name, section, key)
        compared += 1
    assert compared >= 20, compared


def _run_reference(code: str, *args: str) -> str:
    """Run ``code`` in a process that sees only the reference package (its ``experiments`` package has the same name as ours)."""

    import os
    import subprocess

    env = {**os.environ, "PYTHONPATH": str(REF)}
    done = subprocess.run([sys.executable, "-c", code, *args], capture_output=True, text=True, timeout=600, env=env, cwd=str(REF))
    assert done.returncode == 0, done.stderr[-3000:]
    return done.stdout


def test_study_layer_contracts_and_a_reference_dataset_feeds_our_tools(tmp_path):
    """The study layer keeps the reference's contracts (variants, attribute order, template counts, pool sizes, person split),
    and a dataset written by the reference's generator goes through this repository's cache builder, validator, statistics
    and lineage audit unchanged."""

    import json

    from experiments.synbios_moe.audit import audit_dataset
    from experiments.synbios_moe.artifact_io import read_jsonl
    from experiments.synbios_moe.codec import get_codec
    from experiments.synbios_moe.pretraining import dataset as ours
    from experiments.synbios_moe.pretraining.token_statistics import dataset_token_statistics
    from experiments.synbios_moe.probes.dataset import build_probe_cache, validate_probe_cache

    out = tmp_path / "reference_data"
    facts = json.loads(_run_reference(
        "import json, sys\n"
        "from experiments.synbios_moe.pretraining import dataset as d\n"
        "d.write_dataset(sys.argv[1], num_people=30, variant='multi2+permute', seed=5)\n"
        "pools = d.candidate_pools()\n"
        "variants = ['single', 'single+fullname', 'single+permute1', 'single+permute5', 'multi2', 'multi5', 'multi2+permute', 'multi5+permute', 'multi5+permute+fullname']\n"
        "print(json.dumps({'attributes': list(d.ATTRIBUTES), 'templates': list(d.TEMPLATE_COUNTS), 'pools': {k: len(v) for k, v in pools.items()},\n"
        "                  'entries': {v: d.entries_per_person(v) for v in variants},\n"
        "                  'split': [d.split_for_person(i, 1337) for i in range(200)]}))\n", str(out)))
    assert facts["attributes"] == list(ours.ATTRIBUTES) and facts["templates"] == [ours.TEMPLATE_COUNTS[a] for a in ours.ATTRIBUTES]
    assert facts["entries"] == {v: ours.entries_per_person(v) for v in ours.VARIANTS}
    assert facts["split"] == [ours.split_for_person(i, 1337) for i in range(200)]
    mine = {k: len(v) for k, v in ours.candidate_pools().items()}
    assert {k: mine[k] for k in facts["pools"] if k in mine} == {k: v for k, v in facts["pools"].items() if k in mine} and len(mine) >= 5

    rows = list(read_jsonl(out / "biographies.jsonl"))
    assert len(rows) == 60 and set(rows[0]["attribute_spans"]) == set(ours.ATTRIBUTES)
    lo, hi = rows[0]["attribute_spans"]["university"]
    profile = next(p for p in read_jsonl(out / "profiles.jsonl") if p["person_id"] == rows[0]["person_id"])
    assert rows[0]["text"][lo:hi] == profile["university"]
    cache = build_probe_cache(out, tmp_path / "cache", codec_name="bytes")
    report = validate_probe_cache(cache, out)
    assert report["ok"], report
    stats = dataset_token_statistics(get_codec("bytes"), read_jsonl(out / "biographies.jsonl"), read_jsonl(out / "profiles.jsonl"))
    assert stats["biographies"] == 60
    problems = audit_dataset(out)
    assert problems == [], problems


@pytest.mark.parametrize("kind", ["p", "q"])
def test_probe_heads_are_exchangeable(tmp_path, kind):
    """A probe of the reference (backbone weights, rank-r embedding change, normaliser, classifier) loads into this
    repository's probe class under the same names and reads out the same logits."""

    from experiments.synbios_moe.probes.model import AttributeProbe
    from mini_train_sys_b200.models import MiniTransformer, ModelConfig, get_ops_backend

    blob = tmp_path / "probe.pt"
    _run_reference(
        "import sys, torch\n"
        "from minitrain.model.config import ModelConfig\n"
        "from minitrain.model.ops import get_ops_backend\n"
        "from minitrain.model.transformer import MiniTransformer\n"
        "from experiments.synbios_moe.probes.model import AttributeProbe\n"
        "shape = dict(vocab_size=211, seq_len=24, n_layers=2, n_heads=4, hidden_size=64, intermediate_size=48, ffn_type='moe', num_experts=4, experts_per_token=2, dropout=0.0)\n"
        "torch.manual_seed(11)\n"
        "probe = AttributeProbe(MiniTransformer(ModelConfig(**shape), get_ops_backend('torch')), 9, rank=3, kind=sys.argv[2])\n"
        "torch.nn.init.normal_(probe.delta.b.weight, std=0.5)\n"
        "probe.eval()\n"
        "ids = torch.randint(0, 211, (5, 20)); positions = torch.randint(0, 20, (5, 6 if sys.argv[2] == 'p' else 1))\n"
        "with torch.no_grad():\n"
        "    logits = probe(ids, positions)\n"
        "torch.save({'shape': shape, 'state': probe.state_dict(), 'ids': ids, 'positions': positions, 'logits': logits}, sys.argv[1])\n",
        str(blob), kind)
    data = torch.load(blob, weights_only=False)
    probe = AttributeProbe(MiniTransformer(ModelConfig(**data["shape"]), get_ops_backend("torch")), 9, rank=3, kind=kind)
    assert list(probe.state_dict()) == list(data["state"])
    probe.load_state_dict(data["state"])
    probe.eval()
    with torch.no_grad():
        logits = probe(data["ids"], data["positions"])
    assert logits.shape == data["logits"].shape and torch.allclose(logits, data["logits"], atol=1e-5)


def test_console_lines_are_the_reference_s_lines():
    """Tools that grep the console log of a run keep working: the same event payload prints the same line in both packages."""

    from mini_train_sys_b200.runtime.logger import format_console_event

    with reference_on_path():
        from minitrain.runtime.logger import format_console_event as ref_format

    train = {"event": "train", "step": 120, "step_total": 1000, "epoch": 2, "epochs_total": 10, "batch": 20, "batches_total": 100, "loss": 3.14159,
             "lr": 3e-4, "grad_norm": 1.2345, "tokens_per_sec": 123456.7, "data_wait_percent": 0.4, "progress_percent": 12.0, "eta_seconds": 3725.0,
             "elapsed_seconds": 100.0, "tokens_seen": 5_000_000, "tokens_goal": 40_000_000, "gpu_peak_memory_allocated_mb": 30500.0,
             "gpu_memory_allocated_mb": 20000.0, "gpu_compute_utilization_percent_mean": 97.0, "host_peak_memory_mb": 12.5}
    payloads = [train, {k: v for k, v in train.items() if not k.startswith("gpu_")},
                {"event": "checkpoint", "path": "ckpt/x/epoch_000001_step_000000100"},
                {"event": "resume", "path": "ckpt/x", "epoch": 1, "step": 100, "saved_world_size": 4},
                {"event": "init", "run": "r", "device": "cuda:0", "parallel": "fsdp", "world_size": 8, "params": 293494272},
                {"event": "probe_train", "step": 10, "steps_total": 100, "loss": 1.5, "accuracy_running": 0.5, "progress_percent": 10.0, "eta_seconds": 50},
                {"event": "probe_validation", "example": 40, "examples_total": 400, "accuracy_running": 0.25, "progress_percent": 10.0, "eta_seconds": 9},
                {"event": "evaluate", "batch": 3, "batches_total": 30, "progress_percent": 10.0, "eta_seconds": 5},
                {"event": "probe_checkpoint", "step": 10, "steps_total": 100, "path": "p.pt"},
                {"event": "probe_pipeline", "phase": "training", "step": 3, "steps_total": 22, "tasks_running": 2, "tasks_queued": 17, "tasks_failed": 0,
                 "task": "p-major-first", "action": "finished", "device": "cuda:1", "eta_seconds": 600},
                {"event": "parallel_ready", "strategy": "fsdp", "fsdp_units": 13}]
    for payload in payloads:
        assert format_console_event(payload) == ref_format(payload), payload["event"]
    # what this repository adds to a train event shows up as an extra cell and changes nothing else
    extended = format_console_event({**train, "mfu_percent": 41.2})
    assert "mfu 41.2%" in extended and extended.replace(" | mfu 41.2%", "") == ref_format(train)


def test_every_command_and_most_options_of_the_reference_study_cli_exist_here():
    """``scripts/synbios_moe.py`` accepts every sub-command name of the reference's CLI, and for each the option strings the
    reference defines, so that a launcher written for one parses under the other."""

    import importlib.util
    import json

    out = _run_reference(
        "import argparse, json\n"
        "from pathlib import Path\n"
        "from experiments.synbios_moe import cli\n"
        "parser = cli.build_parser(project_root=Path('.'), handlers={name: (lambda args: 0) for name in cli.PUBLIC_COMMANDS}, default_device='cpu')\n"
        "sub = next(a for a in parser._actions if isinstance(a, argparse._SubParsersAction))\n"
        "print(json.dumps({name: sorted(s for a in p._actions for s in a.option_strings if s.startswith('--') and s != '--help') for name, p in sub.choices.items()}))\n")
    theirs = json.loads(out)
    spec = importlib.util.spec_from_file_location("synbios_cli", ROOT / "scripts" / "synbios_moe.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    import argparse

    parser = module.build_parser()
    sub = next(a for a in parser._actions if isinstance(a, argparse._SubParsersAction))
    assert set(theirs) <= set(sub.choices), sorted(set(theirs) - set(sub.choices))
    missing = {}
    total = 0
    for name, options in theirs.items():
        mine = {s for a in sub.choices[name]._actions for s in a.option_strings}
        total += len(options)
        gone = [o for o in options if o not in mine]
        if gone:
            missing[name] = gone
    assert total > 200 and missing == {}, missing
