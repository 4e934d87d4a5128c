"""Checkpoint commit protocol, retention, resume selectors, resharding across world sizes, host-side fault injection."""

import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from mini_train_sys_b200.models import MiniTransformer, ModelConfig, get_ops_backend  # noqa: E402
from mini_train_sys_b200.parallel.flat_engine import FlatDataParallel  # noqa: E402
from mini_train_sys_b200.runtime.config import OptimizerConfig  # noqa: E402
from mini_train_sys_b200.train import checkpoint as ck  # noqa: E402
from mini_train_sys_b200.train.optim import build_optimizer  # noqa: E402
from mini_train_sys_b200.train.trainer import Trainer  # noqa: E402

CFG = ModelConfig(vocab_size=64, seq_len=16, n_layers=2, n_heads=2, hidden_size=32, intermediate_size=64, tie_word_embeddings=True)


def _model():
    torch.manual_seed(0)
    return MiniTransformer(CFG, get_ops_backend("torch"))


def _batch(seed, n=4):
    t = torch.randint(0, 64, (n, 17), generator=torch.Generator().manual_seed(seed))
    return {"input_ids": t[:, :-1], "targets": t[:, 1:]}


def _fake_committed(root: Path, epoch: int, step: int, *, export=False) -> Path:
    p = ck.checkpoint_path(root, "run", epoch=epoch, step=step)
    p.mkdir(parents=True)
    (p / "COMMITTED").write_text("ok\n")
    if export:
        (p / "model.pt").write_bytes(b"x")
    return p


def test_resume_selectors_ignore_uncommitted(tmp_path):
    a = _fake_committed(tmp_path, 1, 10)
    b = _fake_committed(tmp_path, 2, 20)
    torn = ck.checkpoint_path(tmp_path, "run", epoch=3, step=30)
    torn.mkdir(parents=True)                      # no COMMITTED marker
    assert ck.resolve_resume_checkpoint("latest", checkpoint_dir=tmp_path, run_name="run") == b
    with pytest.raises(FileNotFoundError):
        ck.resolve_resume_checkpoint("safety", checkpoint_dir=tmp_path, run_name="run")
    (a / "SAFETY").write_text("resume fallback\n")
    assert ck.resolve_resume_checkpoint("safety", checkpoint_dir=tmp_path, run_name="run") == a
    with pytest.raises(ValueError):
        ck.resolve_resume_checkpoint(torn, checkpoint_dir=tmp_path, run_name="run")
    with pytest.raises(FileNotFoundError):
        ck.resolve_resume_checkpoint(tmp_path / "nope", checkpoint_dir=tmp_path, run_name="run")


def test_prune_keeps_recent_plus_safety_anchors(tmp_path):
    paths = [_fake_committed(tmp_path, e, e * 10, export=True) for e in range(1, 13)]
    removed = ck.prune_checkpoints(tmp_path, "run", keep_last=2, keep_safety=1, safety_every_epochs=5, keep_model_exports=1)
    kept = sorted(p.name for p in (tmp_path / "run").iterdir())
    assert kept == [paths[9].name, paths[10].name, paths[11].name]          # epoch 10 anchor + the last two
    assert (paths[9] / "SAFETY").is_file() and not (paths[11] / "SAFETY").exists()
    assert len(removed) == 9
    assert [(p / "model.pt").exists() for p in (paths[9], paths[10], paths[11])] == [False, False, True]
    with pytest.raises(ValueError):
        ck.prune_checkpoints(tmp_path, "run", keep_last=0)


def test_single_process_roundtrip_and_export(tmp_path):
    model = _model()
    opt = build_optimizer(model, cfg=OptimizerConfig(lr=1e-2))
    tr = Trainer(model, opt, torch.device("cpu"), precision="fp32", grad_clip_norm=1.0)
    tr.train_step(_batch(1))
    path = ck.save_checkpoint(ck.checkpoint_path(tmp_path, "run", epoch=1, step=1), model, opt, 1, epoch=1, tokens_seen=64,
                              precision="fp32", config={"model": vars(CFG) if False else CFG.__dict__}, export_model=True)
    assert ck.is_committed(path) and (path / "runtime.pt").is_file() and (path / "rng_rank_00000.pt").is_file()
    assert (path / "distributed").is_dir() and not list(tmp_path.rglob(".*.tmp"))
    assert ck.save_checkpoint(path, model, opt, 1) == path             # committed path: idempotent
    want = float(tr.train_step(_batch(2)))
    fresh = _model()
    fresh_opt = build_optimizer(fresh, cfg=OptimizerConfig(lr=1e-2))
    info = ck.restore_training_checkpoint(path, fresh, fresh_opt)
    assert info["step"] == 1 and info["epoch"] == 1 and info["tokens_seen"] == 64 and info["rng_restored"]
    tr2 = Trainer(fresh, fresh_opt, torch.device("cpu"), precision="fp32", grad_clip_norm=1.0)
    assert float(tr2.train_step(_batch(2))) == pytest.approx(want, rel=1e-6)
    state = ck.load_model_state_dict_from_checkpoint(path)
    assert set(state) == set(_model().state_dict())
    assert ck.checkpoint_trainer_state(path)["step"] == 1


def test_crash_before_commit_leaves_no_visible_checkpoint(tmp_path, monkeypatch):
    model = _model()
    opt = build_optimizer(model, cfg=OptimizerConfig())

    def boom(stage):
        if stage == "before_commit":
            raise RuntimeError("injected crash")

    monkeypatch.setattr(ck, "fault_hook", boom)
    target = ck.checkpoint_path(tmp_path, "run", epoch=1, step=5)
    with pytest.raises(RuntimeError, match="injected"):
        ck.save_checkpoint(target, model, opt, 5, epoch=1)
    assert not target.exists()
    with pytest.raises(FileNotFoundError):
        ck.resolve_resume_checkpoint("latest", checkpoint_dir=tmp_path, run_name="run")
    monkeypatch.setattr(ck, "fault_hook", None)
    assert ck.is_committed(ck.save_checkpoint(target, model, opt, 5, epoch=1))   # the stale staging dir is replaced


def _sharded_worker(rank, world, port, root, phase):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        eng = FlatDataParallel(_model(), mode="shard")
        opt = build_optimizer(eng, cfg=OptimizerConfig(lr=1e-2))
        tr = Trainer(eng, opt, torch.device("cpu"), precision="fp32", grad_clip_norm=1.0)
        path = ck.checkpoint_path(root, "run", epoch=1, step=2)
        if phase == "save":
            for seed in (1, 2):
                b = _batch(seed, n=4 * world)
                tr.train_step({k: v[rank::world] for k, v in b.items()})
            ck.save_checkpoint(path, eng, opt, 2, epoch=1, tokens_seen=128, export_model=True)
        else:
            info = ck.restore_training_checkpoint(path, eng, opt)
            assert info["saved_world_size"] == 2 and info["tokens_seen"] == 128 * 2 // world
            b = _batch(3, n=8)
            loss = tr.train_step({k: v[rank::world] for k, v in b.items()})
            full = eng.full_state_dict()     # collective: every rank takes part
            if rank == 0:
                torch.save({"full": full, "loss": float(loss)}, Path(root) / f"after_{world}.pt")
    finally:
        dist.destroy_process_group()


def test_sharded_checkpoint_reshards_from_two_ranks_to_one_and_to_plain_model(tmp_path):
    port = 29800 + os.getpid() % 150
    mp.spawn(_sharded_worker, args=(2, port, str(tmp_path), "save"), nprocs=2, join=True)
    path = ck.checkpoint_path(tmp_path, "run", epoch=1, step=2)
    assert ck.is_committed(path) and (path / "rng_rank_00001.pt").is_file() and (path / "model.pt").is_file()
    mp.spawn(_sharded_worker, args=(2, port + 1, str(tmp_path), "load"), nprocs=2, join=True)
    mp.spawn(_sharded_worker, args=(1, port + 2, str(tmp_path), "load"), nprocs=1, join=True)
    two, one = torch.load(tmp_path / "after_2.pt"), torch.load(tmp_path / "after_1.pt")
    for name in two["full"]:
        assert torch.allclose(two["full"][name], one["full"][name], atol=1e-5), name
    # the same DCP payload also loads into an unwrapped model with a stock optimizer
    plain = _model()
    popt = build_optimizer(plain, cfg=OptimizerConfig(lr=1e-2))
    info = ck.restore_training_checkpoint(path, plain, popt)
    assert info["step"] == 2
    exported = ck.load_model_state_dict_from_checkpoint(path)
    for name, p in plain.state_dict().items():
        assert torch.allclose(exported[name], p, atol=1e-6), name
    tr = Trainer(plain, popt, torch.device("cpu"), precision="fp32", grad_clip_norm=1.0)
    tr.train_step(_batch(3, n=8))
    for name, p in plain.state_dict().items():
        assert torch.allclose(one["full"][name], p, atol=2e-5), name
