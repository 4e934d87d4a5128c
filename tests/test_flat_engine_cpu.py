"""Flat sharding engine on CPU: single rank and two Gloo ranks against plain fp32 AdamW training."""

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
from mini_train_sys_b200.parallel.flat_engine import FlatDataParallel, _merge_segments  # noqa: E402
from mini_train_sys_b200.runtime.config import OptimizerConfig  # noqa: E402
from mini_train_sys_b200.train.optim import build_optimizer  # noqa: E402
from mini_train_sys_b200.train.trainer import Trainer  # noqa: E402

CFG = ModelConfig(vocab_size=96, seq_len=16, n_layers=2, n_heads=2, hidden_size=32, intermediate_size=32, ffn_type="moe",
                  num_experts=4, experts_per_token=2, tie_word_embeddings=True)
OPT = OptimizerConfig(lr=1e-2, weight_decay=0.1)


# Data-parallel ranks see different micro-batches; the MoE balance loss is not linear in the batch, so the
# cross-rank equivalence test uses the dense family (mean cross entropy is linear in the batch).
DENSE = ModelConfig(vocab_size=96, seq_len=16, n_layers=2, n_heads=2, hidden_size=32, intermediate_size=64,
                    tie_word_embeddings=False)


DEEP = ModelConfig(vocab_size=96, seq_len=16, n_layers=5, n_heads=2, hidden_size=32, intermediate_size=32, ffn_type="moe",
                   num_experts=4, experts_per_token=2, tie_word_embeddings=True)   # more blocks than staging slots


def make_model(cfg=CFG):
    torch.manual_seed(0)
    return MiniTransformer(cfg, get_ops_backend("torch"))


def batches(n, seed=1, batch=4):
    g = torch.Generator().manual_seed(seed)
    toks = torch.randint(0, CFG.vocab_size, (n, batch, CFG.seq_len + 1), generator=g)
    return [{"input_ids": t[:, :-1], "targets": t[:, 1:]} for t in toks]


def train_plain(steps, cfg=CFG):
    model = make_model(cfg)
    tr = Trainer(model, build_optimizer(model, cfg=OPT), torch.device("cpu"), precision="fp32", grad_clip_norm=1.0)
    losses = [float(tr.train_step(b)) for b in batches(steps)]
    return model, losses


def test_merge_segments_cover_the_shard():
    segs = _merge_segments([(0, 8, True), (8, 24, True), (24, 32, False), (40, 48, True)], 64)
    assert segs == [(0, 24, True), (24, 40, False), (40, 64, True)]
    assert _merge_segments([], 16) == [(0, 16, False)]


def test_single_rank_engine_matches_plain_adamw():
    plain, want = train_plain(4)
    eng = FlatDataParallel(make_model(), mode="shard")
    assert eng.unit_count() == CFG.n_layers + 1
    opt = build_optimizer(eng, cfg=OPT)
    tr = Trainer(eng, opt, torch.device("cpu"), precision="fp32", grad_clip_norm=1.0)
    got = [float(tr.train_step(b)) for b in batches(4)]
    assert got == pytest.approx(want, rel=1e-5)
    full = eng.full_state_dict()
    for name, p in plain.state_dict().items():
        assert torch.allclose(full[name], p, atol=1e-5), name
    assert "grad_norm" in tr.last_metrics and float(tr.last_metrics["grad_norm"]) > 0


def test_replicate_mode_buckets_match_plain_adamw():
    _, want = train_plain(3)
    eng = FlatDataParallel(make_model(), mode="replicate", bucket_cap_mb=1)
    tr = Trainer(eng, build_optimizer(eng, cfg=OPT), torch.device("cpu"), precision="fp32", grad_clip_norm=1.0)
    got = [float(tr.train_step(b)) for b in batches(3)]
    assert got == pytest.approx(want, rel=1e-5)


def _two_rank_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        eng = FlatDataParallel(make_model(DENSE), mode="shard")
        tr = Trainer(eng, build_optimizer(eng, cfg=OPT), torch.device("cpu"), precision="fp32", grad_clip_norm=1.0)
        data = batches(3, batch=4 * world)
        losses = []
        for b in data:   # each rank takes its slice of the global batch
            local = {k: v[rank::world] for k, v in b.items()}
            losses.append(float(tr.train_step(local)))
        full = eng.full_state_dict()
        if rank == 0:
            torch.save({"full": full, "losses": losses}, Path(out_dir) / "result.pt")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_gloo_ranks_match_single_process_on_the_global_batch(tmp_path, world):
    port = 29640 + os.getpid() % 200
    mp.spawn(_two_rank_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    got = torch.load(tmp_path / "result.pt", weights_only=False)
    # the same global batch on one process
    model = make_model(DENSE)
    tr = Trainer(model, build_optimizer(model, cfg=OPT), torch.device("cpu"), precision="fp32", grad_clip_norm=1.0)
    for b in batches(3, batch=4 * world):
        tr.train_step(b)
    for name, p in model.state_dict().items():
        # Adam divides by sqrt(v): where a gradient is tiny, a different summation order over ranks moves single elements
        diff = (got["full"][name] - p).abs()
        assert float(diff.max()) < 1e-4 and float(diff.mean()) < 1e-6, (name, float(diff.max()), float(diff.mean()))


def test_staged_parameters_on_one_rank_match_plain_adamw():
    """full_shard residency exercised with a world of one: parameters live in staging slots only while their block runs."""

    plain, want = train_plain(4, DEEP)
    eng = FlatDataParallel(make_model(DEEP), mode="shard", stage_single_rank=True)
    assert eng.staged and all(u.gathered is None for u in eng.units) and len(eng._slots) == 2
    tr = Trainer(eng, build_optimizer(eng, cfg=OPT), torch.device("cpu"), precision="fp32", grad_clip_norm=1.0)
    gathers = []
    plain_gather = eng.coll.gather_unit
    eng.coll.gather_unit = lambda unit, dst: (gathers.append(unit.name), plain_gather(unit, dst))[1]
    got = [float(tr.train_step(b)) for b in batches(4)]
    assert got == pytest.approx(want, rel=1e-5)
    # per step: the root, five blocks on the way forward, and on the way back the three that the two slots no longer held
    assert gathers[:9] == ["root", "blocks.0", "blocks.1", "blocks.2", "blocks.3", "blocks.4", "blocks.2", "blocks.1", "blocks.0"]
    assert len(gathers) == 4 * 9
    full = eng.full_state_dict()
    for name, p in plain.state_dict().items():
        assert torch.allclose(full[name], p, atol=1e-5), name
    sizes = eng.parameter_bytes()
    assert sizes["staging"] > 0 and sizes["resident"] == sum(16 * u.shard_numel for u in eng.units)


def test_staged_engine_with_activation_checkpointing_matches_plain_adamw():
    _, want = train_plain(3, DEEP)
    eng = FlatDataParallel(make_model(DEEP), mode="shard", stage_single_rank=True, activation_checkpointing=True)
    tr = Trainer(eng, build_optimizer(eng, cfg=OPT), torch.device("cpu"), precision="fp32", grad_clip_norm=1.0)
    got = [float(tr.train_step(b)) for b in batches(3)]
    assert got == pytest.approx(want, rel=1e-5)


def test_a_parameter_without_gradient_contributes_zeros_not_last_steps_values():
    """One parameter of a unit stops receiving gradients: its range of the flat buffer must be zeroed, not reused."""

    eng = FlatDataParallel(make_model(DENSE), mode="shard")
    opt = build_optimizer(eng, cfg=OptimizerConfig(lr=1e-2, weight_decay=0.0))
    tr = Trainer(eng, opt, torch.device("cpu"), precision="fp32", grad_clip_norm=None)
    data = batches(2)
    tr.train_step(data[0])
    gate = eng.module.blocks[0].ffn.gate.weight
    unit, slot = eng._slot_of[gate]
    before = unit.master.clone()
    m_before = unit.exp_avg.clone()
    gate.requires_grad_(False)           # the operator no longer produces this gradient
    try:
        tr.train_step(data[1])
    finally:
        gate.requires_grad_(True)
    lo, hi = slot.offset, slot.offset + slot.numel
    # a zero gradient decays the first moment by beta1 and nothing else feeds it
    assert torch.allclose(unit.exp_avg[lo:hi], m_before[lo:hi] * 0.9, atol=1e-8)
    assert not torch.equal(unit.master[:lo], before[:lo]) or lo == 0


def test_a_second_backward_before_the_step_is_refused():
    eng = FlatDataParallel(make_model(DENSE), mode="shard")
    b = batches(1)[0]
    loss, _ = eng(b["input_ids"], targets=b["targets"])
    loss.backward()
    loss2, _ = eng(b["input_ids"], targets=b["targets"])
    with pytest.raises(RuntimeError, match="one backward pass per step"):
        loss2.backward()


def test_fp16_loss_scaling_is_refused_by_the_sharded_optimizer():
    from mini_train_sys_b200.train.precision import PrecisionPolicy

    eng = FlatDataParallel(make_model(DENSE), mode="shard")
    opt = build_optimizer(eng, cfg=OPT)
    tr = Trainer.__new__(Trainer)
    policy = PrecisionPolicy("fp16", torch.float16, True, True)
    import mini_train_sys_b200.train.trainer as trainer_mod
    orig = trainer_mod.resolve_precision_policy
    trainer_mod.resolve_precision_policy = lambda *_a, **_k: policy
    try:
        with pytest.raises(ValueError, match="loss scaling"):
            Trainer(eng, opt, torch.device("cpu"), precision="fp16")
    finally:
        trainer_mod.resolve_precision_policy = orig
    del tr


def test_fused_fsdp_refuses_options_it_does_not_implement():
    from mini_train_sys_b200.parallel.fsdp import FSDPStrategy

    for kwargs in ({"cpu_offload": True}, {"sharding_strategy": "hybrid_shard"}, {"precision": "fp16"}):
        strat = FSDPStrategy(engine="fused", **kwargs)
        with pytest.raises(ValueError, match="does not implement"):
            strat.wrap_model(make_model(DENSE))


def test_auto_engine_never_picks_one_that_would_refuse_the_run():
    from mini_train_sys_b200.parallel.fsdp import FSDPStrategy

    plain = dict(cpu_offload=False, sharding_strategy="full_shard", precision="bf16")
    assert FSDPStrategy.choose_engine("auto", "fused", **plain) == "fused"
    assert FSDPStrategy.choose_engine("auto", "nccl", **plain) == "nccl"
    for change in ({"cpu_offload": True}, {"sharding_strategy": "no_shard"}, {"sharding_strategy": "hybrid_shard"}, {"precision": "fp16"}):
        assert FSDPStrategy.choose_engine("auto", "fused", **{**plain, **change}) == "nccl"
        assert FSDPStrategy.choose_engine("fused", "fused", **{**plain, **change}) == "fused"     # explicit: refused at wrap time
    assert FSDPStrategy.fused_unsupported(cpu_offload=True, sharding_strategy="no_shard", precision="fp16") == [
        "cpu_offload", "sharding_strategy=no_shard", "precision=fp16 (loss scaling)"]


def _bytes_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mini_train_sys_b200.parallel.custom_allreduce import allreduce_sum

        full = FlatDataParallel(make_model(DENSE), mode="shard", reshard_after_forward=True)
        kept = FlatDataParallel(make_model(DENSE), mode="shard", reshard_after_forward=False)
        t = torch.arange(10, dtype=torch.float32) + rank
        total = allreduce_sum(t, comm=full.coll)
        if rank == 0:
            torch.save({"full_shard": full.parameter_bytes(), "shard_grad_op": kept.parameter_bytes(), "sum": total,
                        "input": t, "total": sum(u.total for u in full.units)}, Path(out_dir) / "bytes.pt")
    finally:
        dist.destroy_process_group()


def test_full_shard_keeps_one_nth_of_the_parameters_resident(tmp_path):
    seen = {}
    for world in (2, 4):
        port = 29240 + os.getpid() % 200 + world
        mp.spawn(_bytes_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
        seen[world] = torch.load(tmp_path / "bytes.pt", weights_only=False)
        want = torch.arange(10, dtype=torch.float32) * world + sum(range(world))
        assert torch.equal(seen[world]["sum"], want) and torch.equal(seen[world]["input"], torch.arange(10.0))
    for world, rec in seen.items():
        # fp32 master + two moments + the low-precision shard (fp32 on CPU): 16 bytes per local element, nothing else resident
        assert rec["full_shard"]["resident"] == 16 * rec["total"] // world
        assert rec["shard_grad_op"]["resident"] == 16 * rec["total"] // world + 4 * rec["total"]
    assert seen[2]["full_shard"]["resident"] == pytest.approx(2 * seen[4]["full_shard"]["resident"], rel=0.02)
    assert seen[2]["full_shard"]["staging"] == pytest.approx(seen[4]["full_shard"]["staging"], rel=0.05)   # padding only


def test_allreduce_sum_without_a_process_group_is_a_copy():
    from mini_train_sys_b200.parallel.custom_allreduce import allreduce_sum, naive_allreduce_sum

    t = torch.randn(7)
    out = allreduce_sum(t)
    assert torch.equal(out, t) and out.data_ptr() != t.data_ptr()
    assert naive_allreduce_sum is allreduce_sum
