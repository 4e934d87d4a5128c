"""Expert parallelism on two Gloo ranks against a single process holding all experts (dropless and with capacity)."""

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
from mini_train_sys_b200.models.router import capacity_keep_mask, expert_capacity  # noqa: E402
from mini_train_sys_b200.runtime.config import CommConfig, EPConfig, OptimizerConfig  # noqa: E402
from mini_train_sys_b200.train.optim import build_optimizer  # noqa: E402
from mini_train_sys_b200.train.trainer import Trainer  # noqa: E402

# balance losses are not linear in the batch, so the cross-rank comparison switches them off
CFG = ModelConfig(vocab_size=64, seq_len=16, n_layers=2, n_heads=2, hidden_size=32, intermediate_size=32, ffn_type="moe",
                  num_experts=4, experts_per_token=2, router_aux_loss_coef=0.0, router_z_loss_coef=0.0)
OPT = OptimizerConfig(lr=1e-2)


def _model():
    torch.manual_seed(0)
    return MiniTransformer(CFG, get_ops_backend("torch"))


def _batch(seed, n):
    t = torch.randint(0, 64, (n, 17), generator=torch.Generator().manual_seed(seed))
    return {"input_ids": t[:, :-1], "targets": t[:, 1:]}


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    from mini_train_sys_b200.parallel.ep import ExpertParallelStrategy

    strat = ExpertParallelStrategy(process_group_backend="gloo", engine="nccl", comm=CommConfig(engine="nccl"), ep=EPConfig())
    strat.setup()
    try:
        eng = strat.wrap_model(_model())
        assert eng.module.blocks[0].ffn.gate_up_proj.shape[0] == CFG.num_experts // world
        tr = Trainer(eng, build_optimizer(eng, cfg=OPT), torch.device("cpu"), precision="fp32", grad_clip_norm=1.0)
        for seed in (1, 2, 3):
            b = _batch(seed, 4 * world)
            tr.train_step({k: v[rank::world] for k, v in b.items()})
        full = eng.full_state_dict()
        if rank == 0:
            torch.save(full, Path(out_dir) / "ep.pt")
    finally:
        strat.teardown()


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_matches_single_process(tmp_path, world):
    mp.spawn(_worker, args=(world, 29900 + os.getpid() % 90, str(tmp_path)), nprocs=world, join=True)
    got = torch.load(tmp_path / "ep.pt")
    model = _model()
    tr = Trainer(model, build_optimizer(model, cfg=OPT), torch.device("cpu"), precision="fp32", grad_clip_norm=1.0)
    for seed in (1, 2, 3):
        tr.train_step(_batch(seed, 4 * world))
    want = model.state_dict()
    assert got["blocks.0.ffn.gate_up_proj"].shape == want["blocks.0.ffn.gate_up_proj"].shape
    for name, p in want.items():
        diff = (got[name] - p).abs()
        assert float(diff.max()) < 1e-4 and float(diff.mean()) < 2e-6, (name, float(diff.max()), float(diff.mean()))


def test_capacity_mask_admits_highest_weights_first():
    idx = torch.tensor([[0, 1], [0, 1], [0, 2], [0, 3]])
    w = torch.tensor([[0.9, 0.1], [0.6, 0.4], [0.7, 0.3], [0.8, 0.2]])
    keep = capacity_keep_mask(idx, w, 4, capacity=2)
    assert keep[:, 0].tolist() == [True, False, False, True]       # expert 0 keeps its two heaviest routes
    assert keep[:, 1].all()
    cfg = ModelConfig(ffn_type="moe", num_experts=4, experts_per_token=2, expert_capacity_factor=1.0, expert_min_capacity=1)
    assert expert_capacity(cfg, 8) == 4 and expert_capacity(ModelConfig(ffn_type="moe"), 8) is None


def test_router_drops_overflow_and_reports_it():
    cfg = ModelConfig(vocab_size=64, seq_len=16, n_layers=1, n_heads=2, hidden_size=32, intermediate_size=32, ffn_type="moe",
                      num_experts=4, experts_per_token=2, expert_capacity_factor=0.5, expert_min_capacity=1)
    torch.manual_seed(0)
    model = MiniTransformer(cfg, get_ops_backend("torch"))
    router = model.blocks[0].ffn.router
    router.enforce_capacity = True
    router.drop_overflow_routes = True
    out = router(torch.randn(64, 32), model.ops)
    dropped = float(out.metrics["moe/dropped_route_fraction"])
    assert 0.3 < dropped < 0.7
    assert float((out.expert_indices < 0).float().mean()) == pytest.approx(dropped)
    assert float(out.expert_weights[out.expert_indices < 0].abs().sum()) == 0.0
    kept_per_expert = torch.bincount(out.expert_indices[out.expert_indices >= 0].long(), minlength=4)
    assert int(kept_per_expert.max()) <= expert_capacity(cfg, 64)


def test_route_layout_slots_are_dense_per_destination_and_overflow_is_dropped():
    import torch

    from mini_train_sys_b200.parallel.ep import _route_layout

    torch.manual_seed(0)
    world, n_local, t, k = 4, 2, 50, 2
    idx = torch.randint(0, world * n_local, (t, k))
    idx[3, 1] = -1
    dest, slot, local_e, counts, over = _route_layout(idx, n_local, world, cap=1000)
    flat = idx.reshape(-1)
    assert int(over) == 0 and dest[7] == -1 and counts.sum() == t * k - 1
    for d in range(world):
        mine = (dest == d).nonzero().flatten()
        assert slot[mine].tolist() == list(range(len(mine)))            # route order is kept inside a destination
        assert (flat[mine] // n_local == d).all() and (local_e[mine] == flat[mine] % n_local).all()
        assert int(counts[d]) == len(mine)
    # a region of 5 rows: everything past slot 4 is dropped and counted
    dest2, slot2, _, counts2, over2 = _route_layout(idx, n_local, world, cap=5)
    assert int(over2) == int((counts - 5).clamp(min=0).sum()) and int(slot2.max()) <= 4 and (counts2 <= 5).all()
    assert int((dest2 >= 0).sum()) == int(counts2.sum())


def test_route_histogram_matches_bincount_with_and_without_weights():
    from mini_train_sys_b200.models.router import route_histogram

    idx = torch.randint(0, 7, (40, 3))
    assert torch.equal(route_histogram(idx, 9), torch.bincount(idx.reshape(-1), minlength=9).float())
    keep = torch.rand(40, 3) > 0.3
    assert torch.equal(route_histogram(idx, 9, keep), torch.bincount(idx[keep], minlength=9).float())
