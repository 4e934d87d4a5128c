"""Flat engine and peer-memory collectives on one GPU (a world of one still runs every kernel)."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _model(ops_name="native", layers=2):
    from mini_train_sys_b200.models import MiniTransformer, ModelConfig, get_ops_backend

    cfg = ModelConfig(vocab_size=1000, seq_len=128, n_layers=layers, n_heads=4, hidden_size=256, intermediate_size=256,
                      ffn_type="moe", num_experts=4, experts_per_token=2, tie_word_embeddings=True)
    torch.manual_seed(0)
    return MiniTransformer(cfg, get_ops_backend(ops_name), activation_dtype=torch.bfloat16).to(DEV)


def _train(engine_collectives, steps=4, layers=2, **engine_kwargs):
    from mini_train_sys_b200.parallel.flat_engine import FlatDataParallel
    from mini_train_sys_b200.runtime.config import OptimizerConfig
    from mini_train_sys_b200.train.optim import build_optimizer
    from mini_train_sys_b200.train.trainer import Trainer

    eng = FlatDataParallel(_model(layers=layers), mode="shard", collectives=engine_collectives, **engine_kwargs)
    opt = build_optimizer(eng, cfg=OptimizerConfig(lr=1e-3))
    tr = Trainer(eng, opt, torch.device(DEV), use_fused_loss=True, precision="bf16", grad_clip_norm=1.0)
    eng._test_optimizer, eng._test_trainer = opt, tr
    g = torch.Generator().manual_seed(3)
    losses, norms = [], []
    for _ in range(steps):
        t = torch.randint(0, 1000, (4, 129), generator=g)
        losses.append(float(tr.train_step({"input_ids": t[:, :-1], "targets": t[:, 1:]})))
        norms.append(float(tr.last_metrics["grad_norm"]))
    return eng, losses, norms


def test_fused_engine_matches_library_collectives():
    from mini_train_sys_b200.ops.native_backend import check_kernel_status
    from mini_train_sys_b200.parallel.comm import PeerCollectives, TorchCollectives

    dev = torch.device(DEV, 0)
    eng_a, loss_a, norm_a = _train(PeerCollectives(dev, max_units=3))
    eng_b, loss_b, norm_b = _train(TorchCollectives(dev))
    assert eng_a.coll.fused and not eng_b.coll.fused
    assert loss_a == pytest.approx(loss_b, abs=2e-2)
    assert norm_a == pytest.approx(norm_b, rel=5e-2)
    fa, fb = eng_a.full_state_dict(), eng_b.full_state_dict()
    # split-K weight gradients are summed with fp32 atomics, so two runs differ in rounding; an AdamW step moves a
    # weight by at most lr, hence two runs of 4 steps at lr 1e-3 can sit 8e-3 apart where a tiny gradient flips sign
    for name in fa:
        diff = (fa[name] - fb[name]).abs()
        assert float(diff.max()) <= 8.5e-3 and float(diff.mean()) < 3e-4, (name, float(diff.max()), float(diff.mean()))
    check_kernel_status()


def test_clip_coefficient_and_first_update_follow_the_fp32_formula():
    """The gradient norm, the clip coefficient and the first AdamW step of every unit, recomputed in PyTorch from the reduced
    gradient shards the kernels themselves produced: the norm to 1e-5 relative, the updated fp32 weights and both moments to
    float round-off, the pushed bf16 replica to one bf16 rounding of the reference weight."""

    from mini_train_sys_b200.parallel.comm import PeerCollectives
    from mini_train_sys_b200.parallel.flat_engine import FlatDataParallel
    from mini_train_sys_b200.runtime.config import OptimizerConfig
    from mini_train_sys_b200.train.optim import build_optimizer

    dev = torch.device(DEV, 0)
    lr, wd, b1, b2, eps, clip = 1e-3, 0.1, 0.9, 0.95, 1e-8, 0.5
    eng = FlatDataParallel(_model(), mode="shard", collectives=PeerCollectives(dev, max_units=3))
    opt = build_optimizer(eng, cfg=OptimizerConfig(lr=lr, weight_decay=wd, beta1=b1, beta2=b2, eps=eps))
    opt.set_clip_norm(clip)
    t = torch.randint(0, 1000, (4, 129), generator=torch.Generator().manual_seed(11))
    with torch.autocast("cuda", dtype=torch.bfloat16):
        loss, _ = eng(t[:, :-1].to(DEV), targets=t[:, 1:].to(DEV), use_fused_loss=True)
    loss.backward()
    eng._flush_incomplete_units()
    torch.cuda.synchronize()
    grads = [u.grad_shard.clone() for u in eng.units]
    before = [u.master.clone() for u in eng.units]
    total = sum(float(g.double().pow(2).sum()) for g in grads)
    norm = total ** 0.5
    assert norm > clip, "the case must actually clip"
    coef = min(1.0, clip / (norm + 1e-6))
    opt.step()
    torch.cuda.synchronize()
    eng.check_status()
    assert float(eng.grad_norm) == pytest.approx(norm, rel=1e-5)
    assert float(eng.clip_coef) == pytest.approx(coef, rel=1e-5)
    decayed = 0
    for u, g, p0 in zip(eng.units, grads, before):
        for lo, hi, decay in u.segments:
            gg = g[lo:hi].double() * coef
            m = (1 - b1) * gg
            v = (1 - b2) * gg * gg
            w = wd if decay else 0.0
            decayed += int(decay)
            denom = (v / (1 - b2)).sqrt() + eps
            want = p0[lo:hi].double() * (1 - lr * w) - (lr / (1 - b1)) * m / denom
            assert torch.allclose(u.exp_avg[lo:hi].double(), m, rtol=2e-5, atol=1e-12)
            assert torch.allclose(u.exp_avg_sq[lo:hi].double(), v, rtol=4e-5, atol=1e-20)
            # |update| <= lr: an error of 1e-7 absolute is 1e-4 of the step itself
            assert float((u.master[lo:hi].double() - want).abs().max()) < 2e-7, (lo, hi, decay)
    assert decayed > 0
    state = eng.full_state_dict()
    for name, param in eng.module.named_parameters():
        if param.dtype == torch.bfloat16:
            assert torch.equal(param.detach().float().cpu(), state[name].to(torch.bfloat16).float().cpu()), name


def test_staged_parameters_match_resident_replicas():
    """full_shard residency with a world of one: five blocks pass through two staging slots in forward and backward; the
    gathers, the re-pointed parameters and the shard-only AdamW push must reproduce the run that keeps a full replica."""

    from mini_train_sys_b200.ops.native_backend import check_kernel_status
    from mini_train_sys_b200.parallel.comm import PeerCollectives

    dev = torch.device(DEV, 0)
    eng_a, loss_a, norm_a = _train(PeerCollectives(dev, max_units=6), layers=5, stage_single_rank=True)
    eng_b, loss_b, norm_b = _train(PeerCollectives(dev, max_units=6), layers=5)
    assert eng_a.staged and not eng_b.staged and all(u.gathered is None for u in eng_a.units)
    assert loss_a == pytest.approx(loss_b, abs=2e-2)
    assert norm_a == pytest.approx(norm_b, rel=5e-2)
    assert loss_a[0] == pytest.approx(loss_b[0], abs=1e-4)          # before any update the two runs compute the same thing
    sizes = eng_a.parameter_bytes()
    assert sizes["resident"] == sum(14 * u.shard_numel for u in eng_a.units) and sizes["staging"] > 0
    check_kernel_status()


def test_a_wait_that_runs_out_blocks_the_update_and_is_reported():
    """A peer flag that never arrives: the wait gives up, the status word is set, the AdamW launch of that step leaves the
    weights and both moments bit-identical, and the engine's status check raises.  The word is cleared afterwards."""

    from mini_train_sys_b200.ops.native_backend import ext
    from mini_train_sys_b200.parallel.comm import PeerCollectives

    dev = torch.device(DEV, 0)
    eng, _, _ = _train(PeerCollectives(dev, max_units=3), steps=1)
    opt = eng._test_optimizer
    tr = eng._test_trainer
    before = [(u.master.clone(), u.exp_avg.clone(), u.exp_avg_sq.clone()) for u in eng.units]
    flags = torch.zeros(8, dtype=torch.int32, device=DEV)
    ext().comm_wait(flags, 0, 2, 9, 20.0, eng.coll.status)      # waits 20 ms for two peers nobody plays
    t = torch.randint(0, 1000, (4, 129))
    tr.train_step({"input_ids": t[:, :-1], "targets": t[:, 1:]})
    torch.cuda.synchronize()
    for u, (p, m, v) in zip(eng.units, before):
        assert torch.equal(u.master, p) and torch.equal(u.exp_avg, m) and torch.equal(u.exp_avg_sq, v)
    with pytest.raises(RuntimeError, match="status 1"):
        eng.check_status()
    eng.coll.status.zero_()
    tr.train_step({"input_ids": t[:, :-1], "targets": t[:, 1:]})
    torch.cuda.synchronize()
    assert not torch.equal(eng.units[0].master, before[0][0])
    eng.check_status()
    del opt


def test_wait_on_a_flag_nobody_sets_times_out_and_reports():
    from mini_train_sys_b200.ops.native_backend import ext

    e = ext()
    flags = torch.zeros(8, dtype=torch.int32, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    e.comm_wait(flags, 0, 2, 5, 50.0, status)          # waits for epoch 5 from two peers; nothing ever signals
    torch.cuda.synchronize()
    assert int(status[0]) == 1
    flags[:2] = 5                                       # once the epoch is there the same wait passes
    status.zero_()
    e.comm_wait(flags, 0, 2, 5, 50.0, status)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    assert torch.ones(4, device=DEV).sum().item() == 4  # the context is still usable


def test_collective_kernels_world_of_one():
    from mini_train_sys_b200.ops.native_backend import ext

    e = ext()
    n = 4096
    flags = torch.zeros(8, dtype=torch.int32, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    src = torch.randn(n, device=DEV)
    out = torch.empty(n, device=DEV)
    sumsq = torch.zeros(1, device=DEV)
    e.comm_reduce_scatter(out, [src.data_ptr()], 0, 0, 0.5, sumsq, flags, 0, 0, 100.0, status, 16)
    assert torch.allclose(out, src * 0.5)
    assert float(sumsq) == pytest.approx(float((src * 0.5).pow(2).sum()), rel=1e-4)
    low = src.to(torch.bfloat16)
    full = torch.empty(n, dtype=torch.bfloat16, device=DEV)
    e.comm_allgather(full, [low.data_ptr()], n * 2, flags, 0, 0, 100.0, status, 16)
    assert torch.equal(full, low)
    coef, norm = torch.zeros(1, device=DEV), torch.zeros(1, device=DEV)
    slots = torch.zeros(64, device=DEV)
    e.comm_norm_clip(sumsq, [slots.data_ptr()], [flags.data_ptr()], flags, 1, 0, 1, 100.0, 1.0, 1.0, coef, norm, status)
    assert float(norm) == pytest.approx(float(sumsq.sqrt()), rel=1e-5)
    assert float(coef) == pytest.approx(min(1.0, 1.0 / (float(norm) + 1e-6)), rel=1e-5)
    assert int(status[0]) == 0


def test_expert_exchange_kernels_with_one_rank_match_the_local_layer():
    """World of one: every route goes to 'the owner' through the push / pull kernels; results must equal the plain layer."""

    from mini_train_sys_b200.models import ModelConfig, get_ops_backend
    from mini_train_sys_b200.models.blocks import MoEFeedForward
    from mini_train_sys_b200.ops.native_backend import check_kernel_status
    from mini_train_sys_b200.parallel import ep as ep_mod

    cfg = ModelConfig(vocab_size=1000, seq_len=128, n_layers=1, n_heads=4, hidden_size=256, intermediate_size=256, ffn_type="moe",
                      num_experts=4, experts_per_token=2, dropout=0.0)
    ops = get_ops_backend("native")
    got = {}
    for mode in ("plain", "peer"):
        torch.manual_seed(5)
        layer = MoEFeedForward(cfg).to(DEV)
        if mode == "peer":
            class Holder(torch.nn.Module):
                def __init__(self, ffn):
                    super().__init__()
                    self.ffn = ffn
            ep_mod.shard_experts(Holder(layer), 0, 1, ep_mod.ExchangeHolder())
        torch.manual_seed(6)
        x = torch.randn(3, 128, 256, device=DEV, dtype=torch.bfloat16).requires_grad_()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out = layer(x, ops).hidden_states
        g = torch.randn_like(out)
        out.backward(g)
        got[mode] = [t.float().clone() for t in (out.detach(), x.grad, layer.gate_up_proj.grad, layer.down_proj.grad, layer.router.weight.grad)]
    for name, a, b in zip(("out", "dx", "d_gate_up", "d_down", "d_router"), got["peer"], got["plain"]):
        err = float((a - b).abs().max()) / max(float(b.abs().max()), 1e-6)
        assert err < 3e-2, (name, err)
    check_kernel_status()


def _run_steps(cuda_graph: bool, steps: int, dropout: float = 0.0, same_batch: bool = False, layers: int = 3, **engine_kwargs):
    from mini_train_sys_b200.models import MiniTransformer, ModelConfig, get_ops_backend
    from mini_train_sys_b200.parallel.comm import PeerCollectives
    from mini_train_sys_b200.parallel.flat_engine import FlatDataParallel
    from mini_train_sys_b200.runtime.config import LRSchedulerConfig, OptimizerConfig
    from mini_train_sys_b200.train.lr_scheduler import LearningRateScheduler
    from mini_train_sys_b200.train.optim import build_optimizer
    from mini_train_sys_b200.train.trainer import Trainer

    cfg = ModelConfig(vocab_size=1000, seq_len=128, n_layers=layers, n_heads=4, hidden_size=256, intermediate_size=256, ffn_type="moe",
                      num_experts=4, experts_per_token=2, tie_word_embeddings=True, dropout=dropout)
    torch.manual_seed(0)
    model = MiniTransformer(cfg, get_ops_backend("native"), activation_dtype=torch.bfloat16).to(DEV)
    eng = FlatDataParallel(model, mode="shard", collectives=PeerCollectives(torch.device(DEV, 0), max_units=layers + 1), **engine_kwargs)
    opt = build_optimizer(eng, cfg=OptimizerConfig(lr=2e-3))
    sched = LearningRateScheduler(opt, LRSchedulerConfig(schedule="cosine", warmup_steps=4, min_lr_ratio=0.1), total_steps=20)
    tr = Trainer(eng, opt, torch.device(DEV), use_fused_loss=True, precision="bf16", grad_clip_norm=1.0, lr_scheduler=sched,
                 cuda_graph=cuda_graph, graph_warmup_steps=3)
    g = torch.Generator().manual_seed(9)
    first = torch.randint(0, 1000, (4, 129), generator=g)
    losses, lrs = [], []
    for _ in range(steps):
        t = first if same_batch else torch.randint(0, 1000, (4, 129), generator=g)
        losses.append(float(tr.train_step({"input_ids": t[:, :-1], "targets": t[:, 1:]})))
        lrs.append(tr.last_lr)
    torch.cuda.synchronize()
    eng.check_status()
    return eng, tr, losses, lrs


@pytest.mark.parametrize("staged", [False, True])
def test_replayed_step_graph_follows_the_eager_run(staged):
    """Three eager steps, then the captured step is replayed: new batches, the warm-up / cosine learning rate, the AdamW bias
    corrections and the flag sequence numbers all have to advance although nothing about them is baked into the graph."""

    from mini_train_sys_b200.ops.native_backend import ext

    kwargs = {"stage_single_rank": True} if staged else {}
    try:
        eng_g, tr_g, loss_g, lr_g = _run_steps(True, 9, **kwargs)
        assert tr_g._graph is not None and eng_g.step_count == 9 and eng_g.comm_epoch == 9
    finally:
        ext().set_step_context(0, 0, 0, False, 0.0, 0.0, 1.0, 1.0)       # neutral again for whatever runs next
        torch.cuda.synchronize()
    eng_e, tr_e, loss_e, lr_e = _run_steps(False, 9, **kwargs)
    assert lr_g == pytest.approx(lr_e) and len(set(lr_g)) > 5
    assert loss_g == pytest.approx(loss_e, abs=3e-2)
    assert loss_g[:3] == pytest.approx(loss_e[:3], abs=2e-3)             # the eager warm-up steps are the same code (atomics aside)
    fa, fb = eng_g.full_state_dict(), eng_e.full_state_dict()
    for name in fa:
        diff = (fa[name] - fb[name]).abs()
        # nine AdamW steps at lr 1e-3: where an atomically summed gradient is near zero the update is sign-like, so two eager
        # runs already sit this far apart (small tensors such as a router weight show it in the mean)
        assert float(diff.max()) <= 2e-2 and float(diff.mean()) < 3e-3, (name, float(diff.max()), float(diff.mean()))


def test_replays_draw_fresh_dropout_masks():
    from mini_train_sys_b200.ops.native_backend import ext

    try:
        _, _, losses, _ = _run_steps(True, 7, dropout=0.3, same_batch=True)
    finally:
        ext().set_step_context(0, 0, 0, False, 0.0, 0.0, 1.0, 1.0)
        torch.cuda.synchronize()
    replayed = losses[3:]
    # the same batch every step: with one baked mask the loss would fall monotonically; fresh masks make it jitter by more
    # than the optimisation moves it, and in any case no two replays may agree to the last digit
    assert len(set(replayed)) == len(replayed)


def test_graph_mode_refuses_what_it_cannot_replay():
    from mini_train_sys_b200.models import MiniTransformer, ModelConfig, get_ops_backend
    from mini_train_sys_b200.train.optim import build_optimizer
    from mini_train_sys_b200.train.trainer import Trainer

    cfg = ModelConfig(vocab_size=512, seq_len=64, n_layers=1, n_heads=2, hidden_size=128, intermediate_size=128)
    model = MiniTransformer(cfg, get_ops_backend("native"), activation_dtype=torch.bfloat16).to(DEV)
    with pytest.raises(ValueError, match="fused sharding engine"):
        Trainer(model, build_optimizer(model), torch.device(DEV), precision="bf16", cuda_graph=True)
