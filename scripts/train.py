"""Training entry point: config -> data/model/strategy -> Trainer -> TrainingRunner.

Flags and emitted events (``init``, ``parallel_ready``, ``resume``, ``train``, ``checkpoint``)
follow the reference entry point (scripts/train.py:57-281); ``memory_plan`` (planned device memory of the configured batch, on a GPU) and
``ops_dispatch`` (native vs fallback calls per operator, at the end of a run with the native back end) are additions.  Launch one process per GPU with
``torchrun --standalone --nproc_per_node N scripts/train.py --config ... --model-config ...``.
"""

from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

from mini_train_sys_b200.data.dataloader import build_training_dataloader  # noqa: E402
from mini_train_sys_b200.runtime.config import load_experiment  # noqa: E402
from mini_train_sys_b200.runtime.device import resolve_device  # noqa: E402
from mini_train_sys_b200.runtime.factory import build_model, build_ops_backend, build_parallel_strategy  # noqa: E402
from mini_train_sys_b200.runtime.logger import build_event_logger, get_run_log_dir  # noqa: E402
from mini_train_sys_b200.runtime.provenance import collect_provenance  # noqa: E402
from mini_train_sys_b200.runtime.scaling import resolve_batch_scale  # noqa: E402
from mini_train_sys_b200.train.checkpoint import resolve_resume_checkpoint, restore_training_checkpoint  # noqa: E402
from mini_train_sys_b200.train.lr_scheduler import LearningRateScheduler, resolve_total_steps  # noqa: E402
from mini_train_sys_b200.train.optim import build_optimizer  # noqa: E402
from mini_train_sys_b200.train.precision import resolve_precision_policy  # noqa: E402
from mini_train_sys_b200.train.runner import TrainingRunner  # noqa: E402
from mini_train_sys_b200.train.trainer import Trainer  # noqa: E402
from mini_train_sys_b200.utils.seed import seed_everything  # noqa: E402


def parse_args(argv=None) -> argparse.Namespace:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--config", required=True)
    ap.add_argument("--model-config", default="configs/model_default.yaml")
    ap.add_argument("--smoke-steps", type=int, default=0)
    ap.add_argument("--device", choices=["auto", "cpu", "cuda"], default="auto")
    ap.add_argument("--resume", nargs="?", const="latest", default=None, metavar="PATH|latest|safety|auto",
                    help="resume from a checkpoint; no value means latest, 'safety' uses the retained fallback anchor, 'auto' is "
                         "latest when the run has a checkpoint and a fresh start when it has none (for launchers that restart)")
    return ap.parse_args(argv)


def init_event(cfg, *, device, ops, strategy, world_size, model, dataloader, scale, precision, run_log_dir) -> dict:
    mc, d = model.cfg, cfg.data
    return {
        "event": "init", "run": cfg.run.name, "device": str(device), "ops": ops.name, "parallel": strategy.name,
        "comm_engine": getattr(strategy, "resolved_engine", lambda: "none")(), "world_size": world_size,
        "params": sum(p.numel() for p in model.parameters()), "ffn_type": mc.ffn_type,
        "data_source": d.source, "data_shuffle": d.shuffle, "data_shuffle_window": d.shuffle_window,
        "data_max_open_shards": d.max_open_shards, "data_packing": d.packing,
        "data_num_workers": dataloader.num_workers, "data_workers_per_node": getattr(dataloader, "worker_budget", 0),
        "data_prefetch_factor": d.prefetch_factor, "data_pin_memory": d.pin_memory,
        "data_persistent_workers": d.persistent_workers, "data_drop_last": d.drop_last,
        "local_batch_size": scale.local_batch_size, "global_batch_size": scale.global_batch_size,
        "reference_global_batch_size": scale.reference_global_batch_size, "batch_size_scale": scale.scale,
        "seq_len": mc.seq_len, "max_steps": cfg.train.max_steps, "epochs": cfg.train.epochs,
        "checkpoint_every_epochs": cfg.checkpoint.every_epochs, "checkpoint_keep_last": cfg.checkpoint.keep_last,
        "checkpoint_export_model_every_epochs": cfg.checkpoint.export_model_every_epochs,
        "precision": precision.name, "activation_dtype": str(precision.activation_dtype),
        "grad_scaler": precision.grad_scaling_enabled, "optimizer": cfg.optimizer.name,
        "reference_learning_rate": cfg.optimizer.lr, "learning_rate": scale.optimizer.lr,
        "lr_schedule": scale.lr_scheduler.schedule, "warmup_steps": scale.lr_scheduler.warmup_steps,
        "run_log_dir": str(run_log_dir) if run_log_dir is not None else "disabled",
        **collect_provenance(ROOT),
    }


def main(argv=None) -> None:
    args = parse_args(argv)
    cfg = load_experiment(args.config, args.model_config)

    seed_everything(cfg.run.seed)          # before the model exists: identical initial weights on every rank
    device = resolve_device(args.device)
    if device.type == "cuda":
        torch.cuda.set_device(device)
    precision = resolve_precision_policy(cfg.train.precision, device)
    ops = build_ops_backend(cfg.backend)
    model = build_model(cfg.model, ops, activation_dtype=precision.activation_dtype).to(device)
    mc = model.cfg
    world_size = int(os.environ.get("WORLD_SIZE", "1"))
    expect = cfg.parallel.expected_world_size
    if expect is not None and expect != world_size:
        raise RuntimeError(f"Config expects WORLD_SIZE={expect}, got {world_size}")
    scale = resolve_batch_scale(cfg.train, cfg.optimizer, cfg.lr_scheduler, world_size=world_size)
    dataloader = build_training_dataloader(cfg.data, seq_len=mc.seq_len, batch_size=cfg.train.batch_size,
                                           vocab_size=mc.vocab_size, seed=cfg.run.seed)
    strategy = build_parallel_strategy(cfg, resolved_precision=precision.name)
    run_log_dir = get_run_log_dir(cfg.logging, run_name=cfg.run.name)
    logger = build_event_logger(cfg.logging, run_name=cfg.run.name, tensorboard_log_dir=run_log_dir)
    logger.log_event(init_event(cfg, device=device, ops=ops, strategy=strategy, world_size=world_size, model=model,
                                dataloader=dataloader, scale=scale, precision=precision, run_log_dir=run_log_dir))
    try:
        strategy.setup()
        model = strategy.wrap_model(model)
        if strategy.name == "fsdp":
            units = strategy.unit_count(model)
            want = mc.n_layers + 1 if cfg.parallel.fsdp.auto_wrap_policy == "transformer_block" else 1
            if units != want:
                raise RuntimeError(f"FSDP wrap verification failed: found {units} units, expected {want}")
            logger.log_event({"event": "parallel_ready", "strategy": "fsdp", "fsdp_units": units,
                              "auto_wrap_policy": cfg.parallel.fsdp.auto_wrap_policy,
                              "sharding_strategy": cfg.parallel.fsdp.sharding_strategy,
                              "engine": strategy.resolved_engine()})
        if device.type == "cuda" and cfg.backend.ops != "torch":
            # what the configured batch will need under the fused engine, before the first step finds out the hard way
            from mini_train_sys_b200.runtime.memory_plan import memory_plan_event

            planned = memory_plan_event(cfg, world_size=world_size, device_bytes=torch.cuda.get_device_properties(device).total_memory)
            if planned is not None:
                logger.log_event(planned)
        max_steps = args.smoke_steps if args.smoke_steps > 0 else cfg.train.max_steps
        total_steps = resolve_total_steps(max_steps=max_steps, epochs=cfg.train.epochs, steps_per_epoch=len(dataloader))
        optimizer = build_optimizer(model, cfg=scale.optimizer)   # after wrapping: sees sharded parameters
        scheduler = LearningRateScheduler(optimizer, scale.lr_scheduler, total_steps=total_steps)
        trainer = Trainer(model, optimizer, device=device, use_fused_loss=cfg.train.use_fused_loss,
                          precision=precision.name, grad_clip_norm=cfg.train.grad_clip_norm,
                          check_finite=cfg.train.check_finite, lr_scheduler=scheduler,
                          cuda_graph=cfg.train.cuda_graph)

        resume = args.resume if args.resume is not None else cfg.checkpoint.resume_from
        resume_path = None
        if resume is not None:
            resume_path = resolve_resume_checkpoint(resume, checkpoint_dir=cfg.checkpoint.directory, run_name=cfg.run.name)
        if resume_path is not None:
            got = restore_training_checkpoint(resume_path, model, optimizer, grad_scaler=trainer.grad_scaler,
                                              lr_scheduler=scheduler, restore_rng=True)
            st = trainer.state
            st.step, st.epoch, st.tokens_seen, st.lr_step = got["step"], got["epoch"], got["tokens_seen"], got["lr_step"]
            st.epoch_batches_done = int(got.get("epoch_batches_done", 0))      # continue inside the interrupted epoch
            if got.get("saved_world_size", world_size) != world_size:
                st.lr_step = st.epoch * len(dataloader)    # re-express schedule progress in the new layout
                st.epoch_batches_done = 0                  # the rank partition changed: the interrupted epoch starts over
            if not got["rng_restored"]:
                seed_everything(cfg.run.seed + strategy.rank + st.step)
            scheduler.step(st.lr_step)
            logger.log_event({"event": "resume", "path": str(resume_path), **got})

        TrainingRunner(cfg=cfg, trainer=trainer, dataloader=dataloader, strategy=strategy, logger=logger,
                       device=device, world_size=world_size).run(max_steps=max_steps, resume_path=resume_path)
        if hasattr(ops, "dispatch_summary"):
            # how often each operator ran natively and how often it fell back to the PyTorch implementation (eager calls;
            # steps replayed from a CUDA graph repeat the captured step's choices)
            logger.log_event({"event": "ops_dispatch", "step": trainer.state.step, "calls": ops.dispatch_summary()})
    finally:
        logger.close()
        strategy.teardown()


if __name__ == "__main__":
    main()
