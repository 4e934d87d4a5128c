"""Headline benchmark: training throughput (tokens/s) of the 293.49M-parameter top-2 MoE decoder.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        bench.py --gpus 8 --steps 10 --warmup 3

Model / run settings are those of ``configs/synbios_moe/model.yaml`` and ``configs/synbios_moe/base.yaml``
(12 layers, d_model 768, 8 experts top-2, vocab 50257, seq 512, dropout 0.1, tied embeddings, AdamW 1e-3,
grad clip 5.0, fused loss, bf16 autocast) with synthetic uniform-random tokens and random-init weights.
Per-GPU work is fixed (weak scaling): ``--local-batch`` sequences of 512 tokens per rank per step.

Two measurements are taken, each over exactly ``--steps`` optimizer steps after ``--warmup`` untimed ones,
bracketed by barrier + synchronize, timed with CUDA events, max over ranks:
  value      inputs already resident on the device,
  e2e.value  every step copies its batch from pinned host memory and reads the loss back to the host.
``--impl reference`` runs the unmodified reference package from ``baseline/_ref`` (its own model, torch ops
backend, Trainer and stock FSDP) on the same configuration.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
PUBLISHED_TOKENS_PER_SEC = 352_544.0   # published by the reference: CUDA backend, 4x RTX 4090, local batch 96 (README.md:70 of the reference)


def parse_args() -> argparse.Namespace:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["own", "reference"], default="own")
    ap.add_argument("--local-batch", type=int, default=96)
    ap.add_argument("--ops", default="native")
    ap.add_argument("--ref-ops", default="torch", choices=["torch", "triton", "cuda"],
                    help="backend.ops of the reference arm (its documented oracle is torch; triton / cuda are its own kernels)")
    ap.add_argument("--strategy", default=None, help="single | ddp | fsdp | ep (default: fsdp when gpus > 1)")
    ap.add_argument("--engine", default="auto", help="parallel.comm.engine for the own arm")
    ap.add_argument("--model-config", default=str(ROOT / "configs" / "synbios_moe" / "model.yaml"))
    ap.add_argument("--sharding", default="full_shard", choices=["full_shard", "shard_grad_op"],
                    help="parallel.fsdp.sharding_strategy (own arm, fused engine: staged parameters vs resident replica)")
    ap.add_argument("--multimem", action="store_true", help="parallel.comm.use_multimem: gradient sums inside the switch (NVLS)")
    ap.add_argument("--capacity-factor", type=float, default=None, help="parallel.ep.capacity_factor (strategy ep); default: no limit")
    ap.add_argument("--seq-len", type=int, default=None, help="override the model's sequence length")
    ap.add_argument("--cuda-graph", action=argparse.BooleanOptionalAction, default=True,
                    help="own arm: replay the device part of every step from one CUDA graph (train.cuda_graph); ignored where the "
                         "trainer cannot replay (expert parallelism, library engines) and with --comm-timing")
    ap.add_argument("--comm-timing", action="store_true",
                    help="own arm: report, per step, how long the compute stream waited in each communication phase")
    return ap.parse_args()


class ClockSampler(threading.Thread):
    """Reads SM clock and throttle reasons every 200 ms through NVML (queries only)."""

    BAD = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown"}
    NOTED = {0x4: "sw_power_cap"}

    def __init__(self, device_index: int) -> None:
        super().__init__(daemon=True)
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = 0
        self._halt = threading.Event()
        self._handle = None
        try:
            import pynvml

            pynvml.nvmlInit()
            import torch

            want = str(torch.cuda.get_device_properties(device_index).uuid).lower().replace("gpu-", "")
            for i in range(pynvml.nvmlDeviceGetCount()):
                h = pynvml.nvmlDeviceGetHandleByIndex(i)
                uuid = pynvml.nvmlDeviceGetUUID(h)
                uuid = uuid.decode() if isinstance(uuid, bytes) else uuid
                if uuid.lower().replace("gpu-", "") == want:
                    self._handle = h
                    break
            self._nvml = pynvml
            if self._handle is not None:
                self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._handle = None

    def run(self) -> None:
        if self._handle is None:
            return
        nv = self._nvml
        while not self._halt.wait(0.2):
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
                for bit, name in {**self.BAD, **self.NOTED}.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass

    def stop(self) -> dict:
        self._halt.set()
        if self.is_alive():
            self.join(timeout=2)
        med = sorted(self.samples)[len(self.samples) // 2] if self.samples else 0
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def run_payload(args, strategy: str) -> dict:
    """The run configuration both arms share (reference schema)."""

    import yaml

    model = yaml.safe_load(Path(args.model_config).read_text())["model"]
    if getattr(args, "seq_len", None):
        model["seq_len"] = int(args.seq_len)
    return {
        "run": {"name": "bench", "seed": 1337},
        "backend": {"ops": args.ops if args.impl == "own" else args.ref_ops},
        "parallel": {"strategy": strategy, "process_group_backend": "nccl" if strategy != "single" else "auto"},
        "optimizer": {"name": "adamw", "lr": 1e-3, "weight_decay": 0.1, "beta1": 0.9, "beta2": 0.95, "eps": 1e-6},
        "lr_scheduler": {"schedule": "cosine", "warmup_steps": 1000, "min_lr_ratio": 0.1},
        "train": {"batch_size": args.local_batch, "max_steps": 100000, "use_fused_loss": True, "precision": "bf16",
                  "grad_clip_norm": 5.0, "log_interval": 1000},
        "checkpoint": {"every_epochs": None},
        "data": {"source": "random", "num_tokens": args.local_batch * model["seq_len"] * 8 + 1, "num_workers": 0,
                 "persistent_workers": False, "pin_memory": True},
        "logging": {"console": False, "tensorboard": False, "jsonl": False},
        "model": model,
    }


def assemble(args, strategy_name: str):
    """Build model, optimizer and Trainer through the arm's own public API."""

    import torch

    payload = run_payload(args, strategy_name)
    if args.impl == "reference":
        sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
        from minitrain.runtime.config import experiment_config_from_dict
        from minitrain.runtime.factory import build_model, build_ops_backend, build_parallel_strategy
        from minitrain.train.lr_scheduler import LearningRateScheduler
        from minitrain.train.optim import build_optimizer
        from minitrain.train.precision import resolve_precision_policy
        from minitrain.train.trainer import Trainer
        from minitrain.utils.seed import seed_everything
        launches = lambda: 0  # noqa: E731
    else:
        from mini_train_sys_b200.runtime.config import experiment_config_from_dict
        from mini_train_sys_b200.runtime.factory import build_model, build_ops_backend, build_parallel_strategy
        from mini_train_sys_b200.train.lr_scheduler import LearningRateScheduler
        from mini_train_sys_b200.train.optim import build_optimizer
        from mini_train_sys_b200.train.precision import resolve_precision_policy
        from mini_train_sys_b200.train.trainer import Trainer
        from mini_train_sys_b200.utils.seed import seed_everything
        payload["parallel"]["comm"] = {"engine": args.engine, "use_multimem": bool(getattr(args, "multimem", False))}
        payload["parallel"]["fsdp"] = {"sharding_strategy": getattr(args, "sharding", "full_shard")}
        if getattr(args, "capacity_factor", None) is not None:
            payload["parallel"]["ep"] = {"capacity_factor": float(args.capacity_factor)}

        def launches() -> int:
            from mini_train_sys_b200.ops.build import load_extension

            return int(load_extension().launch_count())

    cfg = experiment_config_from_dict(payload)
    seed_everything(cfg.run.seed)
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    precision = resolve_precision_policy(cfg.train.precision, device)
    ops = build_ops_backend(cfg.backend)
    model = build_model(cfg.model, ops, activation_dtype=precision.activation_dtype).to(device)
    strategy = build_parallel_strategy(cfg, resolved_precision=precision.name)
    strategy.setup()
    model = strategy.wrap_model(model)
    optimizer = build_optimizer(model, cfg=cfg.optimizer)
    scheduler = LearningRateScheduler(optimizer, cfg.lr_scheduler, total_steps=100000)
    trainer = Trainer(model, optimizer, device=device, use_fused_loss=True, precision=precision.name,
                      grad_clip_norm=cfg.train.grad_clip_norm, check_finite=True, lr_scheduler=scheduler)
    want_graph = args.impl == "own" and getattr(args, "cuda_graph", False) and not getattr(args, "comm_timing", False)
    if want_graph and trainer._graph_unsupported_reason() is None:
        trainer.cuda_graph = True
    return cfg, trainer, strategy, device, ops, launches


def main() -> None:
    args = parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if args.impl == "reference" and not (ROOT / "baseline" / "_ref" / "minitrain").is_dir():
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is missing: install the reference first"}))
        return
    if args.impl == "reference" and args.strategy not in (None, "single", "ddp", "fsdp"):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"the reference has no {args.strategy!r} strategy (single, ddp, fsdp only)"}))
        return
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29517")

    import torch
    import torch.distributed as dist

    strategy_name = args.strategy or ("fsdp" if world > 1 else "single")
    if args.impl == "reference" and args.ref_ops != "torch":
        # the reference's own kernels are compiled on first use; a backend that cannot be built here is reported, not replaced
        try:
            cfg, trainer, strategy, device, ops, launches = assemble(args, strategy_name)
            probe = torch.randint(0, int(cfg.model["vocab_size"]), (2, int(cfg.model["seq_len"]) + 1))
            trainer.train_step({"input_ids": probe[:, :-1], "targets": probe[:, 1:]})
            torch.cuda.synchronize(device)
        except Exception as exc:  # noqa: BLE001 - any build or launch error of the foreign backend ends the arm
            if rank == 0:
                why = f"{type(exc).__name__}: {exc}".splitlines()[0][:300]
                print(json.dumps({"impl": "reference", "ref_ops": args.ref_ops, "unavailable": f"reference ops backend {args.ref_ops!r} did not run here: {why}"}))
            return
    else:
        cfg, trainer, strategy, device, ops, launches = assemble(args, strategy_name)
    seq_len, vocab = int(cfg.model["seq_len"]), int(cfg.model["vocab_size"])
    steps, warmup, batch = args.steps, max(args.warmup, 0), args.local_batch

    # Synthetic uniform-random token batches, one per step, in pinned host memory.
    gen = torch.Generator().manual_seed(1234 + rank)
    n_batches = warmup + steps
    host = [torch.randint(0, vocab, (batch, seq_len + 1), generator=gen).pin_memory() for _ in range(n_batches)]
    host_batches = [{"input_ids": t[:, :-1], "targets": t[:, 1:]} for t in host]

    def sync_all() -> None:
        if dist.is_initialized():
            dist.barrier(device_ids=[device.index])
        torch.cuda.synchronize(device)

    def timed(run_step, label: str) -> tuple[float, dict, int, float]:
        for i in range(warmup):
            run_step(i)
        sync_all()
        sampler = ClockSampler(device.index)
        sampler.start()
        count0 = launches() + int(getattr(trainer, "kernel_launches_replayed", 0))
        t_host = time.perf_counter()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        last = None
        for i in range(warmup, warmup + steps):
            last = run_step(i)
        stop.record()
        sync_all()
        wall = time.perf_counter() - t_host
        ms = start.elapsed_time(stop)
        clocks = sampler.stop()
        worst = torch.tensor([ms], dtype=torch.float64, device=device)
        if dist.is_initialized():
            dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        count1 = launches() + int(getattr(trainer, "kernel_launches_replayed", 0))
        return float(worst.item()), clocks, count1 - count0, float(last)

    # (1) device-resident inputs
    dev_batches = [{k: v.to(device) for k, v in b.items()} for b in host_batches]

    def step_device(i: int):
        return trainer.train_step(dev_batches[i])

    # (2) end to end: pinned host -> device every step, loss read back every step
    h2d_bytes = sum(v.numel() * v.element_size() for v in host_batches[0].values())

    def step_e2e(i: int):
        return trainer.train_step(host_batches[i]).item()

    if getattr(trainer, "cuda_graph", False):
        # set-up, not warm-up: the trainer runs its first steps eagerly and captures the step graph on the next one; do that
        # here so that neither the warm-up nor the timed region of either pass contains the capture
        for i in range(trainer.graph_warmup_steps + 1):
            trainer.train_step(dev_batches[i % len(dev_batches)])
        sync_all()

    # The end-to-end pass runs first: whatever still warms up after the warm-up steps (allocator growth, lazily built buffers
    # of a wrapped engine) falls into its warm-up, and the device-resident pass that follows is steady-state for both arms.
    e2e_ms, clocks_e2e, _, last_loss_e2e = timed(step_e2e, "e2e")
    engine_timing = getattr(trainer.model, "enable_timing", None) if args.comm_timing else None
    if engine_timing is not None:
        for i in range(warmup):          # the timed region below starts right after these
            step_device(i)
        sync_all()
        engine_timing(True)
    total_ms, clocks, n_launch, last_loss = timed(step_device, "device")
    comm_ms = trainer.model.timing_summary(steps + warmup) if engine_timing is not None else None

    headline = Path(args.model_config).resolve() == (ROOT / "configs" / "synbios_moe" / "model.yaml").resolve()
    if headline:
        model_label = "synbios_moe 293.49M top-2 MoE (12L, d768, 8 experts, vocab 50257, dropout 0.1, tied)"
    else:
        mc = cfg.model
        model_label = (f"{Path(args.model_config).stem} ({mc.get('n_layers')}L, d{mc.get('hidden_size')}, ffn {mc.get('ffn_type', 'dense')}, "
                       f"vocab {mc.get('vocab_size')}, seq {mc.get('seq_len')})")
    tokens_per_step = batch * seq_len * world
    value = tokens_per_step * steps / (total_ms / 1e3)
    e2e_value = tokens_per_step * steps / (e2e_ms / 1e3)
    peak_mb = torch.cuda.max_memory_allocated(device) / 2**20
    record = {
        "metric": "tokens/sec, 293M MoE FSDP (weak scaling, max over ranks)" if headline else
                  f"tokens/sec, {Path(args.model_config).stem} {strategy_name} (weak scaling, max over ranks)", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": round(total_ms / steps, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(value / PUBLISHED_TOKENS_PER_SEC, 3) if headline else None, "dtype": "bf16",
        "data": "synthetic uniform-random tokens, random-init weights", "impl": args.impl,
        "config": {"model": model_label,
                   "global_batch": batch * world, "local_batch": batch, "seq_len": seq_len,
                   "parallelism": f"{strategy_name}{world}", "ops": getattr(ops, "name", "?"),
                   "comm_engine": getattr(strategy, "resolved_engine", lambda: "n/a")(),
                   "optimizer": "adamw lr1e-3 clip5.0 fused_loss",
                   "l2": "per-step working set (activations + weights, many GB) exceeds the 126 MB L2; no explicit flush",
                   "vs_baseline_denominator": "published 352,544 tok/s (4x RTX 4090, reference CUDA backend, batch 96)"},
        "clocks": clocks,
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms / steps, 3),
                "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4, "clocks": clocks_e2e},
        "gpu_launches": n_launch, "peak_memory_mb": round(peak_mb, 1), "final_loss": round(last_loss_e2e, 4),
    }
    if hasattr(ops, "dispatch_summary"):
        record["dispatch"] = ops.dispatch_summary()
    if comm_ms is not None:
        record["comm_wait_ms_per_step"] = comm_ms        # this rank's compute-stream stalls, events also cover the warm-up steps
    if args.impl == "reference":
        record["config"]["ref_ops"] = args.ref_ops
    if args.impl == "own":
        try:
            # the step's roofline: every operator at the measured peak of the unit that bounds it, no gaps (runtime/step_model.py)
            from mini_train_sys_b200.models.config import ModelConfig
            from mini_train_sys_b200.runtime.step_model import step_roofline

            bound = step_roofline(ModelConfig(**cfg.model), batch)
            record["roofline"] = {"step_bound_ms_sustained": bound["bound_ms_sustained"], "step_bound_ms_burst": bound["bound_ms_burst"],
                                  "fraction_of_sustained_bound": round(bound["bound_ms_sustained"] / (total_ms / steps), 3),
                                  "denominators": bound["peaks"].get("source", "measured")}
        except Exception:  # noqa: BLE001 - commentary on the number; it must never cost the benchmark its line
            pass
        record["config"]["sharding"] = args.sharding if strategy_name == "fsdp" else None
        record["config"]["multimem"] = bool(args.multimem)
        record["config"]["cuda_graph"] = bool(getattr(trainer, "_graph", None) is not None)
        dropped = trainer.last_metrics.get("moe/dropped_route_fraction")
        if dropped is not None:
            record["dropped_route_fraction"] = round(float(dropped), 5)
            record["config"]["capacity_factor"] = args.capacity_factor
        sizes = getattr(trainer.model, "parameter_bytes", None)
        if callable(sizes):
            record["parameter_bytes"] = sizes()
    if args.impl == "own":
        from mini_train_sys_b200.ops.native_backend import check_kernel_status

        if getattr(ops, "name", "") == "native":
            check_kernel_status(device)
    if rank == 0:
        print(json.dumps(record), flush=True)
    strategy.teardown()


if __name__ == "__main__":
    main()
