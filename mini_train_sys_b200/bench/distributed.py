"""Distributed training benchmark: worker, suites (weak / capacity / backend), presentation and quality gates.

Role of the reference's ``scripts/run_dist_bench.py`` (worker :75-206, inventory :211-239, suite loop with identity
hashing and result reuse :272-484, ``present-backend`` :487-647, ``present-capacity`` :730-977,
``validate-backend`` :980-1061) and ``benchmarks/distributed/workflow.py`` (settings / facade / quality gates
:129-166).  The timing differs on purpose: each step is bracketed by CUDA events on the compute stream, the elapsed
times are max-reduced over ranks, and host wall time is recorded beside them only as a cross-check.
"""

from __future__ import annotations

import hashlib
import json
import os
import signal
import statistics
import subprocess
import sys
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any

PACKAGE_ROOT = Path(__file__).resolve().parents[1]
SOURCE_SUFFIXES = (".py", ".cu", ".cuh", ".cpp", ".h")


def source_fingerprint(extra: tuple[Path, ...] = ()) -> str:
    """sha256 over every source file of the package (and ``extra``): results are reusable only for identical code."""

    digest = hashlib.sha256()
    files = sorted(p for p in PACKAGE_ROOT.rglob("*") if p.suffix in SOURCE_SUFFIXES and "_build" not in p.parts)
    for path in [*files, *extra]:
        digest.update(str(path.name).encode())
        digest.update(path.read_bytes())
    return digest.hexdigest()


def _run(cmd: list[str]) -> str:
    try:
        return subprocess.run(cmd, capture_output=True, text=True, timeout=30).stdout.strip()
    except (OSError, subprocess.SubprocessError):
        return ""


def inventory() -> dict[str, Any]:
    """What the numbers were measured on: GPUs, topology, versions, revision.  Read-only queries."""

    import torch

    from mini_train_sys_b200.runtime.provenance import collect_provenance

    return {
        "provenance": collect_provenance(),
        "gpus": _run(["nvidia-smi", "--query-gpu=index,name,memory.total,clocks.max.sm,power.limit", "--format=csv,noheader"]).splitlines(),
        "topology": _run(["nvidia-smi", "topo", "-m"]),
        "cuda_device_count": torch.cuda.device_count() if torch.cuda.is_available() else 0,
        "nccl": ".".join(map(str, torch.cuda.nccl.version())) if torch.cuda.is_available() else None,
        "source_fingerprint": source_fingerprint(),
    }


def cfg_param_count(model) -> int:
    inner = getattr(model, "module", model)
    cfg = getattr(inner, "cfg", None)
    return cfg.param_count() if cfg is not None and hasattr(cfg, "param_count") else sum(p.numel() for p in model.parameters())


# ---------------------------------------------------------------------------------------------------------
# worker: one (strategy, world, backend, batch) measurement inside torchrun
# ---------------------------------------------------------------------------------------------------------

def worker(config: str, model_config: str | None, *, strategy: str, ops: str, engine: str, batch_size: int, warmup_steps: int,
           measure_steps: int, output: str | None) -> dict[str, Any]:
    import torch
    import torch.distributed as dist

    from mini_train_sys_b200.data.dataloader import build_training_dataloader
    from mini_train_sys_b200.runtime.config import experiment_config_from_dict, load_yaml_dict
    from mini_train_sys_b200.runtime.factory import build_model, build_ops_backend, build_parallel_strategy
    from mini_train_sys_b200.train.lr_scheduler import LearningRateScheduler
    from mini_train_sys_b200.train.optim import build_optimizer
    from mini_train_sys_b200.train.precision import resolve_precision_policy
    from mini_train_sys_b200.train.trainer import Trainer
    from mini_train_sys_b200.utils.seed import seed_everything

    payload = load_yaml_dict(config)
    if model_config:
        payload["model"] = load_yaml_dict(model_config).get("model", load_yaml_dict(model_config))
    payload.setdefault("parallel", {})["strategy"] = strategy
    payload["parallel"]["expected_world_size"] = None
    if not torch.cuda.is_available():           # CPU smoke runs of the harness: Gloo ranks, library collectives
        payload["parallel"]["process_group_backend"] = "gloo"
        payload.setdefault("train", {})["precision"] = "fp32"
        engine = "nccl"
    payload["parallel"].setdefault("comm", {})["engine"] = engine
    payload.setdefault("backend", {})["ops"] = ops
    payload.setdefault("train", {})["batch_size"] = batch_size
    payload.setdefault("logging", {}).update(console=False, tensorboard=False, jsonl=False)
    data = payload.setdefault("data", {})
    seq_len = int(payload["model"]["seq_len"])
    if data.get("source", "random") == "random":
        data["source"] = "random"
        data["num_tokens"] = max(int(data.get("num_tokens", 0)), batch_size * seq_len * (warmup_steps + measure_steps + 2) + 1)
    cfg = experiment_config_from_dict(payload)

    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    seed_everything(cfg.run.seed)
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    precision = resolve_precision_policy(cfg.train.precision, device)
    backend = build_ops_backend(cfg.backend)
    model = build_model(cfg.model, backend, activation_dtype=precision.activation_dtype).to(device)
    loader = build_training_dataloader(cfg.data, seq_len=seq_len, batch_size=batch_size, vocab_size=model.cfg.vocab_size, seed=cfg.run.seed)
    strat = build_parallel_strategy(cfg, resolved_precision=precision.name)
    strat.setup()
    model = strat.wrap_model(model)
    optimizer = build_optimizer(model, cfg=cfg.optimizer)
    scheduler = LearningRateScheduler(optimizer, cfg.lr_scheduler, total_steps=10**6)
    trainer = Trainer(model, optimizer, device=device, use_fused_loss=cfg.train.use_fused_loss, precision=precision.name,
                      grad_clip_norm=cfg.train.grad_clip_norm, check_finite=cfg.train.check_finite, lr_scheduler=scheduler,
                          cuda_graph=cfg.train.cuda_graph)

    stream = iter(loader)

    def next_batch():
        nonlocal stream
        try:
            return next(stream)
        except StopIteration:
            stream = iter(loader)
            return next(stream)

    def sync():
        if cuda:
            torch.cuda.synchronize(device)

    for _ in range(max(warmup_steps, 3)):
        trainer.train_step(next_batch())
    sync()
    strat.barrier()
    if cuda:
        torch.cuda.reset_peak_memory_stats(device)
    step_ms, data_ms, wall_ms = [], [], []
    events = []
    for _ in range(measure_steps):
        t0 = time.perf_counter()
        batch = next_batch()
        t1 = time.perf_counter()
        if cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            trainer.train_step(batch)
            b.record()
            events.append((a, b))
            b.synchronize()
        else:
            trainer.train_step(batch)
        t2 = time.perf_counter()
        data_ms.append((t1 - t0) * 1e3)
        wall_ms.append((t2 - t1) * 1e3)
    sync()
    step_ms = [a.elapsed_time(b) for a, b in events] if cuda else list(wall_ms)

    stats = torch.tensor([step_ms, data_ms, wall_ms], dtype=torch.float64, device=device)
    mem = torch.zeros(3, dtype=torch.float64, device=device)
    if cuda:
        mem = torch.tensor([torch.cuda.max_memory_allocated(device), torch.cuda.max_memory_reserved(device),
                            torch.cuda.get_device_properties(device).total_memory], dtype=torch.float64, device=device)
    mem_sum = mem.clone()
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(mem, op=dist.ReduceOp.MAX)
        dist.all_reduce(mem_sum, op=dist.ReduceOp.SUM)
    step, data_wait, wall = (stats[i].tolist() for i in range(3))
    global_tokens = batch_size * seq_len * world
    tps = [global_tokens / (ms / 1e3) for ms in step]
    record = {
        "strategy": strategy, "engine": getattr(strat, "resolved_engine", lambda: "n/a")(), "world_size": world, "ops": ops,
        "batch_size": batch_size, "global_batch": batch_size * world, "seq_len": seq_len, "measure_steps": measure_steps,
        "warmup_steps": max(warmup_steps, 3), "timing": "cuda events per step, max over ranks",
        "tokens_per_sec": statistics.fmean(tps), "tokens_per_sec_per_gpu": statistics.fmean(tps) / world,
        "step_ms_mean": statistics.fmean(step), "step_ms_p50": statistics.median(step), "step_ms_max": max(step),
        "host_step_ms_mean": statistics.fmean(wall), "data_wait_ms_mean": statistics.fmean(data_wait),
        "data_stall_fraction": sum(data_wait) / max(sum(data_wait) + sum(step), 1e-9),
        "peak_allocated_mb_max": float(mem[0]) / 2**20, "peak_reserved_mb_max": float(mem[1]) / 2**20,
        "peak_allocated_mb_sum": float(mem_sum[0]) / 2**20, "device_memory_mb": float(mem[2]) / 2**20,
        "parameters": int(cfg_param_count(model)),
        "final_loss": float(trainer.last_metrics["loss/total"]) if "loss/total" in trainer.last_metrics else None,
    }
    if hasattr(backend, "dispatch_summary"):
        record["dispatch"] = backend.dispatch_summary()
    if rank == 0 and output:
        out = Path(output)
        out.parent.mkdir(parents=True, exist_ok=True)
        tmp = out.with_suffix(".tmp")
        tmp.write_text(json.dumps(record, indent=1))
        os.replace(tmp, out)
    strat.teardown()
    return record


# ---------------------------------------------------------------------------------------------------------
# suite driver
# ---------------------------------------------------------------------------------------------------------

@dataclass
class BenchmarkSettings:
    config: str
    model_config: str | None = None
    output_dir: str = "results/distributed"
    strategies: tuple[str, ...] = ("fsdp",)
    world_sizes: tuple[int, ...] = (1, 2, 4, 8)
    ops_backends: tuple[str, ...] = ("native",)
    engines: tuple[str, ...] = ("fused",)
    batch_sizes: tuple[int, ...] = (96,)
    repeats: int = 2
    warmup_steps: int = 5
    measure_steps: int = 20
    timeout_s: float = 1800.0
    master_port: int = 29541
    reuse_stale_results: bool = False
    reuse_failures: bool = False
    rerun_existing: bool = False                  # measure every case again although a stored result matches
    memory_limit: float = 0.92                    # capacity suite: share of device memory a candidate batch may reserve
    min_repeats: int = 2                          # capacity and backend suites: repeats a row needs to count
    env: dict[str, str] = field(default_factory=dict)


def planned_batch_ladder(config: str, model_config: str | None, *, strategies: tuple[str, ...], world_sizes: tuple[int, ...],
                         device_gib: float = 180.0, headroom: float = 0.9, fractions: tuple[float, ...] = (0.125, 0.25, 0.5, 0.75, 0.9, 1.0)
                         ) -> tuple[int, ...]:
    """Batch sizes for a capacity sweep from the memory plan instead of a guess: fractions of the largest local batch that the
    plan admits for EVERY (strategy, world size) of the sweep, rounded down to multiples of 8 (at least 1), ascending, unique.
    The last rung is the planned maximum itself, so that the sweep brackets the limit from below."""

    from mini_train_sys_b200.models.config import ModelConfig
    from mini_train_sys_b200.runtime.config import load_yaml_dict
    from mini_train_sys_b200.runtime.memory_plan import GIB, plan_memory

    payload = load_yaml_dict(config)
    model_payload = (load_yaml_dict(model_config).get("model") if model_config else None) or payload.get("model")
    if not model_payload:
        raise ValueError("the batch ladder needs a model: give --model-config or a config that embeds `model:`")
    model = ModelConfig(**model_payload)
    sharding = ((payload.get("parallel") or {}).get("fsdp") or {}).get("sharding_strategy", "full_shard")
    sharding = sharding if sharding in ("full_shard", "shard_grad_op") else "full_shard"
    limits = []
    for strategy in strategies:
        for world in world_sizes:
            kind = "single" if world == 1 and strategy != "ep" else strategy
            if kind == "ep" and (not model.is_moe or model.num_experts % world):
                continue
            plan = plan_memory(model, strategy=kind, world_size=world, sharding=sharding, local_batch_hint=64)
            limits.append(plan.max_local_batch(device_gib * GIB, headroom=headroom))
    if not limits or min(limits) < 1:
        raise ValueError("the memory plan admits no batch for this sweep")
    top = min(limits)
    rungs = sorted({max(1, int(top * f) // 8 * 8 if top * f >= 8 else int(top * f)) for f in fractions})
    return tuple(rungs)


def case_identity(settings: BenchmarkSettings, *, strategy: str, world: int, ops: str, engine: str, batch: int, repeat: int,
                  fingerprint: str) -> str:
    from mini_train_sys_b200.runtime.config import load_yaml_dict

    resolved = {"config": load_yaml_dict(settings.config)}
    if settings.model_config:
        resolved["model"] = load_yaml_dict(settings.model_config)
    blob = {"strategy": strategy, "world": world, "ops": ops, "engine": engine, "batch": batch, "repeat": repeat,
            "warmup": settings.warmup_steps, "steps": settings.measure_steps, "fingerprint": fingerprint,
            "env": dict(sorted(settings.env.items())), "resolved": resolved}
    return hashlib.sha256(json.dumps(blob, sort_keys=True, default=str).encode()).hexdigest()


def case_name(strategy: str, world: int, ops: str, engine: str, batch: int, repeat: int) -> str:
    return f"{strategy}-{engine}-w{world}-{ops}-b{batch}-r{repeat}"


def run_case(settings: BenchmarkSettings, script: Path, *, strategy: str, world: int, ops: str, engine: str, batch: int,
             output: Path, log: Path) -> dict[str, Any]:
    """One torchrun in its own session; on timeout the process GROUP it started is terminated, then killed."""

    strat = "single" if world == 1 and strategy in ("ddp", "fsdp") and engine == "nccl" else strategy
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(settings.master_port), str(script), "_worker", "--config", settings.config, "--strategy", strat,
           "--ops", ops, "--engine", engine, "--batch-size", str(batch), "--warmup-steps", str(settings.warmup_steps),
           "--measure-steps", str(settings.measure_steps), "--output", str(output)]
    if settings.model_config:
        cmd += ["--model-config", settings.model_config]
    log.parent.mkdir(parents=True, exist_ok=True)
    env = {**os.environ, **settings.env}
    t0 = time.time()
    with open(log, "w") as fh:
        proc = subprocess.Popen(cmd, stdout=fh, stderr=subprocess.STDOUT, env=env, start_new_session=True)
        try:
            rc = proc.wait(timeout=settings.timeout_s)
            timed_out = False
        except subprocess.TimeoutExpired:
            timed_out = True
            for sig in (signal.SIGTERM, signal.SIGKILL):
                try:
                    os.killpg(proc.pid, sig)      # the exact group created above
                except ProcessLookupError:
                    break
                try:
                    proc.wait(timeout=15)
                    break
                except subprocess.TimeoutExpired:
                    continue
            rc = proc.returncode if proc.returncode is not None else -9
    tail = log.read_text(errors="replace")[-4000:]
    if rc == 0 and output.exists():
        rec = json.loads(output.read_text())
        rec["status"] = "ok"
    else:
        rec = {"status": "failed", "returncode": rc, "timeout": timed_out, "oom": "out of memory" in tail.lower(), "log_tail": tail}
    rec["seconds"] = time.time() - t0
    return rec


def run_suite(settings: BenchmarkSettings, suite: str, script: Path) -> dict[str, Any]:
    """weak: fixed local batch across world sizes; capacity: batch sweep at each world; backend: ops back ends at fixed shape."""

    out_dir = Path(settings.output_dir) / suite
    raw = out_dir / "raw"
    raw.mkdir(parents=True, exist_ok=True)
    (out_dir / "inventory.json").write_text(json.dumps(inventory(), indent=1, default=str))
    fingerprint = source_fingerprint((script,))
    rows = []
    worlds = settings.world_sizes if suite != "backend" else settings.world_sizes[:1]
    batches = settings.batch_sizes if suite == "capacity" else settings.batch_sizes[:1]
    backends = settings.ops_backends if suite == "backend" else settings.ops_backends[:1]
    for strategy in settings.strategies:
        for world in worlds:
            for ops in backends:
                for engine in settings.engines:
                    for batch in batches:
                        for repeat in range(settings.repeats):
                            name = case_name(strategy, world, ops, engine, batch, repeat)
                            ident = case_identity(settings, strategy=strategy, world=world, ops=ops, engine=engine, batch=batch,
                                                  repeat=repeat, fingerprint=fingerprint)
                            path = raw / f"{name}.json"
                            prev = json.loads(path.read_text()) if path.exists() else None
                            reusable = prev is not None and not settings.rerun_existing and \
                                (prev.get("identity") == ident or settings.reuse_stale_results) and \
                                (prev.get("status") == "ok" or settings.reuse_failures)
                            if reusable:
                                rec = prev
                                rec["reused"] = True
                            else:
                                rec = run_case(settings, script, strategy=strategy, world=world, ops=ops, engine=engine, batch=batch,
                                               output=raw / f"{name}.worker.json", log=raw / f"{name}.log")
                                rec.update(name=name, identity=ident, strategy=strategy, world_size=world, ops=ops, engine=engine,
                                           batch_size=batch, repeat=repeat)
                                path.write_text(json.dumps(rec, indent=1))
                            rows.append(rec)
    summary = {"suite": suite, "settings": asdict(settings), "rows": rows}
    if suite == "weak":
        summary["weak"] = weak_scaling_table(rows)
    elif suite == "capacity":
        summary["capacity"] = present_capacity(rows, memory_limit=settings.memory_limit, min_repeats=settings.min_repeats)
    else:
        summary["backend"] = present_backend(rows, min_repeats=settings.min_repeats)
    summary["quality_gates"] = quality_gates(summary, repeats=settings.repeats)
    (out_dir / "summary.json").write_text(json.dumps(summary, indent=1, default=str))
    return summary


# ---------------------------------------------------------------------------------------------------------
# presentation
# ---------------------------------------------------------------------------------------------------------

def _ok(rows):
    return [r for r in rows if r.get("status") == "ok"]


def _group(rows, *keys):
    out: dict[tuple, list] = {}
    for r in rows:
        out.setdefault(tuple(r.get(k) for k in keys), []).append(r)
    return out


def weak_scaling_table(rows: list[dict[str, Any]]) -> list[dict[str, Any]]:
    """efficiency = 100 * throughput / (world * mean single-GPU throughput) per (strategy, engine, ops, batch)."""

    table = []
    for (strategy, engine, ops, batch), group in _group(_ok(rows), "strategy", "engine", "ops", "batch_size").items():
        by_world = _group(group, "world_size")
        base = by_world.get((1,))
        base_mean = statistics.fmean(r["tokens_per_sec"] for r in base) if base else None
        for (world,), reps in sorted(by_world.items()):
            thr = [r["tokens_per_sec"] for r in reps]
            mean = statistics.fmean(thr)
            table.append({
                "strategy": strategy, "engine": engine, "ops": ops, "batch_size": batch, "world_size": world, "repeats": len(reps),
                "tokens_per_sec_mean": mean, "tokens_per_sec_std": statistics.pstdev(thr) if len(thr) > 1 else 0.0,
                "step_ms_mean": statistics.fmean(r["step_ms_mean"] for r in reps),
                "efficiency_pct": 100.0 * mean / (base_mean * world) if base_mean else None,
                "data_stall_fraction": max(r["data_stall_fraction"] for r in reps),
                "memory_fraction": max(r["peak_reserved_mb_max"] / max(r["device_memory_mb"], 1.0) for r in reps),
            })
    return table


def present_capacity(rows: list[dict[str, Any]], *, memory_limit: float = 0.92, min_repeats: int = 2) -> dict[str, Any]:
    """Per (strategy, engine, world, ops): the max-throughput batch with enough repeats under the memory limit;
    activation memory per sample from the slope of peak allocation over batch; largest batch common to all groups."""

    out: dict[str, Any] = {"selected": [], "rejected": []}
    feasible_sets = []
    for (strategy, engine, world, ops), group in _group(rows, "strategy", "engine", "world_size", "ops").items():
        by_batch = _group(_ok(group), "batch_size")
        candidates = []
        for (batch,), reps in sorted(by_batch.items()):
            frac = max(r["peak_reserved_mb_max"] / max(r["device_memory_mb"], 1.0) for r in reps)
            if len(reps) < min_repeats or frac > memory_limit:
                out["rejected"].append({"strategy": strategy, "world_size": world, "ops": ops, "batch_size": batch,
                                        "reason": "repeats" if len(reps) < min_repeats else "memory", "memory_fraction": frac})
                continue
            candidates.append((statistics.fmean(r["tokens_per_sec"] for r in reps), batch, frac,
                               statistics.fmean(r["peak_allocated_mb_max"] for r in reps)))
        if not candidates:
            continue
        feasible_sets.append({c[1] for c in candidates})
        best = max(candidates)
        smallest = min(candidates, key=lambda c: c[1])
        per_sample = (best[3] - smallest[3]) / (best[1] - smallest[1]) if best[1] != smallest[1] else None
        tested = sorted(b for (b,) in _group(group, "batch_size"))
        out["selected"].append({"strategy": strategy, "engine": engine, "world_size": world, "ops": ops, "batch_size": best[1],
                                "tokens_per_sec_mean": best[0], "memory_fraction": best[2],
                                "activation_mb_per_sample": per_sample,
                                "selected_is_largest_tested": best[1] == tested[-1]})
    common = set.intersection(*feasible_sets) if feasible_sets else set()
    out["common_fixed_batch"] = max(common) if common else None
    return out


def present_backend(rows: list[dict[str, Any]], *, min_repeats: int = 2) -> list[dict[str, Any]]:
    """Mean throughput per ops back end; native rows must show native dispatches only (no silent fallback)."""

    table = []
    groups = _group(_ok(rows), "strategy", "engine", "world_size", "ops", "batch_size")
    base = {k[:3] + k[4:]: statistics.fmean(r["tokens_per_sec"] for r in v) for k, v in groups.items() if k[3] == "torch"}
    for key, reps in groups.items():
        strategy, engine, world, ops, batch = key
        mean = statistics.fmean(r["tokens_per_sec"] for r in reps)
        dispatch = reps[-1].get("dispatch") or {}
        fallbacks = sum(v for k, v in dispatch.items() if k.endswith(":fallback"))
        natives = sum(v for k, v in dispatch.items() if k.endswith(":native"))
        torch_mean = base.get(key[:3] + key[4:])
        table.append({"strategy": strategy, "engine": engine, "world_size": world, "ops": ops, "batch_size": batch, "repeats": len(reps),
                      "tokens_per_sec_mean": mean, "speedup_vs_torch": mean / torch_mean if torch_mean else None,
                      "native_dispatches": natives, "fallback_dispatches": fallbacks,
                      "valid": len(reps) >= min_repeats and (ops == "torch" or (natives > 0 and fallbacks == 0))})
    return table


def quality_gates(summary: dict[str, Any], *, repeats: int, min_efficiency: float = 80.0, max_data_stall: float = 0.05,
                  max_memory: float = 0.90) -> dict[str, Any]:
    """Scaling efficiency, data stall, memory head-room and completeness of repeats."""

    rows = summary["rows"]
    gates: dict[str, Any] = {"all_repeats_completed": all(r.get("status") == "ok" for r in rows)}
    weak = summary.get("weak") or []
    if weak:
        eff = [w["efficiency_pct"] for w in weak if w["efficiency_pct"] is not None and w["world_size"] > 1]
        gates["scaling_efficiency_ok"] = bool(eff) and min(eff) >= min_efficiency
        gates["min_efficiency_pct"] = min(eff) if eff else None
        gates["data_stall_ok"] = max(w["data_stall_fraction"] for w in weak) <= max_data_stall
        gates["memory_ok"] = max(w["memory_fraction"] for w in weak) <= max_memory
        gates["repeats_ok"] = all(w["repeats"] >= repeats for w in weak)
    cap = summary.get("capacity")
    if cap:
        gates["selected_batch_not_largest"] = all(not s["selected_is_largest_tested"] for s in cap["selected"])
    backend = summary.get("backend")
    if backend:
        gates["backend_rows_valid"] = all(b["valid"] for b in backend)
    gates["passed"] = all(v for k, v in gates.items() if isinstance(v, bool))
    return gates


def validate_backend(device_index: int = 0, *, batch: int = 2, sequence_length: int = 512) -> dict[str, Any]:
    """Native attention against the library back end (forward, dq, dk, dv), a dropout run, and the dispatch counters."""

    import torch

    from mini_train_sys_b200.models import get_ops_backend

    dev = torch.device("cuda", device_index)
    native, lib = get_ops_backend("native"), get_ops_backend("torch")
    torch.manual_seed(0)
    shape = (batch, 12, sequence_length, 64)
    base = [torch.randn(shape, device=dev, dtype=torch.bfloat16) for _ in range(3)]
    grad = torch.randn(shape, device=dev, dtype=torch.bfloat16)
    results = {}
    outs = {}
    for name, ops in (("native", native), ("torch", lib)):
        q, k, v = (t.clone().requires_grad_() for t in base)
        o = ops.attention(q, k, v, is_causal=True, dropout_p=0.0)
        o.backward(grad)
        outs[name] = (o, q.grad, k.grad, v.grad)
    ok = True
    for label, a, e in zip(("out", "dq", "dk", "dv"), outs["native"], outs["torch"]):
        close = bool(torch.allclose(a.float(), e.float(), atol=5e-2, rtol=5e-2))
        results[label] = {"max_abs": float((a.float() - e.float()).abs().max()), "close": close}
        ok &= close
    q, k, v = (t.clone().requires_grad_() for t in base)
    o = native.attention(q, k, v, is_causal=True, dropout_p=0.1)
    o.backward(grad)
    finite = all(bool(torch.isfinite(t).all()) for t in (o, q.grad, k.grad, v.grad))
    summary = native.dispatch_summary()
    counters_ok = summary.get("attention:native", 0) == 2 and summary.get("attention:fallback", 0) == 0
    return {"attention": results, "dropout_finite": finite, "dispatch": summary, "dispatch_ok": counters_ok,
            "passed": ok and finite and counters_ok}


class DistributedBenchmark:
    """Notebook / script facade: preflight, inventory, the three suites, and loading of a finished summary."""

    def __init__(self, settings: BenchmarkSettings, script: Path) -> None:
        self.settings, self.script = settings, Path(script)

    def preflight(self) -> dict[str, Any]:
        from mini_train_sys_b200.runtime.server_check import collect_server_status

        return collect_server_status(expected_gpus=max(self.settings.world_sizes), min_free_disk_gb=1.0, require_nvcc=False)

    def inventory(self) -> dict[str, Any]:
        return inventory()

    def run_weak(self) -> dict[str, Any]:
        return run_suite(self.settings, "weak", self.script)

    def run_capacity(self) -> dict[str, Any]:
        return run_suite(self.settings, "capacity", self.script)

    def run_backend(self) -> dict[str, Any]:
        return run_suite(self.settings, "backend", self.script)

    def load(self, suite: str) -> dict[str, Any]:
        return json.loads((Path(self.settings.output_dir) / suite / "summary.json").read_text())
