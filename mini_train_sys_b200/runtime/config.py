"""Typed experiment configuration loaded from YAML with ``extends`` composition.

The schema (section names, keys, defaults, validation messages) follows
minitrain/runtime/config.py:7-367 so reference run files load unchanged.  Additions,
all optional: ``backend.ops`` accepts ``native``/``reference``; ``parallel.strategy``
accepts ``ep``; ``parallel.comm`` configures the fused-collective engine and
``parallel.ep`` the expert-parallel strategy.
"""

from __future__ import annotations

from dataclasses import dataclass, field, fields
from pathlib import Path
from typing import Any

from mini_train_sys_b200.models.ops import OPS_BACKEND_NAMES


def _require(condition: bool, message: str) -> None:
    if not condition:
        raise ValueError(message)


def _positive_or_none(value, message: str) -> None:
    _require(value is None or value > 0, message)


@dataclass(frozen=True)
class RunConfig:
    name: str = "debug"
    seed: int = 1337

    def __post_init__(self) -> None:
        _require(bool(self.name.strip()), "run.name must not be empty")


@dataclass(frozen=True)
class BackendConfig:
    ops: str = "torch"

    def __post_init__(self) -> None:
        _require(self.ops in OPS_BACKEND_NAMES, "backend.ops must be one of: " + ", ".join(OPS_BACKEND_NAMES))


@dataclass(frozen=True)
class DDPConfig:
    broadcast_buffers: bool = False
    bucket_cap_mb: int = 25
    find_unused_parameters: bool = False
    gradient_as_bucket_view: bool = True
    static_graph: bool = False

    def __post_init__(self) -> None:
        _require(self.bucket_cap_mb > 0, "parallel.ddp.bucket_cap_mb must be positive")


@dataclass(frozen=True)
class FSDPConfig:
    sharding_strategy: str = "full_shard"
    auto_wrap_policy: str = "transformer_block"
    backward_prefetch: str = "backward_pre"
    forward_prefetch: bool = False
    limit_all_gathers: bool = True
    use_orig_params: bool = True
    sync_module_states: bool = True
    cpu_offload: bool = False
    activation_checkpointing: bool = False

    def __post_init__(self) -> None:
        _require(self.sharding_strategy in ("full_shard", "shard_grad_op"),
                 "parallel.fsdp.sharding_strategy must be 'full_shard' or 'shard_grad_op'")
        _require(self.auto_wrap_policy in ("transformer_block", "none"),
                 "parallel.fsdp.auto_wrap_policy must be 'transformer_block' or 'none'")
        _require(self.backward_prefetch in ("backward_pre", "backward_post", "none"),
                 "parallel.fsdp.backward_prefetch must be backward_pre, backward_post, or none")


@dataclass(frozen=True)
class CommConfig:
    """Fused-collective engine.

    ``engine``: ``fused`` = own peer-memory kernels (all-gather, reduce-scatter/all-reduce
    fused with the AdamW update, expert all-to-all); ``nccl`` = stock torch DDP/FSDP (the
    baseline); ``auto`` = fused on CUDA with >1 rank and peer access, else nccl/gloo.
    ``wait_timeout_ms`` bounds every device-side wait on a peer flag; a wait that runs out sets the device's
    status word, the optimizer kernel then leaves the weights untouched and the runner raises at its next
    log or checkpoint boundary.  The default leaves room for a peer that logs, checkpoints or collects garbage.
    ``prefetch_units``: under ``full_shard``, how many units ahead of the running one are gathered (0 or 1).
    """

    engine: str = "auto"
    wait_timeout_ms: int = 20000
    prefetch_units: int = 1
    use_multimem: bool = False
    health_check: bool = False            # host-side heartbeats through the process-group store, checked before every step
    health_max_age_seconds: float = 300.0

    def __post_init__(self) -> None:
        _require(self.engine in ("auto", "fused", "nccl"), "parallel.comm.engine must be auto, fused, or nccl")
        _require(self.wait_timeout_ms > 0, "parallel.comm.wait_timeout_ms must be positive")
        _require(self.prefetch_units in (0, 1), "parallel.comm.prefetch_units must be 0 or 1")
        _require(self.health_max_age_seconds > 0, "parallel.comm.health_max_age_seconds must be positive")


@dataclass(frozen=True)
class EPConfig:
    """Expert parallelism: experts sharded ``E / world`` per rank, dense parts data parallel."""

    capacity_factor: float | None = None
    min_capacity: int = 4

    def __post_init__(self) -> None:
        _positive_or_none(self.capacity_factor, "parallel.ep.capacity_factor must be positive or null")
        _require(self.min_capacity > 0, "parallel.ep.min_capacity must be positive")


@dataclass(frozen=True)
class ParallelConfig:
    strategy: str = "single"
    process_group_backend: str = "auto"
    timeout_minutes: int = 30
    expected_world_size: int | None = None
    ddp: DDPConfig = field(default_factory=DDPConfig)
    fsdp: FSDPConfig = field(default_factory=FSDPConfig)
    comm: CommConfig = field(default_factory=CommConfig)
    ep: EPConfig = field(default_factory=EPConfig)

    def __post_init__(self) -> None:
        _require(self.strategy in ("single", "ddp", "fsdp", "ep"),
                 "parallel.strategy must be one of: single, ddp, fsdp, ep")
        _require(self.process_group_backend in ("auto", "nccl", "gloo"),
                 "parallel.process_group_backend must be auto, nccl, or gloo")
        _require(self.timeout_minutes > 0, "parallel.timeout_minutes must be positive")
        _positive_or_none(self.expected_world_size, "parallel.expected_world_size must be positive or null")


@dataclass(frozen=True)
class OptimizerConfig:
    name: str = "adamw"
    lr: float = 3e-4
    weight_decay: float = 0.1
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    fused: bool | None = None

    def __post_init__(self) -> None:
        _require(self.name == "adamw", "optimizer.name must be 'adamw'")
        _require(self.lr > 0 and self.eps > 0 and self.weight_decay >= 0,
                 "optimizer lr/eps must be positive and weight_decay non-negative")
        _require(0 <= self.beta1 < 1 and 0 <= self.beta2 < 1, "optimizer betas must be in [0, 1)")


@dataclass(frozen=True)
class LRSchedulerConfig:
    schedule: str = "cosine"
    warmup_steps: int = 100
    decay_steps: int | None = None
    min_lr_ratio: float = 0.1

    def __post_init__(self) -> None:
        _require(self.schedule in ("constant", "cosine"), "lr_scheduler.schedule must be 'constant' or 'cosine'")
        _require(self.warmup_steps >= 0, "lr_scheduler.warmup_steps must be non-negative")
        _positive_or_none(self.decay_steps, "lr_scheduler.decay_steps must be positive or null")
        if self.schedule == "cosine" and self.decay_steps is not None:
            _require(self.decay_steps > self.warmup_steps, "cosine decay_steps must be greater than warmup_steps")
        _require(0 <= self.min_lr_ratio <= 1, "lr_scheduler.min_lr_ratio must be in [0, 1]")


@dataclass(frozen=True)
class TrainConfig:
    batch_size: int = 8
    max_steps: int | None = 1000
    epochs: int | None = None
    log_interval: int = 10
    use_fused_loss: bool = False
    precision: str = "auto"
    grad_clip_norm: float | None = 5.0
    check_finite: bool = True
    reference_global_batch_size: int | None = None
    batch_size_scaling: str = "none"
    cuda_graph: bool = False       # replay the device part of a step from one CUDA graph (fused sharding engine, fixed batch shape)

    def __post_init__(self) -> None:
        _require(self.batch_size > 0 and self.log_interval > 0,
                 "train.batch_size and train.log_interval must be positive")
        _require(self.precision in ("auto", "fp32", "bf16", "fp16"),
                 "train.precision must be one of: auto, fp32, bf16, fp16")
        _positive_or_none(self.grad_clip_norm, "train.grad_clip_norm must be positive or null")
        _positive_or_none(self.reference_global_batch_size, "train.reference_global_batch_size must be positive or null")
        _require(self.batch_size_scaling in ("none", "linear"), "train.batch_size_scaling must be 'none' or 'linear'")
        _require(self.batch_size_scaling == "none" or self.reference_global_batch_size is not None,
                 "linear batch scaling requires train.reference_global_batch_size")
        _positive_or_none(self.max_steps, "train.max_steps must be positive or null")
        _positive_or_none(self.epochs, "train.epochs must be positive or null")
        _require(self.max_steps is not None or self.epochs is not None,
                 "train.max_steps and train.epochs cannot both be null")


@dataclass(frozen=True)
class CheckpointConfig:
    directory: str = "checkpoints"
    every_epochs: int | None = 1
    every_steps: int | None = None       # also save inside an epoch; such a checkpoint resumes behind the batches it saw
    keep_last: int | None = None
    keep_safety: int = 0
    safety_every_epochs: int | None = None
    keep_model_exports: int | None = None
    save_final: bool = False
    resume_from: str | None = None
    export_model: bool = False
    export_model_every_epochs: int | None = None
    cpu_offload: bool = True

    def __post_init__(self) -> None:
        _positive_or_none(self.every_epochs, "checkpoint.every_epochs must be positive or null")
        _positive_or_none(self.every_steps, "checkpoint.every_steps must be positive or null")
        _positive_or_none(self.keep_last, "checkpoint.keep_last must be positive or null")
        _require(self.keep_safety >= 0, "checkpoint.keep_safety must be non-negative")
        if self.keep_safety:
            _require(self.keep_last is not None, "checkpoint.keep_safety requires checkpoint.keep_last")
            _require(self.safety_every_epochs is not None and self.safety_every_epochs > 0,
                     "checkpoint.safety_every_epochs must be positive when keep_safety is enabled")
        _positive_or_none(self.keep_model_exports, "checkpoint.keep_model_exports must be positive or null")
        _positive_or_none(self.export_model_every_epochs, "checkpoint.export_model_every_epochs must be positive or null")
        _require(self.export_model_every_epochs is None or self.export_model,
                 "checkpoint.export_model_every_epochs requires checkpoint.export_model=true")
        _require(bool(self.directory.strip()), "checkpoint.directory must not be empty")


@dataclass(frozen=True)
class DataConfig:
    source: str = "random"
    path: str | None = None
    num_tokens: int = 100_000
    shuffle: bool = True
    packing: str = "contiguous"
    tokenizer_fingerprint: str | None = None
    shuffle_window: int = 1024
    max_open_shards: int = 8
    num_workers: int | None = None       # None = derive from the host's core budget; 0 = synchronous
    worker_budget: int | None = 32
    max_workers_per_rank: int = 4
    worker_cpu_affinity: bool = True
    prefetch_factor: int = 2
    pin_memory: bool = True
    persistent_workers: bool = True
    drop_last: bool = True
    device_prefetch: bool = False        # copy the next batch to the device on a side stream while the current step runs

    def __post_init__(self) -> None:
        _require(self.source in ("random", "tokens", "token_shards"),
                 "data.source must be 'random', 'tokens', or 'token_shards'")
        _require(self.source == "random" or bool(self.path), f"data.path is required when data.source={self.source!r}")
        _require(self.packing in ("contiguous", "randomized_documents"),
                 "data.packing must be 'contiguous' or 'randomized_documents'")
        _require(self.packing == "contiguous" or self.source == "token_shards",
                 "data.packing='randomized_documents' requires data.source='token_shards'")
        _require(self.num_tokens > 0, "data.num_tokens must be positive")
        _require(self.shuffle_window > 0, "data.shuffle_window must be positive")
        _require(self.max_open_shards > 0, "data.max_open_shards must be positive")
        _require(self.num_workers is None or self.num_workers >= 0, "data.num_workers must be non-negative or null")
        _positive_or_none(self.worker_budget, "data.worker_budget must be positive or null")
        _require(self.max_workers_per_rank > 0, "data.max_workers_per_rank must be positive")
        _require(self.prefetch_factor > 0, "data.prefetch_factor must be positive")
        _require(not (self.persistent_workers and self.num_workers == 0),
                 "data.persistent_workers requires data.num_workers > 0")


@dataclass(frozen=True)
class LoggingConfig:
    console: bool = True
    tensorboard: bool = True
    jsonl: bool = True
    log_dir: str = "runs"
    flush_secs: int = 10

    def __post_init__(self) -> None:
        _require(self.flush_secs > 0, "logging.flush_secs must be positive")


@dataclass(frozen=True)
class ExperimentConfig:
    run: RunConfig = field(default_factory=RunConfig)
    backend: BackendConfig = field(default_factory=BackendConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    optimizer: OptimizerConfig = field(default_factory=OptimizerConfig)
    lr_scheduler: LRSchedulerConfig = field(default_factory=LRSchedulerConfig)
    train: TrainConfig = field(default_factory=TrainConfig)
    checkpoint: CheckpointConfig = field(default_factory=CheckpointConfig)
    data: DataConfig = field(default_factory=DataConfig)
    logging: LoggingConfig = field(default_factory=LoggingConfig)
    model: dict[str, Any] = field(default_factory=dict)


def deep_merge(base: dict[str, Any], override: dict[str, Any]) -> dict[str, Any]:
    """Recursive mapping merge; ``override`` wins, neither input is modified."""

    out = dict(base)
    for key, value in override.items():
        if isinstance(value, dict) and isinstance(out.get(key), dict):
            out[key] = deep_merge(out[key], value)
        else:
            out[key] = value
    return out


def load_yaml_dict(path: str | Path, *, _stack: tuple[Path, ...] = ()) -> dict[str, Any]:
    """Load a YAML mapping, first merging its ``extends`` parents (paths relative to the file)."""

    import yaml

    path = Path(path).resolve()
    if path in _stack:
        raise ValueError("Configuration extends cycle: " + " -> ".join(str(p) for p in (*_stack, path)))
    payload = yaml.safe_load(path.read_text(encoding="utf-8")) or {}
    if not isinstance(payload, dict):
        raise ValueError(f"Expected mapping config at {path}")
    parents = payload.pop("extends", [])
    if isinstance(parents, str):
        parents = [parents]
    if not (isinstance(parents, list) and all(isinstance(p, str) for p in parents)):
        raise ValueError(f"extends must be a path or list of paths in {path}")
    merged: dict[str, Any] = {}
    for parent in parents:
        merged = deep_merge(merged, load_yaml_dict(path.parent / parent, _stack=(*_stack, path)))
    return deep_merge(merged, payload)


def _section(cls, payload: dict[str, Any] | None):
    return cls(**(payload or {}))


def experiment_config_from_dict(payload: dict[str, Any]) -> ExperimentConfig:
    par = dict(payload.get("parallel") or {})
    nested = {name: _section(cls, par.pop(name, None))
              for name, cls in (("ddp", DDPConfig), ("fsdp", FSDPConfig), ("comm", CommConfig), ("ep", EPConfig))}
    return ExperimentConfig(
        run=_section(RunConfig, payload.get("run")),
        backend=_section(BackendConfig, payload.get("backend")),
        parallel=ParallelConfig(**par, **nested),
        optimizer=_section(OptimizerConfig, payload.get("optimizer")),
        lr_scheduler=_section(LRSchedulerConfig, payload.get("lr_scheduler")),
        train=_section(TrainConfig, payload.get("train")),
        checkpoint=_section(CheckpointConfig, payload.get("checkpoint")),
        data=_section(DataConfig, payload.get("data")),
        logging=_section(LoggingConfig, payload.get("logging")),
        model=dict(payload.get("model") or {}),
    )


def load_experiment(config_path: str | Path, model_config_path: str | Path | None = None) -> ExperimentConfig:
    """Run YAML + model YAML -> ``ExperimentConfig`` (the model section comes from the model file)."""

    payload = load_yaml_dict(config_path)
    if model_config_path is not None:
        payload["model"] = load_yaml_dict(model_config_path).get("model", {})
    return experiment_config_from_dict(payload)


def section_field_names(cls) -> tuple[str, ...]:
    return tuple(f.name for f in fields(cls))
