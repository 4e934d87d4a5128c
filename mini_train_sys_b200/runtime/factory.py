"""Factories that turn config sections into backend, model and strategy objects."""

from __future__ import annotations

import torch

from mini_train_sys_b200.models import MiniTransformer, ModelConfig
from mini_train_sys_b200.models.ops import OpsBackend, get_ops_backend
from mini_train_sys_b200.parallel.strategy import ParallelStrategy
from mini_train_sys_b200.runtime.config import BackendConfig, ExperimentConfig


def build_ops_backend(cfg: BackendConfig) -> OpsBackend:
    return get_ops_backend(cfg.ops)


def build_model(model_payload: dict, ops: OpsBackend, *, activation_dtype: torch.dtype = torch.float32) -> MiniTransformer:
    return MiniTransformer(ModelConfig(**model_payload), ops, activation_dtype=activation_dtype)


def resolve_comm_engine(cfg: ExperimentConfig) -> str:
    """``fused`` only where its kernels can run: CUDA, NCCL-class process group."""

    engine = cfg.parallel.comm.engine
    cuda = torch.cuda.is_available() and cfg.parallel.process_group_backend != "gloo"
    if engine == "auto":
        # Reference YAMLs carry no comm section: the native backend pairs with the fused engine.
        return "fused" if cuda and cfg.backend.ops in ("native", "triton", "cuda") else "nccl"
    if engine == "fused" and not cuda:
        raise RuntimeError("parallel.comm.engine=fused requires CUDA")
    return engine


def build_parallel_strategy(cfg: ExperimentConfig, *, resolved_precision: str | None = None) -> ParallelStrategy:
    name = cfg.parallel.strategy
    common = dict(process_group_backend=cfg.parallel.process_group_backend, timeout_minutes=cfg.parallel.timeout_minutes)
    if name == "single":
        from mini_train_sys_b200.parallel.single import SingleDeviceStrategy

        return SingleDeviceStrategy(engine=resolve_comm_engine(cfg), comm=cfg.parallel.comm)
    engine = resolve_comm_engine(cfg)
    if name == "ddp":
        from mini_train_sys_b200.parallel.ddp import DDPStrategy

        return DDPStrategy(**common, **vars(cfg.parallel.ddp), engine=engine, comm=cfg.parallel.comm)
    if name == "fsdp":
        from mini_train_sys_b200.parallel.fsdp import FSDPStrategy

        precision = resolved_precision or cfg.train.precision
        options = vars(cfg.parallel.fsdp)
        engine = FSDPStrategy.choose_engine(cfg.parallel.comm.engine, engine, cpu_offload=bool(options.get("cpu_offload", False)),
                                            sharding_strategy=str(options.get("sharding_strategy", "full_shard")), precision=precision)
        return FSDPStrategy(**common, **options, precision=precision, engine=engine, comm=cfg.parallel.comm)
    if name == "ep":
        from mini_train_sys_b200.parallel.ep import ExpertParallelStrategy

        return ExpertParallelStrategy(**common, engine=engine, comm=cfg.parallel.comm, ep=cfg.parallel.ep)
    raise ValueError(f"Unknown parallel strategy: {name}")
