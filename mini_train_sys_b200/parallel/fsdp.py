"""Sharded data parallelism (ZeRO-3 ``full_shard`` / ZeRO-2 ``shard_grad_op``).

* engine ``nccl`` wraps the model with torch FSDP exactly as the reference configures it
  (minitrain/distributed/fsdp.py:25-160): one unit per ``TransformerBlock`` plus the root,
  bf16 parameters / fp32 reduction, backward prefetch, optional CPU offload and
  non-reentrant activation checkpointing.  This is the measured baseline.
* engine ``fused`` (parallel/flat_engine.py) shards flat fp32 master weights and Adam state per unit and reduces
  gradients with the own reduce-scatter kernel, whose result feeds a sharded AdamW kernel.  ``full_shard`` keeps only
  the rank's bf16 shard resident and pulls each unit from the owners' shards over peer memory into a two-slot staging
  buffer one unit ahead of its use (forward and backward); ``shard_grad_op`` keeps a bf16 replica per rank that the
  AdamW kernel refreshes on every rank by peer stores, so no gather runs during the step.  Options the fused engine
  does not implement (CPU offload, ``no_shard`` / ``hybrid_shard``, fp16 loss scaling) are never ignored: an explicit
  ``engine: fused`` with one of them is refused, ``engine: auto`` selects the ``nccl`` engine, which honours them.
"""

from __future__ import annotations

from functools import partial

import torch

from mini_train_sys_b200.models.blocks import TransformerBlock
from mini_train_sys_b200.parallel.strategy import ProcessGroupMixin

_LOW_PRECISION = {"bf16": torch.bfloat16, "fp16": torch.float16}


def build_auto_wrap_policy(name: str):
    from torch.distributed.fsdp.wrap import ModuleWrapPolicy

    if name == "none":
        return None
    if name == "transformer_block":
        return ModuleWrapPolicy({TransformerBlock})
    raise ValueError(f"Unsupported FSDP auto-wrap policy: {name!r}")


class FSDPStrategy(ProcessGroupMixin):
    name = "fsdp"
    require_cuda = True

    def __init__(self, *, process_group_backend: str = "auto", timeout_minutes: int = 30,
                 sharding_strategy: str = "full_shard", auto_wrap_policy: str = "transformer_block",
                 backward_prefetch: str = "backward_pre", forward_prefetch: bool = False,
                 limit_all_gathers: bool = True, use_orig_params: bool = True, sync_module_states: bool = True,
                 cpu_offload: bool = False, activation_checkpointing: bool = False, precision: str = "fp32",
                 engine: str = "nccl", comm=None) -> None:
        if precision != "fp32" and precision not in _LOW_PRECISION:
            raise ValueError(f"Unsupported FSDP precision: {precision!r}")
        if sharding_strategy not in ("full_shard", "shard_grad_op", "no_shard", "hybrid_shard"):
            raise ValueError(f"Unsupported sharding strategy: {sharding_strategy!r}")
        self.process_group_backend = process_group_backend
        self.timeout_minutes = timeout_minutes
        self.sharding_strategy = sharding_strategy
        self.auto_wrap_policy_name = auto_wrap_policy
        self.backward_prefetch = backward_prefetch
        self.forward_prefetch = forward_prefetch
        self.limit_all_gathers = limit_all_gathers
        self.use_orig_params = use_orig_params
        self.sync_module_states = sync_module_states
        self.cpu_offload = cpu_offload
        self.activation_checkpointing = activation_checkpointing
        self.precision = precision
        self.engine = engine
        self.comm = comm

    @staticmethod
    def fused_unsupported(*, cpu_offload: bool, sharding_strategy: str, precision: str) -> list[str]:
        """The requested options the fused engine does not implement (empty: it can run the configuration)."""

        missing = []
        if cpu_offload:
            missing.append("cpu_offload")
        if sharding_strategy not in ("full_shard", "shard_grad_op"):
            missing.append(f"sharding_strategy={sharding_strategy}")
        from mini_train_sys_b200.train.precision import precision_supports_fused_engine

        if not precision_supports_fused_engine(precision):
            missing.append(f"precision={precision} (loss scaling)")
        return missing

    @classmethod
    def choose_engine(cls, requested: str, available: str, **options) -> str:
        """Engine for an FSDP run: ``requested`` is what the configuration says (``auto`` / ``fused`` / ``nccl``),
        ``available`` what the machine and back end allow.  ``auto`` never picks an engine that would have to refuse the run."""

        if requested == "auto" and available == "fused" and cls.fused_unsupported(**options):
            return "nccl"
        return available

    def resolved_engine(self) -> str:
        return "fused" if self.engine in ("auto", "fused") else "nccl"

    def _wrap_torch_fsdp(self, model: torch.nn.Module) -> torch.nn.Module:
        from torch.distributed.fsdp import (BackwardPrefetch, CPUOffload, FullyShardedDataParallel, MixedPrecision,
                                            ShardingStrategy)

        mixed = None
        if self.precision != "fp32":
            low = _LOW_PRECISION[self.precision]
            mixed = MixedPrecision(param_dtype=low, reduce_dtype=torch.float32, buffer_dtype=low,
                                   keep_low_precision_grads=False, cast_forward_inputs=True)
        prefetch = {"backward_pre": BackwardPrefetch.BACKWARD_PRE, "backward_post": BackwardPrefetch.BACKWARD_POST,
                    "none": None}[self.backward_prefetch]
        wrapped = FullyShardedDataParallel(
            model,
            auto_wrap_policy=build_auto_wrap_policy(self.auto_wrap_policy_name),
            sharding_strategy=getattr(ShardingStrategy, self.sharding_strategy.upper()),
            mixed_precision=mixed, backward_prefetch=prefetch, forward_prefetch=self.forward_prefetch,
            limit_all_gathers=self.limit_all_gathers, device_id=torch.device("cuda", self.local_rank),
            use_orig_params=self.use_orig_params, sync_module_states=self.sync_module_states,
            cpu_offload=CPUOffload(offload_params=self.cpu_offload),
        )
        if self.activation_checkpointing:
            from torch.distributed.algorithms._checkpoint.checkpoint_wrapper import (
                CheckpointImpl, apply_activation_checkpointing, checkpoint_wrapper)

            apply_activation_checkpointing(
                wrapped, checkpoint_wrapper_fn=partial(checkpoint_wrapper, checkpoint_impl=CheckpointImpl.NO_REENTRANT),
                check_fn=lambda m: isinstance(m, TransformerBlock))
        return wrapped

    def wrap_model(self, model: torch.nn.Module) -> torch.nn.Module:
        if self.resolved_engine() == "fused":
            from mini_train_sys_b200.parallel.flat_engine import FlatDataParallel

            unsupported = self.fused_unsupported(cpu_offload=self.cpu_offload, sharding_strategy=self.sharding_strategy,
                                                 precision=self.precision)
            if unsupported:
                raise ValueError("parallel.comm.engine=fused does not implement: " + ", ".join(unsupported)
                                 + "; select parallel.comm.engine=nccl for these options")
            return FlatDataParallel(
                model, mode="shard", comm=self.comm, reshard_after_forward=self.sharding_strategy == "full_shard",
                per_block_units=self.auto_wrap_policy_name == "transformer_block",
                activation_checkpointing=self.activation_checkpointing)
        return self._wrap_torch_fsdp(model)

    def unit_count(self, model: torch.nn.Module) -> int:
        """Number of sharding units in a wrapped model (both engines)."""

        own = getattr(model, "unit_count", None)
        if own is not None:
            return int(own())
        from torch.distributed.fsdp import FullyShardedDataParallel

        return sum(isinstance(m, FullyShardedDataParallel) for m in model.modules())
