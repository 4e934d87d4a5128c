"""Linear batch-size scaling of the learning rate and schedule lengths (no gradient accumulation).

With ``train.batch_size_scaling: linear`` the global batch ``batch_size * world`` is compared
to ``reference_global_batch_size``: lr is multiplied by the ratio, warmup/decay steps divided
(reference behaviour: minitrain/runtime/scaling.py:9-50).
"""

from __future__ import annotations

from dataclasses import dataclass, replace

from mini_train_sys_b200.runtime.config import LRSchedulerConfig, OptimizerConfig, TrainConfig


@dataclass(frozen=True)
class ResolvedBatchScale:
    local_batch_size: int
    global_batch_size: int
    reference_global_batch_size: int
    scale: float
    optimizer: OptimizerConfig
    lr_scheduler: LRSchedulerConfig


def _rescale_steps(steps: int | None, scale: float) -> int | None:
    if steps is None or steps == 0:
        return steps
    return max(1, round(steps / scale))


def resolve_batch_scale(train: TrainConfig, optimizer: OptimizerConfig, lr_scheduler: LRSchedulerConfig, *,
                        world_size: int) -> ResolvedBatchScale:
    global_batch = train.batch_size * world_size
    reference = train.reference_global_batch_size or global_batch
    scale = global_batch / reference if train.batch_size_scaling == "linear" else 1.0
    return ResolvedBatchScale(
        local_batch_size=train.batch_size,
        global_batch_size=global_batch,
        reference_global_batch_size=reference,
        scale=scale,
        optimizer=replace(optimizer, lr=optimizer.lr * scale),
        lr_scheduler=replace(lr_scheduler,
                             warmup_steps=_rescale_steps(lr_scheduler.warmup_steps, scale) or 0,
                             decay_steps=_rescale_steps(lr_scheduler.decay_steps, scale)),
    )
