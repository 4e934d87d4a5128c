"""Warmup + cosine/constant learning-rate schedule driven by completed-step count.

Warmup factor is ``(step + 1) / warmup_steps``; cosine decays from 1 to ``min_lr_ratio``
between the end of warmup and ``decay_steps`` (default: total steps)
(reference: minitrain/train/lr_scheduler.py:10-67).
"""

from __future__ import annotations

import math
from typing import Any

import torch

from mini_train_sys_b200.runtime.config import LRSchedulerConfig


def resolve_total_steps(*, max_steps: int | None, epochs: int | None, steps_per_epoch: int) -> int:
    limits = [v for v in (max_steps, None if epochs is None else epochs * steps_per_epoch) if v is not None]
    if not limits:
        raise ValueError("A max_steps or epochs training limit is required")
    return min(limits)


def lr_scale(cfg: LRSchedulerConfig, step: int, total_steps: int) -> float:
    if cfg.warmup_steps and step < cfg.warmup_steps:
        return (step + 1) / cfg.warmup_steps
    if cfg.schedule == "constant":
        return 1.0
    end = cfg.decay_steps or total_steps
    t = (step - cfg.warmup_steps) / max(1, end - cfg.warmup_steps)
    t = min(1.0, max(0.0, t))
    return cfg.min_lr_ratio + (1.0 - cfg.min_lr_ratio) * 0.5 * (1.0 + math.cos(math.pi * t))


class LearningRateScheduler:
    def __init__(self, optimizer: torch.optim.Optimizer, cfg: LRSchedulerConfig, *, total_steps: int) -> None:
        if total_steps <= 0:
            raise ValueError("total_steps must be positive")
        self.optimizer = optimizer
        self.cfg = cfg
        self.total_steps = total_steps
        self.base_lrs = [float(g["lr"]) for g in optimizer.param_groups]
        self.last_step = 0
        self.step(0)

    def step(self, completed_steps: int) -> None:
        self.last_step = completed_steps
        factor = lr_scale(self.cfg, completed_steps, self.total_steps)
        for base, group in zip(self.base_lrs, self.optimizer.param_groups):
            group["lr"] = base * factor

    def get_last_lr(self) -> list[float]:
        return [float(g["lr"]) for g in self.optimizer.param_groups]

    def state_dict(self) -> dict[str, Any]:
        return {"last_step": self.last_step, "total_steps": self.total_steps}

    def load_state_dict(self, state: dict[str, Any]) -> None:
        self.step(int(state["last_step"]))
