"""One optimizer step: H2D, forward under autocast, backward, clip, update, schedule.

The trainer knows nothing about kernels (the model owns its ``OpsBackend``) or about
distribution (the model may be wrapped by a strategy).  Step order and bookkeeping follow
minitrain/train/trainer.py:13-159.  Two hooks let sharded engines fuse work:
``model.clip_grad_norm_(max_norm)`` replaces the utility clip, and an optimizer exposing
``owns_clipping`` receives the clip threshold and applies the coefficient inside its
update kernel, so no separate pass over the gradients is made.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from mini_train_sys_b200.train.lr_scheduler import LearningRateScheduler
from mini_train_sys_b200.train.precision import PrecisionPolicy, resolve_precision_policy


@dataclass
class TrainState:
    step: int = 0
    lr_step: int = 0       # schedule progress; remapped on elastic resume
    tokens_seen: int = 0   # local tokens; multiplied by world size when logged
    epoch: int = 0


class Trainer:
    def __init__(self, model: torch.nn.Module, optimizer: torch.optim.Optimizer, device: torch.device,
                 use_fused_loss: bool = False, precision: str = "auto", grad_clip_norm: float | None = None,
                 check_finite: bool = True, lr_scheduler: LearningRateScheduler | None = None) -> None:
        self.model = model
        self.optimizer = optimizer
        self.device = device
        self.use_fused_loss = use_fused_loss
        self.precision: PrecisionPolicy = resolve_precision_policy(precision, device)
        self.grad_clip_norm = grad_clip_norm
        self.check_finite = check_finite
        self.lr_scheduler = lr_scheduler
        self.last_lr = float(optimizer.param_groups[0]["lr"])
        self.last_metrics: dict[str, torch.Tensor] = {}
        self.last_visualizations: dict[str, torch.Tensor] = {}
        self.last_grad_norm: float | None = None
        self.last_grad_clip_coefficient = 1.0
        self.last_grad_was_clipped = False
        if self.precision.grad_scaling_enabled and getattr(optimizer, "owns_clipping", False):
            raise ValueError("precision=fp16 needs loss scaling, which an optimizer that clips inside its update kernel (the fused "
                             "sharding engine) does not implement: use bf16, or parallel.comm.engine=nccl")
        self.grad_scaler = torch.amp.GradScaler(device.type, enabled=self.precision.grad_scaling_enabled)
        self.state = TrainState()
        self.optimizer.zero_grad(set_to_none=True)

    # ---- gradient clipping ---------------------------------------------------
    def _record_norm(self, norm: float) -> None:
        if not math.isfinite(norm):
            raise FloatingPointError("non-finite global gradient norm")
        self.last_grad_norm = norm
        self.last_grad_clip_coefficient = min(1.0, self.grad_clip_norm / (norm + 1e-6))
        self.last_grad_was_clipped = norm > self.grad_clip_norm

    def _clip_gradients(self) -> None:
        if self.grad_clip_norm is None:
            self.last_grad_norm, self.last_grad_clip_coefficient, self.last_grad_was_clipped = None, 1.0, False
            return
        if getattr(self.optimizer, "owns_clipping", False):
            # The sharded optimizer reduces the norm and applies the coefficient in its update kernel.
            self.optimizer.set_clip_norm(self.grad_clip_norm)
            return
        sharded_clip = getattr(self.model, "clip_grad_norm_", None)
        if sharded_clip is not None:
            norm = sharded_clip(self.grad_clip_norm)
        else:
            norm = torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.grad_clip_norm)
        self._record_norm(float(norm.detach()))

    def _after_owned_clip(self) -> dict[str, torch.Tensor]:
        """Clip statistics of an optimizer that clips on the device; nothing is read back to the host."""

        if self.grad_clip_norm is None or not getattr(self.optimizer, "owns_clipping", False):
            return {}
        norm = self.optimizer.last_grad_norm().detach().clone()
        self.last_grad_norm, self.last_grad_clip_coefficient, self.last_grad_was_clipped = None, 1.0, False
        limit = float(self.grad_clip_norm)
        return {"grad_norm": norm, "grad_clip_threshold": torch.tensor(limit),
                "grad_clip_coefficient": (limit / (norm + 1e-6)).clamp(max=1.0),
                "grad_was_clipped": (norm > limit).float()}

    # ---- the step --------------------------------------------------------------
    def train_step(self, batch: dict[str, torch.Tensor]) -> torch.Tensor:
        self.model.train()
        input_ids = batch["input_ids"].to(self.device, non_blocking=True)
        targets = batch["targets"].to(self.device, non_blocking=True)

        with self.precision.autocast_context(self.device):
            loss, _ = self.model(input_ids, targets=targets, use_fused_loss=self.use_fused_loss)
        if loss is None:
            raise RuntimeError("Expected loss during training")
        if self.check_finite:
            ok = torch.isfinite(loss.detach())
            if loss.is_cuda:
                torch._assert_async(ok, "non-finite training loss")
            elif not bool(ok):
                raise FloatingPointError("non-finite training loss")

        source = getattr(self.model, "module", self.model)
        self.last_metrics = dict(getattr(source, "last_training_metrics", {}))
        self.last_visualizations = dict(getattr(source, "last_training_visualizations", {}))
        self.last_lr = float(self.optimizer.param_groups[0]["lr"])

        if self.grad_scaler.is_enabled():
            self.grad_scaler.scale(loss).backward()
            self.grad_scaler.unscale_(self.optimizer)
            self._clip_gradients()
            self.grad_scaler.step(self.optimizer)
            self.grad_scaler.update()
        else:
            loss.backward()
            self._clip_gradients()
            self.optimizer.step()
        device_clip_stats = self._after_owned_clip()
        self.optimizer.zero_grad(set_to_none=True)

        st = self.state
        st.step += 1
        st.lr_step += 1
        st.tokens_seen += input_ids.numel()
        if self.lr_scheduler is not None:
            self.lr_scheduler.step(st.lr_step)
        if self.last_grad_norm is not None:
            self.last_metrics.update({
                "grad_norm": torch.tensor(self.last_grad_norm),
                "grad_clip_threshold": torch.tensor(self.grad_clip_norm),
                "grad_clip_coefficient": torch.tensor(self.last_grad_clip_coefficient),
                "grad_was_clipped": torch.tensor(float(self.last_grad_was_clipped)),
            })
        self.last_metrics.update(device_clip_stats)
        if self.grad_scaler.is_enabled():
            self.last_metrics["grad_scale"] = torch.tensor(self.grad_scaler.get_scale())
        return loss.detach()
