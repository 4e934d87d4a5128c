"""One optimizer step: H2D, forward under autocast, backward, clip, update, schedule.

The trainer knows nothing about kernels (the model owns its ``OpsBackend``) or about
distribution (the model may be wrapped by a strategy).  Step order and bookkeeping follow
minitrain/train/trainer.py:13-159.  Two hooks let sharded engines fuse work:
``model.clip_grad_norm_(max_norm)`` replaces the utility clip, and an optimizer exposing
``owns_clipping`` receives the clip threshold and applies the coefficient inside its
update kernel, so no separate pass over the gradients is made.

CUDA-graph mode (``cuda_graph=True``, sharded engine on CUDA only): after a few eager steps the device part of a step -
forward, backward, gradient reduction, clipping, AdamW - is captured once and replayed, which removes the per-launch host
cost and the gaps between dependent launches.  What changes from step to step is not baked into the graph: the batch is
copied into static input buffers, and dropout salts, flag sequence numbers, learning rates and bias corrections are read by
the kernels from a small per-device block that a one-thread kernel rewrites before every replay.
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
    epoch: int = 0         # complete epochs
    epoch_batches_done: int = 0   # batches of the epoch in progress (epoch + 1) that were already trained on: the resume cursor


class Trainer:
    def __init__(self, model: torch.nn.Module, optimizer: torch.optim.Optimizer, device: torch.device,
                 use_fused_loss: bool = False, precision: str = "auto", grad_clip_norm: float | None = None,
                 check_finite: bool = True, lr_scheduler: LearningRateScheduler | None = None, cuda_graph: bool = False,
                 graph_warmup_steps: int = 3) -> None:
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
        if not self.precision.fused_engine and getattr(optimizer, "owns_clipping", False):
            raise ValueError("precision=fp16 needs loss scaling, which an optimizer that clips inside its update kernel (the fused "
                             "sharding engine) does not implement: use bf16, or parallel.comm.engine=nccl")
        self.grad_scaler = torch.amp.GradScaler(device.type, enabled=self.precision.grad_scaling_enabled)
        self.state = TrainState()
        self.optimizer.zero_grad(set_to_none=True)
        self.cuda_graph = bool(cuda_graph)
        self.graph_warmup_steps = max(int(graph_warmup_steps), 1)
        self._graph = None
        self._graph_static: dict = {}
        self._graph_stream = None      # warm-up steps and the capture run here: autograd binds gradient accumulation to the
                                       # stream of a parameter's first backward, and the legacy default stream cannot be captured
        self._eager_steps = 0
        self.kernel_launches_replayed = 0     # launches of the extension's kernels that ran from graph replays (host counters miss them)
        if self.cuda_graph:
            reason = self._graph_unsupported_reason()
            if reason is not None:
                raise ValueError(f"train.cuda_graph is not available here: {reason}")

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
    def _graph_unsupported_reason(self) -> str | None:
        if self.device.type != "cuda":
            return "it needs a CUDA device"
        engine = getattr(self.optimizer, "engine", None)
        if engine is None or not getattr(self.optimizer, "owns_clipping", False) or not getattr(engine.coll, "fused", False):
            return "it needs the fused sharding engine (parallel.comm.engine = fused)"
        if any(u.local for u in engine.units):
            return "expert parallelism numbers its exchanges per layer, which a replayed graph cannot advance"
        if self.grad_scaler.is_enabled():
            return "loss scaling takes host decisions every step"
        return None

    def _device_step(self, input_ids: torch.Tensor, targets: torch.Tensor, *, check: bool):
        """Everything of a step that runs on the device; captured as a whole in CUDA-graph mode."""

        with self.precision.autocast_context(self.device):
            loss, _ = self.model(input_ids, targets=targets, use_fused_loss=self.use_fused_loss)
        if loss is None:
            raise RuntimeError("Expected loss during training")
        if check:
            self._assert_finite(loss)
        source = getattr(self.model, "module", self.model)
        self.last_metrics = dict(getattr(source, "last_training_metrics", {}))
        self.last_visualizations = dict(getattr(source, "last_training_visualizations", {}))
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
        return loss.detach(), device_clip_stats

    def _assert_finite(self, loss: torch.Tensor) -> None:
        if not self.check_finite:
            return
        ok = torch.isfinite(loss.detach())
        if loss.is_cuda:
            torch._assert_async(ok, "non-finite training loss")
        elif not bool(ok):
            raise FloatingPointError("non-finite training loss")

    def _after_step(self, tokens: int, device_clip_stats: dict) -> None:
        st = self.state
        st.step += 1
        st.lr_step += 1
        st.tokens_seen += tokens
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

    def train_step(self, batch: dict[str, torch.Tensor]) -> torch.Tensor:
        self.model.train()
        if self.cuda_graph and self._eager_steps >= self.graph_warmup_steps:
            return self._graphed_step(batch)
        input_ids = batch["input_ids"].to(self.device, non_blocking=True)
        targets = batch["targets"].to(self.device, non_blocking=True)
        self.last_lr = float(self.optimizer.param_groups[0]["lr"])
        if self.cuda_graph:
            if self._graph_stream is None:
                self._graph_stream = torch.cuda.Stream(self.device)
            outer = torch.cuda.current_stream(self.device)
            self._graph_stream.wait_stream(outer)
            with torch.cuda.stream(self._graph_stream):
                loss, device_clip_stats = self._device_step(input_ids, targets, check=True)
            outer.wait_stream(self._graph_stream)
        else:
            loss, device_clip_stats = self._device_step(input_ids, targets, check=True)
        self._eager_steps += 1
        self._after_step(input_ids.numel(), device_clip_stats)
        return loss

    # ---- CUDA-graph mode -----------------------------------------------------
    def _capture(self, batch: dict[str, torch.Tensor]) -> None:
        from mini_train_sys_b200.ops.native_backend import ext

        engine = self.optimizer.engine
        static = self._graph_static
        static["ids"] = batch["input_ids"].to(self.device).clone()
        static["targets"] = batch["targets"].to(self.device).clone()
        static["shape"] = tuple(static["ids"].shape)
        static["epoch_base"], static["step_base"] = engine.comm_epoch, engine.step_count
        static["seed_calls"] = None
        ext().step_context_tensor(self.device.index or 0)        # allocate the block before anything is captured
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        launched = int(ext().launch_count())
        with torch.cuda.graph(graph, stream=self._graph_stream):
            static["loss"], static["clip"] = self._device_step(static["ids"], static["targets"], check=False)
        static["launches"] = int(ext().launch_count()) - launched      # kernels of this extension inside one replay
        # nothing ran during capture: take back what the host-side counters recorded
        engine.comm_epoch, engine.step_count = static["epoch_base"], static["step_base"]
        static["metrics"], static["images"] = self.last_metrics, self.last_visualizations
        self._graph = graph

    def _graphed_step(self, batch: dict[str, torch.Tensor]) -> torch.Tensor:
        from mini_train_sys_b200.ops.native_backend import ext

        if self._graph is None:
            self._capture(batch)
        static, engine = self._graph_static, self.optimizer.engine
        if tuple(batch["input_ids"].shape) != static["shape"]:
            raise ValueError(f"CUDA-graph mode needs a fixed batch shape: captured {static['shape']}, got {tuple(batch['input_ids'].shape)}")
        static["ids"].copy_(batch["input_ids"], non_blocking=True)
        static["targets"].copy_(batch["targets"], non_blocking=True)
        decay, plain = self.optimizer.param_groups
        self.last_lr = float(decay["lr"])
        step = engine.step_count + 1
        b1, b2 = decay["betas"]
        ext().set_step_context(self.device.index or 0, step, engine.comm_epoch - static["epoch_base"], True, float(decay["lr"]),
                               float(plain["lr"]), 1.0 - b1 ** step, 1.0 - b2 ** step)
        self._graph.replay()
        self.kernel_launches_replayed += static["launches"]
        engine.comm_epoch += 1
        engine.step_count = step
        self.last_metrics, self.last_visualizations = dict(static["metrics"]), dict(static["images"])
        self._assert_finite(static["loss"])
        self._after_step(static["ids"].numel(), static["clip"])
        return static["loss"]

    def leave_graph_mode(self) -> None:
        """Drop the captured step and return the per-device block to its neutral state (eager steps may follow)."""

        if self._graph is not None:
            from mini_train_sys_b200.ops.native_backend import ext

            ext().set_step_context(self.device.index or 0, 0, 0, False, 0.0, 0.0, 1.0, 1.0)
            torch.cuda.synchronize(self.device)
        self._graph, self._graph_static, self.cuda_graph = None, {}, False
