"""Epoch / step orchestration: sampler epochs, interval metrics, logging and checkpoint cadence.

Event fields and cadence rules follow minitrain/train/runner.py:27-330.  Interval metrics are
accumulated on the device and only read at log boundaries, so no step forces a host sync.
This implementation additionally reports device-timed step time (CUDA events around each
interval) and MFU against the measured bf16 peak.
"""

from __future__ import annotations

import time
import tracemalloc
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any

import torch

from mini_train_sys_b200.runtime.health import PeerLostError, RankHealth
from mini_train_sys_b200.models.config import ModelConfig
from mini_train_sys_b200.parallel.strategy import ParallelStrategy
from mini_train_sys_b200.runtime.config import ExperimentConfig
from mini_train_sys_b200.runtime.logger import EventLogger
from mini_train_sys_b200.runtime.monitoring import (GpuUtilizationMonitor, distributed_gpu_utilization,
                                                    distributed_mean, distributed_mean_tensors, memory_metrics)
from mini_train_sys_b200.train.checkpoint import checkpoint_path, prune_checkpoints, save_checkpoint
from mini_train_sys_b200.train.lr_scheduler import resolve_total_steps
from mini_train_sys_b200.train.metrics import estimate_mfu, measured_peaks
from mini_train_sys_b200.train.trainer import Trainer


@dataclass
class _Interval:
    """What accumulates between two log events."""

    started_at: float
    start_step: int
    start_tokens: int
    data_wait: float = 0.0
    clipped: int = 0
    scalars: dict[str, torch.Tensor] = field(default_factory=dict)
    images: dict[str, torch.Tensor] = field(default_factory=dict)
    device_start: Any = None

    def add(self, bucket: dict[str, torch.Tensor], values: dict[str, torch.Tensor]) -> None:
        for key, value in values.items():
            v = value.detach()
            if key in bucket:
                bucket[key].add_(v)
            else:
                bucket[key] = v.clone()


class TrainingRunner:
    def __init__(self, *, cfg: ExperimentConfig, trainer: Trainer, dataloader: Any, strategy: ParallelStrategy,
                 logger: EventLogger, device: torch.device, world_size: int) -> None:
        self.cfg = cfg
        self.trainer = trainer
        self.dataloader = dataloader
        self.strategy = strategy
        self.logger = logger
        self.device = device
        self.world_size = world_size
        self.rank = strategy.rank
        self.gpu_monitor = GpuUtilizationMonitor(device)
        try:
            self._flops_per_token = ModelConfig(**cfg.model).flops_per_token() if cfg.model else 0.0
        except (TypeError, ValueError):
            self._flops_per_token = 0.0
        self._peak_flops = measured_peaks()["bf16_tflops_sustained"] * 1e12
        # what one step of this model and batch would take with every kernel at the machine's measured peak and no gaps
        try:
            from mini_train_sys_b200.runtime.step_model import step_roofline

            self._step_bound_ms = float(step_roofline(ModelConfig(**cfg.model), cfg.train.batch_size)["bound_ms_sustained"]) if cfg.model else 0.0
        except (TypeError, ValueError):
            self._step_bound_ms = 0.0

    # ---- logging -----------------------------------------------------------------
    def _new_interval(self) -> _Interval:
        st = self.trainer.state
        iv = _Interval(time.perf_counter(), st.step, st.tokens_seen)
        if self.device.type == "cuda":
            iv.device_start = torch.cuda.Event(enable_timing=True)
            iv.device_start.record()
        return iv

    def _emit_train_event(self, iv: _Interval, *, epoch: int, batch_index: int, batches_in_epoch: int,
                          total_steps: int, tokens_goal: int, session: tuple[float, int, int]) -> None:
        st = self.trainer.state
        now = time.perf_counter()
        steps = max(st.step - iv.start_step, 1)
        seconds = now - iv.started_at
        started, first_step, first_tokens = session
        scalars = {k: float(v / steps) for k, v in iv.scalars.items()}
        scalars["lr"] = self.trainer.last_lr
        scalars["grad_clip_fraction"] = scalars.get("grad_was_clipped", iv.clipped / steps)
        scalars = distributed_mean(scalars, self.device)
        images = distributed_mean_tensors({k: v / steps for k, v in iv.images.items()}, self.device)
        session_seconds = now - started
        eta = session_seconds / max(st.step - first_step, 1) * max(total_steps - st.step, 0)
        tok_s = (st.tokens_seen - iv.start_tokens) * self.world_size / max(seconds, 1e-12)
        event: dict[str, object] = {
            "event": "train", "step": st.step, "step_total": total_steps, "epoch": epoch, "batch": batch_index,
            "batches_total": batches_in_epoch, "optimizer_step": st.step,
            "loss": round(scalars.pop("loss"), 6), "lr": scalars.pop("lr"),
            "tokens_seen": st.tokens_seen * self.world_size, "tokens_goal": tokens_goal,
            "progress_percent": round(100 * st.step / max(total_steps, 1), 3),
            "elapsed_seconds": round(session_seconds, 3), "eta_seconds": round(eta, 3),
            "tokens_per_sec": round(tok_s, 2),
            "avg_tokens_per_sec": round((st.tokens_seen - first_tokens) * self.world_size / max(session_seconds, 1e-12), 2),
            "step_time_ms": round(1000 * seconds / steps, 3),
            "data_wait_ms": round(1000 * iv.data_wait / steps, 3),
            "data_wait_percent": round(100 * iv.data_wait / max(seconds, 1e-12), 3),
        }
        if iv.device_start is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            end.synchronize()
            event["device_step_time_ms"] = round(iv.device_start.elapsed_time(end) / steps, 3)
            if self._step_bound_ms > 0 and event["device_step_time_ms"] > 0:
                event["roofline_fraction"] = round(self._step_bound_ms / event["device_step_time_ms"], 4)
        if self._step_bound_ms > 0:
            event["roofline_step_bound_ms"] = round(self._step_bound_ms, 3)
        if self._flops_per_token and self.device.type == "cuda":
            event["mfu_percent"] = round(100 * estimate_mfu(tok_s / self.world_size, self._flops_per_token,
                                                            self._peak_flops), 2)
        if self.cfg.train.epochs is not None:
            event["epochs_total"] = self.cfg.train.epochs
        event.update(memory_metrics(self.device, reset_peak_stats=True))
        event.update(distributed_gpu_utilization(self.gpu_monitor.read_interval(), self.device))
        event.update(scalars)
        event.update(images)
        self.logger.log_event(event)

    # ---- checkpoints -------------------------------------------------------------
    def _check_device_status(self) -> None:
        """Raise when a kernel of this process gave up on a bounded wait (a peer that stalled or left): gradients of that
        step were incomplete, the optimizer kernel skipped the update, and going on - or saving - would hide it.  Called where
        the device is synchronised anyway: at every log boundary and before every checkpoint."""

        if self.device.type != "cuda":
            return
        import sys

        if "_mts_b200_ext" in sys.modules:      # only when the native extension is in use
            from mini_train_sys_b200.ops.native_backend import check_kernel_status

            check_kernel_status(self.device)
        checker = getattr(self.trainer.model, "check_status", None)
        if callable(checker):
            checker()

    def _save(self, *, epoch: int, force_model_export: bool = False, inside_epoch: bool = False) -> Path:
        self._check_device_status()
        ck, st = self.cfg.checkpoint, self.trainer.state
        target = checkpoint_path(ck.directory, self.cfg.run.name, epoch=epoch, step=st.step)
        every = ck.export_model_every_epochs
        export = ck.export_model and not inside_epoch and (force_model_export or every is None or epoch % every == 0)
        t0 = time.perf_counter()
        save_checkpoint(target, self.trainer.model, self.trainer.optimizer, st.step, epoch=epoch, lr_step=st.lr_step,
                        tokens_seen=st.tokens_seen, epoch_batches_done=st.epoch_batches_done, grad_scaler=self.trainer.grad_scaler,
                        lr_scheduler=self.trainer.lr_scheduler, precision=self.trainer.precision.name,
                        config=asdict(self.cfg), export_model=export, cpu_offload=ck.cpu_offload)
        if self.rank == 0:
            removed: list[Path] = []
            if ck.keep_last is not None:
                removed = prune_checkpoints(ck.directory, self.cfg.run.name, keep_last=ck.keep_last,
                                            keep_safety=ck.keep_safety, safety_every_epochs=ck.safety_every_epochs,
                                            keep_model_exports=ck.keep_model_exports)
            self.logger.log_event({
                "event": "checkpoint", "path": str(target), "includes_optimizer": True, "exported_model": export,
                "checkpoint_seconds": round(time.perf_counter() - t0, 3),
                "checkpoint_bytes": sum(f.stat().st_size for f in target.rglob("*") if f.is_file()),
                "removed_old_checkpoints": [str(p) for p in removed],
            })
        return target

    def _skip_batches(self, sampler, batches: int) -> None:
        """Position the data stream behind the first ``batches`` batches of the epoch: through the sampler's cursor when it
        has one (nothing is read), else by drawing and dropping them."""

        if hasattr(sampler, "set_start"):
            sampler.set_start(batches * self.cfg.train.batch_size)
            self._drop_batches = 0
        else:
            self._drop_batches = batches

    # ---- main loop ---------------------------------------------------------------
    def run(self, *, max_steps: int | None, resume_path: Path | None = None) -> None:
        on_cuda = self.device.type == "cuda"
        if on_cuda:
            torch.cuda.reset_peak_memory_stats(self.device)
            self.gpu_monitor.start()
        else:
            tracemalloc.start()
        self.strategy.barrier()

        st = self.trainer.state
        session = (time.perf_counter(), st.step, st.tokens_seen)
        total_steps = resolve_total_steps(max_steps=max_steps, epochs=self.cfg.train.epochs,
                                          steps_per_epoch=len(self.dataloader))
        tokens_goal = total_steps * self.cfg.train.batch_size * int(self.cfg.model["seq_len"]) * self.world_size
        iv = self._new_interval()
        done = max_steps is not None and st.step >= max_steps
        epoch = st.epoch
        last_saved = resume_path
        epochs_limit = self.cfg.train.epochs

        comm = self.cfg.parallel.comm
        health = RankHealth() if (comm.health_check and self.world_size > 1) else None
        while not done and (epochs_limit is None or epoch < epochs_limit):
            epoch += 1
            sampler = getattr(self.dataloader, "sampler", None)
            if hasattr(sampler, "set_epoch"):
                sampler.set_epoch(epoch)   # every rank must see the same epoch number
            n_batches = len(self.dataloader)
            # a run that was interrupted inside this epoch continues behind the batches it already trained on
            first_batch = min(st.epoch_batches_done, n_batches) if epoch == st.epoch + 1 else 0
            if first_batch:
                self._skip_batches(sampler, first_batch)
            source = self.dataloader
            if self.cfg.data.device_prefetch:
                from mini_train_sys_b200.data.dataloader import DevicePrefetcher

                source = DevicePrefetcher(self.dataloader, self.device)     # a pass-through on a CPU device
            stream = iter(source)
            for _ in range(getattr(self, "_drop_batches", 0)):
                next(stream)
            self._drop_batches = 0
            finished_epoch = True
            for batch_index in range(first_batch + 1, n_batches + 1):
                t_wait = time.perf_counter()
                batch = next(stream)
                iv.data_wait += time.perf_counter() - t_wait
                if health is not None:
                    # on the host, with nothing of this rank in flight: a peer that left or fell silent ends the run here
                    # instead of in a device-side wait or a collective timeout
                    try:
                        health.check(max_age_seconds=comm.health_max_age_seconds)
                    except PeerLostError as exc:
                        self.logger.log_event({"event": "peer_lost", "step": st.step, "detail": str(exc)})
                        raise SystemExit(3) from exc
                loss = self.trainer.train_step(batch)
                st.epoch_batches_done = batch_index
                if health is not None:
                    health.beat(st.step)
                iv.add(iv.scalars, {"loss": loss})
                iv.add(iv.scalars, self.trainer.last_metrics)
                iv.add(iv.images, self.trainer.last_visualizations)
                iv.clipped += int(self.trainer.last_grad_was_clipped)
                hit_limit = max_steps is not None and st.step >= max_steps
                if (st.step == session[1] + 1 or st.step % self.cfg.train.log_interval == 0
                        or batch_index == n_batches or hit_limit):
                    if on_cuda:
                        torch.cuda.synchronize(self.device)
                        self._check_device_status()
                    self._emit_train_event(iv, epoch=epoch, batch_index=batch_index, batches_in_epoch=n_batches,
                                           total_steps=total_steps, tokens_goal=tokens_goal, session=session)
                    iv = self._new_interval()
                if hit_limit:
                    finished_epoch = batch_index == n_batches
                    done = True
                    break
                every_steps = self.cfg.checkpoint.every_steps
                if every_steps is not None and st.step % every_steps == 0 and batch_index < n_batches:
                    last_saved = self._save(epoch=st.epoch, inside_epoch=True)       # the cursor into the epoch goes with it; no model export

            if finished_epoch:   # a max_steps stop mid-epoch keeps the previous complete epoch (and the cursor into this one)
                st.epoch = epoch
                st.epoch_batches_done = 0
            every = self.cfg.checkpoint.every_epochs
            if finished_epoch and every is not None and epoch % every == 0:
                terminal = (epochs_limit is not None and epoch >= epochs_limit) or \
                           (max_steps is not None and st.step >= max_steps)
                last_saved = self._save(epoch=epoch, force_model_export=terminal)
            self.strategy.barrier()

        if self.cfg.checkpoint.save_final:
            final = checkpoint_path(self.cfg.checkpoint.directory, self.cfg.run.name, epoch=st.epoch, step=st.step)
            if final != last_saved:
                self._save(epoch=st.epoch, force_model_export=True)
        if not on_cuda and tracemalloc.is_tracing():
            tracemalloc.stop()
        self.gpu_monitor.close()
