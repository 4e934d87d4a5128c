"""Structured event sinks: console, JSONL, TensorBoard (rank 0 only).

An event is a dict with an ``event`` name and usually a ``step``.  The sinks and the
directory layout ``<log_dir>/<run>/<timestamp>/events.jsonl`` follow
minitrain/runtime/logger.py:17-438; the ``[layer x expert]`` balance matrices become
fixed-scale RGB heatmaps encoded as PNG without any imaging dependency.
"""

from __future__ import annotations

import json
import os
import struct
import threading
import time
import warnings
import zlib
from pathlib import Path
from typing import Protocol

import torch

from mini_train_sys_b200.runtime.config import LoggingConfig


class EventLogger(Protocol):
    def log_event(self, payload: dict[str, object]) -> None: ...

    def close(self) -> None: ...


def is_primary_rank() -> bool:
    return int(os.environ.get("RANK", "0")) == 0


class NullLogger:
    def log_event(self, payload: dict[str, object]) -> None:
        pass

    def close(self) -> None:
        pass


def _hms(seconds: object) -> str:
    try:
        total = max(0, int(float(seconds)))  # type: ignore[arg-type]
    except (TypeError, ValueError):
        return "?"
    return f"{total // 3600:d}:{total % 3600 // 60:02d}:{total % 60:02d}"


def _num(payload: dict[str, object], key: str, digits: int = 3) -> str:
    value = payload.get(key)
    return f"{value:,.{digits}f}" if isinstance(value, (int, float)) else "-"


_PROGRESS_EVENTS = {"train", "probe_train", "probe_validation", "probe_train_evaluation", "evaluate",
                    "analyze", "model_load", "prepare"}
_UNIT_TOTALS = (("batch", "batches_total"), ("step", "steps_total"), ("example", "examples_total"))


def _format_progress(event: str, p: dict[str, object]) -> str:
    unit, total_key = next(((u, t) for u, t in _UNIT_TOTALS if u in p and t in p), ("batch", "batches_total"))
    head = f"[{event}] {unit} {p.get(unit, p.get('step', '?'))}/{p.get(total_key, p.get('step_total', '?'))}"
    cells = [head]
    if "epoch" in p and "epochs_total" in p:
        cells.append(f"epoch {p['epoch']}/{p['epochs_total']}")
    if "loss" in p:
        cells.append(f"loss {_num(p, 'loss', 5)}")
    if "lr" in p:
        lr = p["lr"]
        cells.append(f"lr {float(lr):.3e}" if isinstance(lr, (int, float)) else "lr -")
    for key in ("accuracy", "accuracy_running"):
        if key in p:
            cells.append(f"acc {_num(p, key, 4)}")
            break
    if "grad_norm" in p:
        cells.append(f"grad {_num(p, 'grad_norm', 3)}")
    if "data_wait_percent" in p:
        cells.append(f"data-wait {_num(p, 'data_wait_percent', 1)}%")
    if "tokens_per_sec" in p:
        cells.append(f"tok/s {_num(p, 'tokens_per_sec', 1)}")
    if "items_per_sec" in p and not p.get("tokens_per_sec"):
        cells.append(f"items/s {_num(p, 'items_per_sec', 1)}")
    if "mfu_percent" in p:
        cells.append(f"mfu {_num(p, 'mfu_percent', 1)}%")
    if "gpu_peak_memory_allocated_mb_max" in p:
        used = float(p["gpu_peak_memory_allocated_mb_max"]) / 1024  # type: ignore[arg-type]
        cap = float(p.get("gpu_memory_capacity_mb_max", 0)) / 1024  # type: ignore[arg-type]
        cells.append(f"gpu-peak {used:.2f}/{cap:.2f} GiB")
    elif "host_peak_memory_mb" in p:
        cells.append(f"host-peak {_num(p, 'host_peak_memory_mb', 1)} MiB")
    for key in ("gpu_compute_utilization_percent_mean", "gpu_compute_utilization_percent_local_mean"):
        if key in p:
            cells.append(f"gpu-util {_num(p, key, 1)}%")
            break
    cells.append(f"{_num(p, 'progress_percent', 1)}%")
    cells.append(f"ETA {_hms(p.get('eta_seconds'))}")
    return " | ".join(cells)


def _format_pipeline(p: dict[str, object]) -> str:
    cells = [f"[probe_pipeline:{p.get('phase', '?')}] tasks {p.get('step', '?')}/{p.get('steps_total', '?')}",
             f"running {p.get('tasks_running', 0)} | queued {p.get('tasks_queued', 0)} | failed {p.get('tasks_failed', 0)}"]
    if p.get("task"):
        cells.append(f"{p.get('action', 'update')} {p['task']} on {p.get('device', '?')}")
    if p.get("worker_step") is not None:
        w = f"worker {p['worker_step']}/{p.get('worker_steps_total', '?')}"
        if "worker_progress_percent" in p:
            w += f" {_num(p, 'worker_progress_percent', 1)}%"
        if "worker_eta_seconds" in p:
            w += f" ETA {_hms(p['worker_eta_seconds'])}"
        if "worker_loss" in p:
            w += f" loss {_num(p, 'worker_loss', 5)}"
        for key in ("worker_accuracy", "worker_accuracy_running"):
            if key in p:
                w += f" acc {_num(p, key, 4)}"
                break
        cells.append(w)
    if p.get("pipeline_step") is not None:
        cells.append(f"overall {p['pipeline_step']}/{p.get('pipeline_steps_total', '?')} "
                     f"{_num(p, 'pipeline_progress_percent', 1)}%")
    cells.append(f"phase ETA {_hms(p.get('phase_eta_seconds', p.get('eta_seconds')))}")
    if "pipeline_eta_seconds" in p:
        cells.append(f"pipeline ETA {_hms(p['pipeline_eta_seconds'])}")
    return " | ".join(cells)


def format_console_event(payload: dict[str, object]) -> str:
    """One stable human-readable line per event."""

    event = str(payload.get("event", "event"))
    if event == "probe_pipeline":
        return _format_pipeline(payload)
    if event in _PROGRESS_EVENTS:
        return _format_progress(event, payload)
    if event == "checkpoint":
        return f"[checkpoint] saved {payload.get('path')} (model+optimizer state)"
    if event == "probe_checkpoint":
        return f"[probe_checkpoint] step {payload.get('step')}/{payload.get('steps_total')} saved {payload.get('path')}"
    if event == "resume":
        return (f"[resume] {payload.get('path')} | epoch={payload.get('epoch')} step={payload.get('step')} "
                f"world={payload.get('saved_world_size')}")
    if event == "init":
        return (f"[init] run={payload.get('run')} device={payload.get('device')} strategy={payload.get('parallel')} "
                f"world={payload.get('world_size')} params={payload.get('params')}")
    return f"[{event}] {json.dumps(payload, ensure_ascii=False, default=str)}"


class ConsoleLogger:
    def __init__(self, *, enabled: bool = True) -> None:
        self.enabled = enabled

    def log_event(self, payload: dict[str, object]) -> None:
        if self.enabled:
            print(format_console_event(payload), flush=True)

    def close(self) -> None:
        pass


class JsonlLogger:
    """Append-only, thread-safe, flush-per-event audit log; closing twice is harmless."""

    def __init__(self, path: str | Path) -> None:
        self.path = Path(path)
        self.path.parent.mkdir(parents=True, exist_ok=True)
        self._fh = self.path.open("a", encoding="utf-8")
        self._lock = threading.Lock()

    def log_event(self, payload: dict[str, object]) -> None:
        line = json.dumps(payload, ensure_ascii=False, default=str)
        with self._lock:
            if not self._fh.closed:
                self._fh.write(line + "\n")
                self._fh.flush()

    def close(self) -> None:
        with self._lock:
            if not self._fh.closed:
                self._fh.close()


def encode_png_rgb(pixels: torch.Tensor) -> bytes:
    """Encode a ``[H, W, 3]`` uint8 tensor as an 8-bit truecolour PNG."""

    height, width, channels = pixels.shape
    if channels != 3 or pixels.dtype != torch.uint8:
        raise ValueError("expected a [H, W, 3] uint8 tensor")
    raw = b"".join(b"\x00" + bytes(pixels[row].reshape(-1).tolist()) for row in range(height))

    def chunk(tag: bytes, body: bytes) -> bytes:
        return struct.pack(">I", len(body)) + tag + body + struct.pack(">I", zlib.crc32(tag + body) & 0xFFFFFFFF)

    return (b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", width, height, 8, 2, 0, 0, 0))
            + chunk(b"IDAT", zlib.compress(raw)) + chunk(b"IEND", b""))


def balance_heatmap(matrix: torch.Tensor) -> torch.Tensor:
    """Map load/uniform ratios in [0, 2] to blue (under-used) - white - red (over-used), ``[3, L, E]``."""

    ratio = (matrix * matrix.shape[1]).clamp(0.0, 2.0)
    one = torch.ones_like(ratio)
    return torch.stack((torch.minimum(ratio, one), 1.0 - (ratio - 1.0).abs(), torch.minimum(2.0 - ratio, one))).clamp(0, 1)


_BALANCE_KEYS = {"moe/expert_load_fraction_by_layer", "moe/expert_probability_by_layer"}


class TensorBoardLogger:
    """Numbers become ``<event>/<key>`` scalars at ``step``; numeric arrays become histograms/heatmaps."""

    def __init__(self, *, log_dir: str | Path, flush_secs: int = 10) -> None:
        try:
            from torch.utils.tensorboard import SummaryWriter
        except ModuleNotFoundError as exc:
            raise RuntimeError("TensorBoard logging is enabled, but the 'tensorboard' package is not installed. "
                               "Install it or set logging.tensorboard=false.") from exc
        self.log_dir = Path(log_dir)
        self.writer = SummaryWriter(log_dir=str(self.log_dir), flush_secs=flush_secs)

    def log_event(self, payload: dict[str, object]) -> None:
        event = str(payload.get("event", "event"))
        step = payload.get("step")
        if not isinstance(step, int):
            body = "\n".join(f"- {k}: {v}" for k, v in sorted(payload.items()))
            self.writer.add_text(event, body, global_step=0)
            return
        worker_step = payload.get("worker_step")
        if event == "probe_pipeline" and isinstance(worker_step, int) and payload.get("task"):
            prefix = f"probe_pipeline/{payload.get('phase', 'phase')}/{payload['task']}"
            for key, value in payload.items():
                if key.startswith("worker_") and isinstance(value, (int, float)) and not isinstance(value, bool):
                    self.writer.add_scalar(f"{prefix}/{key.removeprefix('worker_')}", value, worker_step)
        for key, value in payload.items():
            if key in ("event", "step") or isinstance(value, bool):
                continue
            if event == "probe_pipeline" and key.startswith("worker_"):
                continue
            if isinstance(value, (int, float)):
                self.writer.add_scalar(f"{event}/{key}", value, step)
            elif isinstance(value, (list, tuple)):
                self._log_array(f"{event}/{key}", key, value, step)

    def _log_array(self, tag: str, key: str, value: object, step: int) -> None:
        try:
            tensor = torch.tensor(value, dtype=torch.float32)
        except (TypeError, ValueError):
            return
        if tensor.numel() == 0 or not bool(torch.isfinite(tensor).all()):
            return
        if key in _BALANCE_KEYS and tensor.ndim == 2:
            self._add_png(f"{tag}/balance_heatmap", balance_heatmap(tensor), step)
            self.writer.add_histogram(f"{tag}/ratio_histogram", (tensor * tensor.shape[1]).flatten(), step)
        else:
            self.writer.add_histogram(tag, tensor.flatten(), step)

    def _add_png(self, tag: str, image: torch.Tensor, step: int) -> None:
        from tensorboard.compat.proto.summary_pb2 import Summary

        pixels = image.mul(255).round().to(torch.uint8).permute(1, 2, 0).contiguous().cpu()
        img = Summary.Image(height=pixels.shape[0], width=pixels.shape[1], colorspace=3,
                            encoded_image_string=encode_png_rgb(pixels))
        self.writer._get_file_writer().add_summary(Summary(value=[Summary.Value(tag=tag, image=img)]), step)

    def close(self) -> None:
        self.writer.flush()
        self.writer.close()


class CompositeLogger:
    def __init__(self, loggers: list[EventLogger]) -> None:
        self.loggers = loggers

    def log_event(self, payload: dict[str, object]) -> None:
        for sink in self.loggers:
            sink.log_event(payload)

    def close(self) -> None:
        for sink in reversed(self.loggers):
            sink.close()


def make_run_log_dir(base_dir: str | Path, run_name: str) -> Path:
    return Path(base_dir) / run_name / time.strftime("%Y%m%d-%H%M%S")


def get_run_log_dir(cfg: LoggingConfig, *, run_name: str) -> Path | None:
    if not is_primary_rank() or not (cfg.tensorboard or cfg.jsonl):
        return None
    return make_run_log_dir(cfg.log_dir, run_name)


def get_tensorboard_log_dir(cfg: LoggingConfig, *, run_name: str) -> Path | None:
    return get_run_log_dir(cfg, run_name=run_name) if cfg.tensorboard else None


def build_event_logger(cfg: LoggingConfig, *, run_name: str, tensorboard_log_dir: str | Path | None = None) -> EventLogger:
    """Sink stack for this process; non-zero ranks get a ``NullLogger``."""

    if not is_primary_rank():
        return NullLogger()
    sinks: list[EventLogger] = [ConsoleLogger()] if cfg.console else []
    run_dir = Path(tensorboard_log_dir) if tensorboard_log_dir else None
    if cfg.jsonl or cfg.tensorboard:
        run_dir = run_dir or make_run_log_dir(cfg.log_dir, run_name)
    if cfg.jsonl:
        sinks.append(JsonlLogger(run_dir / "events.jsonl"))
    if cfg.tensorboard:
        try:
            sinks.append(TensorBoardLogger(log_dir=run_dir, flush_secs=cfg.flush_secs))
        except RuntimeError as exc:
            warnings.warn(f"{exc} Continuing without TensorBoard.", stacklevel=2)
    return CompositeLogger(sinks) if sinks else NullLogger()
