"""Cross-rank metric reduction, memory accounting, NVML sampling and progress events.

Behaviour follows minitrain/runtime/monitoring.py:17-345, with one change on the
communication side: each helper packs its values into a single buffer and issues one
collective per reduce-op instead of one per value.
"""

from __future__ import annotations

import math
import threading
import time
import tracemalloc
from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist

from mini_train_sys_b200.runtime.logger import EventLogger


def _dist_on() -> bool:
    return dist.is_available() and dist.is_initialized()


def _reduce_device(device: torch.device) -> torch.device:
    return device if _dist_on() and dist.get_backend() == "nccl" else torch.device("cpu")


def distributed_mean(values: dict[str, float], device: torch.device) -> dict[str, float]:
    if not values:
        return {}
    keys = sorted(values)
    buf = torch.tensor([float(values[k]) for k in keys], dtype=torch.float64, device=_reduce_device(device))
    if _dist_on():
        dist.all_reduce(buf)
        buf /= dist.get_world_size()
    return dict(zip(keys, buf.cpu().tolist()))


def distributed_mean_tensors(values: dict[str, torch.Tensor], device: torch.device) -> dict[str, object]:
    """Rank-average same-shaped tensors (one packed all-reduce) and return nested lists."""

    if not values:
        return {}
    keys = sorted(values)
    rdev = _reduce_device(device)
    flat = torch.cat([values[k].detach().to(device=rdev, dtype=torch.float32).reshape(-1) for k in keys])
    if _dist_on():
        dist.all_reduce(flat)
        flat /= dist.get_world_size()
    out: dict[str, object] = {}
    offset = 0
    for k in keys:
        n = values[k].numel()
        out[k] = flat[offset:offset + n].view(values[k].shape).cpu().tolist()
        offset += n
    return out


def memory_metrics(device: torch.device, *, reset_peak_stats: bool = False) -> dict[str, float]:
    world = dist.get_world_size() if _dist_on() else 1
    if device.type != "cuda":
        peak = tracemalloc.get_traced_memory()[1] if tracemalloc.is_tracing() else 0
        return {"host_peak_memory_mb": round(peak / 2**20, 2)}
    local = torch.tensor([torch.cuda.memory_allocated(device), torch.cuda.memory_reserved(device),
                          torch.cuda.max_memory_allocated(device),
                          torch.cuda.get_device_properties(device).total_memory],
                         dtype=torch.float64, device=_reduce_device(device))
    hi, total = local.clone(), local.clone()
    if _dist_on():
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        dist.all_reduce(total, op=dist.ReduceOp.SUM)
    loc, hi, total = (t.cpu().tolist() for t in (local, hi, total))
    mib = float(2**20)
    cap = max(hi[3], 1.0)
    out = {
        "gpu_memory_allocated_mb": round(loc[0] / mib, 2),
        "gpu_memory_reserved_mb": round(loc[1] / mib, 2),
        "gpu_peak_memory_allocated_mb": round(loc[2] / mib, 2),
        "gpu_memory_allocated_mb_max": round(hi[0] / mib, 2),
        "gpu_memory_reserved_mb_max": round(hi[1] / mib, 2),
        "gpu_peak_memory_allocated_mb_max": round(hi[2] / mib, 2),
        "gpu_memory_allocated_mb_total": round(total[0] / mib, 2),
        "gpu_memory_reserved_mb_total": round(total[1] / mib, 2),
        "gpu_memory_capacity_mb_max": round(hi[3] / mib, 2),
        "gpu_memory_capacity_mb_total": round(total[3] / mib, 2),
        "gpu_memory_current_percent_max": round(100 * hi[0] / cap, 2),
        "gpu_memory_reserved_percent_max": round(100 * hi[1] / cap, 2),
        "gpu_memory_peak_percent_max": round(100 * hi[2] / cap, 2),
        "monitored_world_size": world,
    }
    if reset_peak_stats:
        torch.cuda.reset_peak_memory_stats(device)
    return out


def _uuid_key(value: object) -> str:
    if isinstance(value, bytes):
        value = value.decode("ascii")
    return str(value).lower().removeprefix("gpu-").replace("-", "")


class GpuUtilizationMonitor:
    """Background NVML sampler (read-only queries) for this rank's device.

    ``nvml`` may be injected (tests pass a fake module); by default ``pynvml`` is
    imported lazily and a missing module simply disables sampling.
    """

    def __init__(self, device: torch.device, *, sample_interval_seconds: float = 0.2, nvml: Any | None = None,
                 device_uuid: str | None = None) -> None:
        self.device = device
        self.sample_interval_seconds = sample_interval_seconds
        self._nvml = nvml
        self._injected = nvml is not None
        self._uuid = device_uuid
        self._handle: Any | None = None
        self._halt = threading.Event()
        self._lock = threading.Lock()
        self._thread: threading.Thread | None = None
        self._samples: list[tuple[float, float]] = []

    @property
    def available(self) -> bool:
        return self._handle is not None

    def start(self) -> None:
        if self._thread is not None or (self.device.type != "cuda" and not self._injected):
            return
        nvml = self._nvml
        if nvml is None:
            try:
                import pynvml as nvml  # type: ignore[no-redef]
            except ImportError:
                return
        try:
            nvml.nvmlInit()
            want = _uuid_key(self._uuid if self._uuid is not None
                             else torch.cuda.get_device_properties(self.device).uuid)
            for index in range(nvml.nvmlDeviceGetCount()):
                handle = nvml.nvmlDeviceGetHandleByIndex(index)
                if _uuid_key(nvml.nvmlDeviceGetUUID(handle)) == want:
                    self._handle = handle
                    break
            if self._handle is None:
                nvml.nvmlShutdown()
                return
            self._nvml = nvml
            self._take()
            self._thread = threading.Thread(target=self._loop, name=f"mts-nvml-{self.device.index}", daemon=True)
            self._thread.start()
        except Exception:  # NVML errors must never stop training
            self._handle = None
            if not self._injected:
                self._nvml = None

    def _take(self) -> None:
        if self._nvml is None or self._handle is None:
            return
        try:
            rates = self._nvml.nvmlDeviceGetUtilizationRates(self._handle)
        except Exception:
            return
        with self._lock:
            self._samples.append((float(rates.gpu), float(rates.memory)))

    def _loop(self) -> None:
        while not self._halt.wait(self.sample_interval_seconds):
            self._take()

    def read_interval(self) -> dict[str, float]:
        self._take()
        with self._lock:
            samples, self._samples = self._samples, []
        if not samples:
            return {}
        out: dict[str, float] = {}
        for column, prefix in enumerate(("gpu_compute_utilization_percent", "gpu_memory_controller_utilization_percent")):
            vals = [s[column] for s in samples]
            out[f"{prefix}_local_min"] = min(vals)
            out[f"{prefix}_local_mean"] = sum(vals) / len(vals)
            out[f"{prefix}_local_max"] = max(vals)
        out["gpu_utilization_samples_local"] = float(len(samples))
        return out

    def close(self) -> None:
        self._halt.set()
        if self._thread is not None:
            self._thread.join(timeout=max(1.0, 2 * self.sample_interval_seconds))
        if self._nvml is not None and self._handle is not None:
            try:
                self._nvml.nvmlShutdown()
            except Exception:
                pass
        self._thread = None
        self._handle = None


_UTIL_PREFIXES = ("gpu_compute_utilization_percent", "gpu_memory_controller_utilization_percent")


def distributed_gpu_utilization(local: dict[str, float], device: torch.device) -> dict[str, float]:
    """Job-wide min/mean/max from per-rank NVML summaries using three packed all-reduces."""

    rdev = _reduce_device(device)
    have = bool(local)
    # MIN-reduce: [available, samples, min_compute, min_memctl]; values absent -> 0/inf
    mins = torch.tensor([float(have), local.get("gpu_utilization_samples_local", 0.0),
                         *(local.get(f"{p}_local_min", math.inf) for p in _UTIL_PREFIXES)],
                        dtype=torch.float64, device=rdev)
    sums = torch.tensor([local.get(f"{p}_local_mean", 0.0) for p in _UTIL_PREFIXES], dtype=torch.float64, device=rdev)
    maxs = torch.tensor([local.get(f"{p}_local_max", -math.inf) for p in _UTIL_PREFIXES], dtype=torch.float64, device=rdev)
    world = 1
    if _dist_on():
        world = dist.get_world_size()
        dist.all_reduce(mins, op=dist.ReduceOp.MIN)
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
        dist.all_reduce(maxs, op=dist.ReduceOp.MAX)
    mins, sums, maxs = mins.cpu().tolist(), sums.cpu().tolist(), maxs.cpu().tolist()
    if not mins[0]:
        return {"gpu_utilization_available": 0}
    out: dict[str, float] = {}
    for i, prefix in enumerate(_UTIL_PREFIXES):
        out[f"{prefix}_min"] = round(mins[2 + i], 2)
        out[f"{prefix}_mean"] = round(sums[i] / world, 2)
        out[f"{prefix}_max"] = round(maxs[i], 2)
    out["gpu_utilization_samples_per_rank_min"] = int(mins[1])
    out["gpu_utilization_available"] = 1
    return out


@dataclass
class ProgressReporter:
    """Uniform progress events (rate, ETA, memory) for bounded loops such as evaluation or probes."""

    event: str
    total: int
    logger: EventLogger
    device: torch.device
    log_interval: int = 1
    unit: str = "batch"
    tokens_goal: int | None = None

    def __post_init__(self) -> None:
        if self.total <= 0:
            raise ValueError("progress total must be positive")
        if self.log_interval <= 0:
            raise ValueError("progress log_interval must be positive")
        self.started_at = self.last_at = time.perf_counter()
        self.processed_items = 0
        self.processed_tokens = 0
        self.last_payload: dict[str, object] = {}
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
            torch.cuda.reset_peak_memory_stats(self.device)
        elif not tracemalloc.is_tracing():
            tracemalloc.start()

    def update(self, completed: int, *, metrics: dict[str, float] | None = None, items: int = 0, tokens: int = 0,
               force: bool = False) -> None:
        self.processed_items += items
        self.processed_tokens += tokens
        boundary = completed in (1, self.total) or completed % self.log_interval == 0
        if not (force or boundary):
            return
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        now = time.perf_counter()
        elapsed = max(now - self.started_at, 1e-12)
        frac = min(max(completed / self.total, 0.0), 1.0)
        eta = elapsed * (1 - frac) / frac if frac > 0 else math.inf
        plural = {"batch": "batches", "example": "examples"}.get(self.unit, f"{self.unit}s")
        payload: dict[str, object] = {
            "event": self.event, "step": completed, self.unit: completed, f"{plural}_total": self.total,
            "progress_percent": round(100 * frac, 3), "elapsed_seconds": round(elapsed, 3),
            "eta_seconds": round(eta, 3) if math.isfinite(eta) else -1.0,
            "items_processed": self.processed_items, "items_per_sec": round(self.processed_items / elapsed, 3),
            "tokens_processed": self.processed_tokens, "tokens_per_sec": round(self.processed_tokens / elapsed, 3),
        }
        if self.tokens_goal is not None:
            payload["tokens_goal"] = self.tokens_goal
        payload.update(metrics or {})
        payload.update(memory_metrics(self.device))
        self.last_payload = payload
        self.logger.log_event(payload)
        self.last_at = now

    def summary(self) -> dict[str, object]:
        return dict(self.last_payload)
