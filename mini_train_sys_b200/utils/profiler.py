"""Peak-memory helpers, CUDA-event timers and NVTX ranges (enabled with MTS_NVTX=1)."""

from __future__ import annotations

import contextlib
import os

import torch

_NVTX = os.environ.get("MTS_NVTX", "0") == "1"


def reset_cuda_peak_memory() -> None:
    if torch.cuda.is_available():
        torch.cuda.reset_peak_memory_stats()


def cuda_peak_memory_mb() -> float:
    return torch.cuda.max_memory_allocated() / 2**20 if torch.cuda.is_available() else 0.0


@contextlib.contextmanager
def nvtx_range(name: str):
    if _NVTX and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class CudaTimer:
    """Device-side interval timer on the current stream; ``elapsed_ms`` synchronises the end event."""

    def __init__(self) -> None:
        self._start = torch.cuda.Event(enable_timing=True)
        self._stop = torch.cuda.Event(enable_timing=True)

    def start(self) -> None:
        self._start.record()

    def stop(self) -> None:
        self._stop.record()

    def elapsed_ms(self) -> float:
        self._stop.synchronize()
        return self._start.elapsed_time(self._stop)
