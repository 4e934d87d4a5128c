"""Device selection: ``cuda:{LOCAL_RANK}`` when CUDA is present, else CPU."""

from __future__ import annotations

import os

import torch


def local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", "0"))


def get_default_device() -> torch.device:
    return torch.device("cuda", local_rank()) if torch.cuda.is_available() else torch.device("cpu")


def resolve_device(name: str) -> torch.device:
    if name == "auto":
        return get_default_device()
    if name == "cpu":
        return torch.device("cpu")
    if name == "cuda":
        if not torch.cuda.is_available():
            raise RuntimeError("--device cuda was requested, but CUDA is not available")
        return torch.device("cuda", local_rank())
    raise ValueError(f"Unknown device: {name}")
