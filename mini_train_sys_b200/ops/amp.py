"""Autocast helpers: cast activations (never parameters) to the active CUDA autocast dtype."""

from __future__ import annotations

import torch

_LOW = (torch.float16, torch.bfloat16)


def autocast_dtype(device_type: str = "cuda") -> torch.dtype | None:
    if not torch.is_autocast_enabled(device_type):
        return None
    dtype = torch.get_autocast_dtype(device_type)
    if dtype not in _LOW:
        raise RuntimeError(f"Unsupported autocast activation dtype: {dtype}")
    return dtype


def cast_activations(*tensors: torch.Tensor) -> tuple[torch.Tensor, ...]:
    dtype = autocast_dtype("cuda")
    if dtype is None:
        return tensors
    return tuple(t.to(dtype) if (t.is_cuda and t.is_floating_point() and t.dtype != dtype) else t for t in tensors)


# the names the reference's helper module uses (minitrain/kernels/amp.py:7-36)
cuda_autocast_activation_dtype = lambda: autocast_dtype("cuda")   # noqa: E731
cast_cuda_autocast_activations = cast_activations
