"""Precision policy: fp32 parameters always; bf16/fp16 autocast for activations.

``auto`` resolves to bf16 on CUDA (fp16 with loss scaling on devices without bf16) and
fp32 on CPU (reference: minitrain/train/precision.py:16-67).
"""

from __future__ import annotations

from contextlib import nullcontext
from dataclasses import dataclass
from typing import ContextManager

import torch

PRECISION_DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


def recommended_precision(device: torch.device) -> str:
    if device.type != "cuda":
        return "fp32"
    return "bf16" if torch.cuda.is_bf16_supported() else "fp16"


@dataclass(frozen=True)
class PrecisionPolicy:
    name: str
    activation_dtype: torch.dtype
    autocast_enabled: bool
    grad_scaling_enabled: bool

    def autocast_context(self, device: torch.device) -> ContextManager:
        if not self.autocast_enabled:
            return nullcontext()
        return torch.autocast(device_type=device.type, dtype=self.activation_dtype)


def resolve_precision_policy(name: str, device: torch.device) -> PrecisionPolicy:
    key = name.lower()
    if key == "auto":
        key = recommended_precision(device)
    if key not in PRECISION_DTYPES:
        raise ValueError(f"Unknown precision {name!r}; expected one of: auto, " + ", ".join(PRECISION_DTYPES))
    if key == "fp16" and device.type != "cuda":
        raise ValueError("fp16 mixed-precision training is supported only on CUDA")
    if key == "bf16" and device.type == "cuda" and not torch.cuda.is_bf16_supported():
        raise RuntimeError("bf16 was requested, but the selected CUDA device does not support bf16")
    return PrecisionPolicy(key, PRECISION_DTYPES[key], key != "fp32", key == "fp16")
