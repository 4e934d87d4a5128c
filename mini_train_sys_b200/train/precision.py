"""Precision policy of a run: what dtype flows between operators, and whether the loss is scaled.

Parameters and optimizer state are fp32 under every policy; a policy only decides the autocast dtype of activations.
The public contract is the reference's (minitrain/train/precision.py:16-67): ``resolve_precision_policy(name, device)``
returns a ``PrecisionPolicy(name, activation_dtype, autocast_enabled, grad_scaling_enabled)`` and refuses impossible
requests with the same messages.  Here the policies are rows of one table, and each row also says which parts of this
framework can run under it (the native sm_100a kernels and the fused sharding engine are bf16-only; see
``PrecisionPolicy.native_kernels`` and ``PrecisionPolicy.fused_engine``), so that callers ask the policy instead of
comparing strings.
"""

from __future__ import annotations

import contextlib
from dataclasses import dataclass
from typing import ContextManager, NamedTuple

import torch


class _Row(NamedTuple):
    dtype: torch.dtype
    autocast: bool
    loss_scaling: bool
    native_kernels: bool       # the sm_100a back end computes in this dtype (fp32 inputs are accepted by a few operators only)
    fused_engine: bool         # the flat sharding engine can drive it (it takes no host decision per step, so no loss scaler)


_TABLE: dict[str, _Row] = {
    "fp32": _Row(torch.float32, autocast=False, loss_scaling=False, native_kernels=False, fused_engine=True),
    "bf16": _Row(torch.bfloat16, autocast=True, loss_scaling=False, native_kernels=True, fused_engine=True),
    "fp16": _Row(torch.float16, autocast=True, loss_scaling=True, native_kernels=False, fused_engine=False),
}
PRECISION_DTYPES = {name: row.dtype for name, row in _TABLE.items()}


def _device_has_bf16(device: torch.device) -> bool:
    return device.type != "cuda" or torch.cuda.is_bf16_supported()


def recommended_precision(device: torch.device) -> str:
    """``auto``: bf16 on a GPU that has it (every B200), fp16 with loss scaling on one that does not, fp32 on a CPU."""

    if device.type == "cuda":
        return "bf16" if _device_has_bf16(device) else "fp16"
    return "fp32"


@dataclass(frozen=True)
class PrecisionPolicy:
    name: str
    activation_dtype: torch.dtype
    autocast_enabled: bool
    grad_scaling_enabled: bool

    @property
    def native_kernels(self) -> bool:
        return _TABLE[self.name].native_kernels

    @property
    def fused_engine(self) -> bool:
        return _TABLE[self.name].fused_engine

    def autocast_context(self, device: torch.device) -> ContextManager:
        if self.autocast_enabled:
            return torch.autocast(device_type=device.type, dtype=self.activation_dtype)
        return contextlib.nullcontext()


def precision_supports_fused_engine(name: str) -> bool:
    """Whether a resolved precision name (``bf16`` / ``fp16`` / ``fp32``; ``auto`` counts as what it usually resolves to on a
    GPU) can run under the fused sharding engine."""

    row = _TABLE.get("bf16" if name.lower() == "auto" else name.lower())
    return row is not None and row.fused_engine


def resolve_precision_policy(name: str, device: torch.device) -> PrecisionPolicy:
    key = recommended_precision(device) if name.lower() == "auto" else name.lower()
    row = _TABLE.get(key)
    if row is None:
        raise ValueError(f"Unknown precision {name!r}; expected one of: auto, " + ", ".join(_TABLE))
    if row.loss_scaling and device.type != "cuda":
        raise ValueError("fp16 mixed-precision training is supported only on CUDA")
    if key == "bf16" and not _device_has_bf16(device):
        raise RuntimeError("bf16 was requested, but the selected CUDA device does not support bf16")
    return PrecisionPolicy(key, row.dtype, row.autocast, row.loss_scaling)
