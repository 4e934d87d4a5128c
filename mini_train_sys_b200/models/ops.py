"""Operator boundary between model code and kernels.

The model only ever sees this eight-method protocol (reference contract:
minitrain/model/ops.py:18-90).  Three implementations exist:

* ``reference`` - fp32 restatement used as the numerical oracle in tests,
* ``torch``     - library ops (cuBLAS / SDPA); the measured baseline,
* ``native``    - hand-written sm_100a kernels (the product path).

The reference names ``triton`` and ``cuda`` are accepted as aliases of ``native`` so
that reference run YAMLs keep loading.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Protocol, runtime_checkable

import torch


@dataclass
class RouterPostprocessOutput:
    expert_weights: torch.Tensor          # [T, K] fp32, differentiable
    expert_indices: torch.Tensor          # [T, K] int32
    probability_per_expert: torch.Tensor  # [E] mean full-softmax probability, differentiable
    z_loss: torch.Tensor                  # scalar mean(lse^2), differentiable
    entropy: torch.Tensor                 # scalar, detached
    # Optional, from backends whose routing kernel counts as it goes (no gradient):
    expert_counts: torch.Tensor | None = None   # [E] fp32 routes per expert
    balance_stats: torch.Tensor | None = None   # [5 + E] fp32: max count, min count, load cv, max / mean load, dead experts, load fractions


@runtime_checkable
class OpsBackend(Protocol):
    name: str

    def rmsnorm(self, x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor: ...

    def rope(self, q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor
             ) -> tuple[torch.Tensor, torch.Tensor]: ...

    def swiglu(self, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor: ...

    def attention(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, is_causal: bool,
                  dropout_p: float) -> torch.Tensor: ...

    def cross_entropy(self, logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor: ...

    def fused_linear_cross_entropy(self, x: torch.Tensor, weight: torch.Tensor,
                                   targets: torch.Tensor) -> torch.Tensor: ...

    def router_postprocess(self, logits: torch.Tensor, top_k: int, *, normalize: bool
                           ) -> RouterPostprocessOutput: ...

    def fused_moe(self, x: torch.Tensor, gate_up_proj: torch.Tensor, down_proj: torch.Tensor,
                  top_k_index: torch.Tensor, top_k_weights: torch.Tensor) -> torch.Tensor: ...


OPS_BACKEND_NAMES = ("torch", "reference", "native", "triton", "cuda")
_NATIVE_ALIASES = {"native", "triton", "cuda"}


def get_ops_backend(name: str) -> OpsBackend:
    """Lazy constructor; importing the native backend loads the CUDA extension."""

    if name == "torch":
        from mini_train_sys_b200.ops.torch_backend import TorchOpsBackend

        return TorchOpsBackend()
    if name == "reference":
        from mini_train_sys_b200.ops.reference import ReferenceOpsBackend

        return ReferenceOpsBackend()
    if name in _NATIVE_ALIASES:
        from mini_train_sys_b200.ops.native_backend import NativeOpsBackend

        return NativeOpsBackend()
    raise ValueError(f"Unknown ops backend: {name}")
