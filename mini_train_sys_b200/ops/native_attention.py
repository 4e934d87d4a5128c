"""Autograd bridge for the tcgen05 FlashAttention kernels (``csrc/attention.cu``)."""

from __future__ import annotations

import torch


def supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, is_causal: bool, dropout_p: float) -> bool:
    """No-load capability predicate, mirrored by the checks at the C++ boundary."""

    return False


def flash_attention(q, k, v, *, is_causal: bool, dropout_p: float) -> torch.Tensor:
    raise NotImplementedError
