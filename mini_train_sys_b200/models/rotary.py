"""Rotary position cache (half-split / HF-LLaMA convention).

Angles are built once in fp32 and stored in the activation dtype as non-persistent
buffers, so checkpoints never contain them (reference: minitrain/model/rotary.py:6-46).
"""

from __future__ import annotations

import torch
from torch import nn


def rope_tables(head_dim: int, max_seq_len: int, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 ``cos``/``sin`` tables of shape ``[max_seq_len, head_dim]`` (two identical halves)."""

    if head_dim % 2:
        raise ValueError("RoPE requires an even head_dim")
    exponent = torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim
    inv_freq = 1.0 / (theta ** exponent)
    phase = torch.outer(torch.arange(max_seq_len, dtype=torch.float32), inv_freq)
    phase = torch.cat((phase, phase), dim=-1)
    return phase.cos(), phase.sin()


class RotaryEmbedding(nn.Module):
    def __init__(self, head_dim: int, max_seq_len: int, theta: float, *, cache_dtype: torch.dtype) -> None:
        super().__init__()
        cos, sin = rope_tables(head_dim, max_seq_len, theta)
        self.register_buffer("cos", cos.to(cache_dtype), persistent=False)
        self.register_buffer("sin", sin.to(cache_dtype), persistent=False)

    @property
    def max_seq_len(self) -> int:
        return int(self.cos.shape[0])

    def forward(self, seq_len: int) -> tuple[torch.Tensor, torch.Tensor]:
        if seq_len > self.max_seq_len:
            raise ValueError(f"seq_len={seq_len} exceeds configured max seq_len={self.max_seq_len}")
        return self.cos[:seq_len], self.sin[:seq_len]
