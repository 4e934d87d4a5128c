"""Architecture description of the Dense / top-k MoE decoder.

Field names and defaults follow the reference schema (minitrain/model/config.py:5-78)
so that every reference model YAML loads unchanged.  Validation is table driven.
"""

from __future__ import annotations

from dataclasses import dataclass, fields


@dataclass(frozen=True)
class ModelConfig:
    vocab_size: int = 32000
    seq_len: int = 2048
    n_layers: int = 12
    n_heads: int = 12
    hidden_size: int = 768
    intermediate_size: int = 2048
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    dropout: float = 0.0
    tie_word_embeddings: bool = False
    ffn_type: str = "dense"
    num_experts: int = 8
    experts_per_token: int = 2
    router_aux_loss_coef: float = 1e-2
    router_z_loss_coef: float = 1e-3
    router_normalize_topk: bool = True
    router_jitter_noise: float = 0.0
    # Capacity-aware routing.  ``None`` keeps the dropless behaviour of the
    # reference; the expert-parallel strategy reads these two fields to size its
    # receive buffers and to drop overflow routes.
    expert_capacity_factor: float | None = None
    expert_min_capacity: int = 4

    def __post_init__(self) -> None:
        for name in ("vocab_size", "seq_len", "n_layers", "n_heads", "hidden_size", "intermediate_size"):
            if getattr(self, name) <= 0:
                raise ValueError(f"all model dimensions must be positive (got {name}={getattr(self, name)})")
        if not (0.0 <= self.dropout < 1.0):
            raise ValueError("dropout must be in [0, 1)")
        if self.norm_eps <= 0 or self.rope_theta <= 0:
            raise ValueError("norm_eps and rope_theta must be positive")
        if self.ffn_type not in ("dense", "moe"):
            raise ValueError("ffn_type must be either 'dense' or 'moe'")
        if self.hidden_size % self.n_heads:
            raise ValueError("hidden_size must be divisible by n_heads")
        if self.ffn_type != "moe":
            return
        if self.num_experts <= 0:
            raise ValueError("num_experts must be positive")
        if not (0 < self.experts_per_token <= self.num_experts):
            raise ValueError("experts_per_token must be in [1, num_experts]")
        if self.router_aux_loss_coef < 0:
            raise ValueError("router_aux_loss_coef must be non-negative")
        if self.router_z_loss_coef < 0:
            raise ValueError("router_z_loss_coef must be non-negative")
        if not (0.0 <= self.router_jitter_noise < 1.0):
            raise ValueError("router_jitter_noise must be in [0, 1)")
        if self.expert_capacity_factor is not None and self.expert_capacity_factor <= 0:
            raise ValueError("expert_capacity_factor must be positive or null")
        if self.expert_min_capacity <= 0:
            raise ValueError("expert_min_capacity must be positive")

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.n_heads

    @property
    def is_moe(self) -> bool:
        return self.ffn_type == "moe"

    # ---- derived sizes used by the sharding planners and the benchmark -----
    def block_param_count(self) -> int:
        h, i = self.hidden_size, self.intermediate_size
        attn = 4 * h * h + 2 * h  # qkv + out + two norms
        if self.is_moe:
            return attn + self.num_experts * (h + 3 * h * i)
        return attn + 3 * h * i

    def param_count(self) -> int:
        root = self.vocab_size * self.hidden_size + self.hidden_size
        if not self.tie_word_embeddings:
            root += self.vocab_size * self.hidden_size
        return root + self.n_layers * self.block_param_count()

    def active_param_count(self) -> int:
        """Parameters touched per token (top-k experts only) excluding the embedding gather."""

        h, i = self.hidden_size, self.intermediate_size
        ffn = 3 * h * i * (self.experts_per_token if self.is_moe else 1)
        router = self.num_experts * h if self.is_moe else 0
        return self.n_layers * (4 * h * h + ffn + router) + self.vocab_size * h

    def flops_per_token(self) -> float:
        """Training FLOPs per token: 6·active params + causal attention (fwd+bwd)."""

        attn = 6 * self.n_layers * self.seq_len * self.hidden_size  # 12·L·S·H halved by causality
        return 6.0 * self.active_param_count() + attn

    @classmethod
    def field_names(cls) -> tuple[str, ...]:
        return tuple(f.name for f in fields(cls))


@dataclass(frozen=True)
class MoEModelConfig(ModelConfig):
    """Same schema with ``ffn_type`` defaulting to ``moe``."""

    ffn_type: str = "moe"
