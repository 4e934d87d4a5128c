"""Transformer building blocks: RMSNorm, causal attention, dense SwiGLU FFN, MoE FFN.

Parameter names, shapes, construction order and initialisation match the reference
(minitrain/model/blocks.py:13-136) so that state dicts interchange and a given seed
produces the same initial weights.  All heavy math goes through the ``OpsBackend``.

Projections call ``ops.linear`` when the backend provides one (the native backend
routes them to its tcgen05 GEMM); otherwise the ``nn.Linear`` module runs as is.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch import nn

from mini_train_sys_b200.models.config import ModelConfig
from mini_train_sys_b200.models.ops import OpsBackend
from mini_train_sys_b200.models.router import TopKRouter


@dataclass
class FeedForwardOutput:
    hidden_states: torch.Tensor
    router_aux_loss: torch.Tensor | None = None
    router_z_loss: torch.Tensor | None = None
    router_metrics: dict[str, torch.Tensor] | None = None


def project(ops: OpsBackend, layer: nn.Linear, x: torch.Tensor) -> torch.Tensor:
    """``x @ W^T`` through the backend GEMM if it has one, else through the module."""

    fn = getattr(ops, "linear", None)
    return layer(x) if fn is None else fn(x, layer.weight)


def add_dropped(ops: OpsBackend, drop: nn.Dropout, y: torch.Tensor, residual: torch.Tensor | None) -> torch.Tensor:
    """``residual + dropout(y)``; one fused pass when the backend offers ``dropout_add``, and plain ``dropout(y)`` when the
    caller keeps the residual sum to itself (``residual is None``)."""

    if residual is None:
        return drop(y)
    fused = getattr(ops, "dropout_add", None)
    if fused is not None and y.is_cuda:
        return fused(y, residual, drop.p if drop.training else 0.0)
    return residual + drop(y)


def _scaled_std(cfg: ModelConfig) -> float:
    return 0.02 / math.sqrt(2 * cfg.n_layers)


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.eps = eps

    def forward(self, x: torch.Tensor, ops: OpsBackend) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps)

    def with_residual(self, x: torch.Tensor, ops: OpsBackend) -> tuple[torch.Tensor, torch.Tensor]:
        """``(norm(x), x)`` for a pre-norm block.  A backend that offers ``rmsnorm_residual`` returns its own handle on x,
        through which the residual branch's gradient comes back into the norm's backward kernel."""

        fused = getattr(ops, "rmsnorm_residual", None)
        if fused is not None and x.is_cuda:
            return fused(x, self.weight, self.eps)
        return ops.rmsnorm(x, self.weight, self.eps), x


class CausalSelfAttention(nn.Module):
    def __init__(self, cfg: ModelConfig) -> None:
        super().__init__()
        self.cfg = cfg
        h = cfg.hidden_size
        self.qkv = nn.Linear(h, 3 * h, bias=False)
        self.out = nn.Linear(h, h, bias=False)
        self.resid_dropout = nn.Dropout(cfg.dropout)
        nn.init.normal_(self.qkv.weight, mean=0.0, std=0.02)
        nn.init.normal_(self.out.weight, mean=0.0, std=_scaled_std(cfg))

    def forward(self, x: torch.Tensor, ops: OpsBackend, rope_cos: torch.Tensor, rope_sin: torch.Tensor,
                residual: torch.Tensor | None = None) -> torch.Tensor:
        b, s, h = x.shape
        nh, hd = self.cfg.n_heads, self.cfg.head_dim
        # [B, S, 3, heads, D] -> three strided [B, heads, S, D] views of the fused projection
        fused = project(ops, self.qkv, x).view(b, s, 3, nh, hd)
        p = self.cfg.dropout if self.training else 0.0
        ctx = None
        fused_path = getattr(ops, "attention_qkv", None)   # optional backend hook: RoPE + attention in one node
        if fused_path is not None:
            ctx = fused_path(fused, rope_cos, rope_sin, is_causal=True, dropout_p=p)
        if ctx is None:
            q, k, v = (fused[:, :, j].transpose(1, 2) for j in range(3))
            q, k = ops.rope(q, k, rope_cos, rope_sin)
            ctx = ops.attention(q, k, v, is_causal=True, dropout_p=p)
        ctx = ctx.transpose(1, 2).contiguous().view(b, s, h)
        return add_dropped(ops, self.resid_dropout, project(ops, self.out, ctx), residual)


class DenseFeedForward(nn.Module):
    def __init__(self, cfg: ModelConfig) -> None:
        super().__init__()
        h, i = cfg.hidden_size, cfg.intermediate_size
        self.gate = nn.Linear(h, i, bias=False)
        self.up = nn.Linear(h, i, bias=False)
        self.down = nn.Linear(i, h, bias=False)
        self.dropout = nn.Dropout(cfg.dropout)
        nn.init.normal_(self.gate.weight, mean=0.0, std=0.02)
        nn.init.normal_(self.up.weight, mean=0.0, std=0.02)
        nn.init.normal_(self.down.weight, mean=0.0, std=_scaled_std(cfg))

    def forward(self, x: torch.Tensor, ops: OpsBackend, residual: torch.Tensor | None = None) -> FeedForwardOutput:
        act = ops.swiglu(project(ops, self.gate, x), project(ops, self.up, x))
        return FeedForwardOutput(add_dropped(ops, self.dropout, project(ops, self.down, act), residual))


class MoEFeedForward(nn.Module):
    """Routed SwiGLU experts: ``gate_up_proj [E, 2I, H]`` and ``down_proj [E, H, I]``."""

    def __init__(self, cfg: ModelConfig) -> None:
        super().__init__()
        self.cfg = cfg
        e, h, i = cfg.num_experts, cfg.hidden_size, cfg.intermediate_size
        self.router = TopKRouter(cfg)
        self.gate_up_proj = nn.Parameter(torch.empty(e, 2 * i, h))
        self.down_proj = nn.Parameter(torch.empty(e, h, i))
        self.dropout = nn.Dropout(cfg.dropout)
        nn.init.normal_(self.gate_up_proj, mean=0.0, std=0.02)
        nn.init.normal_(self.down_proj, mean=0.0, std=_scaled_std(cfg))
        # Set by the expert-parallel strategy: callable(x, indices, weights, module) -> y
        self.expert_dispatch = None

    def forward(self, x: torch.Tensor, ops: OpsBackend, residual: torch.Tensor | None = None) -> FeedForwardOutput:
        tokens = x.reshape(-1, x.shape[-1])
        route = self.router(tokens, ops)
        if self.expert_dispatch is not None:
            mixed = self.expert_dispatch(tokens, route.expert_indices, route.expert_weights, self, ops)
        else:
            mixed = ops.fused_moe(tokens, self.gate_up_proj, self.down_proj,
                                  route.expert_indices, route.expert_weights)
        return FeedForwardOutput(
            hidden_states=add_dropped(ops, self.dropout, mixed.view(x.shape), residual),
            router_aux_loss=route.auxiliary_loss,
            router_z_loss=route.z_loss,
            router_metrics=route.metrics,
        )


def build_feed_forward(cfg: ModelConfig) -> nn.Module:
    return MoEFeedForward(cfg) if cfg.is_moe else DenseFeedForward(cfg)


class TransformerBlock(nn.Module):
    """Pre-norm residual block; this is also the FSDP sharding unit."""

    def __init__(self, cfg: ModelConfig) -> None:
        super().__init__()
        self.attn_norm = RMSNorm(cfg.hidden_size, cfg.norm_eps)
        self.attn = CausalSelfAttention(cfg)
        self.ffn_norm = RMSNorm(cfg.hidden_size, cfg.norm_eps)
        self.ffn = build_feed_forward(cfg)

    # legacy attribute names used by some analysis code
    mlp_norm = property(lambda self: self.ffn_norm)
    mlp = property(lambda self: self.ffn)

    def forward(self, x: torch.Tensor, ops: OpsBackend, rope_cos: torch.Tensor, rope_sin: torch.Tensor) -> FeedForwardOutput:
        h, res = self.attn_norm.with_residual(x, ops)
        x = self.attn(h, ops, rope_cos, rope_sin, residual=res)
        h, res = self.ffn_norm.with_residual(x, ops)
        return self.ffn(h, ops, residual=res)      # hidden_states already include the residual


SwiGLUMLP = DenseFeedForward
