"""Top-k token router (dropless by default, optional capacity limit).

Semantics follow minitrain/model/moe_router.py:13-144: the router runs in fp32 outside
autocast, the auxiliary load-balancing loss uses non-differentiable assignment counts
times the differentiable mean probability, and a dictionary of balance metrics is
published per layer.  The module boundary is kept (``block.ffn.router``) so analysis
code can attach forward hooks and read ``expert_indices``.

Unlike the reference, a finite ``expert_capacity_factor`` is honoured here when
``enforce_capacity`` is switched on (the expert-parallel strategy does that): routes
ranked beyond the per-expert capacity get weight zero and are reported as dropped.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from mini_train_sys_b200.models.config import ModelConfig
from mini_train_sys_b200.models.ops import OpsBackend


@dataclass
class RouterOutput:
    expert_indices: torch.Tensor
    expert_weights: torch.Tensor
    auxiliary_loss: torch.Tensor
    z_loss: torch.Tensor
    metrics: dict[str, torch.Tensor]


def expert_capacity(cfg: ModelConfig, tokens: int) -> int | None:
    """Rows one expert accepts for ``tokens`` routed tokens, or ``None`` when dropless."""

    if cfg.expert_capacity_factor is None:
        return None
    even = tokens * cfg.experts_per_token / cfg.num_experts
    return max(cfg.expert_min_capacity, math.ceil(cfg.expert_capacity_factor * even))


def route_histogram(indices: torch.Tensor, bins: int, weights: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 counts (or weight sums) per bin without a device-to-host round trip: ``torch.bincount`` reads the maximum index
    back to size its output, which stalls the launch queue; ``scatter_add_`` into a tensor of known size does not."""

    flat = indices.reshape(-1).long()
    src = torch.ones_like(flat, dtype=torch.float32) if weights is None else weights.reshape(-1).float()
    return torch.zeros(bins, dtype=torch.float32, device=flat.device).scatter_add_(0, flat, src)


def capacity_keep_mask(expert_indices: torch.Tensor, expert_weights: torch.Tensor, num_experts: int,
                       capacity: int | None) -> torch.Tensor:
    """Boolean ``[T, K]`` mask of routes that fit within ``capacity`` rows per expert.

    Within an expert, routes are admitted in order of decreasing weight (ties by
    flattened position), which is what minitrain/model/moe_router.py:29-61 describes.
    """

    if capacity is None:
        return torch.ones_like(expert_weights, dtype=torch.bool)
    flat_e = expert_indices.reshape(-1).long()
    flat_w = expert_weights.reshape(-1).float()
    # One composite key sorts by expert first, then by descending weight.
    order = torch.argsort(flat_w, descending=True, stable=True)
    order = order[torch.argsort(flat_e[order], stable=True)]
    counts = route_histogram(flat_e, num_experts).long()
    starts = torch.cumsum(counts, 0) - counts
    rank = torch.arange(order.numel(), device=order.device) - starts[flat_e[order]]
    keep = torch.empty_like(flat_e, dtype=torch.bool)
    keep[order] = rank < capacity
    return keep.view_as(expert_weights)


class TopKRouter(nn.Module):
    def __init__(self, cfg: ModelConfig) -> None:
        super().__init__()
        self.cfg = cfg
        self.weight = nn.Parameter(torch.empty(cfg.num_experts, cfg.hidden_size))
        nn.init.normal_(self.weight, mean=0.0, std=0.02)
        self.enforce_capacity = False
        self.drop_overflow_routes = False   # expert parallelism: mark dropped routes with index -1 so they are not sent

    def forward(self, hidden_states: torch.Tensor, ops: OpsBackend) -> RouterOutput:
        cfg = self.cfg
        n_exp = cfg.num_experts
        jitter = self.training and cfg.router_jitter_noise
        fused_logits = None if jitter else getattr(ops, "router_logits", None)   # optional backend hook

        with torch.autocast(device_type=hidden_states.device.type, enabled=False):
            if fused_logits is not None:
                logits = fused_logits(hidden_states, self.weight)
            else:
                x32 = hidden_states.float()
                if jitter:
                    span = cfg.router_jitter_noise
                    x32 = x32 * torch.empty_like(x32).uniform_(1.0 - span, 1.0 + span)
                logits = F.linear(x32, self.weight.float())
            post = ops.router_postprocess(logits, cfg.experts_per_token, normalize=cfg.router_normalize_topk)
            weights, indices = post.expert_weights, post.expert_indices
            n_routes = indices.numel()
            # Routes per expert: from the routing kernel when it counts as it goes, else a histogram that needs no
            # device-to-host round trip.
            counts = getattr(post, "expert_counts", None)
            balance = getattr(post, "balance_stats", None)
            if counts is None:
                counts = route_histogram(indices, n_exp)
            # Assignment fractions carry no gradient; the probability mean does.
            aux = torch.dot(counts, post.probability_per_expert) * (n_exp / n_routes)

            dropped = weights.new_zeros(())
            if self.enforce_capacity and cfg.expert_capacity_factor is not None:
                keep = capacity_keep_mask(indices, weights, n_exp, expert_capacity(cfg, indices.shape[0]))
                weights = weights * keep
                if cfg.router_normalize_topk:
                    denom = weights.sum(-1, keepdim=True)
                    weights = torch.where(denom > 0, weights / denom.clamp_min(torch.finfo(weights.dtype).eps), weights)
                dropped = 1.0 - keep.float().mean()
                counts = route_histogram(indices, n_exp, keep)
                balance = None                       # the kernel's figures describe the routing before the capacity limit
                if self.drop_overflow_routes:
                    indices = torch.where(keep, indices, torch.full_like(indices, -1))

            log_e = math.log(n_exp) if n_exp > 1 else 1.0
            metrics = {
                "moe/router_entropy": post.entropy,
                "moe/router_entropy_normalized": (post.entropy / log_e).detach(),
                "moe/dropped_route_fraction": dropped.detach(),
            }
            if balance is not None:                  # slices of one small tensor: no launches
                metrics.update({
                    "moe/max_expert_load": balance[0], "moe/min_expert_load": balance[1], "moe/expert_load_cv": balance[2],
                    "moe/max_to_mean_load": balance[3], "moe/dead_expert_count": balance[4],
                    "moe/expert_load_fraction": balance[5:],
                })
            else:
                load = counts / max(n_routes, 1)
                uniform = 1.0 / n_exp
                metrics.update({
                    "moe/max_expert_load": counts.max().detach(),
                    "moe/min_expert_load": counts.min().detach(),
                    "moe/expert_load_cv": (load.std(unbiased=False) / uniform).detach(),
                    "moe/max_to_mean_load": (load.max() / uniform).detach(),
                    "moe/dead_expert_count": (counts == 0).sum().detach(),
                    "moe/expert_load_fraction": load.detach(),
                })
            # per-expert vectors are stacked over layers into [layer, expert] heatmaps by the logger
            metrics["moe/expert_probability"] = post.probability_per_expert.detach()
        return RouterOutput(
            expert_indices=indices.to(torch.int32),
            expert_weights=weights.to(hidden_states.dtype),
            auxiliary_loss=aux,
            z_loss=post.z_loss,
            metrics=metrics,
        )
