"""Expert parallelism: the experts of every MoE layer are sharded ``E / world`` per rank.

The reference has no expert-parallel mode (experts are replicated by DDP or parameter-sharded by FSDP,
minitrain/kernels/README.md:29); this strategy is an addition.

Layout
    dense parameters (attention, norms, router, embedding / head)  data parallel through the flat engine
    expert parameters ``gate_up_proj`` / ``down_proj``                local slice ``[E / world, ...]``, never reduced

A MoE layer then runs: route locally -> *dispatch* every kept route to the rank that owns its expert
(all-to-all of token rows, sorted by destination) -> grouped SwiGLU experts on the receiver through the same
``ops.fused_moe`` the single-GPU path uses -> *return* the rows to their source rank (the inverse all-to-all)
-> weighted sum per token.  Backward is the same two exchanges in reverse, supplied by autograd.

Because every rank's loss is the mean over its own tokens and the global objective is the mean over ranks,
expert gradients (which already collect the tokens of all ranks) are scaled by ``1 / world`` instead of being
all-reduced; the flat engine does that for parameters registered as rank-local.

Capacity: with ``parallel.ep.capacity_factor`` (or ``model.expert_capacity_factor``) set, each expert accepts
at most ``ceil(factor * tokens * top_k / experts)`` routes per rank-local batch; overflow routes are dropped
before the exchange (their weight is zero and they are reported in ``moe/dropped_route_fraction``).
"""

from __future__ import annotations

from dataclasses import replace

import torch
import torch.distributed as dist

from mini_train_sys_b200.models.blocks import MoEFeedForward
from mini_train_sys_b200.parallel.strategy import ProcessGroupMixin


class _AllToAllRows(torch.autograd.Function):
    """Variable-split all-to-all of matrix rows; backward is the all-to-all with the splits swapped."""

    @staticmethod
    def forward(ctx, rows, send_counts, recv_counts):
        ctx.counts = (send_counts, recv_counts)
        out = rows.new_empty(sum(recv_counts), rows.shape[1])
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv_counts, input_split_sizes=send_counts)
        else:
            out.copy_(rows)
        return out

    @staticmethod
    def backward(ctx, grad):
        send_counts, recv_counts = ctx.counts
        out = grad.new_empty(sum(send_counts), grad.shape[1])
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_to_all_single(out, grad.contiguous(), output_split_sizes=send_counts, input_split_sizes=recv_counts)
        else:
            out.copy_(grad)
        return out, None, None


def exchange_counts(per_dest_expert: torch.Tensor, world: int) -> torch.Tensor:
    """``[world, local_experts]`` routes this rank sends -> ``[world, local_experts]`` routes it receives (row = source)."""

    received = torch.empty_like(per_dest_expert)
    if world > 1:
        dist.all_to_all_single(received, per_dest_expert.contiguous())
    else:
        received.copy_(per_dest_expert)
    return received


def expert_parallel_moe(tokens: torch.Tensor, expert_indices: torch.Tensor, expert_weights: torch.Tensor,
                        module: MoEFeedForward, ops) -> torch.Tensor:
    """Dispatch / expert / return / combine for one MoE layer whose module holds only the local experts.

    ``expert_indices`` are global expert ids in ``[0, E)``; negative ids mark dropped routes.
    """

    world = dist.get_world_size() if dist.is_initialized() else 1
    n_local = module.gate_up_proj.shape[0]
    t, k = expert_indices.shape
    flat_e = expert_indices.reshape(-1).long()
    kept = flat_e >= 0
    route_ids = torch.nonzero(kept, as_tuple=False).squeeze(1)
    e_kept = flat_e[route_ids]
    # sort kept routes by (destination rank, local expert); stable, so token order survives inside every group
    order = torch.argsort(e_kept, stable=True)
    route_sorted = route_ids[order]
    counts = torch.bincount(e_kept, minlength=world * n_local).view(world, n_local)
    received = exchange_counts(counts, world)                       # [source rank, local expert]
    send_counts = counts.sum(1).tolist()
    recv_counts = received.sum(1).tolist()
    rows = tokens[route_sorted // k]
    arrived = _AllToAllRows.apply(rows, send_counts, recv_counts)   # grouped by source rank, then by local expert
    # local expert id of every arrived row
    local_expert = torch.repeat_interleave(torch.arange(n_local, device=tokens.device).repeat(world), received.reshape(-1))
    ones = torch.ones(arrived.shape[0], 1, dtype=tokens.dtype, device=tokens.device)
    if arrived.shape[0] > 0:
        y = ops.fused_moe(arrived, module.gate_up_proj, module.down_proj, local_expert.view(-1, 1).to(torch.int32), ones)
    else:   # keep the expert parameters in the autograd graph even when nothing was routed here
        y = arrived + 0.0 * (module.gate_up_proj.sum() + module.down_proj.sum()).to(arrived.dtype)
    back = _AllToAllRows.apply(y, recv_counts, send_counts)         # same order as `rows`
    w = expert_weights.reshape(-1)[route_sorted].unsqueeze(1).to(back.dtype)
    out = torch.zeros_like(tokens)
    return out.index_add(0, route_sorted // k, back * w)


def shard_experts(model: torch.nn.Module, rank: int, world: int) -> list[str]:
    """Replace every MoE layer's expert tensors by this rank's slice; returns the names of the local parameters."""

    local: list[str] = []
    for name, mod in model.named_modules():
        if not isinstance(mod, MoEFeedForward):
            continue
        n_exp = mod.gate_up_proj.shape[0]
        if n_exp % world:
            raise ValueError(f"num_experts={n_exp} is not divisible by the expert-parallel world size {world}")
        per = n_exp // world
        for attr in ("gate_up_proj", "down_proj"):
            full = getattr(mod, attr)
            setattr(mod, attr, torch.nn.Parameter(full.detach()[rank * per:(rank + 1) * per].clone()))
            local.append(f"{name}.{attr}")
        mod.expert_dispatch = expert_parallel_moe
        mod.router.enforce_capacity = mod.cfg.expert_capacity_factor is not None
        mod.router.drop_overflow_routes = True
    return local


class ExpertParallelStrategy(ProcessGroupMixin):
    name = "ep"

    def __init__(self, *, process_group_backend: str = "auto", timeout_minutes: int = 30, engine: str = "nccl", comm=None,
                 ep=None) -> None:
        self.process_group_backend = process_group_backend
        self.timeout_minutes = timeout_minutes
        self.engine = engine
        self.comm = comm
        self.ep = ep

    def resolved_engine(self) -> str:
        return "fused" if self.engine in ("auto", "fused") and torch.cuda.is_available() else "nccl"

    def wrap_model(self, model: torch.nn.Module) -> torch.nn.Module:
        from mini_train_sys_b200.parallel.flat_engine import FlatDataParallel

        if self.ep is not None and self.ep.capacity_factor is not None:
            new_cfg = replace(model.cfg, expert_capacity_factor=self.ep.capacity_factor, expert_min_capacity=self.ep.min_capacity)
            model.cfg = new_cfg
            for mod in model.modules():
                if hasattr(mod, "cfg"):
                    mod.cfg = new_cfg
        local = shard_experts(model, self.rank, self.world_size)
        comm = self.comm if self.resolved_engine() == "fused" else replace(self.comm, engine="nccl") if self.comm else None
        return FlatDataParallel(model, mode="shard", comm=comm, local_params=local)

    def unit_count(self, model) -> int:
        return int(model.unit_count())
