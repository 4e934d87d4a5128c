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



# ---------------------------------------------------------------------------------------------------------
# peer-memory exchange (fused engine): rows are stored straight into the owning rank's receive regions
# ---------------------------------------------------------------------------------------------------------

class PeerExchange:
    """Symmetric buffers, flags and epochs of the row exchange; one instance serves every MoE layer of a model.

    Receive layout on each rank: ``world`` regions of ``cap_rows`` rows, region ``s`` filled by source rank ``s``.  A source
    that has more than ``cap_rows`` routes for one destination drops the excess (counted in ``overflow``); with the default
    factor the regions hold twice the balanced load, and a capacity factor on the router bounds the load exactly.
    Buffer reuse across layers is ordered by the exchange itself: a rank writes a peer's region for layer L+1 only after that
    peer signalled the step of layer L that consumed the region (see the comments in ``csrc/comm.cu``).
    """

    CH_X, CH_Y, CH_DY, CH_DX = 0, 1, 2, 3

    def __init__(self, device: torch.device, hidden: int, cap_rows: int, *, timeout_ms: float = 2000.0, max_ctas: int = 296) -> None:
        from mini_train_sys_b200.ops.native_backend import ext
        from mini_train_sys_b200.parallel.comm import PeerCollectives

        self.ext = ext()
        self.device, self.hidden, self.cap = device, hidden, int(cap_rows)
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.timeout_ms, self.max_ctas = float(timeout_ms), int(max_ctas)
        alloc = PeerCollectives.alloc.__get__(self)        # same symmetric allocator; needs .world / .device / ._keep / .use_multimem
        self._keep, self.use_multimem = [], False
        rows = self.world * self.cap
        self.recv_x = alloc(rows * hidden, torch.bfloat16, shared=True)
        self.y_buf = alloc(rows * hidden, torch.bfloat16, shared=True)
        self.recv_dy = alloc(rows * hidden, torch.bfloat16, shared=True)
        self.dx_buf = alloc(rows * hidden, torch.bfloat16, shared=True)
        self.recv_e = alloc(rows, torch.int32, shared=True)
        self.recv_cnt = alloc(max(self.world, 64), torch.int32, shared=True)
        self.flags = alloc(4 * self.world, torch.int32, shared=True)
        self.status = self.ext.status_tensor(device.index or 0)
        self.epoch = [0, 0, 0, 0]
        self.overflow = torch.zeros((), dtype=torch.int64, device=device)

    def rendezvous(self, channel: int) -> None:
        """Tell every peer that this rank's stores of the phase are done, then wait (on the device, bounded) for theirs."""

        self.epoch[channel] += 1
        if self.world == 1:
            return
        self.ext.comm_signal(self.flags.peer_ptrs, channel, self.rank, self.epoch[channel], self.flags.tensor)
        self.ext.comm_wait(self.flags.tensor, channel, self.world, self.epoch[channel], self.timeout_ms, self.status)

    def rows_view(self, buf) -> torch.Tensor:
        return buf.tensor[: self.world * self.cap * self.hidden].view(self.world * self.cap, self.hidden)


class ExchangeHolder:
    """Creates the exchange on first use (the region size depends on the batch: routes per rank x ``region_factor`` / world,
    never more than all routes) and re-creates it if a larger batch shows up.  Creation is collective: every rank reaches the
    first MoE layer of a step with the same batch shape."""

    def __init__(self, *, region_factor: float = 2.0, timeout_ms: float = 2000.0) -> None:
        self.region_factor, self.timeout_ms = float(region_factor), float(timeout_ms)
        self.exchange: PeerExchange | None = None

    def get(self, device: torch.device, hidden: int, routes: int) -> PeerExchange:
        world = dist.get_world_size() if dist.is_initialized() else 1
        want = min(routes, -(-int(self.region_factor * routes) // world))
        want = -(-want // 256) * 256
        if self.exchange is None or self.exchange.cap < want or self.exchange.hidden != hidden:
            self.exchange = PeerExchange(device, hidden, want, timeout_ms=self.timeout_ms)
        return self.exchange


def _route_layout(expert_indices: torch.Tensor, n_local: int, world: int, cap: int):
    """Per route (flattened ``[T * K]``): destination rank (-1 = dropped), slot inside the (source -> destination) region,
    expert id local to the destination; plus routes per destination.  Device ops only, no host synchronisation."""

    flat = expert_indices.reshape(-1).long()
    kept = flat >= 0
    dest = torch.where(kept, flat // n_local, torch.full_like(flat, world))
    order = torch.argsort(dest, stable=True)
    counts = torch.zeros(world + 1, dtype=torch.long, device=flat.device).scatter_add_(0, dest, torch.ones_like(dest))[:world]
    starts = torch.cumsum(counts, 0) - counts
    ds = dest[order]
    slot_sorted = torch.arange(flat.numel(), device=flat.device) - torch.cat([starts, starts.new_zeros(1)])[ds]
    slot = torch.empty_like(flat)
    slot[order] = slot_sorted
    over = kept & (slot >= cap)
    dest = torch.where(kept & ~over, dest, torch.full_like(dest, -1))
    return dest.int(), slot.clamp(max=cap - 1).int(), (flat % n_local).int(), counts.clamp(max=cap).int(), over.sum()


class _PeerDispatchFn(torch.autograd.Function):
    """tokens -> rows at the experts' ranks (forward: push; backward: pull of the row gradients)."""

    @staticmethod
    def forward(ctx, tokens, ex: PeerExchange, dest, slot, local_expert, counts, k):
        t = tokens.shape[0]
        route_token = (torch.arange(dest.numel(), device=tokens.device) // k).int()
        ex.ext.ep_push_rows(tokens.contiguous(), route_token, dest, slot, local_expert, None, ex.recv_x.peer_ptrs, ex.recv_e.peer_ptrs,
                            counts, ex.recv_cnt.peer_ptrs, ex.rank, ex.cap, ex.max_ctas)
        ex.rendezvous(ex.CH_X)
        ctx.ex, ctx.shape, ctx.k = ex, (t, tokens.shape[1]), k
        ctx.save_for_backward(dest, slot)
        return ex.rows_view(ex.recv_x)   # a view of the receive buffer: consumers copy what they keep (the expert op gathers)

    @staticmethod
    def backward(ctx, d_arrived):
        ex, (t, h), k = ctx.ex, ctx.shape, ctx.k
        dest, slot = ctx.saved_tensors
        ex.rows_view(ex.dx_buf).copy_(d_arrived)
        ex.rendezvous(ex.CH_DX)
        d_tokens = torch.empty(t, h, dtype=torch.bfloat16, device=d_arrived.device)
        ex.ext.ep_pull_combine(d_tokens, dest.view(t, k), slot.view(t, k), None, ex.dx_buf.peer_ptrs, ex.rank, ex.cap, None, ex.max_ctas)
        return d_tokens, None, None, None, None, None, None


class _PeerCombineFn(torch.autograd.Function):
    """expert outputs at the experts' ranks + routing weights -> per-token sums at the source (forward: pull; backward: push)."""

    @staticmethod
    def forward(ctx, y, weights, ex: PeerExchange, dest, slot, t, k):
        ex.rows_view(ex.y_buf).copy_(y)
        ex.rendezvous(ex.CH_Y)
        out = torch.empty(t, ex.hidden, dtype=torch.bfloat16, device=y.device)
        saved = torch.empty(t * k, ex.hidden, dtype=torch.bfloat16, device=y.device)
        w32 = weights.reshape(t, k).float().contiguous()
        ex.ext.ep_pull_combine(out, dest.view(t, k), slot.view(t, k), w32, ex.y_buf.peer_ptrs, ex.rank, ex.cap, saved, ex.max_ctas)
        ctx.ex, ctx.dims, ctx.w_dtype = ex, (t, k), weights.dtype
        ctx.save_for_backward(saved, w32, dest, slot)
        return out

    @staticmethod
    def backward(ctx, dout):
        ex, (t, k) = ctx.ex, ctx.dims
        saved, w32, dest, slot = ctx.saved_tensors
        go = dout.contiguous()
        dw = (go.float().unsqueeze(1) * saved.view(t, k, -1).float()).sum(-1)
        dw = torch.where(dest.view(t, k) >= 0, dw, torch.zeros_like(dw))
        route_token = (torch.arange(t * k, device=go.device) // k).int()
        ex.ext.ep_push_rows(go, route_token, dest, slot, None, w32.reshape(-1), ex.recv_dy.peer_ptrs, ex.recv_dy.peer_ptrs, None,
                            ex.recv_cnt.peer_ptrs, ex.rank, ex.cap, ex.max_ctas)
        ex.rendezvous(ex.CH_DY)
        return ex.rows_view(ex.recv_dy).detach(), dw.to(ctx.w_dtype).view_as(w32), None, None, None, None, None


def expert_parallel_moe_peer(tokens: torch.Tensor, expert_indices: torch.Tensor, expert_weights: torch.Tensor,
                             module: MoEFeedForward, ops) -> torch.Tensor:
    """Same contract as ``expert_parallel_moe``; the two exchanges are own kernels over peer memory."""

    n_local = module.gate_up_proj.shape[0]
    t, k = expert_indices.shape
    ex: PeerExchange = module._ep_exchange.get(tokens.device, tokens.shape[1], t * k)
    dest, slot, local_expert, counts, over = _route_layout(expert_indices, n_local, ex.world, ex.cap)
    ex.overflow += over
    arrived = _PeerDispatchFn.apply(tokens.to(torch.bfloat16), ex, dest, slot, local_expert, counts, k)
    valid = torch.arange(ex.cap, device=tokens.device)[None, :] < ex.recv_cnt.tensor[: ex.world, None]
    idx = torch.where(valid, ex.recv_e.tensor[: ex.world * ex.cap].view(ex.world, ex.cap), torch.full_like(valid, -1, dtype=torch.int32))
    ones = torch.ones(ex.world * ex.cap, 1, dtype=torch.float32, device=tokens.device)
    y = ops.fused_moe(arrived, module.gate_up_proj, module.down_proj, idx.reshape(-1, 1), ones)
    return _PeerCombineFn.apply(y, expert_weights, ex, dest, slot, t, k)


def shard_experts(model: torch.nn.Module, rank: int, world: int, exchange: "ExchangeHolder | None" = None) -> list[str]:
    """Replace every MoE layer's expert tensors by this rank's slice; returns the names of the local parameters.

    With ``exchange`` the layers dispatch and combine through own peer-memory kernels, otherwise through ``all_to_all_single``."""

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
        mod.expert_dispatch = expert_parallel_moe if exchange is None else expert_parallel_moe_peer
        mod._ep_exchange = exchange
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
        fused = self.resolved_engine() == "fused"
        holder = ExchangeHolder(timeout_ms=float(getattr(self.comm, "wait_timeout_ms", 2000))) if fused else None
        local = shard_experts(model, self.rank, self.world_size, holder)
        comm = self.comm if fused else replace(self.comm, engine="nccl") if self.comm else None
        return FlatDataParallel(model, mode="shard", comm=comm, local_params=local)

    def unit_count(self, model) -> int:
        return int(model.unit_count())
