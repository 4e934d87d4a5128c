"""Collective back ends used by the flat sharding engine.

``PeerCollectives`` drives the kernels of ``csrc/comm.cu`` over symmetric (peer-mapped) memory: every
buffer that another rank reads or writes is allocated through ``torch.distributed._symmetric_memory``
once at start-up, the rendezvous yields one device pointer per rank, and from then on gradients are
reduced, weights updated and replicas refreshed by plain kernels that load and store through those
pointers (optionally ``multimem`` on the NVLS multicast mapping).  No NCCL call is made on that path.

``TorchCollectives`` implements the same five operations with ``torch.distributed`` (NCCL or Gloo) or,
for a world of one, with local copies; it is the CPU-testable twin and the baseline engine.

Both expose: ``alloc``, ``reduce_scatter``, ``norm_and_clip``, ``adamw_update``, ``refresh_done`` and the
public ``all_reduce_``.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class SymBuffer:
    """A local tensor plus, for peer-mapped buffers, the address of the same allocation on every rank."""

    tensor: torch.Tensor
    peer_ptrs: list[int] | None = None
    multicast_ptr: int = 0


def _world_rank() -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(), dist.get_rank()
    return 1, 0


class TorchCollectives:
    """Library collectives (or none at all for a single rank)."""

    fused = False

    def __init__(self, device: torch.device) -> None:
        self.device = device
        self.world, self.rank = _world_rank()

    def alloc(self, numel: int, dtype: torch.dtype, *, shared: bool = False) -> SymBuffer:
        return SymBuffer(torch.zeros(numel, dtype=dtype, device=self.device))

    # grad_full: [total] fp32 -> grad_shard: [total / world] fp32, mean over ranks; returns sum of squares (tensor)
    def reduce_scatter(self, unit, epoch: int) -> None:
        shard = unit.shard_numel
        if unit.local:
            unit.grad_shard.copy_(unit.grad_full.tensor).mul_(1.0 / self.world)
        elif self.world > 1:
            if dist.get_backend() == "nccl":
                dist.reduce_scatter_tensor(unit.grad_shard, unit.grad_full.tensor, op=dist.ReduceOp.SUM)
                unit.grad_shard.mul_(1.0 / self.world)
            else:   # gloo has no reduce-scatter
                dist.all_reduce(unit.grad_full.tensor)
                unit.grad_shard.copy_(unit.grad_full.tensor[self.rank * shard:(self.rank + 1) * shard])
                unit.grad_shard.mul_(1.0 / self.world)
        else:
            unit.grad_shard.copy_(unit.grad_full.tensor)
        unit.sumsq.add_(unit.grad_shard.double().pow(2).sum().float())

    def norm_and_clip(self, sumsq: torch.Tensor, max_norm: float | None, epoch: int, coef: torch.Tensor,
                      norm: torch.Tensor) -> None:
        total = sumsq.clone()
        if self.world > 1:
            dist.all_reduce(total)
        norm.copy_(total.sqrt())
        if max_norm is None:
            coef.fill_(1.0)
        else:
            coef.copy_((max_norm / (norm + 1e-6)).clamp(max=1.0))

    def adamw_update(self, unit, seg, *, lr, beta1, beta2, eps, weight_decay, step, coef) -> None:
        lo, hi = seg
        p, g = unit.master[lo:hi], unit.grad_shard[lo:hi] * coef
        m, v = unit.exp_avg[lo:hi], unit.exp_avg_sq[lo:hi]
        m.mul_(beta1).add_(g, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
        bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
        p.mul_(1 - lr * weight_decay).addcdiv_(m, (v / bc2).sqrt_().add_(eps), value=-lr / bc1)

    def refresh_replicas(self, unit, epoch: int) -> None:
        """Make the low-precision replica of ``unit`` reflect the fp32 shards of every rank."""

        low = unit.master.to(unit.gathered.tensor.dtype)
        if self.world > 1 and not unit.local:
            dist.all_gather_into_tensor(unit.gathered.tensor, low)
        else:
            unit.gathered.tensor.copy_(low)

    def refresh_shard(self, unit) -> None:
        """``full_shard``: only the rank's own low-precision shard is kept; rebuild it from the fp32 master."""

        unit.low_shard.tensor[:unit.shard_numel].copy_(unit.master.to(unit.low_shard.tensor.dtype))

    def gather_unit(self, unit, dst: torch.Tensor) -> None:
        """All-gather the low-precision shards of ``unit`` into ``dst`` (``[unit.total]``)."""

        mine = unit.low_shard.tensor[:unit.shard_numel]
        if self.world > 1 and not unit.local:
            dist.all_gather_into_tensor(dst[:unit.total], mine.contiguous())
        else:
            dst[:unit.total].copy_(mine)

    def refresh_done(self, epoch: int) -> None:
        pass

    def all_reduce_(self, tensor: torch.Tensor) -> torch.Tensor:
        """In-place sum over ranks through the library (identity for a single rank)."""

        if self.world > 1:
            dist.all_reduce(tensor, op=dist.ReduceOp.SUM)
        return tensor

    def check_status(self) -> None:
        pass

    def close(self) -> None:
        pass


class PeerCollectives:
    """Own kernels over NVLink peer memory (see ``csrc/comm.cu``)."""

    fused = True
    CH_NORM = 0
    CH_PARAMS = 1
    CH_ALLREDUCE = 2  # the public all-reduce
    CH_UNIT0 = 3      # one "gradients complete" channel per unit from here on
    ALLREDUCE_ONE_SHOT_BYTES = 256 * 1024

    def __init__(self, device: torch.device, *, max_units: int, wait_timeout_ms: float = 2000.0,
                 use_multimem: bool = False, max_ctas: int = 296) -> None:
        from mini_train_sys_b200.ops.native_backend import ext

        self.ext = ext()
        self.device = device
        self.world, self.rank = _world_rank()
        self.timeout_ms = float(wait_timeout_ms)
        self.use_multimem = bool(use_multimem) and self.world > 1
        self.max_ctas = int(max_ctas)
        self.status = self.ext.status_tensor(device.index or 0)
        self._keep = []   # symmetric allocations and their handles stay alive with the engine
        channels = self.CH_UNIT0 + max_units
        self.flags = self.alloc(channels * self.world, torch.int32, shared=True)
        self.slots = self.alloc(4 * max(self.world, 4), torch.float32, shared=True)
        self.comm_stream = torch.cuda.Stream(device)
        self._ar_stage: SymBuffer | None = None     # all-reduce staging: two halves used alternately
        self._ar_part: SymBuffer | None = None      # this rank's reduced slice, read by every peer
        self._ar_result: torch.Tensor | None = None
        self._ar_calls = 0
        self.allreduce_capacity = 16 * 2**20        # fp32 elements per pass (64 MiB); larger tensors go in passes

    def alloc(self, numel: int, dtype: torch.dtype, *, shared: bool = False) -> SymBuffer:
        numel = -(-numel // 64) * 64
        if not shared or self.world == 1:
            t = torch.zeros(numel, dtype=dtype, device=self.device)
            return SymBuffer(t, [t.data_ptr()])
        import torch.distributed._symmetric_memory as symm

        t = symm.empty(numel, dtype=dtype, device=self.device)
        t.zero_()
        handle = symm.rendezvous(t, dist.group.WORLD.group_name)
        self._keep.append((t, handle))
        ptrs = [int(p) for p in handle.buffer_ptrs]
        mc = int(handle.multicast_ptr) if (self.use_multimem and getattr(handle, "multicast_ptr", 0)) else 0
        return SymBuffer(t, ptrs, mc)

    # -- gradient reduce-scatter: runs on the communication stream behind the backward pass --
    def reduce_scatter(self, unit, epoch: int) -> None:
        ready = torch.cuda.Event()
        ready.record()
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(ready)
            channel = self.CH_UNIT0 + unit.index
            shared = self.world > 1 and not unit.local
            if shared:
                self.ext.comm_signal(self.flags.peer_ptrs, channel, self.rank, epoch, unit.grad_shard)
            # rank-local units read only their own buffer (one pointer) but still take the 1 / world of the global mean
            self.ext.comm_reduce_scatter(unit.grad_shard, unit.grad_full.peer_ptrs, unit.grad_full.multicast_ptr,
                                         unit.rank * unit.shard_numel, 1.0 / self.world, unit.sumsq, self.flags.tensor,
                                         channel, epoch if shared else 0, self.timeout_ms, self.status, self.max_ctas)

    def norm_and_clip(self, sumsq: torch.Tensor, max_norm: float | None, epoch: int, coef: torch.Tensor,
                      norm: torch.Tensor) -> None:
        torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
        self.ext.comm_norm_clip(sumsq, self.slots.peer_ptrs, self.flags.peer_ptrs, self.flags.tensor, self.CH_NORM,
                                self.rank, epoch, self.timeout_ms, 0.0 if max_norm is None else float(max_norm), 1.0,
                                coef, norm, self.status)

    def adamw_update(self, unit, seg, *, lr, beta1, beta2, eps, weight_decay, step, coef) -> None:
        lo, hi = seg
        if getattr(unit, "staged", False):      # full_shard: the new weights go into the rank's own shard only
            dests, offset, low = [unit.low_shard.tensor.data_ptr()], lo, unit.low_shard.tensor
        else:
            dests, offset, low = unit.gathered.peer_ptrs, unit.rank * unit.shard_numel + lo, unit.gathered.tensor
        self.ext.comm_adamw_push(unit.master[lo:hi], unit.grad_shard[lo:hi], unit.exp_avg[lo:hi], unit.exp_avg_sq[lo:hi],
                                 dests, offset, low.dtype == torch.bfloat16, lr, beta1, beta2,
                                 eps, weight_decay, step, coef, 1.0, self.max_ctas * 4, self.status)

    def adamw_update_table(self, table, n_rows: int, chunks: int, *, lr, weight_decay, betas, eps, step, coef) -> None:
        """Every segment of every unit in one launch (the table comes from ``ext.comm_adamw_table``)."""

        self.ext.comm_adamw_push_table(table, n_rows, chunks, lr[0], lr[1], weight_decay[0], weight_decay[1], betas[0], betas[1],
                                       eps, step, coef, 1.0, self.status, self.max_ctas * 4)

    def refresh_shard(self, unit) -> None:
        """``full_shard`` start-up / restore: rebuild the own low-precision shard, then let every rank finish before any gathers."""

        unit.low_shard.tensor[:unit.shard_numel].copy_(unit.master.to(unit.low_shard.tensor.dtype))
        if self.world > 1 and not unit.local:
            torch.cuda.synchronize(self.device)
            dist.barrier(device_ids=[self.device.index])

    def gather_unit(self, unit, dst: torch.Tensor) -> None:
        """Pull every owner's shard of ``unit`` into ``dst`` on the current stream.  No flag wait is needed: the shards were
        completed before ``refresh_done`` of the last step returned on every rank, and they are next written after the
        global-norm exchange of this step, which every rank enters only after its last gather."""

        low = unit.low_shard
        self.ext.comm_allgather(dst, low.peer_ptrs, unit.shard_numel * low.tensor.element_size(), self.flags.tensor,
                                self.CH_PARAMS, 0, self.timeout_ms, self.status, self.max_ctas)

    def refresh_replicas(self, unit, epoch: int) -> None:
        """Pull all-gather of the low-precision shards (used at start-up and after a checkpoint load)."""

        low = unit.low_shard
        low.tensor[:unit.shard_numel].copy_(unit.master.to(low.tensor.dtype))
        if unit.local:
            unit.gathered.tensor[:unit.shard_numel].copy_(low.tensor[:unit.shard_numel])
            return
        if self.world > 1:
            torch.cuda.synchronize(self.device)
            dist.barrier(device_ids=[self.device.index])   # start-up / restore path only
        self.ext.comm_allgather(unit.gathered.tensor, low.peer_ptrs, unit.shard_numel * low.tensor.element_size(),
                                self.flags.tensor, self.CH_PARAMS, 0, self.timeout_ms, self.status, self.max_ctas)
        if self.world > 1:
            torch.cuda.synchronize(self.device)
            dist.barrier(device_ids=[self.device.index])

    def refresh_done(self, epoch: int) -> None:
        """After the AdamW pushes of a step: tell every peer, then wait until every peer has told us."""

        if self.world == 1:
            return
        self.ext.comm_signal(self.flags.peer_ptrs, self.CH_PARAMS, self.rank, epoch, self.flags.tensor)
        self.ext.comm_wait(self.flags.tensor, self.CH_PARAMS, self.world, epoch, self.timeout_ms, self.status)

    # -- public all-reduce ----------------------------------------------------------------------------------------
    def _allreduce_buffers(self) -> None:
        if self._ar_stage is None:
            cap = self.allreduce_capacity
            self._ar_stage = self.alloc(2 * cap, torch.float32, shared=True)
            self._ar_part = self.alloc(cap // self.world + 64, torch.float32, shared=True)
            self._ar_result = torch.empty(cap, dtype=torch.float32, device=self.device)

    @torch.no_grad()
    def all_reduce_(self, tensor: torch.Tensor) -> torch.Tensor:
        """In-place sum of ``tensor`` over all ranks with the peer-memory kernels (no library collective).

        Every rank must call this with the same shape, in the same order, on its current stream.  Small inputs take one
        pass (stage, signal, every rank sums all peers' copies); larger ones take two (each rank sums its slice of all
        peers' copies, then gathers the reduced slices).  With ``use_multimem`` the sums are done inside the switch.
        Sums are formed in fp32 in rank order, so every rank obtains bit-identical results."""

        if self.world == 1 or tensor.numel() == 0:
            return tensor
        if not tensor.is_cuda:
            raise ValueError("PeerCollectives.all_reduce_ needs a CUDA tensor")
        self._allreduce_buffers()
        flat = tensor.reshape(-1) if tensor.is_contiguous() else tensor.contiguous().view(-1)
        work = flat if flat.dtype == torch.float32 else flat.float()
        cap = self.allreduce_capacity
        for lo in range(0, work.numel(), cap):
            self._allreduce_pass(work[lo:lo + cap])
        if work is not flat:
            flat.copy_(work)
        if flat.data_ptr() != tensor.data_ptr():
            tensor.copy_(flat.view(tensor.shape))
        return tensor

    def _allreduce_pass(self, part: torch.Tensor) -> None:
        n = part.numel()
        quantum = 4 * self.world
        padded = -(-n // quantum) * quantum
        self._ar_calls += 1
        call = self._ar_calls
        half = (call & 1) * self.allreduce_capacity
        stage = self._ar_stage.tensor[half:half + padded]
        stage[:n].copy_(part)
        if padded > n:
            stage[n:].zero_()
        stage_ptrs = [p + half * 4 for p in self._ar_stage.peer_ptrs]
        mc = self._ar_stage.multicast_ptr + half * 4 if self._ar_stage.multicast_ptr else 0
        ch = self.CH_ALLREDUCE
        self.ext.comm_signal(self.flags.peer_ptrs, ch, self.rank, 2 * call - 1, stage)            # my copy is staged
        if padded * 4 <= self.ALLREDUCE_ONE_SHOT_BYTES:
            out = self._ar_result[:padded]
            self.ext.comm_reduce_scatter(out, stage_ptrs, mc, 0, 1.0, None, self.flags.tensor, ch, 2 * call - 1,
                                         self.timeout_ms, self.status, self.max_ctas)
            # Alternating halves make the next call's staging safe: a peer signals call c + 1 only after its reads of call c.
            self.ext.comm_signal(self.flags.peer_ptrs, ch, self.rank, 2 * call, stage)
        else:
            per = padded // self.world
            mine = self._ar_part.tensor[:per]
            self.ext.comm_reduce_scatter(mine, stage_ptrs, mc, self.rank * per, 1.0, None, self.flags.tensor, ch, 2 * call - 1,
                                         self.timeout_ms, self.status, self.max_ctas)
            self.ext.comm_signal(self.flags.peer_ptrs, ch, self.rank, 2 * call, stage)             # my slice is reduced
            out = self._ar_result[:padded]
            self.ext.comm_allgather(out, self._ar_part.peer_ptrs, per * 4, self.flags.tensor, ch, 2 * call, self.timeout_ms,
                                    self.status, self.max_ctas)
        part.copy_(out[:n])

    def check_status(self) -> None:
        word = int(self.status[0].item())
        if word != 0:
            raise RuntimeError(f"a peer-memory collective reported status {word} (1 = a wait on a peer flag timed out)")

    def close(self) -> None:
        self._keep.clear()
