"""Flat-buffer data-parallel engine: sharded fp32 master weights + low-precision replicas.

One engine serves both strategies of this package:

* ``mode="shard"`` (FSDP): one unit per ``TransformerBlock`` plus a root unit (embedding, final norm,
  head) - the same 13-unit split the reference gets from torch FSDP for the 12-layer model
  (minitrain/distributed/fsdp.py:38-45, scripts/train.py:179-203).
* ``mode="replicate"`` (DDP): units are size-bounded buckets in reverse parameter order, so the
  first buckets complete early in backward (the reference uses torch DDP with 25 MB buckets,
  minitrain/distributed/ddp.py:54-65).

Per unit and per rank the engine holds: the rank's slice of the fp32 master weights and of both
Adam moments, a full fp32 gradient buffer (input of the reduce-scatter) and the low-precision
weights the module's parameters are views of.  Where those low-precision weights live depends on
the sharding strategy:

* ``shard_grad_op`` / DDP (``reshard_after_forward=False``): a full replica per rank stays resident; the fused AdamW
  kernel stores the new weights into every rank's replica, so there is no separate parameter all-gather.
* ``full_shard`` (``reshard_after_forward=True``, more than one rank): only the rank's own low-precision shard is
  resident (parameter memory ~ 1 / world).  A unit is gathered from the owners' shards over peer memory into one of two
  staging slots one unit ahead of its use - block i + 1 while block i runs in forward, block i - 1 in backward (the
  analogue of torch FSDP's forward / ``BACKWARD_PRE`` prefetch, minitrain/distributed/fsdp.py:128-153) - and the
  parameters are re-pointed at the slot.  The root unit (embedding, final norm, head) has a staging buffer of its own
  that is gathered at the start of every step.  Gradient buffers stay full-size per unit in both modes.

A training step is then

    backward      parameter hooks copy each gradient into the unit's flat buffer (or the operator writes it there);
                  when a unit is complete its reduce-scatter runs on a side stream, overlapping the rest of backward
    optimizer     one cross-rank sum gives the global gradient norm and the clip coefficient on the
                  device (no host synchronisation); ONE fused AdamW launch walks a table of all shard segments,
                  updates the fp32 state and stores the new low-precision weights (into the replicas or the shard)

``collectives`` decides how the cross-rank parts run: ``PeerCollectives`` (own kernels over NVLink
peer memory) or ``TorchCollectives`` (NCCL / Gloo / single rank).  Optimizer state is always sharded.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch
import torch.distributed as dist
from torch import nn

from mini_train_sys_b200.parallel.comm import PeerCollectives, SymBuffer, TorchCollectives
from mini_train_sys_b200.runtime.config import OptimizerConfig

ALIGN = 8   # parameter offsets inside a unit are multiples of 8 elements (16 bytes in bf16)


@dataclass
class ParamSlot:
    name: str
    param: nn.Parameter
    offset: int
    numel: int
    shape: torch.Size
    decay: bool
    late: bool = False     # several uses per step (embedding, tied head): writers ADD into the flat buffer, which is zeroed after
                           # every step, and the slot counts as arrived when the optimizer step begins


@dataclass
class Unit:
    index: int
    name: str
    slots: list[ParamSlot]
    total: int = 0                  # padded element count of the whole unit
    shard_numel: int = 0
    master: torch.Tensor = None     # fp32 [shard]
    exp_avg: torch.Tensor = None
    exp_avg_sq: torch.Tensor = None
    grad_shard: torch.Tensor = None
    grad_full: SymBuffer = None     # fp32 [total]
    gathered: SymBuffer = None      # low precision [total]; parameters are views of this
    low_shard: SymBuffer = None     # low precision [shard]; source of pull all-gathers
    sumsq: torch.Tensor = None
    pending: int = 0
    local: bool = False             # rank-local parameters (expert shards): never reduced across ranks, scaled by 1 / world
    world: int = 1                  # number of ranks sharing this unit (1 for local units)
    rank: int = 0
    segments: list[tuple[int, int, bool]] = field(default_factory=list)   # (lo, hi, decay) inside the local shard
    staged: bool = False            # parameters live in a staging slot only while the unit is in use (full_shard)
    reported: set = field(default_factory=set)   # offsets of the slots whose gradient arrived this step


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


def _partition(model: nn.Module, mode: str, per_block_units: bool, bucket_bytes: int, local_names: frozenset[str] = frozenset()
               ) -> list[tuple[str, list[tuple[str, nn.Parameter]]]]:
    """Units as ``(name, [(param name, param)])``; names starting with ``local:`` hold rank-local parameters."""

    everything = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
    named = [(n, p) for n, p in everything if n not in local_names]
    local = [(n, p) for n, p in everything if n in local_names]
    if local:
        groups: dict[str, list] = {}
        for n, p in local:
            key = ".".join(n.split(".")[:2]) if n.startswith("blocks.") else "root"
            groups.setdefault(f"local:{key}", []).append((n, p))
        shared = _partition_shared(model, named, mode, per_block_units, bucket_bytes)
        return shared + list(groups.items())
    return _partition_shared(model, named, mode, per_block_units, bucket_bytes)


def _partition_shared(model: nn.Module, named, mode: str, per_block_units: bool, bucket_bytes: int):
    frozen = [n for n, p in model.named_parameters() if not p.requires_grad]
    if frozen:
        raise ValueError(f"the flat engine expects every parameter to be trainable; frozen: {frozen[:3]}...")
    if mode == "shard":
        if not per_block_units:
            return [("root", named)]
        blocks: dict[str, list] = {}
        root = []
        for n, p in named:
            if n.startswith("blocks."):
                blocks.setdefault(".".join(n.split(".")[:2]), []).append((n, p))
            else:
                root.append((n, p))
        return [("root", root)] + [(k, v) for k, v in blocks.items()]
    buckets, current, size = [], [], 0
    for n, p in reversed(named):
        current.append((n, p))
        size += p.numel() * 4
        if size >= bucket_bytes:
            buckets.append((f"bucket{len(buckets)}", current))
            current, size = [], 0
    if current:
        buckets.append((f"bucket{len(buckets)}", current))
    return buckets


class FlatDataParallel(nn.Module):
    def __init__(self, module: nn.Module, *, mode: str = "shard", comm: Any = None, bucket_cap_mb: int = 25,
                 reshard_after_forward: bool = True, per_block_units: bool = True,
                 activation_checkpointing: bool = False, collectives: Any = None,
                 local_params: list[str] | None = None, stage_single_rank: bool = False) -> None:
        super().__init__()
        if mode not in ("shard", "replicate"):
            raise ValueError("mode must be 'shard' or 'replicate'")
        self.module = module
        self.mode = mode
        self.reshard_after_forward = reshard_after_forward
        first = next(module.parameters())
        self.device = first.device
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        act = getattr(module, "activation_dtype", torch.float32)
        self.param_dtype = act if (self.device.type == "cuda" and act in (torch.bfloat16,)) else torch.float32

        layout = _partition(module, mode, per_block_units, bucket_cap_mb * 2**20, frozenset(local_params or ()))
        if collectives is None:
            engine = getattr(comm, "engine", "auto") if comm is not None else "auto"
            want_fused = self.device.type == "cuda" and engine in ("auto", "fused") and self.param_dtype == torch.bfloat16
            if want_fused:
                collectives = PeerCollectives(self.device, max_units=len(layout),
                                              wait_timeout_ms=getattr(comm, "wait_timeout_ms", 20000),
                                              use_multimem=getattr(comm, "use_multimem", False))
            else:
                collectives = TorchCollectives(self.device)
        self.coll = collectives
        self.step_count = 0      # optimizer steps taken (restored from checkpoints; feeds the bias corrections)
        self.comm_epoch = 0      # sequence number of the peer flags: only ever grows, never restored, so that a flag left
                                 # by a later step can not satisfy a wait after an older checkpoint is loaded
        # full_shard: only the own low-precision shard is resident; units are gathered into staging slots around their use
        self.staged = (mode == "shard" and reshard_after_forward and per_block_units
                       and (self.world > 1 or stage_single_rank))
        self.prefetch = int(getattr(comm, "prefetch_units", 1)) > 0
        self._timing: dict[str, list] | None = None   # phase -> [(start event, end event)] while enable_timing() is on
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.clip_coef = torch.ones(1, dtype=torch.float32, device=self.device)
        self.grad_norm = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.units: list[Unit] = []
        self._slot_of: dict[nn.Parameter, tuple[Unit, ParamSlot]] = {}
        for index, (name, params) in enumerate(layout):
            self.units.append(self._build_unit(index, name, params))
        self._adamw_table = None
        self._setup_staging()
        for unit in self.units:
            self._refresh_unit(unit)
        if activation_checkpointing:
            self._enable_activation_checkpointing()

    # ---- construction -----------------------------------------------------------------------------
    def _build_unit(self, index: int, name: str, params: list[tuple[str, nn.Parameter]]) -> Unit:
        slots, offset = [], 0
        for pname, p in params:
            slots.append(ParamSlot(pname, p, offset, p.numel(), p.shape, p.ndim >= 2))
            offset += _round_up(p.numel(), ALIGN)
        unit = Unit(index, name, slots)
        unit.local = name.startswith("local:")
        unit.world, unit.rank = (1, 0) if unit.local else (self.world, self.rank)
        unit.total = _round_up(offset, unit.world * 64)
        unit.shard_numel = unit.total // unit.world
        dev, f32 = self.device, torch.float32
        lo, hi = unit.rank * unit.shard_numel, (unit.rank + 1) * unit.shard_numel
        flat = torch.zeros(unit.total, dtype=f32, device=dev)
        for s in slots:
            flat[s.offset:s.offset + s.numel].copy_(s.param.detach().reshape(-1).float())
        unit.master = flat[lo:hi].clone()
        del flat
        unit.exp_avg = torch.zeros(unit.shard_numel, dtype=f32, device=dev)
        unit.exp_avg_sq = torch.zeros(unit.shard_numel, dtype=f32, device=dev)
        unit.grad_shard = torch.zeros(unit.shard_numel, dtype=f32, device=dev)
        shared = not unit.local
        unit.staged = self.staged and not unit.local
        unit.grad_full = self.coll.alloc(unit.total, f32, shared=shared)
        unit.gathered = None if unit.staged else self.coll.alloc(unit.total, self.param_dtype, shared=shared)
        unit.low_shard = self.coll.alloc(unit.shard_numel, self.param_dtype, shared=shared)
        unit.sumsq = self.sumsq
        # weight-decay segments: intersections of the parameters with the local shard
        for s in slots:
            a, b = max(s.offset, lo), min(s.offset + _round_up(s.numel, ALIGN), hi)
            if a < b:
                unit.segments.append((a - lo, b - lo, s.decay))
        unit.segments = _merge_segments(unit.segments, unit.shard_numel)
        for s in slots:
            if not unit.staged:
                s.param.data = unit.gathered.tensor[s.offset:s.offset + s.numel].view(s.shape)
            self._slot_of[s.param] = (unit, s)
            s.param.register_post_accumulate_grad_hook(self._on_grad)
            if self._sink_ok(s):
                dst = unit.grad_full.tensor[s.offset:s.offset + s.numel].view(s.shape)
                s.param._mts_grad_sink = (dst, self._on_sunk_grad, False)
            elif self._late_sink_ok(s):
                s.late = True
                dst = unit.grad_full.tensor[s.offset:s.offset + s.numel].view(s.shape)
                s.param._mts_grad_sink = (dst, lambda _p: None, True)
        unit.pending = len(slots)
        return unit

    def _late_sink_ok(self, slot) -> bool:
        """The embedding matrix (which is also the output matrix when the two are tied): its gradient is complete only after
        the very last operator of backward, so nothing is lost by closing its unit when the optimizer step begins."""

        return self.coll.fused and slot.param.dim() == 2 and slot.name == "embed.weight"

    def _sink_ok(self, slot) -> bool:
        """Parameters whose backward may write the fp32 gradient in place: matrices used once per step by an operator that
        knows the protocol (linear layers and expert stacks inside the blocks; never tied or embedding weights)."""

        name = slot.name
        if self.coll.fused and name == "lm_head.weight" and slot.param.dim() == 2:
            return True        # an output matrix of its own (not tied to the embedding): one use, by the loss
        if not (self.coll.fused and ".blocks." in f".{name}"):
            return False
        if slot.param.dim() == 1:      # the two norm weights of a block: RMSNorm backward accumulates dw in fp32 anyway
            return name.endswith(("attn_norm.weight", "ffn_norm.weight"))
        return name.endswith(("qkv.weight", "out.weight", "gate.weight", "up.weight", "down.weight", "gate_up_proj", "down_proj"))

    def _arrived(self, unit: Unit, slot: ParamSlot) -> None:
        if slot.offset in unit.reported:
            raise RuntimeError(f"parameter {slot.name!r} received a second gradient before optimizer.step(): the flat engine "
                               "supports one backward pass per step (no gradient accumulation)")
        unit.reported.add(slot.offset)
        unit.pending -= 1
        if unit.pending == 0:
            self.coll.reduce_scatter(unit, self.comm_epoch + 1)

    def _on_sunk_grad(self, param: nn.Parameter) -> None:
        self._arrived(*self._slot_of[param])

    def _enable_activation_checkpointing(self) -> None:
        from torch.utils.checkpoint import checkpoint

        from mini_train_sys_b200.models.blocks import TransformerBlock

        for m in self.module.modules():
            if isinstance(m, TransformerBlock) and not hasattr(m, "_plain_forward"):
                m._plain_forward = m.forward
                m.forward = lambda *a, _f=m._plain_forward, **k: checkpoint(_f, *a, use_reentrant=False, **k)

    # ---- forward / backward -------------------------------------------------------------------------
    def forward(self, *args, **kwargs):
        if self.staged:
            self._begin_step()
        return self.module(*args, **kwargs)

    def unit_count(self) -> int:
        return len(self.units)

    @torch.no_grad()
    def _on_grad(self, param: nn.Parameter) -> None:
        if param.grad is None:
            return      # the operator wrote this gradient through the parameter's sink and already reported it
        unit, slot = self._slot_of[param]
        dst = unit.grad_full.tensor[slot.offset:slot.offset + slot.numel].view(slot.shape)
        if slot.late:      # contributions that came through autograd join the ones written in place
            dst.add_(param.grad)
            param.grad = None
            return
        dst.copy_(param.grad)
        param.grad = None
        self._arrived(unit, slot)

    def _flush_incomplete_units(self) -> None:
        """Units with parameters that received no gradient this step still have to take part: the ranges of exactly those
        parameters (padding included) are zeroed, so that last step's values are not reduced and applied again."""

        for unit in self.units:
            if unit.pending > 0:
                for s in unit.slots:
                    if s.param.grad is not None:
                        self._on_grad(s.param)
                if unit.pending > 0:
                    for s in unit.slots:
                        if s.offset not in unit.reported and not s.late:
                            unit.grad_full.tensor[s.offset:s.offset + _round_up(s.numel, ALIGN)].zero_()
                    unit.pending = 0
                    self.coll.reduce_scatter(unit, self.comm_epoch + 1)

    # ---- staging of sharded parameters (full_shard) --------------------------------------------------------------
    def _setup_staging(self) -> None:
        self._block_units: dict[int, Unit] = {}
        self._root_unit: Unit | None = None
        self._slots: list[torch.Tensor] = []
        self._slot_unit: list[int | None] = []
        self._slot_event: list[Any] = []
        self._root_stage: torch.Tensor | None = None
        self._root_fresh = False
        if not self.staged:
            return
        blocks = [u for u in self.units if u.staged and u.name != "root"]
        for u in self.units:
            if u.staged and u.name == "root":
                self._root_unit = u
                self._root_stage = torch.zeros(u.total, dtype=self.param_dtype, device=self.device)
                self._point(u, self._root_stage)
        if blocks:
            widest = max(u.total for u in blocks)
            self._slots = [torch.zeros(widest, dtype=self.param_dtype, device=self.device) for _ in range(2)]
            self._slot_unit = [None, None]
            self._slot_event = [None, None]
        order = {u.index: i for i, u in enumerate(blocks)}
        self._block_order = blocks
        for u in blocks:
            module = self.module.get_submodule(u.name)
            pos = order[u.index]
            nxt = blocks[pos + 1] if pos + 1 < len(blocks) else None
            prv = blocks[pos - 1] if pos > 0 else None
            module.register_forward_pre_hook(lambda _m, _a, u=u, nxt=nxt: self._use(u, nxt))
            module.register_forward_hook(lambda _m, _a, out, u=u, prv=prv: self._watch_output(out, u, prv))

    def _watch_output(self, out, unit: Unit, prefetch: Unit | None) -> None:
        """Backward of a block starts when the gradient of its hidden-state output arrives: a hook on that tensor brings the
        unit's weights back before any of the block's backward nodes runs (the block returns a record, not a tensor, so
        module-level backward hooks do not apply).  Every other backward node of the block that touches a weight depends,
        directly or through the routed weights, on this gradient."""

        hidden = getattr(out, "hidden_states", None)
        if hidden is None:
            hidden = out[0] if isinstance(out, (tuple, list)) else out
        if isinstance(hidden, torch.Tensor) and hidden.requires_grad:
            hidden.register_hook(lambda _g, u=unit, p=prefetch: self._use(u, p))

    def _point(self, unit: Unit, buffer: torch.Tensor) -> None:
        for s in unit.slots:
            s.param.data = buffer[s.offset:s.offset + s.numel].view(s.shape)

    def _gather_into(self, unit: Unit, dst: torch.Tensor):
        """All-gather of ``unit``'s low-precision shards into ``dst`` on the communication stream; returns the event that marks
        its end.  Every kernel already queued on the compute stream finishes first (it may still read the slot's old content)."""

        stream = getattr(self.coll, "comm_stream", None)
        if stream is None:      # CPU / library twin: gather in line
            self.coll.gather_unit(unit, dst)
            return None
        before = torch.cuda.Event()
        before.record()
        with torch.cuda.stream(stream):
            stream.wait_event(before)
            self.coll.gather_unit(unit, dst)
            done = torch.cuda.Event()
            done.record()
        return done

    def _use(self, unit: Unit, prefetch: Unit | None) -> None:
        """Called right before ``unit``'s block runs (forward, recomputation or backward): make its weights resident, then start
        gathering the unit that runs next into the other slot."""

        slot = self._slot_unit.index(unit.index) if unit.index in self._slot_unit else None
        if slot is None:
            slot = self._free_slot(keep=None)
            self._slot_event[slot] = self._gather_into(unit, self._slots[slot][:unit.total])
            self._slot_unit[slot] = unit.index
        if self._slot_event[slot] is not None:
            with self._timed("gather_wait"):       # exposed part of the parameter gather: zero when the prefetch was in time
                torch.cuda.current_stream(self.device).wait_event(self._slot_event[slot])
            self._slot_event[slot] = None
        self._point(unit, self._slots[slot])
        if self.prefetch and prefetch is not None and prefetch.index not in self._slot_unit:
            other = self._free_slot(keep=slot)
            self._slot_event[other] = self._gather_into(prefetch, self._slots[other][:prefetch.total])
            self._slot_unit[other] = prefetch.index

    def _free_slot(self, keep: int | None) -> int:
        for i, held in enumerate(self._slot_unit):
            if held is None and i != keep:
                return i
        return 1 - keep if keep is not None else 0

    def _begin_step(self) -> None:
        """Start of a forward pass in staged mode: the root unit (needed first and last) and the first block."""

        if self._root_unit is not None and not self._root_fresh:
            ev = self._gather_into(self._root_unit, self._root_stage)
            if ev is not None:
                with self._timed("gather_wait"):
                    torch.cuda.current_stream(self.device).wait_event(ev)
            self._root_fresh = True
        if self._block_order and self._block_order[0].index not in self._slot_unit:
            first = self._block_order[0]
            slot = self._free_slot(keep=None)
            self._slot_event[slot] = self._gather_into(first, self._slots[slot][:first.total])
            self._slot_unit[slot] = first.index

    def _after_update(self) -> None:
        """The shards changed: nothing that sits in a staging buffer is current any more."""

        if self.staged:
            self._slot_unit = [None] * len(self._slot_unit)
            self._slot_event = [None] * len(self._slot_event)
            self._root_fresh = False

    def _refresh_unit(self, unit: Unit) -> None:
        """Start-up and checkpoint restore: rebuild the low-precision weights of ``unit`` from the fp32 shards."""

        if unit.staged:
            self.coll.refresh_shard(unit)
            self._after_update()
        else:
            self.coll.refresh_replicas(unit, 0)

    def parameter_bytes(self) -> dict[str, int]:
        """Bytes this rank holds for parameters: ``resident`` stays allocated between steps (fp32 master, both moments and the
        low-precision weights), ``staging`` is the fixed pool that units pass through under ``full_shard``."""

        low = torch.empty(0, dtype=self.param_dtype).element_size()
        resident = staging = 0
        for u in self.units:
            resident += 3 * 4 * u.shard_numel + low * u.shard_numel
            if u.gathered is not None:
                resident += low * u.total
        staging += sum(t.numel() * low for t in self._slots)
        if self._root_stage is not None:
            staging += self._root_stage.numel() * low
        return {"resident": resident, "staging": staging}

    # ---- where a step waits for communication (CUDA events on the compute stream) ----------------------------------
    def enable_timing(self, on: bool = True) -> None:
        self._timing = {} if on else None

    def _timed(self, phase: str):
        """Context manager: brackets what the compute stream does inside with two events (no-op unless timing is on)."""

        engine = self

        class _Span:
            def __enter__(self_inner):
                if engine._timing is not None and engine.device.type == "cuda":
                    self_inner.a = torch.cuda.Event(enable_timing=True)
                    self_inner.a.record()
                return self_inner

            def __exit__(self_inner, *exc):
                if engine._timing is not None and engine.device.type == "cuda":
                    b = torch.cuda.Event(enable_timing=True)
                    b.record()
                    engine._timing.setdefault(phase, []).append((self_inner.a, b))
                return False

        return _Span()

    def timing_summary(self, steps: int) -> dict[str, float]:
        """Milliseconds per step the compute stream spent in each bracketed phase since timing was enabled (synchronises)."""

        if not self._timing:
            return {}
        torch.cuda.synchronize(self.device)
        out = {k: round(sum(a.elapsed_time(b) for a, b in v) / max(steps, 1), 4) for k, v in self._timing.items()}
        self._timing = {}
        return out

    def check_status(self) -> None:
        """Raise if a device-side wait of this engine's collectives ran out (synchronises the device)."""

        self.coll.check_status()

    # ---- optimizer ------------------------------------------------------------------------------------
    def build_sharded_optimizer(self, cfg: OptimizerConfig) -> "ShardedAdamW":
        return ShardedAdamW(self, cfg)

    # ---- state dicts ------------------------------------------------------------------------------------
    def _full_flat(self, shard: torch.Tensor, unit: "Unit | None" = None) -> torch.Tensor:
        if self.world == 1 or (unit is not None and unit.local):
            return shard
        full = torch.empty(shard.numel() * self.world, dtype=shard.dtype, device=shard.device)
        dist.all_gather_into_tensor(full, shard.contiguous())
        return full

    def _mesh(self):
        from torch.distributed.device_mesh import init_device_mesh

        if not hasattr(self, "_device_mesh"):
            self._device_mesh = init_device_mesh(self.device.type, (self.world,))
        return self._device_mesh

    def _as_sharded(self, full: torch.Tensor, cpu_offload: bool, local: bool = False):
        if cpu_offload and self.world == 1:
            return full.cpu()
        if self.world == 1:
            return full.clone()
        from torch.distributed.tensor import DTensor, Shard, distribute_tensor

        if local:   # this rank's slice along dim 0 of a tensor that no rank holds in full (expert shards)
            return DTensor.from_local(full.contiguous().clone(), self._mesh(), [Shard(0)], run_check=False)
        return distribute_tensor(full.contiguous(), self._mesh(), [Shard(0)])

    def sharded_state_dict(self, optimizer: "ShardedAdamW", *, cpu_offload: bool = True):
        """``(model_state, optim_state)`` keyed by plain parameter names; tensors are dim-0 sharded DTensors."""

        model_state: dict[str, Any] = {}
        opt_state: dict[str, Any] = {}
        for unit in self.units:
            flats = {k: self._full_flat(t, unit) for k, t in (("p", unit.master), ("m", unit.exp_avg), ("v", unit.exp_avg_sq))}
            for s in unit.slots:
                pick = lambda key: flats[key][s.offset:s.offset + s.numel].view(s.shape)  # noqa: E731
                model_state[s.name] = self._as_sharded(pick("p"), cpu_offload, unit.local)
                opt_state[s.name] = {"step": torch.tensor(float(self.step_count)),
                                     "exp_avg": self._as_sharded(pick("m"), cpu_offload, unit.local),
                                     "exp_avg_sq": self._as_sharded(pick("v"), cpu_offload, unit.local)}
        # tied parameters appear under every name a plain model's state dict uses
        owner = {id(p): n for n, p in self.module.named_parameters()}
        for alias, p in self.module.named_parameters(remove_duplicate=False):
            if alias not in model_state and id(p) in owner:
                model_state[alias] = model_state[owner[id(p)]]
        persistent = set(self.module.state_dict().keys())
        for extra, buf in self.module.named_buffers():
            if extra in persistent:
                model_state[extra] = buf
        groups = optimizer.describe_groups() if optimizer is not None else []
        return model_state, {"state": opt_state, "param_groups": groups}

    @torch.no_grad()
    def load_sharded_state_dict(self, model_state, optim_state, optimizer: "ShardedAdamW | None" = None) -> None:
        def full(t, slot=None, local=False):
            t = t.full_tensor() if hasattr(t, "full_tensor") else t
            if local and t.shape[0] != slot.shape[0]:   # a full [E, ...] tensor: keep this rank's experts
                per = slot.shape[0]
                t = t[self.rank * per:(self.rank + 1) * per]
            return t.to(self.device, torch.float32).reshape(-1)

        steps = []
        for unit in self.units:
            lo, hi = unit.rank * unit.shard_numel, (unit.rank + 1) * unit.shard_numel
            for key, dst in (("p", unit.master), ("m", unit.exp_avg), ("v", unit.exp_avg_sq)):
                flat = torch.zeros(unit.total, dtype=torch.float32, device=self.device)
                for s in unit.slots:
                    if key == "p":
                        src = model_state[s.name]
                    else:
                        entry = optim_state.get("state", {}).get(s.name)
                        if entry is None:
                            continue
                        src = entry["exp_avg" if key == "m" else "exp_avg_sq"]
                        if key == "m" and "step" in entry:
                            steps.append(float(entry["step"]))
                    flat[s.offset:s.offset + s.numel].copy_(full(src, s, unit.local))
                dst.copy_(flat[lo:hi])
        if steps:
            self.step_count = int(max(steps))
        if optimizer is not None:
            optimizer.adopt_groups(optim_state.get("param_groups", []))
        for unit in self.units:
            self._refresh_unit(unit)

    def full_state_dict(self) -> dict[str, torch.Tensor]:
        """Consolidated fp32 CPU weights under the plain parameter names (tied weights appear under both names)."""

        out: dict[str, torch.Tensor] = {}
        for unit in self.units:
            flat = self._full_flat(unit.master, unit)
            for s in unit.slots:
                value = flat[s.offset:s.offset + s.numel].view(s.shape).detach()
                if unit.local and self.world > 1:
                    parts = [torch.empty_like(value) for _ in range(self.world)]
                    dist.all_gather(parts, value.contiguous())
                    value = torch.cat(parts, dim=0)
                out[s.name] = value.cpu().clone()
        by_param = {id(p): n for n, p in self.module.named_parameters()}
        for name, p in self.module.named_parameters(remove_duplicate=False):
            if name not in out and id(p) in by_param:
                out[name] = out[by_param[id(p)]]
        ordered = {k: out[k] for k in self.module.state_dict().keys() if k in out}
        return ordered

    def state_dict(self, *args, **kwargs):
        return self.module.state_dict(*args, **kwargs)


def _merge_segments(segs: list[tuple[int, int, bool]], shard_numel: int) -> list[tuple[int, int, bool]]:
    """Cover ``[0, shard_numel)`` with maximal runs of equal decay flag (padding joins its left neighbour)."""

    if not segs:
        return [(0, shard_numel, False)] if shard_numel else []
    segs = sorted(segs)
    out = [[0, segs[0][1], segs[0][2]]]
    for lo, hi, decay in segs[1:]:
        if decay == out[-1][2]:
            out[-1][1] = hi
        else:
            out[-1][1] = lo
            out.append([lo, hi, decay])
    out[-1][1] = shard_numel
    return [(a, b, d) for a, b, d in out if a < b]


class ShardedAdamW(torch.optim.Optimizer):
    """AdamW over the engine's flat shards; gradient clipping is folded into the update kernel."""

    owns_clipping = True

    def __init__(self, engine: FlatDataParallel, cfg: OptimizerConfig) -> None:
        self.engine = engine
        self._clip: float | None = None
        dummy = [torch.zeros(1, device=engine.device, requires_grad=True), torch.zeros(1, device=engine.device, requires_grad=True)]
        defaults = dict(lr=cfg.lr, betas=(cfg.beta1, cfg.beta2), eps=cfg.eps, weight_decay=cfg.weight_decay)
        super().__init__([{"params": [dummy[0]], "weight_decay": cfg.weight_decay},
                          {"params": [dummy[1]], "weight_decay": 0.0}], defaults)

    def set_clip_norm(self, max_norm: float | None) -> None:
        self._clip = max_norm

    def last_grad_norm(self) -> torch.Tensor:
        return self.engine.grad_norm[0]

    def zero_grad(self, set_to_none: bool = True) -> None:
        for unit in self.engine.units:
            for s in unit.slots:
                s.param.grad = None

    def _segment_table(self):
        """Device table of every (unit, weight-decay run) of the local shards, built once: the update is one launch."""

        eng = self.engine
        if eng._adamw_table is None:
            rows = []
            low_bf16 = eng.param_dtype == torch.bfloat16
            for unit in eng.units:
                for lo, hi, decay in unit.segments:
                    if unit.staged:
                        dests, offset = [unit.low_shard.tensor.data_ptr()], lo
                    else:
                        dests, offset = list(unit.gathered.peer_ptrs), unit.rank * unit.shard_numel + lo
                    rows.append([unit.master[lo:hi].data_ptr(), unit.grad_shard[lo:hi].data_ptr(), unit.exp_avg[lo:hi].data_ptr(),
                                 unit.exp_avg_sq[lo:hi].data_ptr(), hi - lo, offset, 0 if decay else 1, int(low_bf16), *dests])
            table, chunks = eng.coll.ext.comm_adamw_table(rows, eng.sumsq)
            eng._adamw_table = (table, len(rows), int(chunks))
        return eng._adamw_table

    @torch.no_grad()
    def step(self, closure=None):
        eng = self.engine
        eng._flush_incomplete_units()
        epoch = eng.comm_epoch + 1
        step = eng.step_count + 1
        stream = getattr(eng.coll, "comm_stream", None)
        if stream is not None:
            with eng._timed("reduce_scatter_tail"):     # what is left of the gradient reductions once backward has finished
                torch.cuda.current_stream(eng.device).wait_stream(stream)
        with eng._timed("norm_and_clip"):
            eng.coll.norm_and_clip(eng.sumsq, self._clip, epoch, eng.clip_coef, eng.grad_norm)
        decay_group, plain_group = self.param_groups
        if eng.coll.fused and decay_group["betas"] == plain_group["betas"] and decay_group["eps"] == plain_group["eps"]:
            table, n_rows, chunks = self._segment_table()
            with eng._timed("adamw"):
                eng.coll.adamw_update_table(table, n_rows, chunks, lr=(float(decay_group["lr"]), float(plain_group["lr"])),
                                            weight_decay=(float(decay_group["weight_decay"]), float(plain_group["weight_decay"])),
                                            betas=decay_group["betas"], eps=decay_group["eps"], step=step, coef=eng.clip_coef)
            for unit in eng.units:
                unit.pending = len(unit.slots)
                unit.reported.clear()
        else:
            for unit in eng.units:
                for lo, hi, decay in unit.segments:
                    g = decay_group if decay else plain_group
                    eng.coll.adamw_update(unit, (lo, hi), lr=float(g["lr"]), beta1=g["betas"][0], beta2=g["betas"][1],
                                          eps=g["eps"], weight_decay=float(g["weight_decay"]), step=step, coef=eng.clip_coef)
                if not eng.coll.fused:
                    eng._refresh_unit(unit)
                unit.pending = len(unit.slots)
                unit.reported.clear()
        for unit in eng.units:          # multi-use parameters accumulate in place: start the next step from zero
            for s in unit.slots:
                if s.late:
                    unit.grad_full.tensor[s.offset:s.offset + s.numel].zero_()
        with eng._timed("refresh_done"):
            eng.coll.refresh_done(epoch)
        eng._after_update()
        eng.sumsq.zero_()
        eng.comm_epoch = epoch
        eng.step_count = step
        return None

    # ---- checkpoint helpers ----
    def describe_groups(self) -> list[dict[str, Any]]:
        names = {True: [], False: []}
        for unit in self.engine.units:
            for s in unit.slots:
                names[s.decay].append(s.name)
        out = []
        for g, decay in zip(self.param_groups, (True, False)):
            out.append({"lr": g["lr"], "betas": tuple(g["betas"]), "eps": g["eps"], "weight_decay": g["weight_decay"],
                        # remaining torch.optim.AdamW group options, so the payload also loads into a stock optimizer
                        "amsgrad": False, "maximize": False, "foreach": None, "capturable": False, "differentiable": False,
                        "fused": None, "decoupled_weight_decay": True, "params": names[decay]})
        return out

    def adopt_groups(self, groups: list[dict[str, Any]]) -> None:
        for mine, theirs in zip(self.param_groups, groups):
            for key in ("lr", "betas", "eps", "weight_decay"):
                if key in theirs:
                    mine[key] = theirs[key]

    def state_dict(self):
        return {"step": self.engine.step_count, "param_groups": self.describe_groups()}

    def load_state_dict(self, state):
        self.engine.step_count = int(state.get("step", self.engine.step_count))
        self.adopt_groups(state.get("param_groups", []))
