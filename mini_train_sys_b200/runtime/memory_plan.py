"""Device-memory plan of a training run under the fused sharding engine: what is resident, what grows with the batch, and
the largest local batch that fits a device.

The plan is arithmetic over the same rules the engine and the operators follow, not a measurement:

* **static** (``parallel/flat_engine.py``).  Per unit of ``P`` parameters on ``W`` ranks: fp32 master weights, both AdamW
  moments and the reduced gradient shard (``16 P / W`` bytes); the full fp32 gradient buffer every weight-gradient GEMM
  writes into (``4 P``); the bf16 weights the kernels read: a full replica (``2 P``) under ``ddp`` and ``shard_grad_op``, or
  only this rank's shard (``2 P / W``) plus two staging slots of the widest block and one of the root unit under
  ``full_shard``.  With more than one rank the gradient buffer and the bf16 buffers live in symmetric (peer-mapped) memory,
  which the caching allocator does not own: ``torch.cuda.max_memory_allocated`` does not see them, the device does.
  Expert parallelism keeps ``E / W`` experts per rank as rank-local units (24 bytes per parameter) and four exchange
  regions.
* **activations** (what the autograd functions of ``ops/native_backend.py`` save), in bf16 per token and block: the block
  input, the two normalised inputs, the fused QKV projection and the rotated q and k beside it, the attention output, the
  post-attention residual; for the feed-forward either
  ``gate, up, silu(gate) * up`` (dense) or, per route, the gathered row, the ``[gate | up]`` pre-activations, the SwiGLU
  output and the expert output (MoE); dropout saves nothing (masks are recomputed).  The peak is reached inside the fused
  loss at the end of the forward pass: on top of everything saved there are the bf16 logits of one chunk (at most 65,536
  rows, ``MTS_FUSED_CE_CHUNK_ROWS``; they are gone before backward starts), the gradient of the final hidden states and the
  fp32 gradient of the output matrix.  With activation checkpointing only block inputs stay and one block is live at a time.

Against ``max_memory_allocated`` of this repository's benchmark runs on B200 the plan is within 2.5 % on all sixteen
recorded points: the 293M MoE on 1 to 8 GPUs at local batch 24 and 96 under both sharding modes, the 125M dense preset under
``ddp`` on 2, 4 and 8, the 125M MoE preset under ``fsdp`` and ``ep`` on 2 and 4 (``tests/test_runtime_cpu.py`` holds the points).
One constant is fitted (``WORKSPACE_BYTES``, 0.15 GiB); everything else is counted.  The reference has no counterpart: it finds the largest batch by running a sweep
(benchmarks/distributed/workflow.py ``run_capacity``), which this repository's capacity suite also does; the plan says where
to start that sweep and why a configuration does not fit.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

from mini_train_sys_b200.models.config import ModelConfig

GIB = float(2**30)
LOW_BYTES = 2                      # bf16
STRATEGIES = ("single", "ddp", "fsdp", "ep")
# caching-allocator slack, cuBLAS-free workspaces, router statistics, routing plans, CUDA-graph pools: fitted once as the
# intercept left over on the measured points, identical for every model size tried
WORKSPACE_BYTES = int(0.15 * GIB)


def _units(model: ModelConfig) -> tuple[int, int]:
    """(parameters of the root unit, parameters of one block)."""

    return model.param_count() - model.n_layers * model.block_param_count(), model.block_param_count()


def _expert_params_per_block(model: ModelConfig) -> int:
    return model.num_experts * 3 * model.hidden_size * model.intermediate_size if model.is_moe else 0


@dataclass(frozen=True)
class MemoryPlan:
    strategy: str
    world_size: int
    sharding: str
    tokens_per_sample: int
    static: dict[str, int]                                  # bytes, by buffer
    symmetric: frozenset[str]                               # static entries outside the caching allocator (world > 1)
    per_token: dict[str, int]                               # activation bytes per token, by part
    logits_bytes_per_token: int = 0                         # bf16 logits of the fused loss: a buffer of at most `logits_chunk_rows` rows
    logits_chunk_rows: int = 65536
    workspace: int = WORKSPACE_BYTES
    notes: tuple[str, ...] = field(default_factory=tuple)

    def static_bytes(self, *, allocator_only: bool = False) -> int:
        return sum(v for k, v in self.static.items() if not (allocator_only and k in self.symmetric))

    def activation_bytes(self, local_batch: int) -> int:
        tokens = local_batch * self.tokens_per_sample
        return tokens * sum(self.per_token.values()) + min(tokens, self.logits_chunk_rows) * self.logits_bytes_per_token

    def total_bytes(self, local_batch: int, *, allocator_only: bool = False) -> int:
        """Peak bytes at ``local_batch``; ``allocator_only`` gives what ``torch.cuda.max_memory_allocated`` reports."""

        return self.static_bytes(allocator_only=allocator_only) + self.activation_bytes(local_batch) + self.workspace

    def max_local_batch(self, device_bytes: float, *, headroom: float = 0.9) -> int:
        """Largest local batch whose peak stays under ``headroom`` of the device (0 when even the static part does not fit)."""

        limit = headroom * device_bytes
        if self.total_bytes(1) > limit:
            return 0
        low, high = 1, 2
        while self.total_bytes(high) <= limit and high < 1 << 24:
            low, high = high, high * 2
        while high - low > 1:                                # peak memory grows monotonically with the batch: bisect
            mid = (low + high) // 2
            low, high = (mid, high) if self.total_bytes(mid) <= limit else (low, mid)
        return low

    def summary(self, local_batch: int) -> dict[str, object]:
        return {"strategy": self.strategy, "world_size": self.world_size, "sharding": self.sharding, "local_batch": local_batch,
                "static_gib": {k: round(v / GIB, 3) for k, v in self.static.items()},
                "static_total_gib": round(self.static_bytes() / GIB, 3),
                "outside_caching_allocator_gib": round((self.static_bytes() - self.static_bytes(allocator_only=True)) / GIB, 3),
                "activation_bytes_per_token": {**self.per_token, "logits_up_to_chunk": self.logits_bytes_per_token},
                "activation_gib_per_sample": round(self.activation_bytes(1) / GIB, 4),
                "activations_gib": round(self.activation_bytes(local_batch) / GIB, 3), "workspace_gib": round(self.workspace / GIB, 3),
                "total_gib": round(self.total_bytes(local_batch) / GIB, 3),
                "max_memory_allocated_gib": round(self.total_bytes(local_batch, allocator_only=True) / GIB, 3), "notes": list(self.notes)}


def activation_bytes_per_token(model: ModelConfig, *, moe_row_factor: float = 1.0, activation_checkpointing: bool = False,
                               low_bytes: int = LOW_BYTES) -> dict[str, int]:
    """Bytes saved for backward per token, by part (see the module docstring for the list of tensors)."""

    h, i, layers = model.hidden_size, model.intermediate_size, model.n_layers
    if model.is_moe:
        ffn = model.experts_per_token * (2 * h + 3 * i) * low_bytes * moe_row_factor
        router = model.num_experts * 4 * 3 + model.experts_per_token * 10          # fp32 logits, probabilities, gradients' inputs; routes
    else:
        ffn, router = 3 * i * low_bytes, 0
    # seven hidden-sized tensors per block: the block input, both normalised inputs, the attention output, the post-attention
    # residual, and the rotated q and k that the fused RoPE + attention node keeps beside the projection it was given
    # (``_QKVAttentionFn`` saves ``qr, kr, fused``; recomputing the rotation in backward would trade them for two RoPE passes)
    block = {"hidden_sized_tensors": 7 * h * low_bytes, "qkv": 3 * h * low_bytes, "feed_forward": int(ffn), "router": router,
             "statistics": 4 * (2 + model.n_heads)}
    if activation_checkpointing:
        # every block keeps its input; the tensors of ONE block exist while it is recomputed and differentiated
        parts = {"checkpointed_block_inputs": layers * h * low_bytes, "one_live_block": sum(block.values())}
    else:
        parts = {k: layers * v for k, v in block.items()}
    parts["final_norm_and_loss_input_gradient"] = 3 * h * low_bytes        # final norm's input and output; d(hidden) from the fused loss
    return parts


def plan_memory(model: ModelConfig, *, strategy: str = "single", world_size: int = 1, sharding: str = "full_shard",
                local_batch_hint: int = 1, activation_checkpointing: bool = False, ep_region_factor: float = 2.0,
                low_bytes: int = LOW_BYTES, logits_chunk_rows: int = 65536) -> MemoryPlan:
    """Plan for the fused engine (``parallel.comm.engine: fused`` with ``backend.ops: native``).

    ``local_batch_hint`` only sizes the expert-parallel exchange regions, which the engine allocates for the batch it sees.
    """

    if strategy not in STRATEGIES:
        raise ValueError(f"strategy must be one of {STRATEGIES}")
    if strategy == "single":
        world_size = 1
    if world_size < 1:
        raise ValueError("world_size must be positive")
    if sharding not in ("full_shard", "shard_grad_op"):
        raise ValueError("the fused engine implements full_shard and shard_grad_op")
    if strategy == "ep" and (not model.is_moe or model.num_experts % world_size):
        raise ValueError("expert parallelism needs an MoE model whose expert count is a multiple of the world size")
    w = world_size
    root, block = _units(model)
    total = model.param_count()
    notes: list[str] = []
    static: dict[str, int] = {}
    symmetric: set[str] = set()

    expert = _expert_params_per_block(model) * model.n_layers if strategy == "ep" else 0
    shared = total - expert                                  # parameters handled data-parallel / sharded over all ranks
    static["fp32_master_moments_and_gradient_shard"] = 16 * shared // w
    static["fp32_gradient_buffer"] = 4 * shared
    staged = strategy == "fsdp" and sharding == "full_shard" and w > 1
    if staged:
        static["bf16_weight_shard"] = low_bytes * shared // w
        static["bf16_staging_slots"] = low_bytes * (2 * block + root)
        notes.append("full_shard: a block's bf16 weights exist only while it computes (two staging slots), the root unit in its own")
    else:
        static["bf16_weight_replica"] = low_bytes * shared
        static["bf16_weight_shard"] = low_bytes * shared // w
    if w > 1:
        symmetric.update(k for k in ("fp32_gradient_buffer", "bf16_weight_replica", "bf16_weight_shard") if k in static)
    moe_row_factor = 1.0
    if strategy == "ep":
        static["local_experts_all_buffers"] = 24 * expert // w      # rank-local units: 16 + 4 + 2 + 2 bytes per parameter
        routes = local_batch_hint * model.seq_len * model.experts_per_token
        cap = min(routes, math.ceil(ep_region_factor * routes / w))
        cap = -(-cap // 256) * 256
        static["expert_exchange_regions"] = 4 * w * cap * model.hidden_size * low_bytes + w * cap * 4
        symmetric.add("expert_exchange_regions")
        moe_row_factor = w * cap / max(routes, 1)
        notes.append(f"expert parallelism: the grouped GEMMs run over all {w} x {cap} region rows "
                     f"({moe_row_factor:.2f} x the routes of this rank); regions sized for local batch {local_batch_hint}")
    per_token = activation_bytes_per_token(model, moe_row_factor=moe_row_factor, activation_checkpointing=activation_checkpointing,
                                           low_bytes=low_bytes)
    if strategy == "ep":
        # the combine keeps the rows it pulled back (one per route) for its backward pass
        per_token["expert_parallel_pulled_rows"] = ((1 if activation_checkpointing else model.n_layers)
                                                    * model.experts_per_token * model.hidden_size * low_bytes)
    # every expert's segment of the routing plan is padded to the GEMM's 256-row tile: on average half a tile per expert and layer
    extra = 0
    if model.is_moe:
        extra_rows = model.num_experts * 128 * (1 if activation_checkpointing else model.n_layers)
        extra = extra_rows * (2 * model.hidden_size + 3 * model.intermediate_size) * low_bytes
    if 4 * total > 0.5 * 180 * GIB:
        notes.append("the fp32 gradient buffer is full-size on every rank (4 bytes per parameter): it, not the optimizer state, "
                     "bounds the model size per 180 GB device")
    loss_weight_gradient = 4 * model.vocab_size * model.hidden_size       # fp32 dW of the fused loss, made during the forward pass
    return MemoryPlan(strategy=strategy, world_size=w, sharding=sharding if strategy == "fsdp" else "n/a", tokens_per_sample=model.seq_len,
                      static=static, symmetric=frozenset(symmetric), per_token=per_token,
                      logits_bytes_per_token=model.vocab_size * low_bytes, logits_chunk_rows=logits_chunk_rows,
                      workspace=WORKSPACE_BYTES + extra + loss_weight_gradient, notes=tuple(notes))


def memory_plan_event(cfg, *, world_size: int, device_bytes: float, headroom: float = 0.9) -> dict[str, object] | None:
    """The ``memory_plan`` event of a training run: planned peak of the configured batch, whether it fits the device, and the
    largest batch that would.  ``cfg`` is an ``ExperimentConfig``; ``None`` when the run is outside what the plan covers (no
    model section, a strategy or sharding mode of the library engine only)."""

    if not cfg.model:
        return None
    strategy = cfg.parallel.strategy
    sharding = cfg.parallel.fsdp.sharding_strategy
    if strategy not in STRATEGIES or (strategy == "fsdp" and sharding not in ("full_shard", "shard_grad_op")):
        return None
    try:
        model = ModelConfig(**cfg.model)
        plan = plan_memory(model, strategy=strategy, world_size=world_size, sharding=sharding if strategy == "fsdp" else "full_shard",
                           local_batch_hint=cfg.train.batch_size,
                           activation_checkpointing=bool(strategy == "fsdp" and cfg.parallel.fsdp.activation_checkpointing))
    except (TypeError, ValueError):
        return None
    batch = cfg.train.batch_size
    return {"event": "memory_plan", "local_batch": batch, "planned_peak_gib": round(plan.total_bytes(batch) / GIB, 2),
            "planned_max_memory_allocated_gib": round(plan.total_bytes(batch, allocator_only=True) / GIB, 2),
            "resident_gib": round(plan.static_bytes() / GIB, 2), "gib_per_sample": round(plan.activation_bytes(1) / GIB, 4),
            "device_gib": round(device_bytes / GIB, 1), "fits": plan.total_bytes(batch) <= headroom * device_bytes,
            "max_local_batch": plan.max_local_batch(device_bytes, headroom=headroom)}
