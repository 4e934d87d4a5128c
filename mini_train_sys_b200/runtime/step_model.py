"""Work of one training step, item by item, and the time it would take at the machine's measured peaks.

A step of the decoder is a fixed list of operators.  For each the module states the algorithmic work (FLOPs of a
contraction, bytes of a streaming pass: every tensor read or written once) and divides by the denominators measured on
the machine (``MEASURED_PEAKS.json``: copy bandwidth, cuBLAS bf16 rate, burst and sustained).  The sum is the roofline of the
whole step: what it would cost if every kernel ran at its bound with no launch gaps.  ``achieved = bound / measured`` is
then one number for a step and one per item, next to which the per-kernel captures in ``profiles/`` explain the gap.

Conventions: one token = one row; ``T`` tokens per step and rank; expert rows are ``T * K`` (the routing plan's padding to
the GEMM tile is not counted as work); backward of a contraction costs two contractions; the attention FLOPs follow the
FlashAttention convention (``4 S^2 D`` per head forward, halved by causality, backward 2.5 x forward); AdamW reads four fp32
values and writes three fp32 and one bf16 per parameter.  The reference reports speed-ups over PyTorch per operator
(reports/engineering/kernels.md); it has no whole-step roofline.
"""

from __future__ import annotations

from dataclasses import dataclass

from mini_train_sys_b200.models.config import ModelConfig
from mini_train_sys_b200.train.metrics import measured_peaks

LOW, F32 = 2, 4


@dataclass(frozen=True)
class WorkItem:
    name: str
    kind: str                   # "gemm" | "attention" | "memory"
    count: int                  # launches of this shape per step
    flops: float = 0.0          # per launch
    bytes: float = 0.0          # per launch

    def bound_ms(self, peaks: dict[str, float], *, gemm_rate: str = "bf16_tflops_sustained") -> float:
        """Milliseconds per step for all ``count`` launches at the measured peak of the unit that bounds the item."""

        if self.kind == "memory":
            return self.count * self.bytes / (peaks["hbm_gbs"] * 1e9) * 1e3
        return self.count * self.flops / (peaks[gemm_rate] * 1e12) * 1e3


def step_work(model: ModelConfig, local_batch: int) -> list[WorkItem]:
    """The operators of one forward + backward + update, with their algorithmic work."""

    t = local_batch * model.seq_len
    h, i, v, layers, s = model.hidden_size, model.intermediate_size, model.vocab_size, model.n_layers, model.seq_len
    rows = t * model.experts_per_token if model.is_moe else t
    th = t * h * LOW                                         # one hidden-sized bf16 tensor
    gemm = lambda name, m, n, k, count=layers: WorkItem(name, "gemm", count, flops=2.0 * m * n * k)     # noqa: E731
    mem = lambda name, nbytes, count=layers: WorkItem(name, "memory", count, bytes=float(nbytes))       # noqa: E731
    items = [
        # ---- attention half of a block ------------------------------------------------------------------------------
        mem("rmsnorm forward (x2 per block)", 2 * th, 2 * layers),
        gemm("qkv projection", t, 3 * h, h), gemm("qkv projection, data gradient", t, h, 3 * h), gemm("qkv projection, weight gradient", 3 * h, h, t),
        WorkItem("attention forward (rope inside)", "attention", layers, flops=4.0 * local_batch * model.n_heads * s * s * model.head_dim * 0.5),
        WorkItem("attention backward", "attention", layers, flops=2.5 * 4.0 * local_batch * model.n_heads * s * s * model.head_dim * 0.5),
        gemm("attention output projection", t, h, h), gemm("output projection, data gradient", t, h, h), gemm("output projection, weight gradient", h, h, t),
        mem("residual + dropout forward (x2 per block)", 3 * th, 2 * layers), mem("residual + dropout backward (x2 per block)", 2 * th, 2 * layers),
        mem("rmsnorm backward (x2 per block)", 3 * th, 2 * layers),
    ]
    if model.is_moe:
        e = model.num_experts
        rh, ri = rows * h * LOW, rows * i * LOW
        items += [
            mem("router projection + post-processing, forward and backward", 2 * th + 6 * t * e * F32),
            mem("route gather", th + rh), mem("route combine", rh + th), mem("route combine backward", th + 2 * rh), mem("expert input gradient combine", rh + th),
            gemm("expert up-projection + SwiGLU", rows, 2 * i, h), gemm("expert down-projection", rows, h, i),
            gemm("d(gate, up) with SwiGLU derivative", rows, i, h), gemm("expert input gradient", rows, h, 2 * i),
            gemm("expert up-projection, weight gradient", 2 * i, h, rows), gemm("expert down-projection, weight gradient", h, i, rows),
        ]
        del ri
    else:
        items += [
            gemm("gate and up projections", t, 2 * i, h), gemm("down projection", t, h, i),
            mem("swiglu forward", 3 * t * i * LOW), mem("swiglu backward", 5 * t * i * LOW),
            gemm("gate / up data gradient", t, h, 2 * i), gemm("down data gradient", t, i, h),
            gemm("gate / up weight gradient", 2 * i, h, t), gemm("down weight gradient", h, i, t),
        ]
    items += [
        # ---- once per step --------------------------------------------------------------------------------------------
        mem("embedding gather and gradient scatter", 2 * th + t * 8, 1),
        mem("final rmsnorm forward and backward", 5 * th, 1),
        gemm("logits", t, v, h, 1), gemm("d(hidden) from d(logits)", t, h, v, 1), gemm("output matrix, weight gradient", v, h, t, 1),
        mem("cross-entropy forward (read logits)", t * v * LOW, 1), mem("cross-entropy backward (read and rewrite logits)", 2 * t * v * LOW, 1),
        mem("AdamW (four fp32 reads; three fp32 and one bf16 write per parameter)", model.param_count() * (4 * F32 + 3 * F32 + LOW), 1),
    ]
    return items


def step_roofline(model: ModelConfig, local_batch: int, *, peaks: dict[str, float] | None = None, measured_ms: float | None = None) -> dict:
    """Bound per item and in total at the measured peaks; with ``measured_ms`` also the achieved fraction of the step."""

    peaks = peaks or measured_peaks()
    table = []
    for item in step_work(model, local_batch):
        table.append({"item": item.name, "kind": item.kind, "launches": item.count,
                      "tflop_per_step": round(item.count * item.flops / 1e12, 4), "gb_per_step": round(item.count * item.bytes / 1e9, 4),
                      "bound_ms_sustained": round(item.bound_ms(peaks), 4),
                      "bound_ms_burst": round(item.bound_ms(peaks, gemm_rate="bf16_tflops"), 4)})
    totals = {kind: round(sum(r["bound_ms_sustained"] for r in table if r["kind"] == kind), 3) for kind in ("gemm", "attention", "memory")}
    bound = round(sum(totals.values()), 3)
    burst = round(sum(r["bound_ms_burst"] for r in table), 3)
    out = {"tokens_per_step": local_batch * model.seq_len, "peaks": peaks, "items": table, "bound_ms_by_kind": totals,
           "bound_ms_sustained": bound, "bound_ms_burst": burst,
           "gemm_tflop_per_step": round(sum(r["tflop_per_step"] for r in table if r["kind"] == "gemm"), 3)}
    if measured_ms:
        out["measured_ms"] = measured_ms
        out["achieved_fraction_of_sustained_bound"] = round(bound / measured_ms, 3)
        out["achieved_fraction_of_burst_bound"] = round(burst / measured_ms, 3)
    return out


NVLINK_GBS_MEASURED = 770.0        # peer copy per direction per GPU on this pool (nominal 900)


def comm_work(model: ModelConfig, local_batch: int, *, strategy: str, world_size: int, sharding: str = "full_shard",
              multimem: bool = False, link_gbs: float = NVLINK_GBS_MEASURED) -> list[dict]:
    """Bytes that cross NVLink per rank and step on each path of the fused engine, and the time they take alone at ``link_gbs``
    per direction.  A path is bounded by the larger of what a rank receives and what it sends; overlap with compute is what
    the engine is for, so these are the times to hide, not times to add to the step."""

    w = world_size
    if w <= 1 or strategy == "single":
        return []
    far = (w - 1) / w
    params = model.param_count()
    expert = model.n_layers * model.num_experts * 3 * model.hidden_size * model.intermediate_size if (strategy == "ep" and model.is_moe) else 0
    shared = params - expert
    paths = []

    def add(name: str, received: float, sent: float, launches: int) -> None:
        paths.append({"path": name, "launches": launches, "gb_in": round(received / 1e9, 4), "gb_out": round(sent / 1e9, 4),
                      "alone_ms": round(max(received, sent) / (link_gbs * 1e9) * 1e3, 4)})

    units = model.n_layers + 1
    if multimem:
        add("gradient reduce-scatter, summed inside the switch (multimem)", F32 * shared / w, 0.0, units)
    else:
        add("gradient reduce-scatter, pull of this rank's slice from every peer", far * F32 * shared, far * F32 * shared, units)
    if strategy == "fsdp" and sharding == "full_shard":
        add("parameter all-gather into staging slots, forward and backward", 2 * far * LOW * shared, 2 * far * LOW * shared, 2 * units - 2)
        add("AdamW: bf16 result stored into the own shard only", 0.0, 0.0, 1)
    else:
        add("AdamW: bf16 shard pushed into every peer's replica", far * LOW * shared, far * LOW * shared, 1)
    add("global gradient norm (one float per peer)", 4.0 * (w - 1), 4.0 * (w - 1), 1)
    if strategy == "ep":
        # per layer and pass a rank stores the rows of foreign experts at their owners and reads its results back, while its
        # peers do the same with it: two row transfers in and two out
        rows = local_batch * model.seq_len * model.experts_per_token
        per_pass = 2 * model.n_layers * far * rows * model.hidden_size * LOW
        add("expert dispatch and combine, forward (rows to the owners, results back)", per_pass, per_pass, 2 * model.n_layers)
        add("expert dispatch and combine, backward (row gradients to the owners, input gradients back)", per_pass, per_pass, 2 * model.n_layers)
    return paths
