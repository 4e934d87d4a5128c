#!/usr/bin/env python
# %% [markdown]
# # Planning walkthrough: will it fit, and how far from the roofline is it?
#
# Two pieces of arithmetic that need no GPU: the device-memory plan of a run under the fused sharding engine
# (`runtime/memory_plan.py`) and the roofline of one training step against the machine's measured peaks
# (`runtime/step_model.py`).  The cells reproduce the figures quoted in `docs/memory_planning.md` and in the benchmark report
# for the 293M top-2 MoE, and compare the plan with peaks that were measured on B200.

# %%
from __future__ import annotations

import sys
from pathlib import Path

import yaml


def repo_root() -> Path:
    here = Path(globals().get("__file__", Path.cwd() / "notebook")).resolve()
    for folder in (here, *here.parents):
        if (folder / "__graft_entry__.py").is_file():
            return folder
    raise RuntimeError("run this walkthrough from inside the repository")


ROOT = repo_root()
sys.path.insert(0, str(ROOT))

from mini_train_sys_b200.models.config import ModelConfig  # noqa: E402
from mini_train_sys_b200.runtime.memory_plan import GIB, plan_memory  # noqa: E402
from mini_train_sys_b200.runtime.step_model import comm_work, step_roofline  # noqa: E402

model = ModelConfig(**yaml.safe_load((ROOT / "configs" / "synbios_moe" / "model.yaml").read_text())["model"])
print(f"[model] {model.param_count():,} parameters, {model.active_param_count():,} touched per token, sequence {model.seq_len}")

# %% [markdown]
# ## 1. What is resident, what a sample adds
# Eight ranks, `full_shard`: optimizer state and master weights are sharded, the fp32 gradient buffer is not.

# %%
plan = plan_memory(model, strategy="fsdp", world_size=8, sharding="full_shard")
for name, nbytes in plan.static.items():
    where = "symmetric memory" if name in plan.symmetric else "caching allocator"
    print(f"[resident] {name:42s} {nbytes / GIB:7.3f} GiB  ({where})")
print(f"[sample]   {plan.activation_bytes(1) / GIB:.4f} GiB per sample of {model.seq_len} tokens")
assert plan.static["fp32_gradient_buffer"] == 4 * model.param_count()
assert abs(plan.static["fp32_master_moments_and_gradient_shard"] - 16 * model.param_count() / 8) < 64

# %% [markdown]
# ## 2. The plan against measured peaks
# `torch.cuda.max_memory_allocated` of benchmark runs on B200 (GiB) against the plan's allocator-visible total.

# %%
measured = [("single", 1, 96, 30.51), ("single", 1, 24, 12.88), ("fsdp", 2, 96, 26.23), ("fsdp", 4, 96, 25.14), ("fsdp", 8, 96, 24.59), ("fsdp", 8, 24, 6.96)]
for strategy, world, batch, gib in measured:
    p = plan_memory(model, strategy=strategy, world_size=world, local_batch_hint=batch)
    planned = p.total_bytes(batch, allocator_only=True) / GIB
    print(f"[check] {strategy:6s} x{world}  batch {batch:3d}: measured {gib:6.2f}  planned {planned:6.2f}  ({100 * (planned / gib - 1):+.1f} %)")
    assert abs(planned / gib - 1) < 0.02

# %% [markdown]
# ## 3. The largest batch on a 180 GB device

# %%
best = plan.max_local_batch(180 * GIB, headroom=0.9)
print(f"[limit] largest local batch under 0.9 x 180 GiB: {best} samples = {best * model.seq_len:,} tokens per rank and step")
assert plan.total_bytes(best) <= 0.9 * 180 * GIB < plan.total_bytes(best + 1)

# %% [markdown]
# ## 4. The roofline of one step
# Every operator's algorithmic work divided by the measured peak of the unit that bounds it.

# %%
roof = step_roofline(model, 96, measured_ms=62.69)
for kind, ms in roof["bound_ms_by_kind"].items():
    print(f"[bound] {kind:9s} {ms:6.2f} ms")
print(f"[bound] whole step {roof['bound_ms_sustained']:.2f} ms at the sustained GEMM rate; measured 62.69 ms -> "
      f"{roof['achieved_fraction_of_sustained_bound']:.2f} of the bound ({roof['peaks'].get('source', 'measured')} peaks)")
top = sorted(roof["items"], key=lambda r: -r["bound_ms_sustained"])[:5]
for row in top:
    print(f"[largest] {row['item'][:58]:58s} {row['bound_ms_sustained']:6.3f} ms")
assert 0.3 < roof["achieved_fraction_of_sustained_bound"] < 1.0

# %% [markdown]
# ## 5. What has to hide behind compute
# Bytes over NVLink per rank and step on eight GPUs, and the time they take alone at the measured 770 GB/s per direction.

# %%
for row in comm_work(model, 96, strategy="fsdp", world_size=8):
    print(f"[nvlink] {row['path'][:64]:64s} {row['gb_in']:6.3f} GB in  {row['alone_ms']:6.3f} ms alone")
total_alone = sum(row["alone_ms"] for row in comm_work(model, 96, strategy="fsdp", world_size=8))
assert total_alone < 0.1 * 62.69          # a twentieth of the step: hidden behind compute, it does not set the pace
print("walkthrough ok")
