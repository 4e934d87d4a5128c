#!/usr/bin/env python
# %% [markdown]
# # Distributed benchmark walkthrough
#
# The checks of the reference's `benchmarks/distributed/distributed_server_benchmark.ipynb`: inventory of the machine, a
# weak-scaling run (fixed work per GPU, 1 → N GPUs), the scaling table, and the quality gates (efficiency, data stall,
# memory head-room, complete repeats).
#
# On a machine with GPUs the cells run the 293M MoE under FSDP with the native back end and the fused engine on 1, 2, 4 …
# GPUs (a short run; `scripts/bash/distributed_benchmark.sh` is the full protocol).  Without a GPU they run the debug model
# on one and two Gloo ranks, which checks the harness (launch, identity hashing, reuse, reduction over ranks), not speed.

# %%
from __future__ import annotations

import json
import subprocess
import sys
import tempfile
from pathlib import Path

import torch


def repo_root() -> Path:
    here = Path(globals().get("__file__", Path.cwd() / "notebook")).resolve()
    for folder in (here, *here.parents):
        if (folder / "__graft_entry__.py").is_file():
            return folder
    raise RuntimeError("run this walkthrough from inside the repository")


ROOT = repo_root()
CLI = [sys.executable, str(ROOT / "scripts" / "run_dist_bench.py")]
GPUS = torch.cuda.device_count() if torch.cuda.is_available() else 0
scratch = tempfile.TemporaryDirectory()
out_dir = Path(scratch.name)


def run(*args: str, check: bool = True) -> subprocess.CompletedProcess:
    done = subprocess.run([*CLI, *args], capture_output=True, text=True, cwd=ROOT, timeout=3600)
    if check and done.returncode != 0:
        raise SystemExit(f"FAILED: {' '.join(args)}\n{done.stdout[-2000:]}\n{done.stderr[-3000:]}")
    return done


# %% [markdown]
# ## 1. Inventory
# What the harness records about the machine beside every result: devices, driver, library versions, code fingerprint.

# %%
inventory = json.loads(run("inventory").stdout)
print("[inventory]", {k: inventory[k] for k in list(inventory)[:6]})

# %% [markdown]
# ## 2. Weak scaling
# One `torchrun` per case, in its own session; every step is timed with CUDA events (host clock on a CPU) and the figure of
# a case is the maximum over its ranks.  A case whose identity hash (code, resolved configuration, sizes) matches a stored
# result is reused instead of run again.

# %%
if GPUS:
    worlds = [w for w in (1, 2, 4, 8) if w <= GPUS]
    arguments = ["--config", str(ROOT / "configs" / "bench" / "synbios_moe_fsdp.yaml"), "--strategies", "fsdp", "--ops-backends", "native",
                 "--engines", "fused", "--batch-sizes", "24", "--repeats", "2", "--warmup-steps", "5", "--measure-steps", "20"]
else:
    worlds = [1, 2]
    arguments = ["--config", str(ROOT / "configs" / "bench" / "debug_moe.yaml"), "--strategies", "ddp", "--ops-backends", "torch",
                 "--engines", "nccl", "--batch-sizes", "4", "--repeats", "1", "--warmup-steps", "1", "--measure-steps", "3"]
command = ["run", "--suite", "weak", "--output-dir", str(out_dir), "--world-sizes", ",".join(map(str, worlds)), "--master-port", "29671",
           "--timeout", "1200", *arguments]
first = run(*command, check=False)          # the exit code reflects the quality gates; the rows are checked below
print(first.stdout[-1500:])
summary = json.loads((out_dir / "weak" / "summary.json").read_text())
assert all(row["status"] == "ok" for row in summary["rows"]), [(r["name"], r["status"]) for r in summary["rows"]]
assert {w["world_size"] for w in summary["weak"]} == set(worlds)

# %% [markdown]
# ## 3. The table and the gates
# Efficiency is tokens/s at N GPUs divided by N times tokens/s at one.  The gates ask for at least 80 % efficiency, at
# most 5 % of the time spent waiting for data, at most 90 % of device memory in use, and every repeat complete.

# %%
for w in summary["weak"]:
    print({k: w[k] for k in ("strategy", "engine", "ops", "batch_size", "world_size", "tokens_per_sec_mean", "step_ms_mean", "efficiency_pct") if k in w})
print("[gates]", json.dumps(summary["quality_gates"]))
if GPUS > 1:
    assert summary["quality_gates"]["passed"], summary["quality_gates"]

# %% [markdown]
# ## 4. Reuse
# Running the same command again measures nothing: every row is found by its identity hash.

# %%
run(*command, check=False)
again = json.loads((out_dir / "weak" / "summary.json").read_text())
assert all(row.get("reused") for row in again["rows"])
print(run("present-weak", str(out_dir)).stdout[-800:])
scratch.cleanup()
print("walkthrough ok")
