#!/usr/bin/env python
# %% [markdown]
# # Operator benchmark walkthrough
#
# The checks of the reference's `benchmarks/operators/{operator_bench,moe_operator_bench}.ipynb`: every operator of the
# back-end protocol is first compared with the PyTorch implementation (forward and all gradients, random upstream
# gradients), and only then timed; a case that fails parity reports no time.
#
# On a B200 the cells compare the native sm_100a kernels with PyTorch on the shapes of the 293M model at one token count
# (`scripts/bash/operator_benchmark.sh` runs the whole ladder).  Without a GPU they run the same harness on two small
# operators with the fp32 oracle back end in the place of the native one, which checks the harness, not the kernels.

# %%
from __future__ import annotations

import json
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
sys.path.insert(0, str(ROOT))

from mini_train_sys_b200.bench import operators  # noqa: E402
from mini_train_sys_b200.bench.plots import write_kernel_plots  # noqa: E402

ON_GPU = torch.cuda.is_available()
PROVIDERS = ["torch", "native"] if ON_GPU else ["torch", "reference"]
KERNELS = list(operators.DENSE_KERNELS + operators.MOE_KERNELS) if ON_GPU else ["rmsnorm", "swiglu"]
TOKENS = 8192 if ON_GPU else 512
SCRIPT = ROOT / "scripts" / "bench_ops.py"
print(f"[setup] device={'cuda' if ON_GPU else 'cpu'} providers={PROVIDERS} kernels={len(KERNELS)} tokens={TOKENS}")

# %% [markdown]
# ## 1. One process per case
# A case is (operator, shape profile, token count).  Each runs in a fresh process, so that an out-of-memory case or a
# failed launch cannot poison the next one; the record comes back as one JSON line.

# %%
results = []
for kernel in KERNELS:
    tokens = 16384 if (kernel == "router" and ON_GPU) else TOKENS
    record = operators.run_case_subprocess(kernel, "project_formal", tokens, PROVIDERS, warmup=3 if ON_GPU else 1,
                                           iters=10 if ON_GPU else 2, check=True, timeout_s=900.0, script=SCRIPT)
    record.update(kernel=kernel, profile="project_formal", tokens=tokens)
    results.append(record)
    print(f"[case] {kernel:28s} {record['status']}")
assert all(r["status"] == "ok" for r in results), [(r["kernel"], r["status"], r.get("log_tail", "")[-300:]) for r in results if r["status"] != "ok"]

# %% [markdown]
# ## 2. Parity comes first
# Every provider other than `torch` carries a `correctness` verdict per output and gradient (max absolute and relative
# error, relative L2, cosine).  The quality gate fails when a case did not run or a verdict is negative.

# %%
gate = operators.quality_gate(results)
print(json.dumps(gate))
assert gate["quality_gate_passed"], gate
checked = [row for r in results for row in r["rows"] if row["provider"] != "torch"]
assert checked and all(row["correctness"]["passed"] for row in checked)

# %% [markdown]
# ## 3. The headline table
# p50 of forward, forward + backward and backward alone, the speed-up over PyTorch, and the fraction of the measured copy
# bandwidth or GEMM rate of this machine that the operator reaches.

# %%
table = operators.headline_table(results)
columns = ["kernel", "tokens", "provider", "fwd_ms", "full_ms", "speedup_full", "frac_of_gemm_peak", "frac_of_copy_peak", "parity"]
for row in table:
    print(" | ".join("" if row.get(c) is None else (f"{row[c]:.4g}" if isinstance(row[c], float) else str(row[c])) for c in columns))
assert {row["provider"] for row in table} == set(PROVIDERS)
# calls of the native back end that were answered by the PyTorch implementation instead (none expected on these shapes)
fallbacks = {k: v for r in results for row in r["rows"] for k, v in (row.get("dispatch") or {}).items() if k.endswith(":fallback") and v}
print(f"[dispatch] fallbacks: {fallbacks or 'none'}")

# %% [markdown]
# ## 4. Figures
# One SVG per operator: latency and speed-up over the token counts that were measured.

# %%
with tempfile.TemporaryDirectory() as tmp:
    written = write_kernel_plots(table, tmp)
    assert written and all("<svg" in (Path(tmp) / Path(p).name).read_text()[:400] for p in written)
    print(f"[plots] {len(written)} files, e.g. {Path(written[0]).name}")
print("walkthrough ok")
