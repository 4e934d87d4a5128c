#!/usr/bin/env python
# %% [markdown]
# # Training walkthrough
#
# The checks of the reference's `examples/notebooks/training_walkthrough.ipynb`, as cells that run as a plain script
# (`python examples/training_walkthrough.py`), unattended (`python scripts/run_server_notebook.py examples/training_walkthrough.py`)
# or as the notebook generated from this file (`examples/notebooks/training_walkthrough.ipynb`).
#
# Runs on CPU in a minute: load a config with `extends`, check the learning-rate curve, run a dense and an MoE model forward and
# backward, train a few steps, save a checkpoint, export `model.pt` and load it into a fresh fp32 model.  With a GPU present it
# repeats the forward / backward with the native sm_100a back end and compares the loss.  Every cell asserts what it shows.

# %%
from __future__ import annotations

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

from mini_train_sys_b200.models import MiniTransformer, ModelConfig, get_ops_backend  # noqa: E402
from mini_train_sys_b200.runtime.config import LRSchedulerConfig, OptimizerConfig, load_experiment  # noqa: E402
from mini_train_sys_b200.train.lr_scheduler import LearningRateScheduler  # noqa: E402
from mini_train_sys_b200.train.optim import build_optimizer  # noqa: E402
from mini_train_sys_b200.train.trainer import Trainer  # noqa: E402

# %% [markdown]
# ## 1. Configuration
# A run file is YAML with `extends`; the loader returns typed sections.

# %%
cfg = load_experiment(ROOT / "configs" / "train_debug.yaml")
print(f"[config] run={cfg.run.name} strategy={cfg.parallel.strategy} ops={cfg.backend.ops} model_keys={sorted(cfg.model)[:3]}")
assert cfg.parallel.strategy == "single" and cfg.train.batch_size > 0

# %% [markdown]
# ## 2. Learning-rate curve
# Linear warm-up, cosine decay to `min_lr_ratio`.

# %%
probe = torch.nn.Linear(2, 2)
opt = build_optimizer(probe, cfg=OptimizerConfig(lr=1e-3))
sched = LearningRateScheduler(opt, LRSchedulerConfig(schedule="cosine", warmup_steps=10, min_lr_ratio=0.1), total_steps=100)
curve = []
for step in range(100):
    sched.step(step)
    curve.append(opt.param_groups[0]["lr"])
assert abs(curve[0] - 1e-4) < 1e-9 and abs(curve[9] - 1e-3) < 1e-9 and curve[99] < 1.1e-4 and max(curve) <= 1e-3 + 1e-12
print(f"[lr] warm-up {curve[0]:.2e} -> {curve[9]:.2e}, end {curve[-1]:.2e}")

# %% [markdown]
# ## 3. Tiny dense and MoE models
# Forward, backward, finite gradients.

# %%
for ffn in ("dense", "moe"):
    mc = ModelConfig(vocab_size=512, seq_len=32, n_layers=2, n_heads=2, hidden_size=64, intermediate_size=96, ffn_type=ffn,
                     num_experts=4, experts_per_token=2)
    torch.manual_seed(0)
    model = MiniTransformer(mc, get_ops_backend("torch"), activation_dtype=torch.float32)
    tokens = torch.randint(0, 512, (4, 33))
    loss, _ = model(tokens[:, :-1], targets=tokens[:, 1:], use_fused_loss=True)
    loss.backward()
    assert torch.isfinite(loss) and all(torch.isfinite(p.grad).all() for p in model.parameters() if p.grad is not None)
    print(f"[model] {ffn}: params={mc.param_count():,} loss={loss.item():.4f}")

# %% [markdown]
# ## 4. A few optimizer steps, a checkpoint, the exported `model.pt`, a reload

# %%
from mini_train_sys_b200.train.checkpoint import load_model_state_dict_from_checkpoint, save_checkpoint  # noqa: E402

mc = ModelConfig(vocab_size=512, seq_len=32, n_layers=2, n_heads=2, hidden_size=64, intermediate_size=96, ffn_type="moe",
                 num_experts=4, experts_per_token=2)
torch.manual_seed(1)
model = MiniTransformer(mc, get_ops_backend("torch"), activation_dtype=torch.float32)
optimizer = build_optimizer(model, cfg=OptimizerConfig(lr=3e-3))
trainer = Trainer(model, optimizer, device=torch.device("cpu"), use_fused_loss=True, precision="fp32", grad_clip_norm=1.0)
gen = torch.Generator().manual_seed(2)
fixed = torch.randint(0, 512, (8, 33), generator=gen)
losses = [float(trainer.train_step({"input_ids": fixed[:, :-1], "targets": fixed[:, 1:]})) for _ in range(8)]
assert losses[-1] < losses[0], losses
print(f"[train] loss {losses[0]:.4f} -> {losses[-1]:.4f} over 8 steps on one batch")
with tempfile.TemporaryDirectory() as tmp:
    path = Path(tmp) / "ckpt"
    save_checkpoint(path, model, optimizer, step=8, export_model=True)
    state = load_model_state_dict_from_checkpoint(path)
    fresh = MiniTransformer(mc, get_ops_backend("torch"), activation_dtype=torch.float32)
    fresh.load_state_dict(state)
    a, _ = model(fixed[:, :-1], targets=fixed[:, 1:], use_fused_loss=True)
    b, _ = fresh(fixed[:, :-1], targets=fixed[:, 1:], use_fused_loss=True)
    assert abs(float(a) - float(b)) < 1e-6
    print(f"[checkpoint] round trip ok ({sorted(p.name for p in path.iterdir())})")

# %% [markdown]
# ## 5. The native back end on a GPU
# Skipped without one.

# %%
if torch.cuda.is_available():
    mc = ModelConfig(vocab_size=1024, seq_len=128, n_layers=2, n_heads=4, hidden_size=256, intermediate_size=256, ffn_type="moe",
                     num_experts=4, experts_per_token=2)
    tokens = torch.randint(0, 1024, (4, 129), device="cuda")
    out = {}
    for name in ("torch", "native"):
        torch.manual_seed(3)
        m = MiniTransformer(mc, get_ops_backend(name), activation_dtype=torch.bfloat16).cuda()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss, _ = m(tokens[:, :-1], targets=tokens[:, 1:], use_fused_loss=True)
        loss.backward()
        out[name] = float(loss)
    assert abs(out["torch"] - out["native"]) < 2e-2, out
    print(f"[native] loss torch={out['torch']:.4f} native={out['native']:.4f}")
print("walkthrough ok")
