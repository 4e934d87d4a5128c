#!/usr/bin/env python
# %% [markdown]
# # SynBioS walkthrough
#
# The checks of the reference's `synbios_moe_walkthrough.ipynb` (CPU, a few minutes), as cells that run as a plain script,
# unattended through `scripts/run_server_notebook.py`, or as the generated notebook `examples/notebooks/synbios_moe_walkthrough.ipynb`:
#
# prepare (byte codec, 40 people) -> train 2 steps through `scripts/train.py` on the generated shards -> evaluate recall and cloze
# from the exported `model.pt` -> build and validate the probe cache -> train one probe -> run the probe pipeline on two workers
# -> router analysis -> resume the training run to step 3.

# %%
from __future__ import annotations

import json
import subprocess
import sys
import tempfile
from pathlib import Path


def repo_root() -> Path:
    here = Path(globals().get("__file__", Path.cwd() / "notebook")).resolve()
    for folder in (here, *here.parents):
        if (folder / "__graft_entry__.py").is_file():
            return folder
    raise RuntimeError("run this walkthrough from inside the repository")


ROOT = repo_root()
PY = sys.executable


def run(*args: str) -> str:
    done = subprocess.run([PY, *args], capture_output=True, text=True, cwd=ROOT, timeout=1200)
    if done.returncode != 0:
        raise SystemExit(f"FAILED: {' '.join(args)}\n{done.stdout[-2000:]}\n{done.stderr[-3000:]}")
    return done.stdout


scratch = tempfile.TemporaryDirectory()
work = Path(scratch.name)
data = work / "data"
cli = str(ROOT / "scripts" / "synbios_moe.py")

# %% [markdown]
# ## 1. Data
# Profiles, biographies (two paraphrases per person, shuffled sentences), token shards.

# %%
run(cli, "prepare", "--output", str(data), "--variant", "multi2+permute", "--num-people", "40", "--codec", "bytes", "--quiet")
print("[prepare]", json.loads((data / "manifest.json").read_text())["num_biographies"], "biographies")

# %% [markdown]
# ## 2. Two training steps through `scripts/train.py`

# %%
model_yaml = work / "model.yaml"
model_yaml.write_text(json.dumps({"model": {"vocab_size": 257, "seq_len": 768, "n_layers": 2, "n_heads": 2, "hidden_size": 32,
                                            "intermediate_size": 32, "ffn_type": "moe", "num_experts": 4, "experts_per_token": 2,
                                            "dropout": 0.0}}))
train_yaml = work / "train.yaml"
train_yaml.write_text(json.dumps({
    "run": {"name": "walkthrough", "seed": 7}, "backend": {"ops": "torch"}, "parallel": {"strategy": "single"},
    "train": {"batch_size": 4, "max_steps": 2, "epochs": 50, "precision": "fp32", "log_interval": 1, "use_fused_loss": True},
    "optimizer": {"lr": 1e-3}, "lr_scheduler": {"schedule": "constant", "warmup_steps": 0},
    "data": {"source": "token_shards", "path": str(data / "token_shards"), "num_workers": 0, "persistent_workers": False,
             "pin_memory": False, "packing": "contiguous"},
    "checkpoint": {"directory": str(work / "ckpt"), "every_epochs": 1, "save_final": True, "export_model": True, "keep_last": 3},
    "logging": {"console": False, "jsonl": True, "tensorboard": False, "log_dir": str(work / "runs")}}))
run(str(ROOT / "scripts" / "train.py"), "--config", str(train_yaml), "--model-config", str(model_yaml), "--device", "cpu")
ckpts = sorted((work / "ckpt" / "walkthrough").glob("epoch_*"))
assert ckpts and (ckpts[-1] / "model.pt").is_file() and (ckpts[-1] / "COMMITTED").is_file(), ckpts
model_pt = ckpts[-1] / "model.pt"
print("[train] 2 steps, checkpoint", ckpts[-1].name)

# %% [markdown]
# ## 3. Recall and cloze from the exported `model.pt`

# %%
common = ["--data", str(data), "--model-config", str(model_yaml), "--checkpoint", str(model_pt), "--codec", "bytes", "--device", "cpu"]
run(cli, "evaluate", *common, "--output", str(work / "recall.json"), "--max-items", "10")
run(cli, "cloze-evaluate", *common, "--output", str(work / "cloze.json"), "--max-items", "4", "--batch-size", "8")
run(cli, "cloze-evaluate", *common, "--output", str(work / "cloze_progressive.json"), "--protocol", "progressive", "--max-items", "3",
    "--batch-size", "3", "--max-new-tokens", "4")
print("[evaluate] recall", json.loads((work / "recall.json").read_text())["overall"], "| cloze exact",
      json.loads((work / "cloze.json").read_text())["overall_exact_match"], "| progressive cloze biographies",
      json.loads((work / "cloze_progressive.json").read_text())["biographies"])

# %% [markdown]
# ## 4. Probe cache, one probe, the probe pipeline on two workers

# %%
cache = work / "cache"
run(cli, "cache-probes", "--data", str(data), "--output", str(cache), "--codec", "bytes")
assert json.loads(run(cli, "validate-probe-cache", "--probe-cache", str(cache), "--data", str(data)))["ok"]
run(cli, "probe", *common, "--probe-cache", str(cache), "--attribute", "university", "--target", "whole", "--kind", "q", "--steps", "5",
    "--batch-size", "8", "--output", str(work / "probe" / "q-university-whole.json"), "--quiet", "--max-eval-items", "16")
print("[probe] validation accuracy", json.loads((work / "probe" / "q-university-whole.json").read_text())["validation"]["accuracy"])

out = run(cli, "probe-pipeline", *common, "--probe-cache", str(cache), "--stage", "smoke", "--steps", "3", "--attributes", "major",
          "--devices", "cpu,cpu", "--output", str(work / "pipeline"), "--heartbeat-seconds", "1", "--max-eval-items", "8", "--quiet")
summary = json.loads(out.strip().splitlines()[-1])
assert summary["ok"], summary
print("[pipeline]", summary["counts"])

# %% [markdown]
# ## 5. Router analysis

# %%
run(cli, "analyze", *common, "--output", str(work / "routes.json"), "--max-items", "12")
print("[router] NMI per layer", {k: round(v["nmi_attribute_expert"], 3) for k, v in json.loads((work / "routes.json").read_text()).items()})

# %% [markdown]
# ## 6. Resume the training run to step 3

# %%
cfg = json.loads(train_yaml.read_text())
cfg["train"]["max_steps"] = 3
train_yaml.write_text(json.dumps(cfg))
run(str(ROOT / "scripts" / "train.py"), "--config", str(train_yaml), "--model-config", str(model_yaml), "--device", "cpu", "--resume", "latest")
events = [json.loads(line) for f in (work / "runs").rglob("*.jsonl") for line in f.read_text().splitlines()]
assert any(e.get("event") == "resume" for e in events) and max(e.get("step", 0) for e in events if e.get("event") == "train") == 3
print("[resume] continued to step 3")
scratch.cleanup()
print("walkthrough ok")
