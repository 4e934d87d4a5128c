"""End-to-end CLI runs on CPU: train (events, checkpoints, resume), evaluate, sample, data preparation."""

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import yaml

ROOT = Path(__file__).resolve().parents[1]
PY = sys.executable


def run(args, cwd):
    env = {**os.environ, "PYTHONPATH": str(ROOT)}
    done = subprocess.run([PY, *args], cwd=cwd, env=env, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-2000:]
    return done.stdout


def events(cwd):
    files = sorted(Path(cwd).rglob("events.jsonl"))
    return [json.loads(line) for f in files for line in f.read_text().splitlines()]


def test_debug_moe_run_reproduces_the_reference_loss_curve(tmp_path):
    out = run([str(ROOT / "scripts" / "train.py"), "--config", str(ROOT / "configs" / "train_debug.yaml"), "--model-config",
               str(ROOT / "configs" / "model_debug_moe.yaml"), "--device", "cpu"], tmp_path)
    assert "[init] run=debug device=cpu strategy=single world=1 params=1050240" in out
    log = events(tmp_path)
    train = [e for e in log if e["event"] == "train"]
    assert log[0]["event"] == "init" and log[0]["ops"] == "torch" and len(train) == 10
    # the unmodified reference prints 7.689 at step 1 and 7.662 at step 10 for this config and seed
    assert train[0]["loss"] == pytest.approx(7.68907, abs=2e-4) and train[-1]["loss"] == pytest.approx(7.66168, abs=2e-3)
    for key in ("lr", "tokens_seen", "tokens_per_sec", "step_time_ms", "data_wait_percent", "grad_norm", "moe/aux_loss",
                "loss/lm_cross_entropy", "moe/expert_load_fraction_by_layer", "host_peak_memory_mb", "roofline_step_bound_ms"):
        assert key in train[0], key
    assert len(train[0]["moe/expert_load_fraction_by_layer"]) == 2 and len(train[0]["moe/expert_load_fraction_by_layer"][0]) == 4


def test_device_prefetch_option_feeds_the_same_batches(tmp_path):
    """``data.device_prefetch`` routes the loader through the side-stream prefetcher (a pass-through on a CPU): same batches,
    same order, same number of steps."""

    losses = {}
    for flag in (False, True):
        cfg = yaml.safe_load((ROOT / "configs" / "train_debug.yaml").read_text())
        cfg["run"]["name"] = f"prefetch_{flag}"
        cfg["train"].update(max_steps=6, log_interval=1)
        cfg["data"]["device_prefetch"] = flag
        cfg["logging"]["tensorboard"] = False
        work = tmp_path / str(flag)
        work.mkdir()
        (work / "run.yaml").write_text(yaml.safe_dump(cfg))
        run([str(ROOT / "scripts" / "train.py"), "--config", "run.yaml", "--model-config", str(ROOT / "configs" / "model_debug_dense.yaml"),
             "--device", "cpu"], work)
        losses[flag] = [e["loss"] for e in events(work) if e["event"] == "train"]
    assert len(losses[True]) == 6 and losses[True] == losses[False]


def test_resume_inside_an_epoch_continues_behind_the_batches_already_seen(tmp_path):
    """A run stopped in the middle of an epoch and resumed sees exactly the batches the uninterrupted run sees (the reference
    restarts the interrupted epoch): same loss at every step, also across the next epoch boundary."""

    def config(name, max_steps, packing=None):
        cfg = yaml.safe_load((ROOT / "configs" / "train_debug.yaml").read_text())
        cfg["run"]["name"] = name
        cfg["train"].update(max_steps=max_steps, epochs=None, log_interval=1)
        cfg["data"]["num_tokens"] = 64 * cfg["train"]["batch_size"] * 6 + 1            # six batches per epoch
        cfg["checkpoint"] = {"directory": "ckpt", "every_epochs": 1, "export_model": False, "keep_last": 5, "save_final": True}
        cfg["logging"]["tensorboard"] = False
        return cfg

    model_cfg = str(ROOT / "configs" / "model_debug_moe.yaml")
    whole = tmp_path / "whole"
    whole.mkdir()
    (whole / "run.yaml").write_text(yaml.safe_dump(config("cursor", 10)))
    run([str(ROOT / "scripts" / "train.py"), "--config", "run.yaml", "--model-config", model_cfg, "--device", "cpu"], whole)
    want = {e["step"]: e["loss"] for e in events(whole) if e["event"] == "train"}
    assert sorted(want) == list(range(1, 11))

    parts = tmp_path / "parts"
    parts.mkdir()
    (parts / "run.yaml").write_text(yaml.safe_dump(config("cursor", 4)))                  # stops after batch 4 of 6 of the first epoch
    run([str(ROOT / "scripts" / "train.py"), "--config", "run.yaml", "--model-config", model_cfg, "--device", "cpu"], parts)
    (parts / "run.yaml").write_text(yaml.safe_dump(config("cursor", 10)))
    run([str(ROOT / "scripts" / "train.py"), "--config", "run.yaml", "--model-config", model_cfg, "--device", "cpu", "--resume", "latest"], parts)
    log = events(parts)
    resumed = [e for e in log if e["event"] == "resume"]
    assert len(resumed) == 1 and resumed[0]["step"] == 4 and resumed[0]["epoch"] == 0 and resumed[0]["epoch_batches_done"] == 4
    got = {e["step"]: e["loss"] for e in log if e["event"] == "train"}
    assert sorted(got) == list(range(1, 11))
    for step in range(1, 11):
        assert got[step] == pytest.approx(want[step], abs=1e-6), (step, got[step], want[step])
    first_after = next(e for e in log if e["event"] == "train" and e["step"] == 5)
    assert first_after["epoch"] == 1 and first_after["batch"] == 5 and first_after["batches_total"] == 6

    # periodic checkpoints inside an epoch (checkpoint.every_steps): resume from the one at step 4 as after a crash at step 5
    periodic = tmp_path / "periodic"
    periodic.mkdir()
    cfg = config("cursor", 5)
    cfg["checkpoint"]["every_steps"] = 2
    (periodic / "run.yaml").write_text(yaml.safe_dump(cfg))
    run([str(ROOT / "scripts" / "train.py"), "--config", "run.yaml", "--model-config", model_cfg, "--device", "cpu"], periodic)
    saved = sorted(p.name for p in (periodic / "ckpt" / "cursor").iterdir())
    assert saved == ["epoch_000000_step_000000002", "epoch_000000_step_000000004", "epoch_000000_step_000000005"], saved
    assert not (periodic / "ckpt" / "cursor" / saved[0] / "model.pt").exists()
    cfg["train"]["max_steps"] = 10
    (periodic / "run.yaml").write_text(yaml.safe_dump(cfg))
    run([str(ROOT / "scripts" / "train.py"), "--config", "run.yaml", "--model-config", model_cfg, "--device", "cpu", "--resume",
         str(periodic / "ckpt" / "cursor" / saved[1])], periodic)
    after = {}
    for e in events(periodic):
        if e["event"] == "train":
            after[e["step"]] = e["loss"]            # the second session overwrites step 5 of the first
    for step in range(1, 11):
        assert after[step] == pytest.approx(want[step], abs=1e-6), (step, after[step], want[step])


def test_sampler_cursor_skips_exactly_this_ranks_first_samples():
    import torch

    from mini_train_sys_b200.data.dataloader import ShardAwareBlockSampler, TokenBlockDataset

    data = TokenBlockDataset(torch.arange(0, 16 * 40 + 1), 16)
    for world in (1, 2, 3):
        for rank in range(world):
            sampler = ShardAwareBlockSampler(data, shuffle=True, seed=5, rank=rank, world_size=world, shuffle_window=7)
            sampler.set_epoch(3)
            full = list(sampler)
            sampler.set_start(4)
            assert list(sampler) == full[4:] and list(sampler) == full          # the cursor applies to one iteration only
            sampler.set_start(10**6)
            assert list(sampler) == []
    with pytest.raises(ValueError):
        sampler.set_start(-1)


@pytest.fixture()
def run_cfg(tmp_path):
    cfg = yaml.safe_load((ROOT / "configs" / "train_debug.yaml").read_text())
    cfg["run"]["name"] = "cli"
    cfg["train"].update(max_steps=None, epochs=2, log_interval=5)
    cfg["data"]["num_tokens"] = 64 * 2 * 6 + 1
    cfg["checkpoint"] = {"directory": "ckpt", "every_epochs": 1, "export_model": True, "keep_last": 3}
    cfg["logging"]["tensorboard"] = False
    path = tmp_path / "run.yaml"
    path.write_text(yaml.safe_dump(cfg))
    return path


def test_train_checkpoint_resume_eval_sample(tmp_path, run_cfg):
    model_cfg = str(ROOT / "configs" / "model_debug_dense.yaml")
    base = [str(ROOT / "scripts" / "train.py"), "--config", str(run_cfg), "--model-config", model_cfg, "--device", "cpu"]
    run(base, tmp_path)
    ckpts = sorted((tmp_path / "ckpt" / "cli").iterdir())
    assert [p.name for p in ckpts] == ["epoch_000001_step_000000006", "epoch_000002_step_000000012"]
    assert all((p / "COMMITTED").is_file() and (p / "model.pt").is_file() and (p / "distributed").is_dir() for p in ckpts)
    saved = [e for e in events(tmp_path) if e["event"] == "checkpoint"]
    assert len(saved) == 2 and saved[0]["includes_optimizer"]
    # one more epoch from the latest checkpoint
    cfg = yaml.safe_load(run_cfg.read_text())
    cfg["train"]["epochs"] = 3
    run_cfg.write_text(yaml.safe_dump(cfg))
    out = run([*base, "--resume"], tmp_path)
    assert "[resume]" in out and "epoch=2 step=12" in out
    assert (tmp_path / "ckpt" / "cli" / "epoch_000003_step_000000018" / "COMMITTED").is_file()
    last = tmp_path / "ckpt" / "cli" / "epoch_000003_step_000000018"
    res = json.loads(run([str(ROOT / "scripts" / "eval.py"), "--checkpoint", str(last), "--device", "cpu", "--max-batches", "2"],
                         tmp_path).strip().splitlines()[-1])
    assert res["event"] == "evaluate" and 5.0 < res["loss"] < 9.0 and res["tokens"] > 0
    gen = json.loads(run([str(ROOT / "scripts" / "sample.py"), "--checkpoint", str(last), "--device", "cpu", "--prompt-ids", "1,2,3",
                          "--max-new-tokens", "5", "--greedy"], tmp_path).strip().splitlines()[-1])
    assert gen["tokens"][:3] == [1, 2, 3] and len(gen["tokens"]) == 8


def test_prepare_data_cli_and_training_on_shards(tmp_path):
    script = str(ROOT / "scripts" / "prepare_data.py")
    out = json.loads(run([script, "random-shards", "--output", "shards", "--vocab-size", "2048", "--num-tokens", "3000"], tmp_path))
    assert (tmp_path / out["manifest"]).is_file()
    info = json.loads(run([script, "inspect", str(tmp_path / "shards")], tmp_path))
    assert info["splits"]["train"]["tokens"] == 3000 and info["vocab_size"] == 2048
    cfg = yaml.safe_load((ROOT / "configs" / "train_debug.yaml").read_text())
    cfg["data"].update(source="token_shards", path=str(tmp_path / "shards"), packing="randomized_documents")
    cfg["train"]["max_steps"] = 3
    cfg["logging"]["tensorboard"] = False
    (tmp_path / "run.yaml").write_text(yaml.safe_dump(cfg))
    run([str(ROOT / "scripts" / "train.py"), "--config", "run.yaml", "--model-config", str(ROOT / "configs" / "model_debug_dense.yaml"),
         "--device", "cpu"], tmp_path)
    assert len([e for e in events(tmp_path) if e["event"] == "train"]) == 3


def test_walkthrough_runner_records_cells_and_fails_on_errors(tmp_path):
    import json
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    runner = [sys.executable, str(root / "scripts" / "run_server_notebook.py")]
    good = tmp_path / "good.py"
    good.write_text("# %% first\nx = 2\nprint('x is', x)\n# %% second\nassert x == 2\nprint('done')\n")
    done = subprocess.run([*runner, str(good), "--output", str(tmp_path / "good.json"), "--quiet"], capture_output=True, text=True)
    assert done.returncode == 0, done.stderr
    rec = json.loads((tmp_path / "good.json").read_text())
    assert rec["cells"] == 2 and rec["failed_cells"] == [] and rec["records"][0]["stdout"] == "x is 2\n"
    notebook = {"cells": [{"cell_type": "markdown", "source": ["# title"]},
                          {"cell_type": "code", "source": ["%matplotlib inline\n", "y = 1\n"], "outputs": []},
                          {"cell_type": "code", "source": "raise ValueError('boom')", "outputs": []},
                          {"cell_type": "code", "source": "print('never reached')", "outputs": []}], "metadata": {}, "nbformat": 4}
    bad = tmp_path / "bad.ipynb"
    bad.write_text(json.dumps(notebook))
    done = subprocess.run([*runner, str(bad), "--output", str(tmp_path / "bad.json"), "--executed-notebook", str(tmp_path / "bad.out.ipynb"),
                           "--quiet"], capture_output=True, text=True)
    assert done.returncode == 1
    rec = json.loads((tmp_path / "bad.json").read_text())
    assert rec["executed"] == 2 and rec["failed_cells"] == [1] and "ValueError: boom" in rec["records"][1]["error"]
    executed = json.loads((tmp_path / "bad.out.ipynb").read_text())
    assert executed["cells"][2]["outputs"][0]["output_type"] == "error"
    # the reference's options: everything into one directory, a limit per cell
    slow = tmp_path / "slow.ipynb"
    slow.write_text(json.dumps({"cells": [{"cell_type": "code", "source": "print('fast')", "outputs": []},
                                          {"cell_type": "code", "source": "import time\ntime.sleep(30)", "outputs": []}], "metadata": {}, "nbformat": 4}))
    done = subprocess.run([*runner, str(slow), "--output-dir", str(tmp_path / "out"), "--timeout-seconds", "1", "--kernel", "ignored", "--quiet"],
                          capture_output=True, text=True, timeout=60)
    assert done.returncode == 1
    rec = json.loads((tmp_path / "out" / "slow.run.json").read_text())
    assert rec["failed_cells"] == [1] and "CellTimeout" in rec["records"][1]["error"] and rec["records"][1]["seconds"] < 10
    assert (tmp_path / "out" / "slow.executed.ipynb").is_file()


def test_committed_notebooks_equal_their_percent_format_sources_and_run(tmp_path):
    import importlib.util
    import json
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    spec = importlib.util.spec_from_file_location("run_server_notebook", root / "scripts" / "run_server_notebook.py")
    runner = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(runner)
    cells = runner.percent_cells("#!/usr/bin/env python\n# %% [markdown]\n# # Title\n#\n# text\n\n# %%\nx = 1\n\n\n# %% named\nprint(x)\n")
    assert cells == [("markdown", "# Title\n\ntext"), ("code", "x = 1"), ("code", "print(x)")]
    for name in ("training_walkthrough", "synbios_moe_walkthrough", "operator_benchmark_walkthrough", "distributed_benchmark_walkthrough",
                 "planning_walkthrough"):
        source = root / "examples" / f"{name}.py"
        committed = json.loads((root / "examples" / "notebooks" / f"{name}.ipynb").read_text(encoding="utf-8"))
        assert committed == runner.notebook_from_script(source.read_text(encoding="utf-8")), f"regenerate {name}.ipynb with --export-ipynb"
        kinds = [c["cell_type"] for c in committed["cells"]]
        assert kinds[0] == "markdown" and kinds.count("code") >= 4 and all(c["outputs"] == [] for c in committed["cells"] if c["cell_type"] == "code")
    notebook = root / "examples" / "notebooks" / "training_walkthrough.ipynb"
    done = subprocess.run([sys.executable, str(root / "scripts" / "run_server_notebook.py"), str(notebook), "--output", str(tmp_path / "run.json"),
                           "--executed-notebook", str(tmp_path / "executed.ipynb"), "--quiet"], capture_output=True, text=True, cwd=tmp_path)
    assert done.returncode == 0, done.stderr[-2000:]
    record = json.loads((tmp_path / "run.json").read_text())
    assert record["failed_cells"] == [] and "walkthrough ok" in record["records"][-1]["stdout"]
    executed = json.loads((tmp_path / "executed.ipynb").read_text())
    assert any(o.get("text", "").startswith("[lr]") for c in executed["cells"] if c["cell_type"] == "code" for o in c["outputs"])
    exported = tmp_path / "again.ipynb"
    done = subprocess.run([sys.executable, str(root / "scripts" / "run_server_notebook.py"), str(root / "examples" / "training_walkthrough.py"),
                           "--export-ipynb", str(exported)], capture_output=True, text=True)
    assert done.returncode == 0 and json.loads(exported.read_text()) == json.loads(notebook.read_text())


def test_planning_walkthrough_notebook_runs(tmp_path):
    import json
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    done = subprocess.run([sys.executable, str(root / "scripts" / "run_server_notebook.py"), str(root / "examples" / "notebooks" / "planning_walkthrough.ipynb"),
                           "--output", str(tmp_path / "run.json"), "--quiet"], capture_output=True, text=True, timeout=300, cwd=tmp_path)
    assert done.returncode == 0, done.stderr[-2000:]
    record = json.loads((tmp_path / "run.json").read_text())
    assert record["failed_cells"] == [] and "walkthrough ok" in record["records"][-1]["stdout"]


def test_operator_benchmark_walkthrough_runs_cell_by_cell_on_a_cpu(tmp_path):
    import json
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    done = subprocess.run([sys.executable, str(root / "scripts" / "run_server_notebook.py"), str(root / "examples" / "operator_benchmark_walkthrough.py"),
                           "--output", str(tmp_path / "run.json"), "--quiet"], capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-2000:]
    record = json.loads((tmp_path / "run.json").read_text())
    assert record["failed_cells"] == [] and "walkthrough ok" in record["records"][-1]["stdout"]
    assert any("quality_gate_passed" in r["stdout"] for r in record["records"])


def test_ground_truth_first_audit_lists_every_violation(tmp_path):
    import json
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    rec = {"protocol": "ground_truth_first_whole_rank_matched_v1", "ground_truth_first_token": True, "backbone_parameters_updated": False,
           "target": "whole", "identity": {"kind": "p", "rank": 2, "steps": 20}, "reference_rank": 2, "steps": 20, "final_loss": 1.5,
           "resumed_from_step": 10, "whole_accuracy_validation_by_source_position": [0.5] * 6,
           "whole_correct_validation_by_source_position": [2] * 6, "whole_total_validation_by_source_position": [4] * 6,
           "first_token_text": {"32": " "}}
    path = tmp_path / "p_university.json"
    path.write_text(json.dumps(rec))
    path.with_suffix(".pt").write_bytes(b"x")
    cmd = [sys.executable, str(root / "scripts" / "audit_ground_truth_first_probe.py"), str(path), "--expect-resumed-from", "10"]
    done = subprocess.run(cmd, capture_output=True, text=True)
    assert done.returncode == 0 and json.loads(done.stdout)["ok"], done.stdout + done.stderr
    rec.update(backbone_parameters_updated=True, resumed_from_step=None)
    rec["whole_total_validation_by_source_position"] = [4, 4, 4, 4, 4, 9]
    path.write_text(json.dumps(rec))
    done = subprocess.run(cmd, capture_output=True, text=True)
    errors = json.loads(done.stdout)["errors"]
    assert done.returncode == 1 and len(errors) >= 3 and any("frozen" in e for e in errors) and any("resumed" in e for e in errors)


def _launcher_sandbox(tmp_path):
    """A copy of the bash launchers under a scratch checkout whose `python` prints its arguments instead of running them."""

    import shutil
    import stat

    checkout = tmp_path / "checkout"
    shutil.copytree(ROOT / "scripts" / "bash", checkout / "scripts" / "bash")
    shutil.copytree(ROOT / "configs", checkout / "configs")
    stub = tmp_path / "python_stub"
    stub.write_text('#!/usr/bin/env bash\necho "ARGS: $*"\necho "TMPDIR=${TMPDIR:-} STORAGE=${MTS_STORAGE_ROOT:-}"\n')
    stub.chmod(stub.stat().st_mode | stat.S_IEXEC)
    env = {"PATH": os.environ["PATH"], "PYTHON": str(stub), "HOME": str(tmp_path)}
    run = lambda script, *args, **extra: subprocess.run(["bash", str(checkout / "scripts" / "bash" / script), *args], capture_output=True,   # noqa: E731
                                                        text=True, timeout=120, env={**env, **extra})
    return checkout, run


def test_storage_setup_links_artifacts_to_the_data_disk_and_launchers_pick_it_up(tmp_path):
    checkout, run = _launcher_sandbox(tmp_path)
    disk = tmp_path / "disk"
    disk.mkdir()
    refused = run("setup_storage.sh", str(disk))
    if refused.returncode == 0:
        pytest.skip("the scratch directory is on a filesystem of its own")
    assert refused.returncode == 2 and "root filesystem" in refused.stderr and not (checkout / "artifacts").exists()
    assert run("setup_storage.sh", "relative/path").returncode == 2
    done = run("setup_storage.sh", str(disk), ALLOW_SYSTEM_DISK_STORAGE="1")
    assert done.returncode == 0, done.stderr
    store = disk / "mini-train-sys"
    assert (checkout / "artifacts").is_symlink() and (checkout / "artifacts").resolve() == (store / "artifacts").resolve()
    assert (store / "artifacts" / "synbios_moe" / "checkpoints").is_dir() and (store / "cache" / "torch_extensions").is_dir() and (store / "tmp").is_dir()
    settings = (checkout / ".mts-storage.env").read_text()
    assert f"export MTS_STORAGE_ROOT={store}" in settings and f"export TMPDIR={store}/tmp" in settings
    assert run("setup_storage.sh", str(disk), ALLOW_SYSTEM_DISK_STORAGE="1").returncode == 0            # a second run changes nothing
    # a storage root outside the disk, and a link that points elsewhere, are refused
    assert run("setup_storage.sh", str(disk), ALLOW_SYSTEM_DISK_STORAGE="1", MTS_STORAGE_ROOT=str(tmp_path / "elsewhere")).returncode == 2
    other = tmp_path / "disk2"
    other.mkdir()
    clash = run("setup_storage.sh", str(other), ALLOW_SYSTEM_DISK_STORAGE="1")
    assert clash.returncode == 2 and "already links" in clash.stderr
    # the launchers read the settings
    out = run("train.sh")
    assert out.returncode == 0 and f"TMPDIR={store}/tmp STORAGE={store}" in out.stdout, out.stdout + out.stderr
    # files already in a real artifacts directory are never moved
    (checkout / "artifacts").unlink()
    (checkout / "artifacts").mkdir()
    (checkout / "artifacts" / "keep.txt").write_text("x")
    kept = run("setup_storage.sh", str(disk), ALLOW_SYSTEM_DISK_STORAGE="1")
    assert kept.returncode == 2 and "left alone" in kept.stderr and (checkout / "artifacts" / "keep.txt").exists()


def test_launchers_take_their_settings_from_the_environment(tmp_path):
    checkout, run = _launcher_sandbox(tmp_path)
    out = run("train.sh", CONFIG="configs/train_debug.yaml", MODEL_CONFIG="configs/model_debug_moe.yaml", DEVICE="cpu", RESUME="latest")
    assert "scripts/train.py --config configs/train_debug.yaml --device cpu --model-config configs/model_debug_moe.yaml --resume latest" in out.stdout, out.stdout + out.stderr
    out = run("train.sh", "configs/train_single.yaml", "--max-steps", "3")
    assert "--config configs/train_single.yaml --device auto --max-steps 3" in out.stdout
    out = run("distributed.sh", "fsdp", NPROC="4", MASTER_PORT="29777")
    assert out.returncode == 0 and "--nproc-per-node 4 --master-addr 127.0.0.1 --master-port 29777 scripts/train.py --config configs/server/b200_180gb/runs/fsdp_4gpu.yaml " \
        "--model-config configs/synbios_moe/model.yaml --resume auto" in out.stdout, out.stdout + out.stderr
    out = run("distributed.sh", "ddp", "2", "--max-steps", "5", RESUME="safety", MAX_RESTARTS="2")
    assert "--rdzv-backend c10d" in out.stdout and "--max-restarts 2" in out.stdout and "ddp_2gpu.yaml" in out.stdout and "--resume safety --max-steps 5" in out.stdout
    assert run("distributed.sh", "zero3", "2").returncode == 2 and run("distributed.sh", "fsdp", "3").returncode == 2
    # the study launcher: data present -> no prepare; AUTO_RESUME=0 drops --resume; people that differ across variants stop it
    data = checkout / "artifacts" / "synbios_moe" / "data"
    for variant, people in (("single", "a\n"), ("multi5_permute", "a\n")):
        (data / variant).mkdir(parents=True)
        (data / variant / "manifest.json").write_text("{}")
        (data / variant / "profiles.jsonl").write_text(people)
    out = run("synbios_moe.sh", "single", "fsdp", NPROC="8")
    assert out.returncode == 0 and "prepare" not in out.stdout and "--nproc-per-node 8" in out.stdout and "--resume auto" in out.stdout, out.stdout + out.stderr
    out = run("synbios_moe.sh", "single", "single", AUTO_RESUME="0")
    assert out.returncode == 0 and "--resume" not in out.stdout and "single_single.yaml" in out.stdout
    (checkout / "artifacts" / "synbios_moe" / "checkpoints" / "synbios_moe_single_fsdp" / "epoch_000001_step_000000010").mkdir(parents=True)
    forced = run("synbios_moe.sh", "single", "fsdp", "8", FORCE_PREPARE="1")
    assert forced.returncode == 2 and "refusing" in forced.stderr
    (data / "multi5_permute" / "profiles.jsonl").write_text("b\n")
    differ = run("synbios_moe.sh", "single", "fsdp", "8")
    assert differ.returncode == 2 and "differ" in differ.stderr


def test_probe_launcher_takes_both_call_forms_and_the_study_cli_resolves_checkpoint_directories(tmp_path):
    checkout, run = _launcher_sandbox(tmp_path)
    data = checkout / "artifacts" / "synbios_moe" / "data" / "single"
    data.mkdir(parents=True)
    batches = tmp_path / "recommended.env"
    batches.write_text("P_BATCH_SIZE=64\nQ_BATCH_SIZE=32\n")
    out = run("synbios_probes.sh", "single", "fsdp", STAGE="pilot", PROBE_DEVICES="cuda:0,cuda:1", PROBE_BATCH_ENV=str(batches),
              SKIP_PRETRAIN_GATE="1", PROBE_LOG_INTERVAL="50")
    assert out.returncode == 0, out.stdout + out.stderr
    lines = [line for line in out.stdout.splitlines() if line.startswith("ARGS:")]
    # the stub python "validates" any cache, so only a missing manifest leads to cache-probes
    assert "cache-probes --data artifacts/synbios_moe/data/single" in lines[0] and lines[0].endswith("--codec gpt2 --require-coverage")
    pipeline = [line for line in lines if "probe-pipeline" in line]
    assert len(pipeline) == 1 and "--stage pilot" in pipeline[0] and "--devices cuda:0,cuda:1" in pipeline[0]
    assert "--checkpoint artifacts/synbios_moe/checkpoints/synbios_moe_single_fsdp/latest" in pipeline[0]
    assert pipeline[0].endswith("--quiet --require-coverage --skip-gate --p-batch-size 64 --q-batch-size 32 --log-interval 50")
    assert not any("summarize-probes" in line for line in lines)                 # no formal stage, no summary
    out = run("synbios_probes.sh", str(data), "weights/model.pt", REQUIRE_COVERAGE="0", PROBE_GPUS="0", OUT=str(tmp_path / "study"))
    stages = [line for line in out.stdout.splitlines() if "probe-pipeline" in line]
    assert [s.split("--stage ")[1].split()[0] for s in stages] == ["smoke", "pilot", "formal"] and all("--devices cpu" in s and s.endswith("--quiet") for s in stages)
    assert run("synbios_probes.sh", "multi5_permute", "fsdp").returncode == 2          # no such dataset yet
    assert run("synbios_probes.sh", "single", "fsdp", PROBE_BATCH_ENV=str(tmp_path / "absent.env")).returncode == 2

    sys.path.insert(0, str(ROOT / "scripts"))
    try:
        import synbios_moe as cli
    finally:
        sys.path.pop(0)
    run_dir = tmp_path / "run"
    for step, exported in ((10, True), (20, True), (25, False)):
        ckpt = run_dir / f"epoch_{step // 10:06d}_step_{step:09d}"
        ckpt.mkdir(parents=True)
        if exported:
            (ckpt / "model.pt").write_text("x")
        if step != 25:
            (ckpt / "COMMITTED").write_text("ok\n")
    assert cli.exported_model_file(str(run_dir / "latest")) == str(run_dir / "epoch_000002_step_000000020" / "model.pt")
    assert cli.exported_model_file(str(run_dir / "epoch_000001_step_000000010")).endswith("step_000000010/model.pt")
    assert cli.exported_model_file("some/model.pt") == "some/model.pt"
    with pytest.raises(SystemExit, match="not a committed checkpoint"):
        cli.exported_model_file(str(run_dir / "epoch_000002_step_000000025"))
    (run_dir / "epoch_000002_step_000000020" / "model.pt").unlink()
    with pytest.raises(SystemExit, match="no model export"):
        cli.exported_model_file(str(run_dir / "latest"))


def test_full_experiment_launcher_wants_a_confirmation_and_runs_both_variants(tmp_path):
    checkout, run = _launcher_sandbox(tmp_path)
    assert run("synbios_full_experiment.sh", "fsdp").returncode == 2                                   # both variants: not without the confirmation
    refused = run("synbios_full_experiment.sh", "fsdp", CONFIRM_FULL_EXPERIMENT="1")
    assert refused.returncode == 2 and "PROBE_BATCH_ENV" in refused.stderr                             # several GPUs: measured probe batches
    assert run("synbios_full_experiment.sh", "zero3", CONFIRM_FULL_EXPERIMENT="1").returncode == 2
    for variant in ("single", "multi5_permute"):                                                       # a finished pretraining of each variant
        (checkout / "artifacts" / "synbios_moe" / "checkpoints" / f"synbios_moe_{variant}_fsdp" / "epoch_000001_step_000000010").mkdir(parents=True)
        data = checkout / "artifacts" / "synbios_moe" / "data" / variant
        data.mkdir(parents=True)
        (data / "manifest.json").write_text("{}")
    out = run("synbios_full_experiment.sh", "fsdp", CONFIRM_FULL_EXPERIMENT="1", ALLOW_DEFAULT_PROBE_BATCHES="1", NPROC="8", PROBE_GPUS="8")
    assert out.returncode == 0, out.stdout + out.stderr
    calls = [line for line in out.stdout.splitlines() if line.startswith("ARGS:")]
    trainings = [c for c in calls if "scripts/train.py" in c]
    assert len(trainings) == 2 and "single_fsdp.yaml" in trainings[0] and "multi5_permute_fsdp.yaml" in trainings[1]
    assert sum("probe-pipeline" in c for c in calls) == 6 and sum("report-formal-study" in c for c in calls) == 2
    assert "compare-formal-studies --single artifacts/synbios_moe/studies/synbios_moe_single_fsdp/probes/formal --multi " \
        "artifacts/synbios_moe/studies/synbios_moe_multi5_permute_fsdp/probes/formal" in calls[-1]
