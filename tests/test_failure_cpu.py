"""Failure detection without any device fault: ranks are CPU / Gloo processes and every failure is made on the host."""

import os
import socket
import subprocess
import sys
import time
from pathlib import Path

import pytest

WORKER = str(Path(__file__).with_name("failure_worker.py"))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(scenario: str, world: int = 2, **env):
    port = _free_port()
    procs = []
    for rank in range(world):
        e = {**os.environ, "RANK": str(rank), "WORLD_SIZE": str(world), "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port),
             **{k: str(v) for k, v in env.items()}}
        procs.append(subprocess.Popen([sys.executable, WORKER, scenario], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=e))
    return procs


def _finish(procs, limit: float):
    start, out = time.time(), []
    for p in procs:
        try:
            text, _ = p.communicate(timeout=max(1.0, limit - (time.time() - start)))
        except subprocess.TimeoutExpired:
            p.kill()                                 # the exact process started above
            text, _ = p.communicate()
            text += "\nKILLED_BY_TEST"
        out.append((p.returncode, text))
    return out, time.time() - start


def test_healthy_ranks_finish():
    out, _ = _finish(_launch("none"), 120)
    assert [c for c, _ in out] == [0, 0] and all("DONE" in t for _, t in out), out


def test_announced_departure_is_seen_on_the_host_before_the_next_collective():
    out, seconds = _finish(_launch("announced"), 120)
    (c0, t0), (c1, _) = out
    assert c1 == 0 and c0 == 3 and "PEER_LOST" in t0 and "node drained" in t0, out
    assert seconds < 60          # far below any collective timeout: the survivor never entered the collective


def test_silent_crash_ends_the_survivor_with_an_error_not_a_hang():
    out, seconds = _finish(_launch("silent", PG_TIMEOUT_S=6), 120)
    (c0, t0), (c1, _) = out
    assert c1 == 17 and c0 in (3, 4) and "KILLED_BY_TEST" not in t0, out
    assert seconds < 90


def test_stale_heartbeat_of_a_hung_peer_is_detected():
    procs = _launch("stale", MAX_AGE_S=2, PG_TIMEOUT_S=30)
    (c0, t0), = _finish(procs[:1], 120)[0]
    procs[1].kill()                                   # the sleeping rank: started by this test
    procs[1].communicate()
    assert c0 == 3 and "last heartbeat" in t0, t0


def test_rank_health_against_a_fake_store_and_clock():
    from mini_train_sys_b200.runtime.health import PeerLostError, RankHealth

    class FakeStore(dict):
        def set(self, k, v): self[k] = v.encode() if isinstance(v, str) else v
        def get(self, k): return self[k]
        def check(self, keys): return all(k in self for k in keys)

    import torch.distributed as dist
    now = [100.0]
    store = FakeStore()
    real = dist.PrefixStore
    dist.PrefixStore = lambda prefix, s: s          # the fake needs no prefixing
    try:
        a = RankHealth(store, rank=0, world_size=3, clock=lambda: now[0])
        b = RankHealth(store, rank=1, world_size=3, clock=lambda: now[0])
        a.beat(0); b.beat(0)
        a.check(max_age_seconds=5)                   # rank 2 has not posted yet: tolerated unless required
        with pytest.raises(PeerLostError):
            a.check(max_age_seconds=5, require_heartbeat=True)
        now[0] += 10
        a.beat(1)
        with pytest.raises(PeerLostError) as err:
            a.check(max_age_seconds=5)
        assert list(err.value.lost) == [1]
        b.beat(1); b.leave("preempted")
        with pytest.raises(PeerLostError) as err:
            a.check(max_age_seconds=5)
        assert "preempted" in err.value.lost[1]
    finally:
        dist.PrefixStore = real


def test_a_crashed_rank_is_restarted_and_the_run_continues_from_the_last_checkpoint(tmp_path):
    """torchrun --max-restarts + ``--resume auto`` + ``checkpoint.every_steps``: rank 1 dies after step 3; the launcher stops
    rank 0 and starts both again; they resume from the checkpoint of step 2 inside the epoch and finish with the losses of a
    run that never crashed."""

    import json
    import subprocess
    import sys
    from pathlib import Path

    import yaml

    root = Path(__file__).resolve().parents[1]
    cfg = yaml.safe_load((root / "configs" / "train_debug.yaml").read_text())
    cfg["run"]["name"] = "restart"
    cfg["parallel"].update(strategy="ddp", process_group_backend="gloo", timeout_minutes=1)
    cfg["train"].update(max_steps=7, epochs=None, log_interval=1)
    cfg["data"].update(num_tokens=64 * cfg["train"]["batch_size"] * 2 * 5 + 1, num_workers=0, persistent_workers=False)   # five batches per epoch and rank
    cfg["checkpoint"] = {"directory": "ckpt", "every_epochs": 1, "every_steps": 2, "export_model": False, "keep_last": 8, "save_final": True}
    cfg["logging"]["tensorboard"] = False

    def launch(work: Path, script: Path, port: int, extra_env: dict, restarts: int):
        work.mkdir()
        (work / "run.yaml").write_text(yaml.safe_dump(cfg))
        env = {**os.environ, "PYTHONPATH": str(root), **extra_env}
        # the c10d rendezvous (hosted by the launcher, a fresh key prefix per restart), not a static master address: after a
        # restart the workers must not find the dead workers' addresses in the store
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--rdzv-backend", "c10d",
               "--rdzv-endpoint", f"127.0.0.1:{port}", "--local-addr", "127.0.0.1", "--max-restarts", str(restarts), str(script),
               "--config", "run.yaml", "--model-config",
               str(root / "configs" / "model_debug_moe.yaml"), "--device", "cpu", "--resume", "auto"]
        done = subprocess.run(cmd, cwd=work, env=env, capture_output=True, text=True, timeout=600)
        log = [json.loads(line) for f in sorted(work.rglob("events.jsonl")) for line in f.read_text().splitlines()]
        return done, log

    done, log = launch(tmp_path / "whole", root / "scripts" / "train.py", 29731, {}, 0)
    assert done.returncode == 0, done.stderr[-2000:]
    want = {e["step"]: e["loss"] for e in log if e["event"] == "train"}
    assert sorted(want) == list(range(1, 8)) and not [e for e in log if e["event"] == "resume"]

    marker = tmp_path / "crashed"
    done, log = launch(tmp_path / "crash", root / "tests" / "restart_train_worker.py", 29732,
                       {"CRASH_AFTER_STEP": "3", "CRASH_MARKER": str(marker)}, 1)
    assert done.returncode == 0, done.stderr[-3000:]
    assert marker.exists()
    resumed = [e for e in log if e["event"] == "resume"]
    assert len(resumed) == 1 and resumed[0]["step"] == 2 and resumed[0]["epoch_batches_done"] == 2
    got = {}
    for e in log:
        if e["event"] == "train":
            got[e["step"]] = e["loss"]                    # step 3 appears twice: before the crash and after the restart
    assert sorted(got) == list(range(1, 8))
    for step, loss in want.items():
        assert got[step] == pytest.approx(loss, abs=1e-6), (step, got[step], loss)
    # without restarts the same crash ends the job with an error
    done, _ = launch(tmp_path / "fatal", root / "tests" / "restart_train_worker.py", 29733,
                     {"CRASH_AFTER_STEP": "3", "CRASH_MARKER": str(tmp_path / "crashed_again")}, 0)
    assert done.returncode != 0
