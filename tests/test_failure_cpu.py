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
