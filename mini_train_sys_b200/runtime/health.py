"""Host-side rank health: heartbeats and departure notices through the process group's key-value store.

The reference has no in-job failure detection (a lost rank is only noticed when a collective hits the 30-minute
process-group timeout, minitrain/distributed/ddp.py:49-52).  Here every rank posts ``(step, wall time)`` after each
optimizer step and, before its next step launches anything, looks at what its peers posted: a peer that announced its
departure, or whose heartbeat is older than ``max_age_seconds``, raises ``PeerLostError`` on the host.  No kernel or
collective is in flight at that point, so the survivors can checkpoint or exit cleanly instead of spinning on a flag
that will never be set; device-side waits keep their own deadline as the second line of defence.
"""

from __future__ import annotations

import time

import torch.distributed as dist


class PeerLostError(RuntimeError):
    def __init__(self, lost: dict[int, str]) -> None:
        super().__init__("lost ranks: " + ", ".join(f"{r} ({why})" for r, why in sorted(lost.items())))
        self.lost = lost


class RankHealth:
    def __init__(self, store=None, *, rank: int | None = None, world_size: int | None = None, prefix: str = "mts_health",
                 clock=time.time) -> None:
        if store is None:
            store = dist.distributed_c10d._get_default_store()
        self.store = dist.PrefixStore(prefix, store)
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world_size is None else world_size
        self.clock = clock

    def beat(self, step: int) -> None:
        self.store.set(f"hb/{self.rank}", f"{step}:{self.clock():.3f}")

    def leave(self, reason: str = "left") -> None:
        """Announce an orderly departure (call it between steps, with nothing of this rank in flight)."""

        self.store.set(f"left/{self.rank}", reason)

    def peers(self) -> dict[int, dict]:
        out = {}
        now = self.clock()
        for r in range(self.world):
            if r == self.rank:
                continue
            info: dict = {"step": None, "age": None, "left": None}
            if self.store.check([f"left/{r}"]):
                info["left"] = self.store.get(f"left/{r}").decode()
            if self.store.check([f"hb/{r}"]):
                step, stamp = self.store.get(f"hb/{r}").decode().split(":")
                info["step"], info["age"] = int(step), now - float(stamp)
            out[r] = info
        return out

    def check(self, *, max_age_seconds: float | None = None, require_heartbeat: bool = False) -> None:
        lost = {}
        for r, info in self.peers().items():
            if info["left"] is not None:
                lost[r] = f"announced: {info['left']}"
            elif info["age"] is None:
                if require_heartbeat:
                    lost[r] = "no heartbeat yet"
            elif max_age_seconds is not None and info["age"] > max_age_seconds:
                lost[r] = f"last heartbeat {info['age']:.1f} s ago at step {info['step']}"
        if lost:
            raise PeerLostError(lost)
