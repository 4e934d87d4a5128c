"""Rank process of the failure-detection tests (CPU, Gloo): a tiny data-parallel loop with a scripted failure."""

import os
import sys
import time
from datetime import timedelta

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mini_train_sys_b200.runtime.health import PeerLostError, RankHealth  # noqa: E402


def main() -> int:
    scenario = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", timeout=timedelta(seconds=float(os.environ.get("PG_TIMEOUT_S", "8"))))
    health = RankHealth()
    weight = torch.zeros(4)
    try:
        for step in range(6):
            health.beat(step)
            if scenario in ("announced", "stale"):
                health.check(max_age_seconds=float(os.environ.get("MAX_AGE_S", "3")))
            if rank == 1 and step == 2:
                if scenario == "announced":
                    health.leave("node drained")          # orderly: between steps, nothing in flight
                    dist.destroy_process_group()
                    return 0
                if scenario == "silent":
                    os._exit(17)                          # crash without a word
                if scenario == "stale":
                    time.sleep(60)                        # a hung host: alive but silent
            grad = torch.full((4,), float(rank + 1))
            if scenario in ("announced", "stale") and step >= 2:
                time.sleep(0.5 if scenario == "announced" else 4.0)    # give the notice / the silence time to show
                health.check(max_age_seconds=float(os.environ.get("MAX_AGE_S", "3")))
            dist.all_reduce(grad)
            weight -= 0.1 * grad / world
    except PeerLostError as exc:
        print(f"PEER_LOST rank={rank} step={step} {exc}", flush=True)
        return 3
    except RuntimeError as exc:                           # the collective itself failed (timeout / connection reset)
        print(f"COLLECTIVE_FAILED rank={rank} step={step} {type(exc).__name__}", flush=True)
        return 4
    print(f"DONE rank={rank} weight={weight[0].item():.3f}", flush=True)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    code = main()
    sys.stdout.flush()
    os._exit(code)
