"""Fused collectives and the sharded engine on 2+ GPUs (one process per GPU, launched with torchrun)."""

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = Path(__file__).resolve().parents[1]


def _launch(n: int, extra_env=None) -> str:
    env = {**os.environ, "MASTER_ADDR": "127.0.0.1", **(extra_env or {})}
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29733", str(ROOT / "tests" / "mgpu_worker.py")]
    done = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-3000:]
    return done.stdout


@pytest.mark.parametrize("multimem", [False, True])
@pytest.mark.parametrize("ranks", [2, 4, 8])
def test_peer_collectives_and_engine(ranks, multimem):
    """Reduce-scatter, all-reduce, the sharded engine (full_shard and shard_grad_op) and the expert exchange against their
    library twins, on as many GPUs as the box has; ``multimem`` repeats it with the switch-side reductions."""

    if torch.cuda.device_count() < ranks:
        pytest.skip(f"needs {ranks} GPUs")
    out = _launch(ranks, {"MTS_TEST_MULTIMEM": "1" if multimem else "0"})
    for marker in ("PASS reduce_scatter", "PASS all_reduce", "PASS engine", "PASS graph_replay", "PASS fifty_steps", "PASS expert_parallel"):
        assert marker in out, out[-2000:]
    if multimem:
        assert "PASS reduce_scatter multimem=True" in out, "the multicast mapping was not used"


def test_a_rank_that_leaves_between_steps_is_noticed_on_the_host():
    n = min(torch.cuda.device_count(), 4)
    env = {**os.environ, "MASTER_ADDR": "127.0.0.1", "NCCL_NVLS_ENABLE": "0", "TORCH_NCCL_ASYNC_ERROR_HANDLING": "0"}
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29741", str(ROOT / "tests" / "mgpu_exit_worker.py")]
    done = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    out = done.stdout + done.stderr
    assert out.count("PASS survivor") == n - 1 and "LEFT rank" in out and "FAIL" not in out, out[-3000:]
