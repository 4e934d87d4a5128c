"""Run provenance: interpreter, torch/CUDA versions, host, git revision (None outside a checkout)."""

from __future__ import annotations

import os
import platform
import subprocess
import sys
from pathlib import Path

import torch


def _git(root: Path, *args: str) -> str | None:
    try:
        done = subprocess.run(["git", *args], cwd=root, capture_output=True, text=True, check=False)
    except OSError:
        return None
    return done.stdout.strip() if done.returncode == 0 else None


def collect_provenance(repository: str | Path | None = None) -> dict[str, object]:
    root = Path(repository or Path.cwd())
    dirty = _git(root, "status", "--porcelain")
    return {
        "python_version": sys.version.split()[0],
        "torch_version": torch.__version__,
        "cuda_runtime": torch.version.cuda,
        "hostname": platform.node(),
        "platform": platform.platform(),
        "git_revision": _git(root, "rev-parse", "HEAD"),
        "git_branch": _git(root, "branch", "--show-current"),
        "git_dirty": None if dirty is None else bool(dirty),
        "world_size": int(os.environ.get("WORLD_SIZE", "1")),
    }
