"""What a result needs to be traced back to: software versions, host, checkout state, device and kernel build.

The first nine keys (``python_version`` ... ``world_size``) are the reference's record
(minitrain/runtime/provenance.py:11-35) and keep their names because event logs and result files are compared across
both systems.  The rest describes what matters on this hardware: which GPU and driver ran, which NCCL carried the
bootstrap, and the content hash of the sm_100a extension that was loaded (two runs with different hashes did not run the
same kernels, whatever their git revision says).  Every probe is independent and failure-tolerant: outside a checkout,
without a GPU or before the extension is built the affected keys are ``None`` and nothing raises.
"""

from __future__ import annotations

import os
import platform
import subprocess
import sys
from pathlib import Path
from typing import Callable

import torch


def _git_output(root: Path, arguments: tuple[str, ...]) -> str | None:
    try:
        done = subprocess.run(("git", *arguments), cwd=root, capture_output=True, text=True, check=False, timeout=30)
    except (OSError, subprocess.TimeoutExpired):
        return None
    return done.stdout.strip() if done.returncode == 0 else None


def _checkout_state(root: Path) -> dict[str, object]:
    changed = _git_output(root, ("status", "--porcelain"))
    return {"git_revision": _git_output(root, ("rev-parse", "HEAD")),
            "git_branch": _git_output(root, ("branch", "--show-current")),
            "git_dirty": changed if changed is None else len(changed) > 0}


def _device_state() -> dict[str, object]:
    # only a process that already uses its GPU describes it: a launcher that merely records provenance must not initialise
    # CUDA (and hold device memory) as a side effect
    if not (torch.cuda.is_available() and torch.cuda.is_initialized()):
        return {"gpu_name": None, "gpu_capability": None, "gpu_sm_count": None, "gpu_memory_gb": None, "nccl_version": None}
    index = torch.cuda.current_device()
    prop = torch.cuda.get_device_properties(index)
    try:
        nccl = ".".join(str(part) for part in torch.cuda.nccl.version())
    except Exception:                  # noqa: BLE001 - a build without NCCL still has provenance
        nccl = None
    return {"gpu_name": prop.name, "gpu_capability": f"{prop.major}.{prop.minor}", "gpu_sm_count": prop.multi_processor_count,
            "gpu_memory_gb": round(prop.total_memory / 2**30, 1), "nccl_version": nccl}


def _extension_state() -> dict[str, object]:
    """Hash and profile of the in-tree extension as it was built (read from the build record, nothing is compiled)."""

    try:
        from mini_train_sys_b200.ops.build import EXT_PATH, KEY_PATH
    except Exception:                  # noqa: BLE001
        return {"extension_build_key": None, "extension_profile": None}
    built = EXT_PATH.is_file() and KEY_PATH.is_file()
    return {"extension_build_key": KEY_PATH.read_text().strip() if built else None,
            "extension_profile": os.environ.get("MTS_BUILD_PROFILE", "release") if built else None}


def collect_provenance(repository: str | Path | None = None) -> dict[str, object]:
    root = Path(repository) if repository is not None else Path.cwd()
    record: dict[str, object] = {}
    scalar_probes: tuple[tuple[str, Callable[[], object]], ...] = (
        ("python_version", lambda: sys.version.split()[0]),
        ("torch_version", lambda: torch.__version__),
        ("cuda_runtime", lambda: torch.version.cuda),
        ("hostname", platform.node),
        ("platform", platform.platform),
    )
    for key, probe in scalar_probes:
        record[key] = probe()
    record.update(_checkout_state(root))
    record["world_size"] = int(os.environ.get("WORLD_SIZE", "1"))
    record.update(_device_state())
    record.update(_extension_state())
    return record
