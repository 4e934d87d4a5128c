"""Preflight for a B200 training host: software, devices, peer access, toolchain, storage.

Reports errors (exit code 2) and warnings as JSON; every probe only reads state.  The reference's
preflight targets its RTX 4090 server (minitrain/runtime/server_check.py:18-230); this one checks
what the sm_100a build and the peer-memory collectives need instead.
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import os
import platform
import shutil
import subprocess
import sys
from pathlib import Path

import torch

REQUIRED_MODULES = ("numpy", "yaml", "torch")
OPTIONAL_MODULES = ("tensorboard", "tiktoken", "tokenizers", "pyarrow", "pynvml")


def _capture(cmd: list[str]) -> tuple[int, str]:
    try:
        done = subprocess.run(cmd, text=True, capture_output=True, check=False, timeout=60)
    except (OSError, subprocess.TimeoutExpired) as exc:
        return 127, f"{type(exc).__name__}: {exc}"
    return done.returncode, (done.stdout.strip() or done.stderr.strip())


def parse_nvlink_status(text: str) -> dict[int, dict[str, float]]:
    """``nvidia-smi nvlink --status`` -> per GPU: active links, inactive links, and the summed per-direction rate in GB/s.

    The listing has one ``GPU <n>: <name> (UUID: ...)`` line per device followed by ``Link <k>: <rate> GB/s`` or
    ``Link <k>: <inactive>`` lines; anything else is ignored.
    """

    import re

    status: dict[int, dict[str, float]] = {}
    current = None
    for line in text.splitlines():
        head = re.match(r"\s*GPU\s+(\d+)\s*:", line)
        if head:
            current = status.setdefault(int(head.group(1)), {"active_links": 0, "inactive_links": 0, "gbs_per_direction": 0.0})
            continue
        link = re.match(r"\s*Link\s+\d+\s*:\s*(.+)$", line)
        if link is None or current is None:
            continue
        rate = re.match(r"([0-9.]+)\s*GB/s", link.group(1).strip())
        if rate:
            current["active_links"] += 1
            current["gbs_per_direction"] = round(current["gbs_per_direction"] + float(rate.group(1)), 3)
        else:
            current["inactive_links"] += 1
    return status


def nvlink_findings(status: dict[int, dict[str, float]], *, expected_links: int = 18) -> list[str]:
    """Warnings for GPUs whose NVLink fabric is not whole (a B200 has 18 links; fewer active ones cost peer bandwidth)."""

    found = []
    for gpu, info in sorted(status.items()):
        if info["inactive_links"] or 0 < info["active_links"] < expected_links:
            found.append(f"GPU {gpu}: {int(info['active_links'])} of {expected_links} NVLink links active "
                         f"({int(info['inactive_links'])} reported inactive)")
    return found


def find_checkout(start: str | Path | None = None) -> Path | None:
    here = Path(start or Path.cwd()).resolve()
    for cand in (here, *here.parents):
        if (cand / "mini_train_sys_b200").is_dir() and (cand / "configs").is_dir():
            return cand
    pkg_root = Path(__file__).resolve().parents[2]
    return pkg_root if (pkg_root / "configs").is_dir() else None


def collect_server_status(*, expected_gpus: int, min_free_disk_gb: float, require_nvcc: bool,
                          storage_root: str | None = None) -> dict[str, object]:
    errors: list[str] = []
    warnings: list[str] = []
    modules = {m: importlib.util.find_spec(m) is not None for m in (*REQUIRED_MODULES, *OPTIONAL_MODULES)}
    missing = [m for m in REQUIRED_MODULES if not modules[m]]
    if missing:
        errors.append("missing Python modules: " + ", ".join(missing))
    absent = [m for m in OPTIONAL_MODULES if not modules[m]]
    if absent:
        warnings.append("optional modules not installed: " + ", ".join(absent))
    if platform.system() != "Linux":
        errors.append(f"training hosts must run Linux, found {platform.system()}")
    if sys.version_info < (3, 10):
        errors.append(f"Python >= 3.10 is required, found {sys.version_info.major}.{sys.version_info.minor}")

    cuda = torch.cuda.is_available()
    n_gpu = torch.cuda.device_count() if cuda else 0
    devices = []
    if not cuda:
        errors.append("CUDA is not available")
    elif n_gpu < expected_gpus:
        errors.append(f"expected {expected_gpus} GPUs, found {n_gpu}")
    for i in range(n_gpu):
        prop = torch.cuda.get_device_properties(i)
        devices.append({"index": i, "name": prop.name, "capability": f"{prop.major}.{prop.minor}",
                        "memory_gb": round(prop.total_memory / 2**30, 1), "sms": prop.multi_processor_count})
        if (prop.major, prop.minor) != (10, 0):
            errors.append(f"GPU {i} is sm_{prop.major}{prop.minor}; the native kernels are built for sm_100a only")
    peer_ok = True
    for i in range(n_gpu):
        for j in range(n_gpu):
            if i != j and not torch.cuda.can_device_access_peer(i, j):
                peer_ok = False
    if n_gpu > 1 and not peer_ok:
        errors.append("not every GPU pair has peer access; the fused collectives need NVLink peer mappings")
    nccl = torch.distributed.is_available() and torch.distributed.is_nccl_available()
    if cuda and not nccl:
        errors.append("torch.distributed NCCL backend is unavailable")
    if cuda and not torch.cuda.is_bf16_supported():
        errors.append("bf16 is not supported on this device")

    rc_l, smi_list = _capture(["nvidia-smi", "-L"])
    rc_t, topo = _capture(["nvidia-smi", "topo", "-m"])
    if rc_l != 0:
        warnings.append("nvidia-smi -L failed")
    nvlink: dict[int, dict[str, float]] = {}
    if n_gpu > 1:
        rc_n, listing = _capture(["nvidia-smi", "nvlink", "--status"])          # a read-only query
        if rc_n == 0:
            nvlink = parse_nvlink_status(listing)
            warnings.extend(nvlink_findings(nvlink))
    nvcc = shutil.which("nvcc") or ("/usr/local/cuda/bin/nvcc" if Path("/usr/local/cuda/bin/nvcc").exists() else None)
    if nvcc is None and require_nvcc:
        errors.append("nvcc not found (needed to build the sm_100a extension)")
    from mini_train_sys_b200.ops.build import EXT_PATH

    if not EXT_PATH.exists():
        warnings.append(f"native extension not built yet: {EXT_PATH.name}")

    checkout = find_checkout()
    if checkout is None:
        errors.append("repository checkout (mini_train_sys_b200/ + configs/) not found from the working directory")
    root = Path(storage_root or os.environ.get("MTS_STORAGE_ROOT") or os.environ.get("MINITRAIN_STORAGE_ROOT") or Path.cwd())
    free_gb = shutil.disk_usage(root if root.exists() else Path.cwd()).free / 2**30
    if free_gb < min_free_disk_gb:
        errors.append(f"only {free_gb:.1f} GB free under {root}, need {min_free_disk_gb}")
    shm = Path("/dev/shm")
    shm_gb = shutil.disk_usage(shm).free / 2**30 if shm.exists() else 0.0
    if shm_gb < 1.0:
        warnings.append("/dev/shm has less than 1 GB free; DataLoader workers may fail")
    return {"ok": not errors, "errors": errors, "warnings": warnings, "modules": modules, "python": sys.version.split()[0],
            "torch": torch.__version__, "cuda_runtime": torch.version.cuda, "gpu_count": n_gpu, "devices": devices,
            "peer_access_all_pairs": peer_ok, "nccl": nccl, "nvidia_smi": smi_list if rc_l == 0 else None,
            "topology": topo if rc_t == 0 else None, "nvlink": {str(k): v for k, v in nvlink.items()}, "nvcc": nvcc, "extension_built": EXT_PATH.exists(),
            "checkout": str(checkout) if checkout else None, "storage_root": str(root), "free_disk_gb": round(free_gb, 1),
            "shm_free_gb": round(shm_gb, 1)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Preflight checks for a B200 training host")
    ap.add_argument("--expected-gpus", type=int, default=8)
    ap.add_argument("--min-free-disk-gb", type=float, default=50.0)
    ap.add_argument("--skip-nvcc", action="store_true")
    ap.add_argument("--storage-root", default=None)
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--require-nvcc", action="store_true", help="nvcc is required unless --skip-nvcc is given; accepted so that command "
                    "lines written for the reference's check keep working")
    ap.add_argument("--output", help="also write the full report as JSON to this file")
    args = ap.parse_args(argv)
    status = collect_server_status(expected_gpus=args.expected_gpus, min_free_disk_gb=args.min_free_disk_gb,
                                   require_nvcc=not args.skip_nvcc, storage_root=args.storage_root)
    if args.output:
        Path(args.output).parent.mkdir(parents=True, exist_ok=True)
        Path(args.output).write_text(json.dumps(status, indent=2, default=str) + "\n")
    if args.json:
        print(json.dumps(status, indent=2))
    else:
        for line in status["errors"]:
            print(f"ERROR   {line}")
        for line in status["warnings"]:
            print(f"WARNING {line}")
        print("server check " + ("passed" if status["ok"] else "FAILED"))
    return 0 if status["ok"] else 2


if __name__ == "__main__":
    raise SystemExit(main())
