"""Nsight Compute wrapper: kernel registry, command builder and report reducers.

Role of the reference's ``benchmarks/operators/nsight.py`` (registry :90-140, command :449-498, details export
collapsed to one row per launch :256-292,622-629).  Differences that matter on shared B200 machines:

* every command carries ``--clock-control none`` (a killed capture must not leave clocks locked);
* the default capture is a launch list (one pass); ``full`` captures are limited to one kernel and at most three
  launches and the builder refuses anything larger;
* the raw-page reducer keeps the handful of counters a roofline needs (DRAM bytes, DRAM and tensor pipe
  utilisation, registers, warp stalls) and writes them as a short text summary.
"""

from __future__ import annotations

import csv
import io
import shlex
import subprocess
from dataclasses import dataclass
from pathlib import Path
from typing import Iterable


@dataclass(frozen=True)
class NsightKernel:
    name: str            # registry key, e.g. "gemm"
    regex: str           # kernel-name regex handed to ncu -k
    case: tuple[str, ...]  # arguments of the operator-bench worker that launches it on a small case
    skip: int = 0        # matching launches to pass over before the capture (ncu -s)


_REGISTRY: dict[str, NsightKernel] = {}


def register_nsight_kernel(name: str, regex: str, case: Iterable[str], skip: int = 0) -> None:
    _REGISTRY[name] = NsightKernel(name, regex, tuple(case), skip)


def registered() -> dict[str, NsightKernel]:
    return dict(_REGISTRY)


def _case(kernel: str, tokens: int, profile: str = "project_formal") -> tuple[str, ...]:
    return ("_worker", "--kernel", kernel, "--profile", profile, "--tokens", str(tokens), "--providers", "native",
            "--warmup", "1", "--iters", "2", "--no-check")


# small cases: a few hundred MB on the device, inputs larger than L2 where the op is bandwidth bound
register_nsight_kernel("gemm", "gemm_tcgen05_kernel", _case("linear", 24576))
# the fused MoE worker launches its GEMMs in a fixed order: seven forward passes (up projection with the SwiGLU epilogue,
# down projection) while it times the forward, then forward + backward, whose first GEMM is the down-projection dgrad
# with the SwiGLU-derivative epilogue: launch 14 of the kernel
register_nsight_kernel("gemm_swiglu", "gemm_tcgen05_kernel", _case("fused_moe", 24576))
register_nsight_kernel("gemm_swiglu_bwd", "gemm_tcgen05_kernel", _case("fused_moe", 24576), skip=14)
register_nsight_kernel("flash_fwd", "flash_fwd_kernel", _case("attention", 24576))
register_nsight_kernel("flash_bwd_dkdv", "flash_bwd_dkdv_kernel", _case("attention", 24576))
register_nsight_kernel("flash_bwd_dq", "flash_bwd_dq_kernel", _case("attention", 24576))
register_nsight_kernel("rmsnorm_fwd", "rmsnorm_fwd_kernel", _case("rmsnorm", 57344))
register_nsight_kernel("rmsnorm_bwd", "rmsnorm_bwd", _case("rmsnorm", 57344))
register_nsight_kernel("rope", "rope_kernel", _case("rope", 57344))
register_nsight_kernel("swiglu_fwd", "swiglu_fwd_kernel", _case("swiglu", 57344))
register_nsight_kernel("swiglu_bwd", "swiglu_bwd_kernel", _case("swiglu", 57344))
register_nsight_kernel("ce_forward", "ce_forward_kernel", _case("cross_entropy", 8192))
register_nsight_kernel("ce_backward", "ce_backward_kernel", _case("cross_entropy", 8192))
register_nsight_kernel("router_fwd", "router_forward_kernel", _case("router", 262144))
register_nsight_kernel("router_logits_fwd", "router_logits_fwd_kernel", _case("router_logits", 98304))
register_nsight_kernel("router_logits_dx", "router_logits_dx_kernel", _case("router_logits", 98304))
register_nsight_kernel("router_logits_dw", "router_logits_dw_kernel", _case("router_logits", 98304))
register_nsight_kernel("embedding_fwd", "embedding_fwd_kernel", _case("embedding", 98304))
register_nsight_kernel("embedding_bwd", "embedding_bwd_kernel", _case("embedding", 98304))
register_nsight_kernel("moe_gather", "moe_gather_kernel", _case("fused_moe", 24576))
register_nsight_kernel("moe_combine", "moe_combine_kernel", _case("fused_moe", 24576))

MAX_FULL_LAUNCHES = 3
ROOFLINE_METRICS = (
    "gpu__time_duration.sum", "dram__bytes_read.sum", "dram__bytes_write.sum", "dram__cycles_active.avg.pct_of_peak_sustained_elapsed",
    "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed", "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active",
    "sm__warps_active.avg.pct_of_peak_sustained_active", "launch__registers_per_thread", "launch__shared_mem_per_block_dynamic",
    "sm__throughput.avg.pct_of_peak_sustained_elapsed",
)


def build_command(target: list[str], *, mode: str = "launches", kernel_regex: str | None = None, skip: int = 0,
                  count: int | None = None, output: str | Path | None = None, python: str = "python") -> list[str]:
    """``mode``: ``launches`` (device time of every launch, one pass), ``roofline`` (named counters) or ``full``."""

    cmd = ["ncu", "--clock-control", "none"]
    if mode == "launches":
        cmd += ["--metrics", "gpu__time_duration.sum", "--csv"]
        count = 400 if count is None else count
    elif mode in ("roofline", "full"):
        if kernel_regex is None:
            raise ValueError(f"mode {mode!r} captures one kernel: give kernel_regex")
        count = MAX_FULL_LAUNCHES if count is None else count
        if count > MAX_FULL_LAUNCHES:
            raise ValueError(f"a {mode} capture replays every launch many times; at most {MAX_FULL_LAUNCHES} launches")
        cmd += ["--set", "full"] if mode == "full" else ["--metrics", ",".join(ROOFLINE_METRICS)]
    else:
        raise ValueError(f"unknown mode {mode!r}")
    if kernel_regex:
        cmd += ["-k", f"regex:{kernel_regex}"]
    if skip:
        cmd += ["-s", str(skip)]
    cmd += ["-c", str(count)]
    if output is not None:
        cmd += ["--log-file", str(output)] if mode == "launches" else ["-o", str(output)]
    return cmd + [python] + list(target)


def command_for(name: str, script: str | Path, *, mode: str = "full", output: str | Path | None = None) -> str:
    """Shell line for a registered kernel: the plain run first, the capture only if it exits 0."""

    k = _REGISTRY[name]
    target = [str(script), *k.case]
    plain = " ".join(shlex.quote(c) for c in ["python", *target])
    cap = " ".join(shlex.quote(c) for c in build_command(target, mode=mode, kernel_regex=k.regex, skip=k.skip, output=output))
    return f"{plain} > /dev/null && {cap}"


def export_raw_csv(report: str | Path) -> str:
    """``ncu -i report --page raw --csv`` (works without a GPU)."""

    return subprocess.run(["ncu", "-i", str(report), "--page", "raw", "--csv"], capture_output=True, text=True, check=True).stdout


def parse_raw_csv(text: str) -> list[dict[str, str]]:
    """One dict per captured launch; the second CSV row holds units and is folded into ``<metric> [unit]`` keys."""

    rows = list(csv.reader(io.StringIO(text)))
    rows = [r for r in rows if r]
    start = next((i for i, r in enumerate(rows) if r and r[0] == "ID"), None)
    if start is None:
        return []
    header, units = rows[start], rows[start + 1] if len(rows) > start + 1 else []
    out = []
    for r in rows[start + 2:]:
        out.append({(f"{h} [{u}]" if u else h): v for h, u, v in zip(header, units + [""] * len(header), r)})
    return out


def parse_launch_list(text: str) -> list[dict[str, str]]:
    """The ``--csv`` log of a ``launches`` capture: one row per launch with kernel name and duration."""

    lines = [ln for ln in text.splitlines() if ln.startswith('"')]
    if not lines:
        return []
    return list(csv.DictReader(io.StringIO("\n".join(lines))))


def launch_shares(rows: list[dict[str, str]]) -> list[tuple[str, int, float, float]]:
    """(kernel, launches, total microseconds, share) sorted by total time."""

    totals: dict[str, list[float]] = {}
    for r in rows:
        name = r.get("Kernel Name", "?").split("(")[0]
        val = float(r.get("Metric Value", "0").replace(",", "") or 0)
        unit = r.get("Metric Unit", "ns")
        us = val / 1e3 if unit in ("ns", "nsecond") else val if unit in ("us", "usecond") else val * 1e3
        t = totals.setdefault(name, [0, 0.0])
        t[0] += 1; t[1] += us
    grand = sum(t[1] for t in totals.values()) or 1.0
    return sorted(((k, int(n), us, us / grand) for k, (n, us) in totals.items()), key=lambda x: -x[2])


def _pick(row: dict[str, str], needle: str) -> float | None:
    for k, v in row.items():
        if k.startswith(needle):
            try:
                return float(v.replace(",", ""))
            except ValueError:
                return None
    return None


def roofline_summary(rows: list[dict[str, str]], *, algorithmic_bytes: float | None = None) -> str:
    """Short text block per launch: duration, DRAM traffic (and its ratio to the algorithmic bytes), pipe utilisation."""

    out = []
    for r in rows:
        rd, wr = _pick(r, "dram__bytes_read.sum"), _pick(r, "dram__bytes_write.sum")
        dur = _pick(r, "gpu__time_duration.sum")
        line = [f"kernel {r.get('Kernel Name', '?')[:80]}", f"  duration            {dur} (unit as exported)"]
        if rd is not None and wr is not None:
            line.append(f"  dram read / write   {rd:.4g} / {wr:.4g} (units as exported)")
            if algorithmic_bytes:
                line.append(f"  algorithmic bytes   {algorithmic_bytes:.4g}")
        for label, key in (("dram throughput %", "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed"),
                           ("tensor pipe active %", "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active"),
                           ("warps active %", "sm__warps_active.avg.pct_of_peak_sustained_active"),
                           ("sm throughput %", "sm__throughput.avg.pct_of_peak_sustained_elapsed"),
                           ("registers / thread", "launch__registers_per_thread")):
            v = _pick(r, key)
            if v is not None:
                line.append(f"  {label:<19} {v:.4g}")
        out.append("\n".join(line))
    return "\n\n".join(out)
