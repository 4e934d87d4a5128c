"""Task-parallel probe scheduler: one worker thread per device, one subprocess per job, state in ``pipeline.json``.

Reference behaviour kept (experiments/synbios_moe/probes/pipeline.py:179-224,278-283,393-399,507-632): jobs are
skipped when their output marker is newer than their dependencies; completion is judged by marker freshness, not by
the exit code alone; a heartbeat callback reports the tail of each running job's ``events.jsonl``; the pipeline state
is rewritten atomically on every event; an identity hash over the inputs invalidates state left by a different study.
"""

from __future__ import annotations

import json
import os
import queue
import subprocess
import threading
import time
from pathlib import Path
from typing import Callable, Sequence

from experiments.synbios_moe.artifact_io import sha256_file, sha256_json, write_json
from experiments.synbios_moe.probes.spec import JobSpec


def pipeline_identity(*, checkpoint: str | Path, probe_cache: str | Path, model_config: str | Path, settings: dict) -> str:
    """Hash of everything that determines the results: backbone weights, cache manifest, model shape, hyper-parameters."""

    return sha256_json({"checkpoint": sha256_file(checkpoint), "cache": sha256_file(Path(probe_cache) / "manifest.json"),
                        "model_config": sha256_file(model_config), "settings": settings})


def _tail_event(events_root: Path | None) -> dict | None:
    if events_root is None:
        return None
    path = events_root / "events.jsonl"
    try:
        with open(path, "rb") as fh:
            fh.seek(0, os.SEEK_END)
            size = fh.tell()
            fh.seek(max(0, size - 4096))
            lines = fh.read().decode("utf-8", errors="replace").strip().splitlines()
        return json.loads(lines[-1]) if lines else None
    except (OSError, ValueError, IndexError):
        return None


class PipelineState:
    """Thread-safe view of the jobs that is mirrored to ``pipeline.json`` after every change."""

    def __init__(self, path: Path, identity: str, jobs: Sequence[JobSpec]) -> None:
        self.path, self.lock = path, threading.Lock()
        previous = None
        if path.is_file():
            try:
                previous = json.loads(path.read_text())
            except ValueError:
                previous = None
        same = previous is not None and previous.get("identity") == identity
        self.data = {"identity": identity, "started": time.time(), "jobs": {}}
        for job in jobs:
            old = previous["jobs"].get(job.name, {}) if same else {}
            self.data["jobs"][job.name] = {"phase": job.phase, "status": "pending", "attempts": int(old.get("attempts", 0)),
                                           "output": str(job.output), "log": str(job.log), **job.metadata}
        self.flush()

    def update(self, name: str, **fields) -> None:
        with self.lock:
            self.data["jobs"][name].update(fields)
            self.data["updated"] = time.time()
            write_json(self.path, self.data)

    def flush(self) -> None:
        with self.lock:
            write_json(self.path, self.data)

    def counts(self) -> dict[str, int]:
        with self.lock:
            out: dict[str, int] = {}
            for job in self.data["jobs"].values():
                out[job["status"]] = out.get(job["status"], 0) + 1
            return out


def schedule_jobs(jobs: Sequence[JobSpec], devices: Sequence[str], state: PipelineState, *, heartbeat_seconds: float = 30.0,
                  on_heartbeat: Callable[[str, dict | None], None] | None = None, timeout_seconds: float | None = None,
                  env: dict[str, str] | None = None) -> dict[str, str]:
    """Run ``jobs`` over ``devices``; returns ``{job name: status}`` with status in done / skipped / failed."""

    todo: "queue.Queue[JobSpec]" = queue.Queue()
    results: dict[str, str] = {}
    for job in jobs:
        if job.is_fresh():
            results[job.name] = "skipped"
            state.update(job.name, status="skipped")
        else:
            todo.put(job)

    def worker(device: str) -> None:
        while True:
            try:
                job = todo.get_nowait()
            except queue.Empty:
                return
            missing = [str(d) for d in job.dependencies if not d.is_file()]
            if missing:
                results[job.name] = "failed"
                state.update(job.name, status="failed", error=f"missing dependencies: {missing}")
                continue
            job.log.parent.mkdir(parents=True, exist_ok=True)
            job.output.parent.mkdir(parents=True, exist_ok=True)
            argv = [part.replace("{device}", device) for part in job.command]
            launched = time.time()
            attempts = state.data["jobs"][job.name]["attempts"] + 1
            state.update(job.name, status="running", device=device, attempts=attempts, launched=launched)
            with open(job.log, "a") as log:
                log.write(f"\n=== attempt {attempts} on {device}: {' '.join(argv)}\n")
                log.flush()
                proc = subprocess.Popen(argv, stdout=log, stderr=subprocess.STDOUT, env={**os.environ, **(env or {})},
                                        start_new_session=True)
                code = None
                while code is None:
                    try:
                        code = proc.wait(timeout=heartbeat_seconds)
                    except subprocess.TimeoutExpired:
                        last = _tail_event(job.events_root)
                        state.update(job.name, heartbeat=time.time(), last_event=last)
                        if on_heartbeat:
                            on_heartbeat(job.name, last)
                        if timeout_seconds is not None and time.time() - launched > timeout_seconds:
                            try:
                                os.killpg(proc.pid, 15)      # the group started above, nothing else
                            except ProcessLookupError:
                                pass
                            try:
                                code = proc.wait(timeout=10)
                            except subprocess.TimeoutExpired:
                                os.killpg(proc.pid, 9)
                                code = proc.wait()
            fresh = job.output.is_file() and job.output.stat().st_size > 0 and job.output.stat().st_mtime >= launched - 1.0
            status = "done" if code == 0 and fresh else "failed"
            results[job.name] = status
            state.update(job.name, status=status, returncode=code, seconds=time.time() - launched,
                         error=None if status == "done" else ("output marker missing or stale" if code == 0 else f"exit code {code}"))

    threads = [threading.Thread(target=worker, args=(d,), daemon=True) for d in devices]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    return results


def estimate_phase_durations(previous: dict | None, jobs: Sequence[JobSpec], *, steps: int, device_count: int) -> dict[str, float]:
    """Wall-clock seconds per phase of a stage, predicted from the finished prerequisite stage.

    ``previous`` is that stage's ``pipeline.json``.  A phase is estimated only when the earlier stage ran exactly the same
    jobs of that phase and all of them finished with a recorded duration: their seconds are summed (training scaled by the
    ratio of step counts, which is what differs between stages), and divided over the devices that will share them
    (reference: experiments/synbios_moe/probes/pipeline.py:635-675)."""

    if not previous or device_count <= 0:
        return {}
    earlier_steps = (previous.get("settings") or {}).get("steps")
    records = previous.get("jobs")
    if not isinstance(records, dict):
        return {}
    out: dict[str, float] = {}
    for phase in ("training", "validation"):
        mine = {j.name for j in jobs if j.phase == phase}
        theirs = {n: r for n, r in records.items() if r.get("phase") == phase}
        if not mine or set(theirs) != mine:
            continue
        if any(r.get("status") not in ("done", "skipped") or not isinstance(r.get("seconds"), (int, float)) for r in theirs.values()):
            continue
        scale = 1.0
        if phase == "training":
            if not isinstance(earlier_steps, int) or earlier_steps <= 0 or steps <= 0:      # per-task step tables are not scaled
                continue
            scale = steps / earlier_steps
        out[phase] = sum(float(r["seconds"]) for r in theirs.values()) * scale / device_count
    return out


def run_pipeline(root: Path, training: Sequence[JobSpec], validation: Sequence[JobSpec], *, devices: Sequence[str], identity: str,
                 heartbeat_seconds: float = 30.0, on_heartbeat=None, env=None, settings: dict | None = None,
                 estimates: dict[str, float] | None = None) -> dict:
    """Training phase, then validation of everything that trained; the summary is what ``pipeline.json`` ends with.
    ``settings`` (step count and the like) and ``estimates`` (predicted seconds per phase) are recorded beside the jobs."""

    state = PipelineState(root / "pipeline.json", identity, [*training, *validation])
    if settings is not None:
        state.data["settings"] = dict(settings)
    if estimates:
        state.data["estimated_phase_seconds"] = dict(estimates)
    state.flush()
    first = schedule_jobs(training, devices, state, heartbeat_seconds=heartbeat_seconds, on_heartbeat=on_heartbeat, env=env)
    runnable = [v for v in validation if all(d.is_file() for d in v.dependencies)]
    second = schedule_jobs(runnable, devices, state, heartbeat_seconds=heartbeat_seconds, on_heartbeat=on_heartbeat, env=env)
    for v in validation:
        if v not in runnable:
            second[v.name] = "failed"
            state.update(v.name, status="failed", error="training output missing")
    summary = {"training": first, "validation": second, "counts": state.counts(),
               "ok": all(s in ("done", "skipped") for s in [*first.values(), *second.values()])}
    state.data["summary"] = summary
    state.flush()
    return summary
