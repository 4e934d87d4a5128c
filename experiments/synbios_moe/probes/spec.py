"""Job description shared by the command builders and the scheduler (reference: experiments/synbios_moe/probes/spec.py:10-40)."""

from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path


@dataclass(frozen=True)
class JobSpec:
    name: str                              # unique inside a pipeline, e.g. "p-university-whole"
    command: tuple[str, ...]               # subprocess argv; "{device}" is replaced by the worker's device
    output: Path                           # the marker file that proves completion
    log: Path
    events_root: Path | None = None        # directory holding events.jsonl of the job (heartbeat source)
    dependencies: tuple[Path, ...] = ()    # files that must exist and be older than `output`
    phase: str = "training"
    metadata: dict = field(default_factory=dict)

    def is_fresh(self) -> bool:
        """Completed AND newer than everything it depends on (exit codes alone are not trusted)."""

        if not self.output.is_file() or self.output.stat().st_size == 0:
            return False
        stamp = self.output.stat().st_mtime
        return all(dep.is_file() and dep.stat().st_mtime <= stamp for dep in self.dependencies)
