"""Command lines of the probe jobs (reference: experiments/synbios_moe/probes/commands.py:15-146).

Layout under the pipeline root: ``training/<job>.json|.pt`` (result + weights), ``recovery/<job>.pt`` (resumable
state), ``validation/<job>.json``, ``logs/<job>.log``, ``events/<job>/events.jsonl``.
"""

from __future__ import annotations

import sys
from pathlib import Path

from experiments.synbios_moe.probes.dataset import probe_tasks
from experiments.synbios_moe.probes.spec import JobSpec

CLI = str(Path(__file__).resolve().parents[3] / "scripts" / "synbios_moe.py")


def job_name(kind: str, attribute: str, target: str) -> str:
    return f"{kind}-{attribute}-{target}"


def training_job(root: Path, *, kind: str, attribute: str, target: str, data: str, probe_cache: str, model_config: str, checkpoint: str,
                 steps: int, rank: int | None, batch_size: int | None, seed: int, checkpoint_interval_steps: int | None,
                 codec: str, extra: tuple[str, ...] = (), evaluation_batch_size: int | None = None,
                 evaluate_train: bool = False) -> JobSpec:
    name = job_name(kind, attribute, target)
    out = root / "training" / f"{name}.json"
    cmd = [sys.executable, CLI, "probe", "--data", data, "--probe-cache", probe_cache, "--model-config", model_config,
           "--checkpoint", checkpoint, "--attribute", attribute, "--target", target, "--kind", kind, "--steps", str(steps),
           "--seed", str(seed), "--device", "{device}", "--output", str(out), "--recovery-checkpoint", str(root / "recovery" / f"{name}.pt"),
           "--log-dir", str(root / "events" / name), "--codec", codec, "--quiet"]
    if rank is not None:
        cmd += ["--rank", str(rank)]
    if batch_size is not None:
        cmd += ["--batch-size", str(batch_size)]
    if checkpoint_interval_steps:
        cmd += ["--checkpoint-interval-steps", str(checkpoint_interval_steps)]
    if evaluation_batch_size is not None:
        cmd += ["--evaluation-batch-size", str(evaluation_batch_size)]
    if evaluate_train:
        cmd += ["--evaluate-train"]
    return JobSpec(name=name, command=tuple(cmd) + tuple(extra), output=out, log=root / "logs" / f"{name}.log",
                   events_root=root / "events" / name, dependencies=(Path(checkpoint), Path(probe_cache) / "manifest.json"),
                   phase="training", metadata={"kind": kind, "attribute": attribute, "target": target})


def validation_job(root: Path, training: JobSpec, *, data: str, probe_cache: str, model_config: str, checkpoint: str, codec: str) -> JobSpec:
    name = training.name
    out = root / "validation" / f"{name}.json"
    state = training.output.with_suffix(".pt")
    cmd = [sys.executable, CLI, "validate-probe", "--probe-cache", probe_cache, "--model-config", model_config, "--checkpoint", checkpoint,
           "--probe-state", str(state), "--device", "{device}", "--output", str(out), "--codec", codec, "--quiet"]
    return JobSpec(name=f"validate-{name}", command=tuple(cmd), output=out, log=root / "logs" / f"validate-{name}.log",
                   dependencies=(state,), phase="validation", metadata=dict(training.metadata))


def all_training_jobs(root: Path, *, kinds=("p", "q"), tasks="all", steps, **kw) -> list[JobSpec]:
    """The 22 jobs of a full study (11 tasks x {P, Q}), or the subset a stage names.

    ``steps`` is one number or a mapping ``{"p_first": ..., "p_whole": ..., "q_first": ..., "q_whole": ...}``;
    ``tasks`` is ``"all"`` or a list of ``{"kind", "attribute", "target"}`` records.
    """

    ranks = kw.pop("ranks", {})
    batches = kw.pop("batch_sizes", {})
    eval_batches = kw.pop("evaluation_batch_sizes", {})
    wanted = None if tasks in (None, "all") else {(t["kind"], t["attribute"], t["target"]) for t in tasks}
    jobs = []
    for kind in kinds:
        for t in probe_tasks():
            if wanted is not None and (kind, t.attribute, t.target) not in wanted:
                continue
            n = steps[f"{kind}_{t.target}"] if isinstance(steps, dict) else steps
            jobs.append(training_job(root, kind=kind, attribute=t.attribute, target=t.target, steps=int(n), rank=ranks.get(kind),
                                     batch_size=batches.get(kind), evaluation_batch_size=eval_batches.get(kind), **kw))
    return jobs
