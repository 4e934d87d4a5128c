"""Durable, reshardable training checkpoints.

Directory layout (kept structurally identical to minitrain/train/checkpoint.py:198-281)::

    <root>/<run>/epoch_{epoch:06d}_step_{step:09d}/
        distributed/             torch.distributed.checkpoint payload {"model", "optimizer"}
        runtime.pt               format_version 4: trainer counters, saved_world_size, precision, config,
                                 grad_scaler / lr_scheduler state
        rng_rank_{rank:05d}.pt   python / torch / cuda generator state of each rank
        model.pt                 optional consolidated fp32 CPU state dict (plain parameter names)
        COMMITTED                written last inside a hidden temp dir, which is then renamed into place
        SAFETY                   marker maintained by ``prune_checkpoints`` on retained fallback anchors

Every rank takes part in the DCP save/load, so model and Adam state stay sharded and can
be loaded at another world size or under another strategy.  Models wrapped by this
package's own sharding engine expose ``sharded_state_dict``/``load_sharded_state_dict``
(DTensor views of the original parameter shapes); anything else goes through
``torch.distributed.checkpoint.state_dict``.

``fault_hook`` (module attribute) is a host-side injection point for tests: it is called
with a stage name (``after_dcp``, ``before_commit``, ``before_rename``) and may raise to
emulate a crash at that point.
"""

from __future__ import annotations

import random
import re
import shutil
import warnings
from pathlib import Path
from typing import Any, Callable

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp
from torch.distributed.checkpoint.state_dict import (StateDictOptions, get_model_state_dict, get_state_dict,
                                                     set_state_dict)

warnings.filterwarnings("ignore", message=r"Please use DTensor instead.*", category=FutureWarning,
                        module=r"torch\.distributed\..*")

FORMAT_VERSION = 4
_NAME = re.compile(r"^epoch_(\d+)_step_(\d+)")
fault_hook: Callable[[str], None] | None = None


def _fault(stage: str) -> None:
    if fault_hook is not None:
        fault_hook(stage)


def _rank() -> int:
    return dist.get_rank() if dist.is_initialized() else 0


def _world() -> int:
    return dist.get_world_size() if dist.is_initialized() else 1


def _sync() -> None:
    if dist.is_initialized():
        dist.barrier()


def _agree(status: int) -> int:
    """Rank 0's decision, shared with every rank."""

    if not dist.is_initialized():
        return status
    box = [status if _rank() == 0 else 0]
    dist.broadcast_object_list(box, src=0)
    return int(box[0])


def checkpoint_path(root: str | Path, run_name: str, *, epoch: int, step: int) -> Path:
    return Path(root) / run_name / f"epoch_{epoch:06d}_step_{step:09d}"


def is_committed(path: Path) -> bool:
    return path.is_dir() and (path / "COMMITTED").is_file()


def _committed_dirs(run_dir: Path) -> list[Path]:
    return [p for p in run_dir.glob("epoch_*_step_*") if is_committed(p)]


def resolve_resume_checkpoint(resume_from: str | Path, *, checkpoint_dir: str | Path, run_name: str) -> Path | None:
    """``latest`` / ``safety`` pick among committed checkpoints of the run; ``auto`` is ``latest`` when the run has one and
    ``None`` (start from scratch) when it has none, which is what a restarted launcher wants; anything else is a path."""

    selector = str(resume_from).lower()
    run_dir = Path(checkpoint_dir) / run_name
    if selector == "auto":
        found = sorted([*_committed_dirs(run_dir), *run_dir.glob("epoch_*_step_*.pt")])
        return found[-1] if found else None
    if selector == "safety":
        anchors = sorted(p for p in _committed_dirs(run_dir) if (p / "SAFETY").is_file())
        if not anchors:
            raise FileNotFoundError(f"No safety checkpoint found in: {run_dir}")
        return anchors[-1]
    if selector == "latest":
        found = sorted([*_committed_dirs(run_dir), *run_dir.glob("epoch_*_step_*.pt")])
        if not found:
            raise FileNotFoundError(f"No committed checkpoints found in: {run_dir}")
        return found[-1]
    path = Path(resume_from)
    if not path.exists():
        raise FileNotFoundError(f"Checkpoint does not exist: {path}")
    if path.is_dir() and not is_committed(path):
        raise ValueError(f"Checkpoint is incomplete (no COMMITTED marker): {path}")
    return path


def prune_checkpoints(checkpoint_dir: str | Path, run_name: str, *, keep_last: int, keep_safety: int = 0,
                      safety_every_epochs: int | None = None, keep_model_exports: int | None = None) -> list[Path]:
    """Keep the newest ``keep_last`` checkpoints plus up to ``keep_safety`` older anchors.

    Anchors are older checkpoints whose epoch is a multiple of ``safety_every_epochs``; while
    too few exist, the oldest remaining checkpoints fill in.  ``SAFETY`` markers are rewritten
    to match, and only the newest ``keep_model_exports`` consolidated exports are kept.
    """

    if keep_last <= 0:
        raise ValueError("keep_last must be positive")
    if keep_safety < 0:
        raise ValueError("keep_safety must be non-negative")
    if keep_safety and not (safety_every_epochs and safety_every_epochs > 0):
        raise ValueError("safety_every_epochs must be positive when keep_safety is enabled")
    if keep_model_exports is not None and keep_model_exports <= 0:
        raise ValueError("keep_model_exports must be positive or null")
    run_dir = Path(checkpoint_dir) / run_name
    dirs = _committed_dirs(run_dir)
    everything = sorted([*dirs, *run_dir.glob("epoch_*_step_*.pt")])
    recent, older = everything[-keep_last:], everything[:-keep_last]
    anchors: list[Path] = []
    if keep_safety and older:
        def epoch_of(p: Path) -> int | None:
            m = _NAME.match(p.name)
            return int(m.group(1)) if m else None

        anchors = [p for p in older if (e := epoch_of(p)) is not None and e % int(safety_every_epochs) == 0][-keep_safety:]
        if len(anchors) < keep_safety:
            spare = [p for p in older if p not in anchors]
            anchors = spare[:keep_safety - len(anchors)] + anchors
    keep = set(recent) | set(anchors)
    removed = [p for p in everything if p not in keep]
    for p in removed:
        shutil.rmtree(p) if p.is_dir() else p.unlink()
    for p in dirs:
        if p in removed:
            continue
        marker = p / "SAFETY"
        if p in anchors:
            marker.write_text("resume fallback\n", encoding="utf-8")
        elif marker.exists():
            marker.unlink()
    if keep_model_exports is not None:
        exports = [p for p in sorted(keep) if p.is_dir() and (p / "model.pt").is_file()]
        for p in exports[:-keep_model_exports]:
            (p / "model.pt").unlink()
    return removed


def capture_rng() -> dict[str, Any]:
    return {"python": random.getstate(), "torch": torch.get_rng_state(),
            "cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None}


def apply_rng_state(state: dict[str, Any]) -> None:
    random.setstate(state["python"])
    torch.set_rng_state(state["torch"])
    if torch.cuda.is_available() and state.get("cuda") is not None:
        torch.cuda.set_rng_state(state["cuda"])


def _gather_states(model, optimizer, cpu_offload: bool):
    own = getattr(model, "sharded_state_dict", None)
    if own is not None:
        return own(optimizer, cpu_offload=cpu_offload)
    return get_state_dict(model, optimizer, options=StateDictOptions(cpu_offload=cpu_offload))


def _full_model_state(model) -> dict[str, torch.Tensor]:
    own = getattr(model, "full_state_dict", None)
    if own is not None:
        return own()
    return get_model_state_dict(model, options=StateDictOptions(full_state_dict=True, cpu_offload=True))


def save_checkpoint(path: str | Path, model: torch.nn.Module, optimizer: torch.optim.Optimizer, step: int, *,
                    epoch: int = 0, lr_step: int | None = None, tokens_seen: int = 0, epoch_batches_done: int = 0,
                    grad_scaler: torch.amp.GradScaler | None = None, lr_scheduler: Any | None = None,
                    precision: str | None = None, config: dict[str, Any] | None = None, export_model: bool = False,
                    cpu_offload: bool = True, write: bool | None = None) -> Path:
    """Collective save; returns the committed directory.  ``write`` is accepted and ignored."""

    del write
    path = Path(path)
    staging = path.with_name(f".{path.name}.tmp")
    verdict = 0
    if _rank() == 0:
        verdict = 1 if is_committed(path) else (2 if path.exists() else 0)
    verdict = _agree(verdict)
    if verdict == 1:
        return path
    if verdict == 2:
        raise FileExistsError(f"Refusing to overwrite incomplete checkpoint path: {path}")
    if _rank() == 0:
        path.parent.mkdir(parents=True, exist_ok=True)
        if staging.exists():
            shutil.rmtree(staging)
        staging.mkdir()
    _sync()

    model_state, optim_state = _gather_states(model, optimizer, cpu_offload)
    dcp.save({"model": model_state, "optimizer": optim_state}, checkpoint_id=staging / "distributed")
    _fault("after_dcp")
    torch.save(capture_rng(), staging / f"rng_rank_{_rank():05d}.pt")
    exported = _full_model_state(model) if export_model else None
    _sync()

    if _rank() == 0:
        runtime: dict[str, Any] = {
            "format_version": FORMAT_VERSION,
            "trainer": {"step": step, "lr_step": step if lr_step is None else lr_step, "epoch": epoch,
                        "tokens_seen": tokens_seen, "epoch_batches_done": int(epoch_batches_done)},
            "saved_world_size": _world(), "precision": precision, "config": config,
        }
        if grad_scaler is not None:
            runtime["grad_scaler"] = grad_scaler.state_dict()
        if lr_scheduler is not None:
            runtime["lr_scheduler"] = lr_scheduler.state_dict()
        torch.save(runtime, staging / "runtime.pt")
        if exported is not None:
            torch.save({k: v.detach().cpu() for k, v in exported.items()}, staging / "model.pt")
        _fault("before_commit")
        (staging / "COMMITTED").write_text("ok\n", encoding="utf-8")
        _fault("before_rename")
        staging.replace(path)
    _sync()
    return path


def _counters(trainer: dict[str, Any], payload: dict[str, Any] | None = None) -> dict[str, int]:
    base = payload or {}
    step = int(trainer.get("step", base.get("step", 0)))
    return {"step": step, "lr_step": int(trainer.get("lr_step", step)), "epoch": int(trainer.get("epoch", 0)),
            "tokens_seen": int(trainer.get("tokens_seen", 0)), "epoch_batches_done": int(trainer.get("epoch_batches_done", 0))}


def _restore_single_file(path: Path, model, optimizer, grad_scaler, lr_scheduler, want_rng: bool) -> dict[str, Any]:
    blob = torch.load(path, map_location="cpu", weights_only=False)
    model.load_state_dict(blob["model"])
    for obj, key in ((optimizer, "optimizer"), (grad_scaler, "grad_scaler"), (lr_scheduler, "lr_scheduler")):
        if obj is not None and key in blob:
            obj.load_state_dict(blob[key])
    got_rng = bool(want_rng and "rng" in blob)
    if got_rng:
        apply_rng_state(blob["rng"])
    return {**_counters(blob.get("trainer", {}), blob), "rng_restored": got_rng}


def _keep_group_options(optimizer: torch.optim.Optimizer, before: list[dict[str, Any]]) -> None:
    """DCP may drop non-tensor group options (betas, eps...); refill only the missing ones."""

    if len(optimizer.param_groups) != len(before):
        raise ValueError("Checkpoint changed the optimizer parameter-group count: "
                         f"expected {len(before)}, got {len(optimizer.param_groups)}")
    for now, old in zip(optimizer.param_groups, before):
        for key, value in old.items():
            if key != "params":
                now.setdefault(key, value)


def restore_training_checkpoint(path: str | Path, model: torch.nn.Module,
                                optimizer: torch.optim.Optimizer | None = None, *,
                                grad_scaler: torch.amp.GradScaler | None = None, lr_scheduler: Any | None = None,
                                restore_rng: bool = True) -> dict[str, Any]:
    """Collective restore; reshards model/Adam state to the current world size and strategy."""

    path = Path(path)
    want_rng = restore_rng
    if path.is_file():
        return _restore_single_file(path, model, optimizer, grad_scaler, lr_scheduler, want_rng)
    if not is_committed(path):
        raise ValueError(f"Checkpoint is incomplete: {path}")
    if optimizer is None:
        raise ValueError("Training restore requires an optimizer")

    own_load = getattr(model, "load_sharded_state_dict", None)
    if own_load is not None:
        model_state, optim_state = model.sharded_state_dict(optimizer, cpu_offload=True)
        bundle = {"model": model_state, "optimizer": optim_state}
        dcp.load(bundle, checkpoint_id=path / "distributed")
        own_load(bundle["model"], bundle["optimizer"], optimizer)
    else:
        opts = StateDictOptions(cpu_offload=True)
        groups_before = [dict(g) for g in optimizer.param_groups]
        model_state, optim_state = get_state_dict(model, optimizer, options=opts)
        bundle = {"model": model_state, "optimizer": optim_state}
        dcp.load(bundle, checkpoint_id=path / "distributed")
        set_state_dict(model, optimizer, model_state_dict=bundle["model"], optim_state_dict=bundle["optimizer"],
                       options=opts)
        _keep_group_options(optimizer, groups_before)

    runtime = torch.load(path / "runtime.pt", map_location="cpu", weights_only=False)
    if grad_scaler is not None and "grad_scaler" in runtime:
        grad_scaler.load_state_dict(runtime["grad_scaler"])
    if lr_scheduler is not None and "lr_scheduler" in runtime:
        lr_scheduler.load_state_dict(runtime["lr_scheduler"])
    rng_file = path / f"rng_rank_{_rank():05d}.pt"
    got_rng = bool(want_rng and rng_file.is_file())
    if got_rng:
        apply_rng_state(torch.load(rng_file, map_location="cpu", weights_only=False))
    counters = _counters(runtime.get("trainer", {}))
    saved_world = int(runtime.get("saved_world_size", 1))
    # tokens_seen is a per-rank count: rescale so that local * world stays the global total
    counters["tokens_seen"] = counters["tokens_seen"] * saved_world // _world()
    return {**counters, "rng_restored": got_rng, "saved_world_size": saved_world}


def load_model_state_dict_from_checkpoint(path: str | Path) -> dict[str, torch.Tensor]:
    """Consolidated weights only (``model.pt`` or a single-file checkpoint), ``module.`` prefixes stripped."""

    path = Path(path)
    if path.is_dir():
        export = path / "model.pt"
        if not export.is_file():
            raise FileNotFoundError("This distributed checkpoint has no consolidated export. Set "
                                    "checkpoint.export_model: true while training.")
        state = torch.load(export, map_location="cpu", weights_only=True, mmap=True)
    else:
        blob = torch.load(path, map_location="cpu", weights_only=False, mmap=True)
        state = blob["model"] if isinstance(blob, dict) and "model" in blob else blob
    if not isinstance(state, dict):
        raise ValueError(f"Checkpoint does not contain a model state dict: {path}")
    if state and all(k.startswith("module.") for k in state):
        state = {k.removeprefix("module."): v for k, v in state.items()}
    return state


def load_checkpoint(path: str | Path, model: torch.nn.Module, optimizer: torch.optim.Optimizer | None = None,
                    **kwargs: Any) -> int:
    return int(restore_training_checkpoint(path, model, optimizer, **kwargs)["step"])


def checkpoint_trainer_state(path: str | Path) -> dict[str, int]:
    path = Path(path)
    blob = torch.load(path / "runtime.pt" if path.is_dir() else path, map_location="cpu", weights_only=False)
    return _counters(blob.get("trainer", {}), blob)
