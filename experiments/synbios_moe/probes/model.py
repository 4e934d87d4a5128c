"""P / Q probes: frozen backbone + rank-r embedding delta + normaliser + linear classifier, and their training loop.

The backbone never learns; what is trained is a low-rank additive change of the input embeddings (``A``: vocabulary x r
embedding, ``B``: r x hidden, zero-initialised, so the probe starts from the unmodified model), a LayerNorm (P) or
BatchNorm (Q) over the selected hidden states, and a linear classifier.  Accuracy therefore measures how linearly
extractable a fact is at a position, not what fine-tuning could add.  Protocol constants follow the reference
(experiments/synbios_moe/probes/model.py:28-33,199-241,282-337): AdamW lr 1e-3, weight decay 0.3, eps 1e-6, linear
decay to zero without warm-up, backbone kept in train mode (dropout active) while frozen.

Training is resumable with exact data-order replay: the order of epoch ``e`` is ``Generator(seed + e).randperm``, so a
recovery checkpoint only needs the step count to continue with the very batches an uninterrupted run would have seen.
"""

from __future__ import annotations

import json
import os
import time
from pathlib import Path
from typing import Callable, Sequence

import numpy as np
import torch
from torch import nn

from experiments.synbios_moe.probes.dataset import CachedProbeDataset, ProbeItem

DEFAULT_RANK = {"p": 2, "q": 16}
DEFAULT_BATCH = {"p": 50, "q": 200}
LEARNING_RATE, WEIGHT_DECAY, ADAM_EPS = 1e-3, 0.3, 1e-6
CHECKPOINT_VERSION = 1


def linear_decay_fraction(step: int, steps: int) -> float:
    """Learning-rate multiplier of optimizer step ``step`` (0-based): 1 at the start, 0 after ``steps``."""

    return max(0.0, 1.0 - step / max(steps, 1))


def collate(items: Sequence[ProbeItem], eos: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    if not items:
        raise ValueError("cannot collate an empty probe batch")
    width = max(int(i.input_ids.shape[0]) for i in items)
    ids = torch.full((len(items), width), eos, dtype=torch.long)
    for row, item in enumerate(items):
        ids[row, :item.input_ids.shape[0]] = torch.from_numpy(item.input_ids.astype(np.int64))
    pos = torch.from_numpy(np.stack([i.positions for i in items]).astype(np.int64))
    return ids, pos, torch.tensor([i.label for i in items], dtype=torch.long)


class LowRankEmbeddingDelta(nn.Module):
    def __init__(self, vocab_size: int, hidden_size: int, rank: int) -> None:
        super().__init__()
        self.a = nn.Embedding(vocab_size, rank)
        self.b = nn.Linear(rank, hidden_size, bias=False)
        nn.init.normal_(self.a.weight, std=0.02)
        nn.init.zeros_(self.b.weight)

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        return self.b(self.a(input_ids))


class AttributeProbe(nn.Module):
    def __init__(self, backbone, num_classes: int, *, rank: int, kind: str) -> None:
        super().__init__()
        if kind not in ("p", "q"):
            raise ValueError("kind must be 'p' or 'q'")
        self.backbone = backbone
        for parameter in backbone.parameters():
            parameter.requires_grad_(False)
        hidden = backbone.cfg.hidden_size
        self.delta = LowRankEmbeddingDelta(backbone.cfg.vocab_size, hidden, rank)
        self.normalizer: nn.Module = nn.LayerNorm(hidden) if kind == "p" else nn.BatchNorm1d(hidden)
        self.classifier = nn.Linear(hidden, num_classes)

    def trainable_state(self) -> dict[str, torch.Tensor]:
        return {k: v for k, v in self.state_dict().items() if not k.startswith("backbone.")}

    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        hidden = self.backbone.hidden_states(input_ids, embedding_delta=self.delta(input_ids))
        hidden = hidden[0] if isinstance(hidden, tuple) else hidden
        rows = torch.arange(hidden.shape[0], device=hidden.device)[:, None]
        picked = hidden[rows, positions].float()                       # [B, P, H]
        shape = picked.shape
        return self.classifier(self.normalizer(picked.reshape(-1, shape[-1]))).view(shape[0], shape[1], -1)


@torch.no_grad()
def evaluate(probe: AttributeProbe, dataset: CachedProbeDataset, *, batch_size: int, device, max_items: int | None = None) -> dict:
    """Accuracy per position (P0..P5, or the single Q position).  The normaliser runs in eval mode, the backbone too."""

    was_training = probe.training
    probe.eval()
    count = len(dataset) if max_items is None else min(len(dataset), max_items)
    hits = None
    for lo in range(0, count, batch_size):
        ids, pos, labels = collate([dataset[i] for i in range(lo, min(lo + batch_size, count))], dataset.eos)
        logits = probe(ids.to(device), pos.to(device))
        ok = (logits.argmax(-1).cpu() == labels[:, None]).sum(0)
        hits = ok if hits is None else hits + ok
    probe.train(was_training)
    per_position = (hits.double() / max(count, 1)).tolist() if hits is not None else []
    return {"examples": count, "accuracy_by_position": per_position, "accuracy": float(np.mean(per_position)) if per_position else 0.0}


def _epoch_order(n: int, seed: int, epoch: int) -> torch.Tensor:
    return torch.randperm(n, generator=torch.Generator().manual_seed(seed + epoch))


def _atomic_torch_save(payload: dict, path: Path) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_suffix(path.suffix + ".tmp")
    torch.save(payload, tmp)
    os.replace(tmp, path)


def train_probe(backbone, cache_dir: str | Path, *, kind: str, attribute: str, target: str, steps: int, device="cpu",
                rank: int | None = None, batch_size: int | None = None, evaluation_batch_size: int | None = None, seed: int = 1337,
                recovery_checkpoint: str | Path | None = None, checkpoint_interval_steps: int | None = None, resume: bool = True,
                evaluate_train: bool = False, skip_final_validation: bool = False, identity: dict | None = None,
                on_event: Callable[[dict], None] | None = None, max_eval_items: int | None = None,
                train_set=None, valid_set=None, return_probe: bool = False) -> dict:
    """Train one probe; returns the result record (also what ``training/<job>.json`` holds).

    ``identity`` is stored in the recovery checkpoint and must match on resume (a checkpoint of another backbone,
    task or hyper-parameter set is refused rather than silently continued).  ``train_set`` / ``valid_set`` replace the
    cached task's examples with a derived dataset (same item type, ``class_names`` and ``eos``): the interventions that
    rebuild probe inputs train through this entry; with ``return_probe`` the trained module is returned under ``"probe"``.
    """

    rank = DEFAULT_RANK[kind] if rank is None else rank
    batch_size = DEFAULT_BATCH[kind] if batch_size is None else batch_size
    evaluation_batch_size = evaluation_batch_size or batch_size
    if train_set is None:
        train_set = CachedProbeDataset(cache_dir, kind=kind, attribute=attribute, target=target, split="train")
    if valid_set is None:
        valid_set = CachedProbeDataset(cache_dir, kind=kind, attribute=attribute, target=target, split="validation")
    if len(train_set) == 0:
        raise ValueError("the training split of this probe task is empty")
    torch.manual_seed(seed)
    probe = AttributeProbe(backbone, len(train_set.class_names), rank=rank, kind=kind).to(device)
    probe.train()                                # dropout of the frozen backbone stays active, as in the protocol
    params = [p for p in probe.parameters() if p.requires_grad]
    optimizer = torch.optim.AdamW(params, lr=LEARNING_RATE, weight_decay=WEIGHT_DECAY, eps=ADAM_EPS)
    identity = {"kind": kind, "attribute": attribute, "target": target, "rank": rank, "batch_size": batch_size, "steps": steps,
                "seed": seed, **(identity or {})}
    step, losses = 0, []
    resumed_from = None
    recovery = Path(recovery_checkpoint) if recovery_checkpoint else None
    if recovery is not None and resume and recovery.is_file():
        saved = torch.load(recovery, map_location="cpu", weights_only=False)
        if saved.get("version") != CHECKPOINT_VERSION or saved.get("identity") != identity:
            raise ValueError(f"recovery checkpoint {recovery} belongs to a different probe job")
        probe.load_state_dict({**probe.state_dict(), **saved["probe"]})
        optimizer.load_state_dict(saved["optimizer"])
        torch.set_rng_state(saved["torch_rng"])
        if saved.get("cuda_rng") is not None and torch.cuda.is_available():
            torch.cuda.set_rng_state_all(saved["cuda_rng"])
        step = resumed_from = int(saved["step"])
        if on_event:
            on_event({"event": "probe_resume", "step": step, "path": str(recovery)})

    def save_recovery() -> None:
        if recovery is None:
            return
        _atomic_torch_save({"version": CHECKPOINT_VERSION, "identity": identity, "step": step, "probe": probe.trainable_state(),
                            "optimizer": optimizer.state_dict(), "torch_rng": torch.get_rng_state(),
                            "cuda_rng": torch.cuda.get_rng_state_all() if torch.cuda.is_available() else None}, recovery)

    n = len(train_set)
    per_epoch = max(n // batch_size, 1)
    started = time.time()
    while step < steps:
        epoch, within = divmod(step, per_epoch)
        order = _epoch_order(n, seed, epoch)
        picks = order[within * batch_size:(within + 1) * batch_size].tolist() or order[:batch_size].tolist()
        ids, pos, labels = collate([train_set[i] for i in picks], train_set.eos)
        for group in optimizer.param_groups:
            group["lr"] = LEARNING_RATE * linear_decay_fraction(step, steps)
        logits = probe(ids.to(device), pos.to(device))
        loss = nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]), labels.to(device)[:, None].expand(-1, logits.shape[1]).reshape(-1))
        optimizer.zero_grad(set_to_none=True)
        loss.backward()
        optimizer.step()
        step += 1
        losses.append(float(loss.detach()))
        if on_event and (step % 10 == 0 or step == steps):
            on_event({"event": "probe_train", "step": step, "steps": steps, "loss": losses[-1], "lr": optimizer.param_groups[0]["lr"]})
        if checkpoint_interval_steps and step % checkpoint_interval_steps == 0 and step < steps:
            save_recovery()
    result = {"identity": identity, "steps": step, "resumed_from_step": resumed_from, "final_loss": losses[-1] if losses else None,
              "train_examples": n,
              "validation_examples": len(valid_set), "classes": len(train_set.class_names), "seconds": time.time() - started,
              "trainable_parameters": sum(p.numel() for p in params)}
    if not skip_final_validation:
        result["validation"] = evaluate(probe, valid_set, batch_size=evaluation_batch_size, device=device, max_items=max_eval_items)
    if evaluate_train:
        result["train"] = evaluate(probe, train_set, batch_size=evaluation_batch_size, device=device, max_items=max_eval_items)
    result["probe_state"] = probe.trainable_state()
    if return_probe:
        result["probe"] = probe
    return result


def active_parameter_estimate(model) -> dict[str, int]:
    """Parameter count of the backbone and how many of them one token touches: with routed experts only ``top_k / experts``
    of the expert weights are active (reference: experiments/synbios_moe/probes/model.py:575-583)."""

    inner = getattr(model, "module", model)
    total = sum(p.numel() for p in inner.parameters())
    cfg = inner.cfg
    if not cfg.is_moe:
        return {"total": total, "active_estimate": total}
    experts = sum(b.ffn.gate_up_proj.numel() + b.ffn.down_proj.numel() for b in inner.blocks if hasattr(b.ffn, "gate_up_proj"))
    return {"total": total, "active_estimate": total - experts + experts * cfg.experts_per_token // cfg.num_experts}


def save_probe_result(result: dict, json_path: str | Path, state_path: str | Path) -> None:
    """``training/<job>.pt`` (trainable weights) first, then ``training/<job>.json``: the marker is written last."""

    result.pop("probe", None)
    state = result.pop("probe_state")
    _atomic_torch_save({"version": CHECKPOINT_VERSION, "identity": result["identity"], "probe": state}, Path(state_path))
    tmp = Path(json_path).with_suffix(".json.tmp")
    Path(json_path).parent.mkdir(parents=True, exist_ok=True)
    tmp.write_text(json.dumps(result, indent=1, default=str))
    os.replace(tmp, json_path)


def load_saved_probe(backbone, state_path: str | Path, num_classes: int, *, expect: dict | None = None, device="cpu") -> AttributeProbe:
    """Rebuild a trained probe from ``training/<job>.pt``; ``expect`` lists identity fields that must match (kind, attribute,
    target, ...), so that a head of another task is refused instead of silently evaluated."""

    saved = torch.load(state_path, map_location="cpu", weights_only=False)
    ident = saved.get("identity")
    if saved.get("version") != CHECKPOINT_VERSION or not isinstance(ident, dict):
        raise ValueError(f"{state_path} is not a probe result of this format")
    for key, want in (expect or {}).items():
        if ident.get(key) != want:
            raise ValueError(f"{state_path}: {key} is {ident.get(key)!r}, expected {want!r}")
    probe = AttributeProbe(backbone, num_classes, rank=int(ident["rank"]), kind=ident["kind"])
    merged = {**probe.state_dict(), **saved["probe"]}
    missing = [k for k in probe.trainable_state() if k not in saved["probe"]]
    if missing:
        raise ValueError(f"{state_path} lacks trainable tensors: {missing[:3]}")
    probe.load_state_dict(merged)
    return probe.to(device)


def validate_saved_probe(backbone, cache_dir: str | Path, state_path: str | Path, *, device="cpu", batch_size: int = 200,
                         max_items: int | None = None) -> dict:
    """Re-evaluate a trained probe from its saved weights (the pipeline's validation phase)."""

    saved = torch.load(state_path, map_location="cpu", weights_only=False)
    ident = saved["identity"]
    data = CachedProbeDataset(cache_dir, kind=ident["kind"], attribute=ident["attribute"], target=ident["target"], split="validation")
    probe = AttributeProbe(backbone, len(data.class_names), rank=ident["rank"], kind=ident["kind"]).to(device)
    probe.load_state_dict({**probe.state_dict(), **saved["probe"]})
    return {"identity": ident, "validation": evaluate(probe, data, batch_size=batch_size, device=device, max_items=max_items)}
