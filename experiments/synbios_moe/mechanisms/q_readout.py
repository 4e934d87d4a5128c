"""Aligned Q-first and Q-whole predictions of two trained probe heads on the held-out people.

A Q probe reads the hidden state right after a person's name (``[EOS] name [EOS]``, last position).  For one attribute
the first-token head and the whole-value head see identical inputs, so their predictions can be paired per person:
this table is the input of the oracle first-token intervention and of the first-vs-whole agreement statistics
(reference: experiments/synbios_moe/mechanisms/q_readout.py:111-215).
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Callable

import numpy as np
import torch

from experiments.synbios_moe.artifact_io import read_json, read_jsonl
from experiments.synbios_moe.probes.commands import job_name
from experiments.synbios_moe.probes.dataset import CachedProbeDataset
from experiments.synbios_moe.probes.model import AttributeProbe, collate, load_saved_probe


@dataclass(frozen=True)
class QPrediction:
    case_id: int
    profile_index: int
    person_id: str
    attribute: str
    input_ids: tuple[int, ...]
    true_first_id: int
    pred_first_id: int
    true_first_token: str
    pred_first_token: str
    true_whole_id: int
    pred_whole_id: int
    true_whole_value: str
    pred_whole_value: str
    whole_true_probability: float

    @property
    def first_correct(self) -> bool:
        return self.true_first_id == self.pred_first_id

    @property
    def whole_correct(self) -> bool:
        return self.true_whole_id == self.pred_whole_id


def task_class_names(cache_root: str | Path, attribute: str, target: str) -> list[str]:
    for task in read_json(Path(cache_root) / "manifest.json")["tasks"]:
        if task["attribute"] == attribute and task["target"] == target:
            return [str(c) for c in task["classes"]]
    raise ValueError(f"the probe cache has no task {attribute}/{target}")


def probe_state_path(probe_dir: str | Path, kind: str, attribute: str, target: str) -> Path:
    """``<probe_dir>/training/<job>.pt`` of a pipeline root, or ``<probe_dir>/<job>.pt`` of a flat directory."""

    root = Path(probe_dir)
    name = f"{job_name(kind, attribute, target)}.pt"
    nested = root / "training" / name
    return nested if nested.is_file() else root / name


@torch.no_grad()
def collect_q_predictions(backbone, *, data_root: str | Path, cache_root: str | Path, probe_dir: str | Path, attribute: str,
                          device="cpu", batch_size: int = 256, max_examples: int | None = None,
                          progress: Callable[[int], None] | None = None) -> tuple[list[QPrediction], AttributeProbe]:
    """One record per held-out person; also returns the whole-value head (the intervention re-uses it unchanged)."""

    first = CachedProbeDataset(cache_root, kind="q", attribute=attribute, target="first", split="validation")
    whole = CachedProbeDataset(cache_root, kind="q", attribute=attribute, target="whole", split="validation")
    if len(first) != len(whole) or not np.array_equal(first.examples, whole.examples):
        raise ValueError("the first and whole Q datasets do not list the same people")
    profiles = read_jsonl(Path(data_root) / "profiles.jsonl")
    heads = {}
    for target, data in (("first", first), ("whole", whole)):
        heads[target] = load_saved_probe(backbone, probe_state_path(probe_dir, "q", attribute, target), len(data.class_names),
                                         expect={"kind": "q", "attribute": attribute, "target": target}, device=device).eval()
    count = len(first) if max_examples is None else min(max_examples, len(first))
    records: list[QPrediction] = []
    for lo in range(0, count, batch_size):
        hi = min(lo + batch_size, count)
        f_items, w_items = [first[i] for i in range(lo, hi)], [whole[i] for i in range(lo, hi)]
        f_ids, f_pos, f_lab = collate(f_items, first.eos)
        w_ids, w_pos, w_lab = collate(w_items, whole.eos)
        if not torch.equal(f_ids, w_ids):
            raise ValueError("first and whole Q inputs differ")
        f_logits = heads["first"](f_ids.to(device), f_pos.to(device))[:, 0]
        w_logits = heads["whole"](w_ids.to(device), w_pos.to(device))[:, 0]
        f_pred, w_pred = f_logits.argmax(-1).cpu(), w_logits.argmax(-1).cpu()
        w_prob = w_logits.softmax(-1).gather(1, w_lab.to(device)[:, None])[:, 0].cpu()
        for off, idx in enumerate(range(lo, hi)):
            row = int(first.examples[idx])
            records.append(QPrediction(
                case_id=idx, profile_index=row, person_id=str(profiles[row]["person_id"]), attribute=attribute,
                input_ids=tuple(int(t) for t in f_items[off].input_ids),
                true_first_id=int(f_lab[off]), pred_first_id=int(f_pred[off]),
                true_first_token=first.class_names[int(f_lab[off])], pred_first_token=first.class_names[int(f_pred[off])],
                true_whole_id=int(w_lab[off]), pred_whole_id=int(w_pred[off]),
                true_whole_value=whole.class_names[int(w_lab[off])], pred_whole_value=whole.class_names[int(w_pred[off])],
                whole_true_probability=float(w_prob[off])))
        if progress is not None:
            progress(hi)
    return records, heads["whole"]


def prediction_row(record: QPrediction) -> dict[str, object]:
    return {"case_id": record.case_id, "profile_index": record.profile_index, "person_id": record.person_id,
            "attribute": record.attribute, "true_first_token": record.true_first_token, "pred_first_token": record.pred_first_token,
            "true_whole_value": record.true_whole_value, "pred_whole_value": record.pred_whole_value,
            "first_correct": record.first_correct, "whole_correct": record.whole_correct,
            "whole_true_probability": record.whole_true_probability}


def agreement_table(records: list[QPrediction]) -> dict[str, float | int]:
    """How the two heads agree: whole accuracy given a right / wrong first token (a whole value whose first token the model
    cannot name is rarely recovered, which is what the oracle intervention then tests causally)."""

    n = len(records)
    first_ok = [r for r in records if r.first_correct]
    first_bad = [r for r in records if not r.first_correct]
    frac = lambda rows: sum(r.whole_correct for r in rows) / len(rows) if rows else 0.0   # noqa: E731
    return {"examples": n, "first_accuracy": len(first_ok) / n if n else 0.0, "whole_accuracy": frac(records),
            "whole_accuracy_given_first_correct": frac(first_ok), "whole_accuracy_given_first_wrong": frac(first_bad)}
