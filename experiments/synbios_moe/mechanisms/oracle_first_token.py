"""Oracle first-token intervention on the Q read-out.

The question asked: when the whole-value head fails on ``[EOS] name [EOS]``, is the missing piece the first token of the
value?  Each held-out input is rebuilt as ``[EOS] name t1 [EOS]`` with the TRUE first token ``t1`` of the value inserted
before the read-out position, and the UNCHANGED Q-whole head is evaluated again.  Nothing is trained; the report counts
recovered errors and harmed successes (reference: experiments/synbios_moe/mechanisms/oracle_first_token.py:19-163).
"""

from __future__ import annotations

from pathlib import Path
from typing import Callable, Sequence

import numpy as np
import torch

from experiments.synbios_moe.artifact_io import write_csv, write_json
from experiments.synbios_moe.mechanisms.q_readout import collect_q_predictions, prediction_row, task_class_names
from experiments.synbios_moe.pretraining.dataset import WHOLE_ATTRIBUTES
from experiments.synbios_moe.probes.dataset import ProbeItem
from experiments.synbios_moe.probes.model import collate

PROTOCOL = "q_whole_oracle_first_token_v1"


def insert_oracle_first_token(input_ids: Sequence[int], token_id: int, eos_id: int) -> list[int]:
    if not len(input_ids) or int(input_ids[-1]) != eos_id:
        raise ValueError("a Q input must end in the read-out EOS token")
    return [*(int(t) for t in input_ids[:-1]), int(token_id), eos_id]


def summarize_oracle_rows(rows: Sequence[dict]) -> dict[str, float | int]:
    n = len(rows)
    before = sum(bool(r["whole_before_correct"]) for r in rows)
    after = sum(bool(r["whole_after_correct"]) for r in rows)
    wrong = [r for r in rows if not r["whole_before_correct"]]
    right = [r for r in rows if r["whole_before_correct"]]
    recovered = sum(bool(r["whole_after_correct"]) for r in wrong)
    harmed = sum(not r["whole_after_correct"] for r in right)
    return {"examples": n, "accuracy_before": before / n if n else 0.0, "accuracy_after": after / n if n else 0.0,
            "accuracy_delta": (after - before) / n if n else 0.0, "baseline_errors": len(wrong), "recovered_errors": recovered,
            "recovery_rate": recovered / len(wrong) if wrong else 0.0, "baseline_correct": len(right), "harmed_correct": harmed,
            "harm_rate": harmed / len(right) if right else 0.0}


def first_token_id(class_name: str) -> int:
    """First-token classes are named by their token id (the birth date's month names are not: it has no whole task)."""

    try:
        return int(class_name)
    except ValueError as exc:
        raise ValueError(f"first-token class {class_name!r} is not a token id") from exc


@torch.no_grad()
def oracle_first_token_validation(backbone, *, data_root: str | Path, cache_root: str | Path, probe_dir: str | Path,
                                  output_dir: str | Path, device="cpu", attributes: Sequence[str] = WHOLE_ATTRIBUTES,
                                  batch_size: int = 256, max_examples: int | None = None,
                                  progress: Callable[[str, int], None] | None = None) -> dict:
    if batch_size <= 0 or (max_examples is not None and max_examples <= 0):
        raise ValueError("batch_size and max_examples must be positive")
    out = Path(output_dir)
    out.mkdir(parents=True, exist_ok=True)
    all_rows: list[dict] = []
    per_attribute: list[dict] = []
    for attribute in attributes:
        records, whole_head = collect_q_predictions(
            backbone, data_root=data_root, cache_root=cache_root, probe_dir=probe_dir, attribute=attribute, device=device,
            batch_size=batch_size, max_examples=max_examples,
            progress=(lambda done, name=attribute: progress(name, done)) if progress else None)
        whole_names = task_class_names(cache_root, attribute, "whole")
        eos = int(records[0].input_ids[-1]) if records else 0
        rows = []
        for lo in range(0, len(records), batch_size):
            chunk = records[lo:lo + batch_size]
            items = []
            for r in chunk:
                ids = insert_oracle_first_token(r.input_ids, first_token_id(r.true_first_token), eos)
                items.append(ProbeItem(np.asarray(ids, dtype=np.int64), np.asarray([len(ids) - 1], dtype=np.int64), r.true_whole_id))
            ids, pos, labels = collate(items, eos)
            logits = whole_head(ids.to(device), pos.to(device))[:, 0]
            pred = logits.argmax(-1).cpu()
            prob = logits.softmax(-1).gather(1, labels.to(device)[:, None])[:, 0].cpu()
            for off, r in enumerate(chunk):
                row = prediction_row(r)
                row.update({"whole_before_correct": r.whole_correct, "whole_after_correct": int(pred[off]) == r.true_whole_id,
                            "pred_whole_after": whole_names[int(pred[off])], "whole_true_probability_after": float(prob[off]),
                            "true_probability_delta": float(prob[off]) - r.whole_true_probability})
                rows.append(row)
        all_rows.extend(rows)
        per_attribute.append({"attribute": attribute, **summarize_oracle_rows(rows)})
        del whole_head
    summary = {"protocol": PROTOCOL, "intervention": "[EOS, name, label_t1, EOS]; the final EOS is read by the unchanged Q-whole head",
               "split": "person-held-out validation", "parameters_updated": False, "data": str(Path(data_root).resolve()),
               "probe_cache": str(Path(cache_root).resolve()), "probe_dir": str(Path(probe_dir).resolve()),
               "overall": summarize_oracle_rows(all_rows), "attributes": per_attribute}
    write_csv(out / "records.csv", all_rows)
    write_csv(out / "summary.csv", per_attribute)
    write_json(out / "summary.json", summary)
    return summary
