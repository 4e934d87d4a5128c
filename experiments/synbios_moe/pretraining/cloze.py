"""Progressive cloze evaluation: can the model *generate* an attribute value from the text that precedes it?

For attribute ``a`` of a biography the prompt is ``[EOS] + tokens`` up to the value; the model then decodes greedily,
one token per forward pass over the growing prefix (there is no KV cache: every step re-runs ``hidden_states`` on the
whole prefix and applies ``lm_head`` to the last position), until the value's token count is reached.  Batches are
right-padded with EOS and every row keeps its own write position
(reference: experiments/synbios_moe/pretraining/cloze.py:101-150).
"""

from __future__ import annotations

from typing import Iterable

import torch

from experiments.synbios_moe.codec import token_span_of_chars
from experiments.synbios_moe.pretraining.dataset import ATTRIBUTES


def cloze_items(codec, row: dict, attributes=ATTRIBUTES) -> list[dict]:
    items = []
    for attribute in attributes:
        start, end = row["attribute_spans"][attribute]
        ids, lo, hi = token_span_of_chars(codec, row["text"], int(start), int(end))
        items.append({"person_id": row["person_id"], "attribute": attribute, "prompt": ids[:lo], "answer": ids[lo:hi]})
    return items


@torch.no_grad()
def greedy_complete(model, prompts: list[list[int]], lengths: list[int], *, eos: int, device) -> list[list[int]]:
    """Decode ``lengths[i]`` tokens after ``prompts[i]``; rows advance in lock step, finished rows are frozen."""

    steps = max(lengths)
    width = max(len(p) for p in prompts) + steps
    tokens = torch.full((len(prompts), width), eos, dtype=torch.long, device=device)
    cursor = torch.tensor([len(p) for p in prompts], device=device)
    for row, p in enumerate(prompts):
        tokens[row, :len(p)] = torch.tensor(p, device=device)
    need = torch.tensor(lengths, device=device)
    rows = torch.arange(len(prompts), device=device)
    out: list[list[int]] = [[] for _ in prompts]
    for step in range(steps):
        active = need > step
        span = int(cursor.max())
        hidden = model.hidden_states(tokens[:, :span])
        hidden = hidden[0] if isinstance(hidden, tuple) else hidden
        last = hidden[rows, cursor - 1]
        nxt = model.lm_head(last).argmax(-1)
        tokens[rows[active], cursor[active]] = nxt[active]
        for row in torch.nonzero(active).flatten().tolist():
            out[row].append(int(nxt[row]))
        cursor = cursor + active.long()
    return out


def evaluate_cloze(model, codec, biographies: Iterable[dict], *, device="cpu", batch_size: int = 16, attributes=ATTRIBUTES,
                   max_items: int | None = None) -> dict:
    model.eval()
    limit = getattr(getattr(model, "cfg", None), "seq_len", 1 << 30)
    pending: list[dict] = []
    tallies = {a: {"items": 0, "exact": 0, "first": 0, "tokens": 0, "token_hits": 0} for a in attributes}
    examples: list[dict] = []

    def flush() -> None:
        if not pending:
            return
        got = greedy_complete(model, [i["prompt"] for i in pending], [len(i["answer"]) for i in pending], eos=codec.eos, device=device)
        for item, pred in zip(pending, got):
            t = tallies[item["attribute"]]
            hits = [a == b for a, b in zip(pred, item["answer"])]
            t["items"] += 1; t["exact"] += int(all(hits)); t["first"] += int(hits[0]); t["tokens"] += len(hits); t["token_hits"] += sum(hits)
            if len(examples) < 20:
                examples.append({"person_id": item["person_id"], "attribute": item["attribute"], "expected": codec.decode(item["answer"]),
                                 "generated": codec.decode(pred), "exact": all(hits)})
        pending.clear()

    for count, row in enumerate(biographies):
        if max_items is not None and count >= max_items:
            break
        for item in cloze_items(codec, row, attributes):
            if not item["answer"] or len(item["prompt"]) + len(item["answer"]) > limit:
                continue
            pending.append(item)
            if len(pending) == batch_size:
                flush()
    flush()
    per_attribute = {a: {"items": t["items"], "exact_match": t["exact"] / max(t["items"], 1), "first_token": t["first"] / max(t["items"], 1),
                         "token_accuracy": t["token_hits"] / max(t["tokens"], 1)} for a, t in tallies.items()}
    total = sum(t["items"] for t in tallies.values())
    return {"per_attribute": per_attribute, "overall_exact_match": sum(t["exact"] for t in tallies.values()) / max(total, 1),
            "items": total, "examples": examples}


def summarize_cloze(reports: dict[str, dict]) -> list[dict]:
    """Rows ``(run, attribute, exact_match, first_token, items)`` from several ``evaluate_cloze`` reports."""

    rows = []
    for run, report in sorted(reports.items()):
        for attribute, stats in report["per_attribute"].items():
            rows.append({"run": run, "attribute": attribute, **stats})
        rows.append({"run": run, "attribute": "overall", "exact_match": report["overall_exact_match"], "items": report["items"]})
    return rows
