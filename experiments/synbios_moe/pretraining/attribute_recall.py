"""Teacher-forced attribute recall: how often the model's arg-max next token equals each token of an attribute value.

For every biography the text is tokenised as ``[EOS] + tokens``; the value of attribute ``a`` occupies a token range
``[lo, hi)``; the prediction for token ``t`` is read from the logits at ``t - 1``.  Reported per attribute: accuracy over
all value tokens, over first tokens only, and the share of values reproduced in full
(reference: experiments/synbios_moe/pretraining/attribute_recall.py:17-133).
"""

from __future__ import annotations

from collections import defaultdict
from typing import Iterable

import torch

from experiments.synbios_moe.codec import token_span_of_chars
from experiments.synbios_moe.pretraining.dataset import ATTRIBUTES


def attribute_token_ranges(codec, text: str, spans: dict) -> tuple[list[int], dict[str, tuple[int, int]]]:
    ids, ranges = None, {}
    for attribute in ATTRIBUTES:
        start, end = spans[attribute]
        ids, lo, hi = token_span_of_chars(codec, text, int(start), int(end))
        ranges[attribute] = (lo, hi)
    return ids, ranges


@torch.no_grad()
def evaluate_attribute_recall(model, codec, biographies: Iterable[dict], *, device: torch.device | str = "cpu", batch_size: int = 32,
                              max_items: int | None = None) -> dict[str, dict[str, float]]:
    """``biographies``: rows of ``biographies.jsonl``.  The model is called as ``model(input_ids)`` -> logits."""

    model.eval()
    tallies = {a: defaultdict(int) for a in ATTRIBUTES}
    batch: list[tuple[list[int], dict]] = []

    def flush() -> None:
        if not batch:
            return
        width = max(len(ids) for ids, _ in batch)
        tokens = torch.full((len(batch), width), codec.eos, dtype=torch.long)
        for row, (ids, _) in enumerate(batch):
            tokens[row, :len(ids)] = torch.tensor(ids)
        out = model(tokens.to(device))
        logits = out[-1] if isinstance(out, tuple) else out           # the model returns (loss, logits)
        guess = logits.argmax(-1).cpu()                       # guess[:, t] predicts token t + 1
        for row, (ids, ranges) in enumerate(batch):
            for attribute, (lo, hi) in ranges.items():
                hits = [int(guess[row, t - 1]) == ids[t] for t in range(lo, hi)]
                tally = tallies[attribute]
                tally["tokens"] += len(hits); tally["token_hits"] += sum(hits)
                tally["values"] += 1; tally["first_hits"] += int(hits[0]) if hits else 0
                tally["whole_hits"] += int(all(hits)) if hits else 0
        batch.clear()

    for count, row in enumerate(biographies):
        if max_items is not None and count >= max_items:
            break
        ids, ranges = attribute_token_ranges(codec, row["text"], row["attribute_spans"])
        limit = getattr(getattr(model, "cfg", None), "seq_len", None)
        if limit is not None and len(ids) > limit:
            continue
        batch.append((ids, ranges))
        if len(batch) == batch_size:
            flush()
    flush()
    report = {}
    for attribute, t in tallies.items():
        report[attribute] = {"values": t["values"], "token_accuracy": t["token_hits"] / max(t["tokens"], 1),
                             "first_token_accuracy": t["first_hits"] / max(t["values"], 1),
                             "whole_value_accuracy": t["whole_hits"] / max(t["values"], 1)}
    total = sum(t["values"] for t in tallies.values())
    report["overall"] = {"values": total, "whole_value_accuracy": sum(t["whole_hits"] for t in tallies.values()) / max(total, 1),
                         "token_accuracy": sum(t["token_hits"] for t in tallies.values()) / max(sum(t["tokens"] for t in tallies.values()), 1)}
    return report
