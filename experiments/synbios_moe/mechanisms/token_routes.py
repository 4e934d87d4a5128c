"""Token-level route analyses: which experts the tokens of each attribute value visit, and how stable that is.

Reference counterpart: experiments/synbios_moe/mechanisms/token_routes.py:22-373 (route capture per attribute token,
route Jaccard between renderings of the same fact, difference-in-differences against other people's facts).
"""

from __future__ import annotations

import random
from collections import defaultdict
from typing import Iterable

import torch

from experiments.synbios_moe.codec import token_span_of_chars
from experiments.synbios_moe.mechanisms.routing import expert_load, normalized_mutual_information, routes_for_batch
from experiments.synbios_moe.pretraining.dataset import ATTRIBUTES


def attribute_token_labels(codec, row: dict) -> tuple[list[int], list[int]]:
    """Token ids of ``[EOS] + text`` and, per token, the index of the attribute it belongs to (-1 outside values)."""

    ids, labels = None, None
    for k, attribute in enumerate(ATTRIBUTES):
        start, end = row["attribute_spans"][attribute]
        ids, lo, hi = token_span_of_chars(codec, row["text"], int(start), int(end))
        if labels is None:
            labels = [-1] * len(ids)
        for t in range(lo, hi):
            labels[t] = k
    return ids, labels


@torch.no_grad()
def collect_token_routes(model, codec, biographies: Iterable[dict], *, device="cpu", max_items: int = 256) -> dict:
    """Per layer: routes of value tokens keyed by (person, attribute), plus flat (label, top-1 expert) pairs."""

    model.eval()
    limit = model.cfg.seq_len
    per_layer_sets: dict[int, dict[tuple[int, str], list[frozenset]]] = defaultdict(lambda: defaultdict(list))
    flat_labels: dict[int, list[int]] = defaultdict(list)
    flat_experts: dict[int, list[int]] = defaultdict(list)
    for n, row in enumerate(biographies):
        if n >= max_items:
            break
        ids, labels = attribute_token_labels(codec, row)
        if len(ids) > limit:
            continue
        routes = routes_for_batch(model, torch.tensor([ids], device=device))
        for layer, r in routes.items():
            r = r[0]                                                  # [seq, K]
            flat_labels[layer] += labels
            flat_experts[layer] += r[:, 0].tolist()
            for k, attribute in enumerate(ATTRIBUTES):
                toks = [t for t, lab in enumerate(labels) if lab == k]
                if toks:
                    per_layer_sets[layer][(row["person_id"], attribute)].append(frozenset(r[toks].reshape(-1).tolist()))
    return {"sets": per_layer_sets, "labels": flat_labels, "experts": flat_experts}


def jaccard(a: frozenset, b: frozenset) -> float:
    return len(a & b) / len(a | b) if (a or b) else 1.0


def route_report(collected: dict, num_experts: int, *, seed: int = 0) -> dict:
    """Per layer: NMI(attribute, expert), expert load over value tokens, and route-set Jaccard of the same fact rendered
    twice against the Jaccard of different people's facts of the same attribute (their difference is the DiD)."""

    rng = random.Random(seed)
    report = {}
    for layer in sorted(collected["labels"]):
        labels = torch.tensor(collected["labels"][layer])
        experts = torch.tensor(collected["experts"][layer])
        on_values = labels >= 0
        same, other = [], []
        sets = collected["sets"][layer]
        by_attribute: dict[str, list[tuple[int, frozenset]]] = defaultdict(list)
        for (person, attribute), renderings in sets.items():
            by_attribute[attribute] += [(person, r) for r in renderings]
            for i in range(len(renderings)):
                for j in range(i + 1, len(renderings)):
                    same.append(jaccard(renderings[i], renderings[j]))
        for attribute, entries in by_attribute.items():
            for _ in range(min(len(entries), 200)):
                (pa, ra), (pb, rb) = rng.choice(entries), rng.choice(entries)
                if pa != pb:
                    other.append(jaccard(ra, rb))
        mean = lambda xs: sum(xs) / len(xs) if xs else None   # noqa: E731
        report[layer] = {"nmi_attribute_expert": normalized_mutual_information(labels, experts, num_experts),
                         "value_token_load": expert_load(experts[on_values], num_experts).tolist() if on_values.any() else [],
                         "jaccard_same_fact": mean(same), "jaccard_other_people": mean(other),
                         "jaccard_did": (mean(same) - mean(other)) if same and other else None,
                         "value_tokens": int(on_values.sum())}
    return report
