"""Token-level route analyses: which experts the tokens of each attribute value visit, and how stable that is.

Reference counterpart: experiments/synbios_moe/mechanisms/token_routes.py:22-373 (route capture per attribute token,
route Jaccard between renderings of the same fact, difference-in-differences against other people's facts; t1 / t2 route
branching on the Q read-out's bad cases, second half of this file).
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


# ---------------------------------------------------------------------------------------------------------------------
# Route branching on the Q read-out's bad cases
#
# A "bad case" is a held-out person whose value the Q-first head names correctly (first token right) while the Q-whole head
# does not, for a value of at least two tokens.  The frozen backbone is run on ``[EOS] name t1 t2 [EOS]`` with the TRUE tokens
# and the experts chosen at the t1 and t2 positions are recorded per layer.  Values that share t1 are then compared in pairs:
# if routing follows the token, pairs with the same t2 overlap at t2 as much as at t1, pairs with different t2 overlap less at
# t2; the drop ("branching score") says how strongly the second token redirects the route
# (reference: experiments/synbios_moe/mechanisms/token_routes.py:61-342, protocol name shared with its comparison report).
# ---------------------------------------------------------------------------------------------------------------------
ROUTE_PROTOCOL = "q_bad_case_t1_t2_route_branching_v1"


@torch.no_grad()
def routes_at_positions(model, input_ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """Experts chosen at selected positions: ``[batch, position, layer, K]`` (layers in model order, MoE layers only)."""

    per_layer = routes_for_batch(model, input_ids)
    if not per_layer:
        raise ValueError("route analysis needs a backbone with routed experts")
    rows = torch.arange(input_ids.shape[0])[:, None]
    picked = [per_layer[layer][rows, positions.cpu()] for layer in sorted(per_layer)]
    return torch.stack(picked, dim=2)


def _pairs_within(groups: dict[int, list[int]], *, same_second: bool, limit: int, rng: random.Random) -> list[tuple[int, int]]:
    """Index pairs of cases that share t1: both from one t2 group, or one from each of two different t2 groups."""

    keys = [k for k, members in groups.items() if len(members) >= (2 if same_second else 1)]
    if (same_second and not keys) or (not same_second and len(keys) < 2):
        return []
    pairs = []
    for _ in range(limit):
        if same_second:
            a, b = rng.sample(groups[rng.choice(keys)], 2)
        else:
            ka, kb = rng.sample(keys, 2)
            a, b = rng.choice(groups[ka]), rng.choice(groups[kb])
        pairs.append((a, b))
    return pairs


def pairwise_branching(cases: list[dict], *, layers: int, pair_limit: int = 2000, seed: int = 1337) -> list[dict]:
    """Per (attribute, layer, pair group): mean route overlap at t1 and at t2 over sampled same-t1 pairs and their difference."""

    rng = random.Random(seed)
    by_first: dict[tuple[str, int], dict[int, list[int]]] = defaultdict(lambda: defaultdict(list))
    for n, case in enumerate(cases):
        by_first[(str(case["attribute"]), int(case["t1_id"]))][int(case["t2_id"])].append(n)
    sums: dict[tuple[str, int, str], list[float]] = defaultdict(lambda: [0.0, 0.0, 0])
    for (attribute, _t1), groups in sorted(by_first.items()):
        for label, same in (("same_t2", True), ("different_t2", False)):
            for a, b in _pairs_within(groups, same_second=same, limit=pair_limit, rng=rng):
                ra, rb = cases[a]["routes"], cases[b]["routes"]
                for layer in range(layers):
                    acc = sums[(attribute, layer, label)]
                    acc[0] += jaccard(frozenset(ra[0][layer]), frozenset(rb[0][layer]))
                    acc[1] += jaccard(frozenset(ra[1][layer]), frozenset(rb[1][layer]))
                    acc[2] += 1
    rows = []
    for (attribute, layer, label), (s1, s2, n) in sorted(sums.items()):
        rows.append({"attribute": attribute, "layer": layer, "pair_group": label, "pair_count": n, "t1_route_overlap": s1 / n,
                     "t2_route_overlap": s2 / n, "branching_score": (s1 - s2) / n})
    return rows


def _path(per_layer: list[list[int]]) -> str:
    return "|".join("+".join(str(e) for e in layer) for layer in per_layer)


def _label_nmi(experts: list[int], labels: list[int], num_experts: int) -> float:
    if not labels:
        return 0.0
    dense = {tok: i for i, tok in enumerate(sorted(set(labels)))}          # token ids are sparse: re-index them
    return normalized_mutual_information(torch.tensor([dense[t] for t in labels]), torch.tensor(experts), num_experts)


@torch.no_grad()
def bad_case_route_validation(backbone, codec, *, data_root, cache_root, probe_dir, output_dir, device="cpu",
                              attributes=None, batch_size: int = 512, max_examples: int | None = None, pair_limit: int = 2000,
                              progress=None) -> dict:
    """Writes ``bad_cases.csv``, ``route_records.csv``, ``pairwise_branching.csv``, ``token_route_nmi.csv`` and ``summary.json``."""

    from pathlib import Path

    import numpy as np

    from experiments.synbios_moe.artifact_io import write_csv, write_json
    from experiments.synbios_moe.mechanisms.q_readout import collect_q_predictions, prediction_row
    from experiments.synbios_moe.pretraining.dataset import WHOLE_ATTRIBUTES
    from experiments.synbios_moe.probes.dataset import ProbeItem
    from experiments.synbios_moe.probes.model import collate

    if batch_size <= 0 or pair_limit <= 0 or (max_examples is not None and max_examples <= 0):
        raise ValueError("batch_size, pair_limit and max_examples must be positive")
    cfg = getattr(backbone, "module", backbone).cfg
    if not cfg.is_moe:
        raise ValueError("route analysis needs a backbone with routed experts")
    top_k = int(cfg.experts_per_token)
    attributes = tuple(attributes) if attributes else tuple(WHOLE_ATTRIBUTES)
    out = Path(output_dir)
    out.mkdir(parents=True, exist_ok=True)
    cases: list[dict] = []
    for attribute in attributes:
        records, head = collect_q_predictions(
            backbone, data_root=data_root, cache_root=cache_root, probe_dir=probe_dir, attribute=attribute, device=device,
            batch_size=batch_size, max_examples=max_examples,
            progress=(lambda done, name=attribute: progress(name, done)) if progress else None)
        del head
        chosen = []
        for r in records:
            value_ids = codec.encode(" " + r.true_whole_value)
            if r.first_correct and not r.whole_correct and len(value_ids) >= 2:
                chosen.append((r, value_ids))
        for lo in range(0, len(chosen), batch_size):
            chunk = chosen[lo:lo + batch_size]
            eos = int(chunk[0][0].input_ids[-1])
            items = []
            for r, value_ids in chunk:
                prefix = [int(t) for t in r.input_ids[:-1]]
                ids = [*prefix, int(value_ids[0]), int(value_ids[1]), eos]
                items.append(ProbeItem(np.asarray(ids, dtype=np.int64), np.asarray([len(prefix), len(prefix) + 1], dtype=np.int64),
                                       r.true_whole_id))
            ids, pos, _ = collate(items, eos)
            routes = routes_at_positions(backbone, ids.to(device), pos)
            for off, (r, value_ids) in enumerate(chunk):
                cases.append({**prediction_row(r), "t1_id": int(value_ids[0]), "t2_id": int(value_ids[1]),
                              "t1_text": codec.decode([int(value_ids[0])]), "t2_text": codec.decode([int(value_ids[1])]),
                              "routes": routes[off].tolist()})
    layers = len(cases[0]["routes"][0]) if cases else 0
    case_rows, route_rows = [], []
    for case in cases:
        row = {k: v for k, v in case.items() if k != "routes"}
        row["t1_route_path"], row["t2_route_path"] = _path(case["routes"][0]), _path(case["routes"][1])
        case_rows.append(row)
        for layer in range(layers):
            first, second = case["routes"][0][layer], case["routes"][1][layer]
            rec = {"case_id": case["case_id"], "person_id": case["person_id"], "attribute": case["attribute"], "t1_id": case["t1_id"],
                   "t2_id": case["t2_id"], "layer": layer}
            for k in range(top_k):
                rec[f"t1_expert_{k}"], rec[f"t2_expert_{k}"] = first[k], second[k]
            rec["within_case_jaccard"] = jaccard(frozenset(first), frozenset(second))
            rec["top1_changed"] = first[0] != second[0]
            route_rows.append(rec)
    pair_rows = pairwise_branching(cases, layers=layers, pair_limit=pair_limit)
    nmi_rows = []
    for attribute in attributes:
        mine = [c for c in cases if c["attribute"] == attribute]
        for layer in range(layers):
            nmi_rows.append({"attribute": attribute, "layer": layer, "examples": len(mine),
                             "t1_top1_token_nmi": _label_nmi([c["routes"][0][layer][0] for c in mine], [c["t1_id"] for c in mine], cfg.num_experts),
                             "t2_top1_token_nmi": _label_nmi([c["routes"][1][layer][0] for c in mine], [c["t2_id"] for c in mine], cfg.num_experts)})
    summary = {"protocol": ROUTE_PROTOCOL, "case_definition": "Q-first correct, Q-whole wrong, whole value has >=2 tokens",
               "route_model": "frozen pretrained backbone without probe embedding delta", "split": "person-held-out validation",
               "parameters_updated": False, "data": str(Path(data_root).resolve()), "probe_cache": str(Path(cache_root).resolve()),
               "probe_dir": str(Path(probe_dir).resolve()), "examples": len(cases),
               "attributes": {a: sum(c["attribute"] == a for c in cases) for a in attributes}, "layers": layers,
               "experts": int(cfg.num_experts), "top_k": top_k}
    write_csv(out / "bad_cases.csv", case_rows)
    write_csv(out / "route_records.csv", route_rows)
    write_csv(out / "pairwise_branching.csv", pair_rows)
    write_csv(out / "token_route_nmi.csv", nmi_rows)
    write_json(out / "summary.json", summary)
    return summary
