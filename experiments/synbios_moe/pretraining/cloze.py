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


# ---------------------------------------------------------------------------------------------------------------------
# Progressive cloze over the original biography
#
# All six holes of a biography are filled from left to right in one growing sequence: what the model generated for an
# earlier fact stays in the context of the later ones, so mistakes propagate exactly as they would in free generation;
# only the text between the facts comes from the source.  A value is generated greedily until the decoded continuation
# contains the source text that follows the value up to and including the next full stop (or ``max_new_tokens`` ran out);
# the prediction is what precedes that stop text (reference: experiments/synbios_moe/pretraining/cloze.py:36-392).
# ---------------------------------------------------------------------------------------------------------------------
PROGRESSIVE_PROTOCOL = "progressive_original_biography_cloze_greedy"
FUZZY_THRESHOLDS = (0.5, 0.8, 0.9)


def character_similarity(predicted: str, expected: str) -> float:
    """1 - Levenshtein distance / longer length, on case-folded text with runs of white space collapsed."""

    a, b = " ".join(predicted.casefold().split()), " ".join(expected.casefold().split())
    if not a and not b:
        return 1.0
    row = list(range(len(b) + 1))
    for i, ca in enumerate(a, start=1):
        nxt = [i]
        for j, cb in enumerate(b, start=1):
            nxt.append(min(nxt[-1] + 1, row[j] + 1, row[j - 1] + (ca != cb)))
        row = nxt
    return 1.0 - row[-1] / max(len(a), len(b), 1)


def biography_fields(codec, row: dict) -> tuple[list[int], list[dict]]:
    """Token ids of ``[EOS] + text`` and the six value spans ``{attribute, lo, hi, expected}`` in textual order."""

    text = str(row["text"])
    ids, fields = None, []
    for attribute in ATTRIBUTES:
        start, end = (int(v) for v in row["attribute_spans"][attribute])
        ids, lo, hi = token_span_of_chars(codec, text, start, end)
        fields.append({"attribute": attribute, "lo": lo, "hi": hi, "expected": text[start:end]})
    fields.sort(key=lambda f: f["lo"])
    if any(f["lo"] >= f["hi"] for f in fields) or any(a["hi"] > b["lo"] for a, b in zip(fields, fields[1:])):
        raise ValueError(f"biography of {row.get('person_id')}: empty or overlapping value spans")
    return ids, fields


@torch.no_grad()
def generate_until(model, codec, prefixes: list[list[int]], stop_texts: list[str], *, device, max_new_tokens: int):
    """Greedy continuation of every prefix until its stop text shows up in the decoded continuation.

    Returns (generated token lists, terminated flags, model tokens processed).  Rows that are done leave the batch."""

    limit = getattr(getattr(model, "cfg", None), "seq_len", 1 << 30)
    seqs = [list(p) for p in prefixes]
    made: list[list[int]] = [[] for _ in prefixes]
    done = [False] * len(prefixes)
    live = list(range(len(prefixes)))
    processed = 0
    for _ in range(max_new_tokens):
        if not live:
            break
        width = max(len(seqs[i]) for i in live)
        if width > limit:
            raise ValueError(f"cloze prompt of {width} tokens exceeds seq_len={limit}")
        batch = torch.full((len(live), width), codec.eos, dtype=torch.long, device=device)
        ends = torch.empty(len(live), dtype=torch.long, device=device)
        for r, i in enumerate(live):
            batch[r, :len(seqs[i])] = torch.tensor(seqs[i], device=device)
            ends[r] = len(seqs[i])
        hidden = model.hidden_states(batch)
        hidden = hidden[0] if isinstance(hidden, tuple) else hidden
        nxt = model.lm_head(hidden[torch.arange(len(live), device=device), ends - 1]).argmax(-1).tolist()
        processed += batch.numel()
        still = []
        for i, tok in zip(live, nxt):
            seqs[i].append(int(tok))
            made[i].append(int(tok))
            if stop_texts[i] in codec.decode(made[i]):
                done[i] = True
            else:
                still.append(i)
        live = still
    return made, done, processed


def evaluate_progressive_cloze(model, codec, biographies: Iterable[dict], *, device="cpu", max_biographies: int, start_index: int = 0,
                               batch_size: int = 16, max_new_tokens: int = 16, sample_biographies: int = 12) -> dict:
    import time

    if start_index < 0 or max_biographies <= 0 or batch_size <= 0 or max_new_tokens <= 0:
        raise ValueError("start_index must be >= 0; max_biographies, batch_size and max_new_tokens must be positive")
    model.eval()
    hits = {a: 0 for a in ATTRIBUTES}
    seen = {a: 0 for a in ATTRIBUTES}
    similarity = {a: 0.0 for a in ATTRIBUTES}
    fuzzy = {t: {a: 0 for a in ATTRIBUTES} for t in FUZZY_THRESHOLDS}
    histogram = {n: 0 for n in range(len(ATTRIBUTES) + 1)}
    counters = {"biographies": 0, "all_exact": 0, "unterminated": 0, "tokens": 0}
    samples: list[dict] = []
    t0 = time.perf_counter()

    def run_batch(rows: list[dict]) -> None:
        states = []
        for row in rows:
            ids, fields = biography_fields(codec, row)
            states.append({"row": row, "ids": ids, "fields": fields, "cursor": 1, "seq": [codec.eos], "pred": {}, "ok": {}, "sim": {}})
        for k in range(len(ATTRIBUTES)):
            prefixes, stops = [], []
            for st in states:
                f = st["fields"][k]
                st["seq"] += st["ids"][st["cursor"]:f["lo"]]
                prefixes.append(st["seq"])
                stops.append(codec.decode(st["ids"][f["hi"]:]).split(".", 1)[0] + ".")
            made, done, processed = generate_until(model, codec, prefixes, stops, device=device, max_new_tokens=max_new_tokens)
            counters["tokens"] += processed
            for st, tokens, ended, stop in zip(states, made, done, stops):
                f = st["fields"][k]
                a = f["attribute"]
                guess = codec.decode(tokens).split(stop, 1)[0].strip()
                sim = character_similarity(guess, f["expected"])
                seen[a] += 1
                hits[a] += int(guess == f["expected"])
                similarity[a] += sim
                for t in FUZZY_THRESHOLDS:
                    fuzzy[t][a] += int(sim >= t)
                counters["unterminated"] += int(not ended)
                st["pred"][a], st["ok"][a], st["sim"][a] = guess, guess == f["expected"], sim
                st["seq"] += tokens
                st["cursor"] = f["hi"]
                if ended:       # the generation already wrote the sentence's full stop: skip the source tokens up to and including it
                    skipped = ""
                    while st["cursor"] < len(st["ids"]) and "." not in skipped:
                        skipped += codec.decode([st["ids"][st["cursor"]]])
                        st["cursor"] += 1
        for st in states:
            st["seq"] += st["ids"][st["cursor"]:]
            exact = sum(bool(v) for v in st["ok"].values())
            histogram[exact] += 1
            counters["all_exact"] += int(exact == len(ATTRIBUTES))
            counters["biographies"] += 1
            if len(samples) < sample_biographies:
                samples.append({"person_id": st["row"]["person_id"], "original_text": st["row"]["text"], "filled_text": codec.decode(st["seq"][1:]),
                                "expected": {f["attribute"]: f["expected"] for f in st["fields"]}, "predicted": st["pred"],
                                "correct": st["ok"], "character_similarity": st["sim"], "exact_fields": exact})

    pending: list[dict] = []
    for n, row in enumerate(biographies):
        if n < start_index:
            continue
        if n >= start_index + max_biographies:
            break
        pending.append(row)
        if len(pending) == batch_size:
            run_batch(pending)
            pending = []
    if pending:
        run_batch(pending)
    n_bio, total = counters["biographies"], max(sum(seen.values()), 1)
    elapsed = time.perf_counter() - t0
    per_attribute = {a: {"items": seen[a], "exact_match": hits[a] / max(seen[a], 1),
                         "mean_character_similarity": similarity[a] / max(seen[a], 1)} for a in ATTRIBUTES}
    return {"protocol": PROGRESSIVE_PROTOCOL,
            "protocol_note": "six holes per original biography filled left to right; generated earlier facts stay in the context",
            "start_index": start_index, "biographies": n_bio, "fields": n_bio * len(ATTRIBUTES),
            "attribute_accuracy": {a: hits[a] / max(seen[a], 1) for a in ATTRIBUTES},
            "attribute_mean_character_similarity": {a: similarity[a] / max(seen[a], 1) for a in ATTRIBUTES},
            "mean_character_similarity": sum(similarity.values()) / total,
            "fuzzy_accuracy_by_threshold": {str(t): {a: fuzzy[t][a] / max(seen[a], 1) for a in ATTRIBUTES} for t in FUZZY_THRESHOLDS},
            "micro_fuzzy_accuracy_by_threshold": {str(t): sum(fuzzy[t].values()) / total for t in FUZZY_THRESHOLDS},
            "micro_field_accuracy": sum(hits.values()) / total, "biography_all_fields_accuracy": counters["all_exact"] / max(n_bio, 1),
            "mean_correct_fields_per_biography": sum(k * v for k, v in histogram.items()) / max(n_bio, 1),
            "biography_correct_field_count_histogram": {str(k): v for k, v in histogram.items()},
            "correct_fields": hits, "total_fields": seen, "unterminated_fields": counters["unterminated"],
            "elapsed_seconds": elapsed, "biographies_per_second": n_bio / max(elapsed, 1e-9), "model_tokens_processed": counters["tokens"],
            # the keys the table builder and the probe pipeline's gate read, so that either protocol can feed them
            "per_attribute": per_attribute, "overall_exact_match": sum(hits.values()) / total, "items": sum(seen.values()),
            "samples": samples}
