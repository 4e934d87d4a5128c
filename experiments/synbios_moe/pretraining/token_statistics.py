"""Token statistics of a generated dataset: lengths, value-token counts, vocabulary coverage, first-token ambiguity.

The first-token statistics matter for the probes: a ``first`` probe task classifies the first token of the value, so
the number of distinct first tokens (and how many values share one) bounds what such a probe can tell apart
(reference: experiments/synbios_moe/pretraining/token_statistics.py:1-254).
"""

from __future__ import annotations

from collections import Counter
from statistics import fmean, median
from typing import Iterable

from experiments.synbios_moe.codec import token_span_of_chars
from experiments.synbios_moe.pretraining.dataset import ATTRIBUTES


def dataset_token_statistics(codec, biographies: Iterable[dict], profiles: Iterable[dict]) -> dict:
    lengths, vocab = [], Counter()
    value_tokens = {a: [] for a in ATTRIBUTES}
    for row in biographies:
        ids = None
        for attribute in ATTRIBUTES:
            start, end = row["attribute_spans"][attribute]
            ids, lo, hi = token_span_of_chars(codec, row["text"], int(start), int(end))
            value_tokens[attribute].append(hi - lo)
        lengths.append(len(ids))
        vocab.update(ids)
    first = {a: Counter() for a in ATTRIBUTES}
    distinct = {a: set() for a in ATTRIBUTES}
    for p in profiles:
        for attribute in ATTRIBUTES:
            value = str(p[attribute])
            distinct[attribute].add(value)
            first[attribute][codec.encode(" " + value)[0]] += 1
    srt = sorted(lengths)
    return {
        "biographies": len(lengths), "tokens_total": sum(lengths), "tokens_mean": fmean(lengths) if lengths else 0.0,
        "tokens_median": median(lengths) if lengths else 0, "tokens_max": srt[-1] if srt else 0,
        "tokens_p95": srt[int(0.95 * (len(srt) - 1))] if srt else 0, "vocabulary_used": len(vocab),
        "vocabulary_fraction": len(vocab) / codec.vocab_size,
        "attributes": {a: {"value_tokens_mean": fmean(value_tokens[a]) if value_tokens[a] else 0.0,
                           "value_tokens_max": max(value_tokens[a], default=0), "distinct_values": len(distinct[a]),
                           "distinct_first_tokens": len(first[a]),
                           "largest_first_token_share": max(first[a].values(), default=0) / max(sum(first[a].values()), 1)}
                       for a in ATTRIBUTES}}
