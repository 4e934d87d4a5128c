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


# ---------------------------------------------------------------------------------------------------------------------
# Distribution of the attribute values' tokens
#
# Every value is encoded the way it appears inside a sentence (``" " + value``).  Per attribute the report gives the token
# length distribution (weighted by profile and over distinct values), what a first-token probe can tell apart (distinct first
# tokens, their entropy, how many whole values share one first token), the token distribution at every position of the
# value, and how much the leading space changes the tokenisation.  The normalised distribution is the same for every
# augmentation of a corpus, because augmentation repeats the same profiles
# (reference: experiments/synbios_moe/pretraining/token_statistics.py:29-237).
# ---------------------------------------------------------------------------------------------------------------------
DISTRIBUTION_PROTOCOL = "synbios_attribute_leading_space_token_distribution_v1"


def entropy_bits(counts: Counter) -> float:
    import math

    total = sum(counts.values())
    return -sum(c / total * math.log2(c / total) for c in counts.values() if c) if total else 0.0


def percentile(values: list[int], q: float) -> float:
    """Linear interpolation between order statistics (``q`` in percent)."""

    if not values:
        return 0.0
    srt = sorted(values)
    at = (len(srt) - 1) * q / 100.0
    lo = int(at)
    hi = min(lo + 1, len(srt) - 1)
    return srt[lo] + (srt[hi] - srt[lo]) * (at - lo)


def attribute_token_distribution(codec, profiles: Iterable[dict], output_dir=None) -> dict:
    """Summary per attribute; with ``output_dir`` also ``attribute_summary.csv``, ``length_distribution.csv``,
    ``position_token_distribution.csv`` and ``summary.json``."""

    people = list(profiles)
    if not people:
        raise ValueError("no profiles")
    summaries: dict[str, dict] = {}
    length_rows, position_rows = [], []
    for attribute in ATTRIBUTES:
        values = [str(p[attribute]) for p in people]
        spaced_all = [tuple(codec.encode(" " + v)) for v in values]
        distinct = sorted(set(values))
        spaced = {v: tuple(codec.encode(" " + v)) for v in distinct}
        bare = {v: tuple(codec.encode(v)) for v in distinct}
        lengths_all, lengths_distinct = [len(s) for s in spaced_all], [len(s) for s in spaced.values()]
        by_position_counts, by_position_entropy = {}, {}
        for pos in range(max(lengths_all)):
            weighted = Counter(s[pos] for s in spaced_all if len(s) > pos)
            among_distinct = Counter(s[pos] for s in spaced.values() if len(s) > pos)
            present = sum(weighted.values())
            by_position_counts[str(pos + 1)] = len(weighted)
            by_position_entropy[str(pos + 1)] = entropy_bits(weighted)
            for token, count in weighted.most_common():
                position_rows.append({"attribute": attribute, "token_position": pos + 1, "token_id": int(token),
                                      "token_text": codec.decode([int(token)]), "profile_count": count,
                                      "profile_probability": count / len(people), "conditional_probability_when_present": count / present,
                                      "unique_value_count": among_distinct[token]})
        sharing = Counter(s[0] for s in spaced.values())            # whole values behind each first token
        changed = sum(spaced[v] != bare[v] for v in distinct)
        summaries[attribute] = {
            "profile_count": len(people), "unique_values": len(distinct), "unique_token_sequences": len(set(spaced.values())),
            "leading_space": True,
            "token_length": {"minimum": min(lengths_all), "mean_profile_weighted": fmean(lengths_all),
                             "median_profile_weighted": median(lengths_all), "p95_profile_weighted": percentile(lengths_all, 95),
                             "maximum": max(lengths_all), "mean_unique_values": fmean(lengths_distinct),
                             "median_unique_values": median(lengths_distinct)},
            "first_token": {"unique_tokens_profile_weighted": len({s[0] for s in spaced_all}), "unique_tokens_unique_values": len(sharing),
                            "entropy_bits_profile_weighted": entropy_bits(Counter(s[0] for s in spaced_all)),
                            "whole_classes_per_first_token": {"minimum": min(sharing.values()), "mean": fmean(sharing.values()),
                                                              "median": median(sharing.values()), "maximum": max(sharing.values())}},
            "position_unique_token_counts": by_position_counts, "position_entropy_bits_profile_weighted": by_position_entropy,
            "leading_space_comparison": {"bare_first_token_classes": len({s[0] for s in bare.values()}),
                                         "space_first_token_classes": len(sharing), "unique_values_with_changed_token_sequence": changed,
                                         "changed_fraction": changed / len(distinct),
                                         "bare_mean_unique_value_length": fmean(len(s) for s in bare.values()),
                                         "space_mean_unique_value_length": fmean(lengths_distinct)}}
        for weighting, counts, total in (("profile_weighted", Counter(lengths_all), len(people)),
                                         ("unique_values", Counter(lengths_distinct), len(distinct))):
            for n_tokens, count in sorted(counts.items()):
                length_rows.append({"attribute": attribute, "weighting": weighting, "token_length": n_tokens, "count": count,
                                    "probability": count / total})
    result = {"protocol": DISTRIBUTION_PROTOCOL, "tokenizer": type(codec).__name__, "encoding_rule": 'codec.encode(" " + attribute_value)',
              "num_people": len(people),
              "data_conditions": {"single": "one biography per profile",
                                  "multi5_permute": "five biographies per profile; the normalised value-token distribution is the same "
                                                    "because the same profiles are repeated"},
              "attributes": summaries,
              "artifacts": {"summary_table": "attribute_summary.csv", "length_distribution": "length_distribution.csv",
                            "position_token_distribution": "position_token_distribution.csv"}}
    if output_dir is not None:
        from pathlib import Path

        from experiments.synbios_moe.artifact_io import write_csv, write_json

        out = Path(output_dir)
        out.mkdir(parents=True, exist_ok=True)
        table = [{"attribute": a, "profiles": s["profile_count"], "unique_values": s["unique_values"],
                  "space_first_token_classes": s["first_token"]["unique_tokens_unique_values"], "minimum_tokens": s["token_length"]["minimum"],
                  "mean_tokens_profile_weighted": s["token_length"]["mean_profile_weighted"],
                  "median_tokens_profile_weighted": s["token_length"]["median_profile_weighted"],
                  "p95_tokens_profile_weighted": s["token_length"]["p95_profile_weighted"], "maximum_tokens": s["token_length"]["maximum"],
                  "first_token_entropy_bits": s["first_token"]["entropy_bits_profile_weighted"],
                  "mean_whole_classes_per_first_token": s["first_token"]["whole_classes_per_first_token"]["mean"],
                  "space_vs_bare_changed_fraction": s["leading_space_comparison"]["changed_fraction"]} for a, s in summaries.items()]
        write_csv(out / "attribute_summary.csv", table, list(table[0]))
        write_csv(out / "length_distribution.csv", length_rows, list(length_rows[0]))
        write_csv(out / "position_token_distribution.csv", position_rows, list(position_rows[0]))
        write_json(out / "summary.json", result)
    return result
