"""Ground-truth-first whole probes: P-whole heads trained on prefixes extended by the true first token of the value.

A P probe reads a biography right BEFORE an attribute value.  Here every read-out prefix is extended by the value's
true first token ``t1`` (as it appears mid-sentence, with its leading space) and the hidden state AT ``t1`` is read.  A
fresh probe of the same architecture and rank as the original P-whole probe is trained on these inputs; the gain over
the original probe, by source position P0..P5, measures how much of the whole value becomes linearly readable once
its first token is known (reference: experiments/synbios_moe/mechanisms/first_token_intervention.py:49-349).
"""

from __future__ import annotations

import heapq
from dataclasses import dataclass
from pathlib import Path
from typing import Sequence

import numpy as np
import torch

from experiments.synbios_moe.artifact_io import sha256_file
from experiments.synbios_moe.mechanisms.q_readout import probe_state_path
from experiments.synbios_moe.pretraining.dataset import WHOLE_ATTRIBUTES
from experiments.synbios_moe.probes.dataset import CachedProbeDataset, ProbeItem
from experiments.synbios_moe.probes.model import AttributeProbe, collate, train_probe

PROTOCOL = "ground_truth_first_whole_rank_matched_v1"
POSITIONS = 6


def first_token_text(class_name: str, codec) -> tuple[int, str]:
    """A cached first-token class back to ``(token id, text)``; the text must start with the mid-sentence space and encode
    back to exactly that one token, otherwise appending it would not reproduce what the model saw in training."""

    try:
        token = int(class_name)
    except ValueError as exc:
        raise ValueError(f"first-token class is not a token id: {class_name!r}") from exc
    if not 0 <= token < codec.vocab_size or token == codec.eos:
        raise ValueError(f"invalid first-token id {token}")
    text = codec.decode([token])
    if not text.startswith(" "):
        raise ValueError(f"first token {token} decodes to {text!r}: expected a leading space")
    if codec.encode(text) != [token]:
        raise ValueError(f"first token {token} does not survive a decode / encode round trip")
    return token, text


def build_ground_truth_first_input(item: ProbeItem, source_position: int, token_id: int) -> ProbeItem:
    """Prefix of the biography up to read-out ``source_position``, then ``token_id``; the new token is the read-out."""

    if not 0 <= source_position < len(item.positions):
        raise IndexError("source position outside the cached item")
    prefix = np.asarray(item.input_ids[: int(item.positions[source_position]) + 1], dtype=np.int64)
    ids = np.concatenate([prefix, np.asarray([int(token_id)], dtype=np.int64)])
    return ProbeItem(ids, np.asarray([ids.shape[0] - 1], dtype=np.int64), item.label)


class GroundTruthFirstWholeDataset:
    """Whole-value labels on inputs rebuilt from the cached first-token labels: ``6 x`` the biographies of the split."""

    kind = "p"

    def __init__(self, first_data: CachedProbeDataset, whole_data: CachedProbeDataset, token_ids_by_class: Sequence[int]) -> None:
        if len(first_data) != len(whole_data) or not np.array_equal(first_data.examples, whole_data.examples):
            raise ValueError("the first and whole datasets are not aligned")
        self.first_data, self.whole_data = first_data, whole_data
        self.token_ids_by_class = tuple(int(t) for t in token_ids_by_class)
        self.class_names = list(whole_data.class_names)
        self.eos = whole_data.eos

    def __len__(self) -> int:
        return len(self.first_data) * POSITIONS

    @staticmethod
    def source_position(index: int) -> int:
        return index % POSITIONS

    def __getitem__(self, index: int) -> ProbeItem:
        source, position = divmod(int(index), POSITIONS)
        first, whole = self.first_data[source], self.whole_data[source]
        if not (np.array_equal(first.input_ids, whole.input_ids) and np.array_equal(first.positions, whole.positions)):
            raise ValueError("first and whole cached items are not input-aligned")
        if not 0 <= first.label < len(self.token_ids_by_class):
            raise ValueError("first-token class out of range")
        rebuilt = build_ground_truth_first_input(first, position, self.token_ids_by_class[first.label])
        return ProbeItem(rebuilt.input_ids, rebuilt.positions, whole.label)

    def longest(self, limit: int) -> list[ProbeItem]:
        """The rebuilt inputs with the largest sequence lengths (what a batch-size benchmark must survive)."""

        if limit <= 0:
            raise ValueError("limit must be positive")
        positions = self.first_data.positions

        def length(index: int) -> int:
            source, position = divmod(index, POSITIONS)
            return int(positions[int(self.first_data.examples[source])][position]) + 2

        return [self[i] for i in heapq.nlargest(min(limit, len(self)), range(len(self)), key=length)]


@dataclass(frozen=True)
class GroundTruthFirstWholeData:
    train_data: GroundTruthFirstWholeDataset
    validation_data: GroundTruthFirstWholeDataset
    token_entries: list[tuple[int, str]]
    reference_whole_checkpoint: Path
    cache_manifest_sha256: str
    rank: int


def prepare_ground_truth_first_whole_data(*, cache_root: str | Path, probe_dir: str | Path, attribute: str, codec,
                                          expected_rank: int | None = None) -> GroundTruthFirstWholeData:
    """Datasets of both splits, with the rank bound to the original P-whole probe of the same attribute."""

    if attribute not in WHOLE_ATTRIBUTES:
        raise ValueError(f"{attribute!r} has no whole-value task")
    cache = Path(cache_root)
    parts = {(t, s): CachedProbeDataset(cache, kind="p", attribute=attribute, target=t, split=s)
             for t in ("first", "whole") for s in ("train", "validation")}
    if parts["first", "train"].class_names != parts["first", "validation"].class_names:
        raise ValueError("first-token class mappings differ between the splits")
    reference = probe_state_path(probe_dir, "p", attribute, "whole")
    saved = torch.load(reference, map_location="cpu", weights_only=False)
    ident = saved.get("identity", {})
    if {k: ident.get(k) for k in ("kind", "attribute", "target")} != {"kind": "p", "attribute": attribute, "target": "whole"}:
        raise ValueError(f"{reference} is not the P-whole probe of {attribute!r}")
    rank = int(ident["rank"])
    if expected_rank is not None and rank != expected_rank:
        raise ValueError(f"the reference P-whole probe has rank {rank}, expected {expected_rank}")
    classes = saved["probe"]["classifier.weight"].shape[0]
    if classes != len(parts["whole", "train"].class_names):
        raise ValueError("the reference P-whole probe was trained on a different class mapping")
    tokens = [first_token_text(name, codec) for name in parts["first", "train"].class_names]
    ids = [t for t, _ in tokens]
    return GroundTruthFirstWholeData(
        train_data=GroundTruthFirstWholeDataset(parts["first", "train"], parts["whole", "train"], ids),
        validation_data=GroundTruthFirstWholeDataset(parts["first", "validation"], parts["whole", "validation"], ids),
        token_entries=tokens, reference_whole_checkpoint=reference, cache_manifest_sha256=sha256_file(cache / "manifest.json"), rank=rank)


@torch.no_grad()
def evaluate_by_source_position(probe: AttributeProbe, dataset: GroundTruthFirstWholeDataset, *, device="cpu", batch_size: int = 256,
                                max_examples: int | None = None) -> dict:
    if max_examples is not None and max_examples <= 0:
        raise ValueError("max_examples must be positive or None")
    was_training = probe.training
    probe.eval()
    count = len(dataset) if max_examples is None else min(len(dataset), max_examples)
    correct, total = [0] * POSITIONS, [0] * POSITIONS
    for lo in range(0, count, batch_size):
        idx = range(lo, min(lo + batch_size, count))
        ids, pos, labels = collate([dataset[i] for i in idx], dataset.eos)
        pred = probe(ids.to(device), pos.to(device))[:, 0].argmax(-1).cpu()
        for i, p, y in zip(idx, pred.tolist(), labels.tolist()):
            total[i % POSITIONS] += 1
            correct[i % POSITIONS] += int(p == y)
    probe.train(was_training)
    return {"accuracy": sum(correct) / max(sum(total), 1), "accuracy_by_position": [c / max(t, 1) for c, t in zip(correct, total)],
            "correct_by_position": correct, "total_by_position": total}


def train_ground_truth_first_whole_probe(backbone, *, cache_root: str | Path, probe_dir: str | Path, attribute: str, codec, device="cpu",
                                         batch_size: int = 50, evaluation_batch_size: int = 256, steps: int = 3000, seed: int = 1337,
                                         recovery_checkpoint: str | Path | None = None, checkpoint_interval_steps: int | None = None,
                                         resume: bool = True, max_validation_examples: int | None = None, on_event=None) -> dict:
    """Train the rank-matched probe and evaluate it per source position; returns the result record (with ``probe_state``)."""

    prepared = prepare_ground_truth_first_whole_data(cache_root=cache_root, probe_dir=probe_dir, attribute=attribute, codec=codec)
    identity = {"protocol": PROTOCOL, "reference_whole_probe_sha256": sha256_file(prepared.reference_whole_checkpoint),
                "probe_cache_manifest_sha256": prepared.cache_manifest_sha256}
    result = train_probe(backbone, cache_root, kind="p", attribute=attribute, target="whole", steps=steps, device=device,
                         rank=prepared.rank, batch_size=batch_size, evaluation_batch_size=evaluation_batch_size, seed=seed,
                         recovery_checkpoint=recovery_checkpoint, checkpoint_interval_steps=checkpoint_interval_steps, resume=resume,
                         skip_final_validation=True, identity=identity, on_event=on_event, train_set=prepared.train_data,
                         valid_set=prepared.validation_data, return_probe=True)
    probe = result.pop("probe")
    validation = evaluate_by_source_position(probe, prepared.validation_data, device=device, batch_size=evaluation_batch_size,
                                             max_examples=max_validation_examples)
    result.update({
        "protocol": PROTOCOL, "attribute": attribute, "target": "whole", "ground_truth_first_token": True,
        "validation": {"accuracy": validation["accuracy"], "accuracy_by_position": validation["accuracy_by_position"],
                       "examples": sum(validation["total_by_position"])},
        "whole_accuracy_validation_by_source_position": validation["accuracy_by_position"],
        "whole_correct_validation_by_source_position": validation["correct_by_position"],
        "whole_total_validation_by_source_position": validation["total_by_position"],
        "first_token_text": {str(t): text for t, text in prepared.token_entries},
        "reference_whole_probe_checkpoint": str(prepared.reference_whole_checkpoint.resolve()), "reference_rank": prepared.rank,
        "input_protocol": "biography prefix through the original read-out, then the true leading-space first token; read at that token",
        "backbone_parameters_updated": False,
        "stage_two_trainable_components": ["low_rank_embedding_delta", "normalizer", "whole_classifier"]})
    return result
