#!/usr/bin/env python
"""Audit one result of the ground-truth-first whole probe (``synbios_moe.py ground-truth-first-whole``).

Checks the fields that make the result comparable with the original P-whole probe: protocol name, frozen backbone, rank
bound to the reference probe, six source positions whose totals add up to the evaluated examples, finite loss, the weights
file next to the record, the hash of the reference probe, and (optionally) that a resumed run continued from the expected
step.  Exit code 0 = every check passed; 1 = at least one failed (all failures are listed)
(reference: scripts/audit_ground_truth_first_probe.py:1-182).
"""

from __future__ import annotations

import argparse
import hashlib
import json
import math
import sys
from pathlib import Path


def audit(path: Path, *, expect_resumed_from: int | None = None, max_validation_examples: int | None = None,
          reference_probe: Path | None = None) -> list[str]:
    errors: list[str] = []
    try:
        rec = json.loads(path.read_text(encoding="utf-8"))
    except (OSError, ValueError) as exc:
        return [f"unreadable result: {exc}"]

    def check(ok: bool, message: str) -> None:
        if not ok:
            errors.append(message)

    check(rec.get("protocol") == "ground_truth_first_whole_rank_matched_v1", f"protocol is {rec.get('protocol')!r}")
    check(rec.get("ground_truth_first_token") is True, "ground_truth_first_token is not true")
    check(rec.get("backbone_parameters_updated") is False, "the backbone must stay frozen")
    check(rec.get("target") == "whole", "target must be 'whole'")
    ident = rec.get("identity", {})
    check(ident.get("kind") == "p", "the probe must be a P probe")
    check(ident.get("rank") == rec.get("reference_rank"), f"rank {ident.get('rank')} differs from the reference probe's {rec.get('reference_rank')}")
    acc, hit, tot = (rec.get(k, []) for k in ("whole_accuracy_validation_by_source_position", "whole_correct_validation_by_source_position",
                                              "whole_total_validation_by_source_position"))
    check(len(acc) == len(hit) == len(tot) == 6, "expected six source positions")
    if len(acc) == len(hit) == len(tot) == 6:
        for i in range(6):
            check(0 <= hit[i] <= tot[i], f"position {i}: {hit[i]} correct of {tot[i]}")
            check(tot[i] == 0 or abs(acc[i] - hit[i] / tot[i]) < 1e-9, f"position {i}: accuracy does not equal correct / total")
        check(max(tot) - min(tot) <= 1, "source positions were not evaluated equally often")
        if max_validation_examples is not None:
            check(sum(tot) <= max_validation_examples, f"{sum(tot)} examples evaluated, limit {max_validation_examples}")
    check(rec.get("final_loss") is not None and math.isfinite(float(rec["final_loss"])), "final loss is missing or not finite")
    check(rec.get("steps") == ident.get("steps"), f"trained {rec.get('steps')} of {ident.get('steps')} steps")
    check(path.with_suffix(".pt").is_file(), f"weights file {path.with_suffix('.pt').name} is missing")
    if expect_resumed_from is not None:
        check(rec.get("resumed_from_step") == expect_resumed_from, f"resumed from step {rec.get('resumed_from_step')}, expected {expect_resumed_from}")
    ref = reference_probe or (Path(rec["reference_whole_probe_checkpoint"]) if rec.get("reference_whole_probe_checkpoint") else None)
    if ref is not None and ref.is_file():
        digest = hashlib.sha256(ref.read_bytes()).hexdigest()
        check(digest == ident.get("reference_whole_probe_sha256"), "the reference P-whole probe changed since this probe was trained")
    elif reference_probe is not None:
        errors.append(f"reference probe {reference_probe} not found")
    tokens = rec.get("first_token_text", {})
    check(bool(tokens) and all(t.startswith(" ") for t in tokens.values()), "first-token texts must start with the mid-sentence space")
    return errors


def audit_protocol(*, probe_cache: Path, probe_dir: Path, model_config: str, checkpoint: str, device: str, codec_name: str,
                   samples_per_split: int = 64) -> dict:
    """The protocol itself on real artifacts, before any GPU time is spent on it (the reference script's mode): for each of
    the five whole-value attributes the rebuilt datasets exist and are aligned, the fresh probe has the rank of the original
    P-whole probe, exactly the embedding change, the normaliser and the classifier are trainable, the backbone is frozen,
    and sampled inputs are the cached prefix up to the read-out followed by the value's true first token, read at that token."""

    import torch

    sys.path.insert(0, str(Path(__file__).resolve().parent))
    from synbios_moe import load_backbone

    from experiments.synbios_moe.artifact_io import sha256_file
    from experiments.synbios_moe.codec import get_codec
    from experiments.synbios_moe.mechanisms.first_token_intervention import POSITIONS, PROTOCOL, prepare_ground_truth_first_whole_data
    from experiments.synbios_moe.pretraining.dataset import WHOLE_ATTRIBUTES
    from experiments.synbios_moe.probes.model import AttributeProbe

    codec = get_codec(codec_name)
    backbone = load_backbone(model_config, checkpoint, device, codec_vocab=codec.vocab_size)
    expected_trainable = ("delta.a.weight", "delta.b.weight", "normalizer.weight", "normalizer.bias", "classifier.weight", "classifier.bias")
    tasks = []
    for attribute in WHOLE_ATTRIBUTES:
        errors: list[str] = []
        try:
            prepared = prepare_ground_truth_first_whole_data(cache_root=probe_cache, probe_dir=probe_dir, attribute=attribute, codec=codec)
        except (ValueError, FileNotFoundError, KeyError) as exc:
            tasks.append({"kind": "p", "attribute": attribute, "passed": False, "errors": [f"{type(exc).__name__}: {exc}"]})
            continue
        probe = AttributeProbe(backbone, len(prepared.train_data.class_names), rank=prepared.rank, kind="p")
        trainable = tuple(name for name, parameter in probe.named_parameters() if parameter.requires_grad)
        if trainable != expected_trainable:
            errors.append(f"trainable parameters are {trainable}")
        if any(parameter.requires_grad for parameter in backbone.parameters()):
            errors.append("the backbone is not frozen")
        if tuple(probe.delta.b.weight.shape) != (backbone.cfg.hidden_size, prepared.rank) or bool(probe.delta.b.weight.abs().sum() != 0):
            errors.append("the embedding change does not start at zero with the reference rank")
        checked = 0
        for data in (prepared.train_data, prepared.validation_data):
            if len(data) != POSITIONS * len(data.first_data):
                errors.append("a split does not hold six rebuilt inputs per source")
            stride = max(len(data) // max(samples_per_split, 1), 1)
            for index in range(0, len(data), stride):
                source, position = divmod(index, POSITIONS)
                first, item = data.first_data[source], data[index]
                prefix_end = int(first.positions[position]) + 1
                token = data.token_ids_by_class[first.label]
                ok = (item.input_ids.shape[0] == prefix_end + 1 and bool((item.input_ids[:prefix_end] == first.input_ids[:prefix_end]).all())
                      and int(item.input_ids[-1]) == token and list(item.positions) == [prefix_end]
                      and item.label == data.whole_data[source].label)
                if not ok:
                    errors.append(f"item {index} is not prefix + true first token read at that token")
                    break
                checked += 1
        tasks.append({"kind": "p", "attribute": attribute, "rank": prepared.rank, "classes": len(prepared.train_data.class_names),
                      "train_sources": len(prepared.train_data.first_data), "validation_sources": len(prepared.validation_data.first_data),
                      "expanded_train_examples": len(prepared.train_data), "expanded_validation_examples": len(prepared.validation_data),
                      "sampled_items_checked": checked, "reference_whole_probe": str(prepared.reference_whole_checkpoint.resolve()),
                      "reference_whole_probe_sha256": sha256_file(prepared.reference_whole_checkpoint), "trainable_parameters": list(trainable),
                      "input_protocol": "P prefix + true_t1, read true_t1", "passed": not errors, "errors": errors})
    return {"schema_version": 1, "protocol": PROTOCOL, "quality_gate_passed": len(tasks) == 5 and all(t["passed"] for t in tasks),
            "probe_cache": str(Path(probe_cache).resolve()), "probe_cache_manifest_sha256": sha256_file(Path(probe_cache) / "manifest.json"),
            "probe_dir": str(Path(probe_dir).resolve()), "backbone_checkpoint": str(Path(checkpoint).resolve()), "tasks": tasks}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("results", nargs="*", type=Path, help="result records of a run (record mode)")
    ap.add_argument("--expect-resumed-from", type=int)
    ap.add_argument("--max-validation-examples", type=int)
    ap.add_argument("--reference-probe", type=Path)
    # protocol mode (the reference script's command line): audit the inputs of a run that has not been made yet
    ap.add_argument("--probe-cache", type=Path); ap.add_argument("--probe-dir", type=Path, help="finished pipeline stage with the original P probes")
    ap.add_argument("--model-config"); ap.add_argument("--checkpoint"); ap.add_argument("--device", default="cpu")
    ap.add_argument("--codec", default="gpt2"); ap.add_argument("--data", help="accepted: the cache names its dataset")
    ap.add_argument("--output", type=Path, help="protocol mode: where the audit record goes")
    args = ap.parse_args(argv)
    if args.probe_dir is not None:
        missing = [name for name in ("probe_cache", "model_config", "checkpoint", "output") if getattr(args, name) is None]
        if missing:
            ap.error("protocol mode needs --" + ", --".join(m.replace("_", "-") for m in missing))
        record = audit_protocol(probe_cache=args.probe_cache, probe_dir=args.probe_dir, model_config=args.model_config,
                                checkpoint=args.checkpoint, device=args.device, codec_name=args.codec)
        args.output.parent.mkdir(parents=True, exist_ok=True)
        temporary = args.output.with_suffix(args.output.suffix + ".tmp")
        temporary.write_text(json.dumps(record, indent=2) + "\n", encoding="utf-8")
        temporary.replace(args.output)
        print(json.dumps({"quality_gate_passed": record["quality_gate_passed"], "tasks": {t["attribute"]: t["passed"] for t in record["tasks"]}}))
        return 0 if record["quality_gate_passed"] else 1
    if not args.results:
        ap.error("give result records, or --probe-dir with --probe-cache, --model-config, --checkpoint and --output")
    failed = False
    for path in args.results:
        errors = audit(path, expect_resumed_from=args.expect_resumed_from, max_validation_examples=args.max_validation_examples,
                       reference_probe=args.reference_probe)
        print(json.dumps({"result": str(path), "ok": not errors, "errors": errors}))
        failed = failed or bool(errors)
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
