#!/usr/bin/env python
"""SynBioS experiment workflow.

    prepare                generate profiles / biographies and tokenise them into training shards
    token-statistics       length, vocabulary and first-token statistics of a generated dataset
    cache-probes           build the memory-mapped probe cache (format 2)
    validate-probe-cache   structural + lineage checks of a cache
    evaluate               teacher-forced attribute recall of a trained model (model.pt)
    cloze-evaluate         progressive greedy cloze generation of attribute values
    summarize-cloze        merge cloze reports into one table
    probe                  train one P / Q probe (resumable)
    validate-probe         re-evaluate a trained probe from its saved weights
    probe-pipeline         schedule all probe jobs over the available devices, then validate them
    summarize-probes       collect probe results into a table
    analyze                router analyses: NMI(attribute, expert), expert load, route Jaccard
    report-formal-study    probe table + cloze table + router report of one study directory
    audit-synbios-repository   lineage audit of dataset / cache / pipeline directories
    oracle-first-token     insert the true first token into the Q inputs and re-read the unchanged Q-whole heads
    ground-truth-first-whole   train one P-whole probe on prefixes extended by the true first token (resumable)
    ground-truth-first-report  table of a ground-truth-first run against the original P probes
    company-relation       exposure-position curve fits of the paired attributes (company / company city)
    probe-batch-benchmark  step time and peak memory of probe steps per batch size, on the longest examples
    summarize-probe-batch-benchmarks   merge benchmark runs of several devices into one recommendation
    compare-formal-studies single vs multi5+permute probe studies: tidy table, headline means, Markdown
    diagnostic-report      oracle and routing evidence of both conditions side by side
    bad-case-routes        experts chosen at the first two value tokens where Q-first is right and Q-whole wrong

The command names of the reference's CLI are accepted as aliases (``validate-probe-oracle-first-token``,
``validate-probe-bad-case-routes``, ``train-ground-truth-first-whole``, ``summarize-ground-truth-first-whole``,
``benchmark-probe-batches``, ``benchmark-ground-truth-first-whole-batches``, ``summarize-probe-benchmarks``,
``report-probe-diagnostics``).

Evaluation and probing always build the model with the library (``torch``) operator back end in fp32 and load only the
exported ``model.pt`` (reference: scripts/synbios_moe.py:141-168), independent of how training was sharded.
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from experiments.synbios_moe.codec import codec_argument  # noqa: E402
from experiments.synbios_moe.pretraining.dataset import ATTRIBUTES, VARIANTS  # noqa: E402


# ---------------------------------------------------------------------------------------------------------
# shared helpers
# ---------------------------------------------------------------------------------------------------------

def load_backbone(model_config: str, checkpoint: str, device: str, *, codec_vocab: int | None = None):
    import torch

    from mini_train_sys_b200.models import MiniTransformer, ModelConfig, get_ops_backend
    from mini_train_sys_b200.runtime.config import load_yaml_dict

    payload = load_yaml_dict(model_config)
    cfg = ModelConfig(**payload.get("model", payload))
    if codec_vocab is not None and codec_vocab > cfg.vocab_size:
        raise ValueError(f"the codec has {codec_vocab} tokens but the model only {cfg.vocab_size}")
    model = MiniTransformer(cfg, get_ops_backend("torch"), activation_dtype=torch.float32)
    state = torch.load(checkpoint, map_location="cpu", weights_only=False)
    state = state.get("model", state) if isinstance(state, dict) else state
    model.load_state_dict(state)
    return model.to(device)


class EventSink:
    """``events.jsonl`` under ``--log-dir`` (the scheduler's heartbeat source) plus optional console lines."""

    def __init__(self, log_dir: str | None, quiet: bool, *, log_interval: int = 1, tensorboard: bool = False) -> None:
        self.quiet = quiet
        self.log_interval = max(int(log_interval or 1), 1)
        self.handle = None
        self.writer = None
        if log_dir:
            Path(log_dir).mkdir(parents=True, exist_ok=True)
            self.handle = open(Path(log_dir) / "events.jsonl", "a", buffering=1)
            if tensorboard:
                try:
                    from torch.utils.tensorboard import SummaryWriter

                    self.writer = SummaryWriter(log_dir=str(log_dir))
                except Exception:       # noqa: BLE001 - event files are an extra; the JSONL log is the record
                    self.writer = None

    @classmethod
    def from_args(cls, args) -> "EventSink":
        return cls(getattr(args, "log_dir", None), getattr(args, "quiet", False), log_interval=getattr(args, "log_interval", 1) or 1,
                   tensorboard=bool(getattr(args, "tensorboard", False)))

    def __call__(self, event: dict) -> None:
        event = {"time": time.time(), **event}
        if self.handle:
            self.handle.write(json.dumps(event, default=str) + "\n")
        step = event.get("step")
        if self.writer is not None and isinstance(step, int):
            for key, value in event.items():
                if key not in ("time", "step") and isinstance(value, (int, float)) and not isinstance(value, bool):
                    self.writer.add_scalar(f"{event.get('event', 'event')}/{key}", value, step)
        # the console shows every log_interval-th progress event (and every event that is not a progress event); the file all
        thin = isinstance(step, int) and self.log_interval > 1 and step % self.log_interval != 0 and step != event.get("steps_total")
        if not self.quiet and not thin:
            print(json.dumps(event, default=str), flush=True)


def _codec(args):
    from experiments.synbios_moe.codec import get_codec

    return get_codec(args.codec)


# ---------------------------------------------------------------------------------------------------------
# handlers
# ---------------------------------------------------------------------------------------------------------

def cmd_prepare(args) -> int:
    from experiments.synbios_moe.pretraining.dataset import write_dataset
    from mini_train_sys_b200.data.documents import CleaningConfig
    from mini_train_sys_b200.data.preprocess import prepare_token_shards

    sink = EventSink.from_args(args)
    out = write_dataset(args.output, num_people=args.num_people, variant=args.variant, seed=args.seed)
    sink({"event": "dataset_written", "path": str(out)})
    if args.codec == "gpt2":
        from mini_train_sys_b200.data.tokenizer import TiktokenTokenizer

        tokenizer = TiktokenTokenizer("gpt2")
    elif args.codec.startswith("bpe:"):
        # a byte-level BPE of the corpus itself: trained on the biographies just written when the directory is new, so
        # that the study has real multi-byte tokens on a machine without the GPT-2 vocabulary
        from experiments.synbios_moe.artifact_io import read_jsonl
        from mini_train_sys_b200.data.tokenizer import ByteLevelBPETokenizer, TOKENIZER_METADATA_FILE

        directory = Path(args.codec[4:])
        if not (directory / TOKENIZER_METADATA_FILE).is_file():
            trained = ByteLevelBPETokenizer.train_from_iterator((row["text"] for row in read_jsonl(out / "biographies.jsonl")),
                                                                vocab_size=args.bpe_vocab_size, min_frequency=2)
            trained.save(directory)
            sink({"event": "tokenizer_trained", "path": str(directory), "vocab_size": trained.vocab_size,
                  "fingerprint": trained.fingerprint})
        tokenizer = ByteLevelBPETokenizer.load(directory)
    else:
        from experiments.synbios_moe.codec import ShardTokenizer, get_codec

        tokenizer = ShardTokenizer(get_codec(args.codec))
    # one document per biography (each starts with the boundary token); nothing is filtered (min_chars=1) and everything
    # trains (validation_fraction=0): the held-out half of the PEOPLE is a probe split, not a language-model validation split
    shards = prepare_token_shards([out / "biographies.jsonl"], output_dir=out / "token_shards", tokenizer=tokenizer,
                                  cleaning=CleaningConfig(min_chars=1, exact_dedup=False), validation_fraction=0.0,
                                  max_shard_tokens=args.max_shard_tokens, split_seed=args.seed)
    sink({"event": "shards_written", "path": str(shards)})
    return 0


def cmd_token_statistics(args) -> int:
    from experiments.synbios_moe.artifact_io import read_jsonl, write_json
    from experiments.synbios_moe.pretraining.token_statistics import dataset_token_statistics

    root = Path(args.data)
    stats = dataset_token_statistics(_codec(args), read_jsonl(root / "biographies.jsonl"), read_jsonl(root / "profiles.jsonl"))
    write_json(args.output, stats)
    if args.distribution_dir:          # the per-attribute value-token distribution with its three tables
        from experiments.synbios_moe.pretraining.token_statistics import attribute_token_distribution

        attribute_token_distribution(_codec(args), read_jsonl(root / "profiles.jsonl"), args.distribution_dir)
    print(json.dumps({k: v for k, v in stats.items() if k != "attributes"}))
    return 0


def cmd_cache_probes(args) -> int:
    from experiments.synbios_moe.probes.dataset import build_probe_cache

    path = build_probe_cache(args.data, args.output, codec_name=args.codec, force=args.force, require_coverage=args.require_coverage)
    print(json.dumps({"probe_cache": str(path)}))
    return 0


def cmd_validate_probe_cache(args) -> int:
    from experiments.synbios_moe.probes.dataset import validate_probe_cache

    verdict = validate_probe_cache(args.probe_cache, args.data)
    print(json.dumps(verdict))
    return 0 if verdict["ok"] else 1


def cmd_evaluate(args) -> int:
    from experiments.synbios_moe.artifact_io import read_jsonl, write_json
    from experiments.synbios_moe.pretraining.attribute_recall import evaluate_attribute_recall

    codec = _codec(args)
    model = load_backbone(args.model_config, args.checkpoint, args.device, codec_vocab=codec.vocab_size)
    report = evaluate_attribute_recall(model, codec, read_jsonl(Path(args.data) / "biographies.jsonl"), device=args.device,
                                       batch_size=args.batch_size, max_items=args.max_items)
    write_json(args.output, report)
    print(json.dumps(report["overall"]))
    return 0


def cmd_cloze(args) -> int:
    from experiments.synbios_moe.artifact_io import read_jsonl, write_json
    from experiments.synbios_moe.pretraining.cloze import evaluate_cloze

    codec = _codec(args)
    model = load_backbone(args.model_config, args.checkpoint, args.device, codec_vocab=codec.vocab_size)
    rows = read_jsonl(Path(args.data) / "biographies.jsonl")
    if getattr(args, "protocol", "independent") == "progressive":
        from experiments.synbios_moe.pretraining.cloze import evaluate_progressive_cloze

        report = evaluate_progressive_cloze(model, codec, rows, device=args.device, batch_size=args.batch_size,
                                            max_biographies=args.examples if args.max_items is None else args.max_items,
                                            start_index=args.start_index, max_new_tokens=args.max_new_tokens,
                                            sample_biographies=args.sample_biographies)
    else:
        report = evaluate_cloze(model, codec, rows, device=args.device, batch_size=args.batch_size, max_items=args.max_items)
    write_json(args.output, report)
    print(json.dumps({"overall_exact_match": report["overall_exact_match"], "items": report["items"]}))
    return 0


def cmd_summarize_cloze(args) -> int:
    from experiments.synbios_moe.artifact_io import read_json, write_csv
    from experiments.synbios_moe.pretraining.cloze import summarize_cloze

    reports = [*args.reports, *args.run]
    if not reports:
        print(json.dumps({"error": "give cloze reports as arguments or with --run"}))
        return 2
    rows = summarize_cloze({Path(p).stem: read_json(p) for p in reports})
    write_csv(args.output, rows, ["run", "attribute", "exact_match", "first_token", "token_accuracy", "items"])
    print(json.dumps({"rows": len(rows), "output": args.output}))
    return 0


def cmd_probe(args) -> int:
    from experiments.synbios_moe.artifact_io import sha256_file
    from experiments.synbios_moe.probes.model import active_parameter_estimate, save_probe_result, train_probe

    sink = EventSink.from_args(args)
    codec = _codec(args)
    model = load_backbone(args.model_config, args.checkpoint, args.device, codec_vocab=codec.vocab_size)
    cache = args.probe_cache or str(Path(args.data) / "probe_cache")
    identity = {"checkpoint_sha256": args.checkpoint_model_sha256 or sha256_file(args.checkpoint), "codec": args.codec}
    result = train_probe(model, cache, kind=args.kind, attribute=args.attribute, target=args.target, steps=args.steps, device=args.device,
                         rank=args.rank, batch_size=args.batch_size, evaluation_batch_size=args.evaluation_batch_size, seed=args.seed,
                         recovery_checkpoint=args.recovery_checkpoint, checkpoint_interval_steps=args.checkpoint_interval_steps,
                         resume=args.resume_probe, evaluate_train=args.evaluate_train, skip_final_validation=args.skip_final_validation,
                         identity=identity, on_event=sink, max_eval_items=args.max_eval_items)
    result["model_parameters"] = active_parameter_estimate(model)
    result["checkpoint"] = str(Path(args.checkpoint).resolve())
    result["checkpoint_bytes"] = Path(args.checkpoint).stat().st_size
    out = Path(args.output)
    save_probe_result(result, out, out.with_suffix(".pt"))
    sink({"event": "probe_done", "output": str(out), "validation": result.get("validation", {}).get("accuracy")})
    return 0


def cmd_validate_probe(args) -> int:
    from experiments.synbios_moe.artifact_io import write_json
    from experiments.synbios_moe.probes.model import validate_saved_probe

    codec = _codec(args)
    model = load_backbone(args.model_config, args.checkpoint, args.device, codec_vocab=codec.vocab_size)
    import torch as _torch

    from experiments.synbios_moe.artifact_io import sha256_file

    trained_on = (_torch.load(args.probe_state, map_location="cpu", weights_only=False).get("identity") or {}).get("checkpoint_sha256")
    if trained_on and not args.allow_checkpoint_mismatch:
        current = args.checkpoint_model_sha256 or sha256_file(args.checkpoint)
        if current != trained_on:
            print(json.dumps({"error": "the probe was trained on another backbone checkpoint (pass --allow-checkpoint-mismatch to evaluate anyway)",
                              "probe_checkpoint_sha256": trained_on, "given_checkpoint_sha256": current}))
            return 3
    verdict = validate_saved_probe(model, args.probe_cache, args.probe_state, device=args.device, batch_size=args.batch_size,
                                   max_items=args.max_eval_items)
    write_json(args.output, verdict)
    if not args.quiet:
        print(json.dumps(verdict["validation"]))
    return 0


def cmd_probe_pipeline(args) -> int:
    """Stages ``smoke`` -> ``pilot`` -> ``formal`` of ``configs/synbios_moe/probe_pipeline.yaml``: a stage needs the marker of
    the stage it ``requires``; an optional cloze gate refuses to probe a model that has not memorised the biographies."""

    import yaml

    from experiments.synbios_moe.artifact_io import read_jsonl, write_json
    from experiments.synbios_moe.probes.commands import all_training_jobs, validation_job
    from experiments.synbios_moe.probes.pipeline import pipeline_identity, run_pipeline
    from experiments.synbios_moe.probes.results import summarize_probe_results

    settings = yaml.safe_load(Path(args.config).read_text()) if args.config else {}
    stage = settings.get("stages", {}).get(args.stage, {})
    runtime = dict(settings.get("runtime", {}))
    # command-line overrides of the pipeline file (the reference's option names)
    if args.num_gpus:
        args.devices = ",".join(f"cuda:{i}" for i in range(args.num_gpus))
    for kind in ("p", "q"):
        if getattr(args, f"{kind}_batch_size"):
            runtime["training_batch_sizes"] = {**runtime.get("training_batch_sizes", {}), kind: getattr(args, f"{kind}_batch_size")}
        if getattr(args, f"{kind}_validation_batch_size"):
            runtime["validation_batch_sizes"] = {**runtime.get("validation_batch_sizes", {}), kind: getattr(args, f"{kind}_validation_batch_size")}
    if args.evaluate_train is not None:
        runtime["evaluate_train"] = bool(args.evaluate_train)
    if args.require_coverage:
        from experiments.synbios_moe.probes.dataset import validate_probe_cache

        from experiments.synbios_moe.artifact_io import read_json

        checked = validate_probe_cache(args.probe_cache, args.data)
        recorded = read_json(Path(args.probe_cache) / "manifest.json").get("coverage", {})
        unseen = {task: c for task, c in recorded.items() if c.get("validation_only_classes")}
        if not checked.get("ok") or unseen:
            print(json.dumps({"error": "the probe cache fails validation, or its validation half has classes the training half never shows",
                              "errors": checked.get("errors", []), "validation_only_classes": unseen}))
            return 3
    steps = args.steps or stage.get("steps", {"smoke": 20, "pilot": 2000, "formal": 30000}[args.stage])
    root = Path(args.output)
    root.mkdir(parents=True, exist_ok=True)
    required = stage.get("requires")
    if required and not args.skip_requirements and not (root.parent / required / "STAGE_OK").is_file():
        print(json.dumps({"error": f"stage {args.stage!r} requires a finished {required!r} stage at {root.parent / required}"}))
        return 3
    gate = settings.get("gate")
    if gate and args.gate_threshold is not None:
        gate = {**gate, "threshold": args.gate_threshold}
    if gate and not args.skip_gate:
        # The gate is the progressive cloze over the original biographies: a model that cannot regenerate the facts it was
        # trained on has nothing for a probe to find.  A gate file of the same checkpoint, data and settings is reused.
        import hashlib

        from experiments.synbios_moe.artifact_io import read_json
        from experiments.synbios_moe.pretraining.cloze import PROGRESSIVE_PROTOCOL, evaluate_progressive_cloze

        wanted = {"checkpoint": str(Path(args.checkpoint).resolve()), "data": str(Path(args.data).resolve()), "codec": args.codec,
                  "examples": int(gate.get("examples", 1000)), "max_new_tokens": int(gate.get("max_new_tokens", 16))}
        wanted["checkpoint_bytes"] = Path(args.checkpoint).stat().st_size
        gate_id = hashlib.sha256(json.dumps(wanted, sort_keys=True).encode()).hexdigest()[:16]
        path = root / "gate.json"
        cached = read_json(path) if path.is_file() else {}
        if (not args.force_gate and cached.get("protocol") == PROGRESSIVE_PROTOCOL and cached.get("identity") == gate_id
                and isinstance(cached.get("exact_match"), (int, float))):
            verdict = {**cached, "reused": True}
        else:
            codec = _codec(args)
            first_device = args.devices.split(",")[0]
            model = load_backbone(args.model_config, args.checkpoint, first_device, codec_vocab=codec.vocab_size)
            report = evaluate_progressive_cloze(model, codec, read_jsonl(Path(args.data) / "biographies.jsonl"), device=first_device,
                                                batch_size=int(gate.get("batch_size", 128)), max_biographies=wanted["examples"],
                                                max_new_tokens=wanted["max_new_tokens"],
                                                sample_biographies=int(gate.get("sample_biographies", 12)))
            verdict = {"protocol": PROGRESSIVE_PROTOCOL, "identity": gate_id, "exact_match": report["micro_field_accuracy"],
                       "all_fields_accuracy": report["biography_all_fields_accuracy"], "biographies": report["biographies"],
                       "items": report["items"], "unterminated_fields": report["unterminated_fields"], "samples": report["samples"], "reused": False}
            del model
        verdict["threshold"] = float(gate.get("threshold", 0.9))
        verdict["passed"] = verdict["exact_match"] >= verdict["threshold"]
        write_json(path, verdict)
        if not verdict["passed"]:
            print(json.dumps({"error": "cloze gate failed", **{k: v for k, v in verdict.items() if k != "samples"}}))
            return 3
    ranks = {"p": args.p_rank, "q": args.q_rank}
    batches = runtime.get("training_batch_sizes", {})
    devices = args.devices.split(",")
    hyper = {"stage": args.stage, "steps": steps, "ranks": ranks, "batches": batches, "seed": args.seed, "codec": args.codec,
             "tasks": stage.get("tasks", "all")}
    identity = pipeline_identity(checkpoint=args.checkpoint, probe_cache=args.probe_cache, model_config=args.model_config, settings=hyper)
    extra = ("--max-eval-items", str(args.max_eval_items)) if args.max_eval_items else ()
    training = all_training_jobs(root, kinds=tuple(args.kinds.split(",")), tasks=stage.get("tasks", "all"), data=args.data,
                                 probe_cache=args.probe_cache, model_config=args.model_config, checkpoint=args.checkpoint, steps=steps,
                                 ranks=ranks, batch_sizes=batches, evaluation_batch_sizes=runtime.get("validation_batch_sizes", {}),
                                 evaluate_train=bool(runtime.get("evaluate_train", False)), seed=args.seed,
                                 checkpoint_interval_steps=args.checkpoint_interval_steps or runtime.get("checkpoint_interval_steps"),
                                 codec=args.codec, extra=extra)
    if args.attributes:
        keep = set(args.attributes.split(","))
        training = [j for j in training if j.metadata["attribute"] in keep]
    validation = [validation_job(root, j, data=args.data, probe_cache=args.probe_cache, model_config=args.model_config,
                                 checkpoint=args.checkpoint, codec=args.codec) for j in training]
    heartbeat = args.heartbeat_seconds or float(runtime.get("heartbeat_seconds", 30))
    estimates = {}
    if required and (root.parent / required / "pipeline.json").is_file():      # how long will this stage take, judging by the last one
        from experiments.synbios_moe.artifact_io import read_json
        from experiments.synbios_moe.probes.pipeline import estimate_phase_durations

        estimates = estimate_phase_durations(read_json(root.parent / required / "pipeline.json"), [*training, *validation],
                                             steps=steps if isinstance(steps, int) else 0, device_count=len(devices))
        if estimates and not args.quiet:
            print(json.dumps({"estimated_phase_seconds": estimates, "from_stage": required}), flush=True)
    summary = run_pipeline(root, training, validation, devices=devices, identity=identity, heartbeat_seconds=heartbeat,
                           settings={"stage": args.stage, "steps": steps, "devices": len(devices)}, estimates=estimates,
                           on_heartbeat=None if args.quiet else (lambda name, ev: print(json.dumps({"job": name, "last_event": ev}), flush=True)))
    if estimates:
        summary["estimated_phase_seconds"] = estimates
    summary["results"] = summarize_probe_results(root)["mean_accuracy"]
    if summary["ok"]:
        (root / "STAGE_OK").write_text(identity + "\n")
    print(json.dumps(summary, default=str))
    return 0 if summary["ok"] else 1


def cmd_summarize_probes(args) -> int:
    from experiments.synbios_moe.artifact_io import write_csv
    from experiments.synbios_moe.probes.results import summarize_probe_results

    if args.run:
        # the reference's form: NAME=DIRECTORY per study; the tables of all of them go into one file with a `run` column
        rows, means = [], {}
        for value in args.run:
            name, _, path = value.partition("=")
            if not name or not path:
                print(json.dumps({"error": "--run must use NAME=DIRECTORY"}))
                return 2
            one = summarize_probe_results(path[:-len("/validation")] if path.rstrip("/").endswith("/validation") else path)
            rows += [{"run": name, **row} for row in one["rows"]]
            means[name] = one.get("mean_accuracy")
        if args.output:
            write_csv(args.output, rows)
        print(json.dumps({"runs": list(means), "rows": len(rows), "mean_accuracy": means}))
        return 0
    if not args.root:
        print(json.dumps({"error": "give a pipeline stage directory, or --run NAME=DIRECTORY"}))
        return 2
    summary = summarize_probe_results(args.root)
    if args.output:
        write_csv(args.output, summary["rows"])
    print(json.dumps({k: v for k, v in summary.items() if k != "rows"}))
    return 0


def cmd_analyze(args) -> int:
    from experiments.synbios_moe.artifact_io import read_jsonl, write_json
    from experiments.synbios_moe.mechanisms.token_routes import collect_token_routes, route_report

    codec = _codec(args)
    model = load_backbone(args.model_config, args.checkpoint, args.device, codec_vocab=codec.vocab_size)
    if not model.cfg.is_moe:
        print(json.dumps({"error": "router analyses need an MoE model"}))
        return 2
    collected = collect_token_routes(model, codec, read_jsonl(Path(args.data) / "biographies.jsonl"), device=args.device,
                                     max_items=args.max_items or 256)
    report = route_report(collected, model.cfg.num_experts)
    write_json(args.output, {str(k): v for k, v in report.items()})
    print(json.dumps({str(k): v["nmi_attribute_expert"] for k, v in report.items()}))
    return 0


def cmd_report(args) -> int:
    from experiments.synbios_moe.artifact_io import read_json, write_json
    from experiments.synbios_moe.probes.results import summarize_probe_results

    if args.single and args.multi:
        from experiments.synbios_moe.probes.comparison_report import build_formal_report_artifacts

        caches = {}
        for side, root_dir, given in (("single", args.single, args.single_cache), ("multi", args.multi, args.multi_cache)):
            caches[side] = Path(given) if given else Path(root_dir).resolve().parent / "cache"
            if not (caches[side] / "manifest.json").is_file():
                print(json.dumps({"error": f"no probe cache at {caches[side]}: pass --{side}-cache"}))
                return 2
        out = build_formal_report_artifacts(args.single, args.multi, args.output, single_cache=caches["single"], multi_cache=caches["multi"])
        cloze = {name: read_json(path) for name, path in (("single", args.single_cloze), ("multi5_permute", args.multi_cloze)) if path and Path(path).is_file()}
        if cloze:
            write_json(Path(args.output) / "cloze_gate.json", {k: {f: v.get(f) for f in ("micro_field_accuracy", "biography_all_fields_accuracy", "overall_exact_match", "biographies", "items") if f in v}
                                                               for k, v in cloze.items()})
        print(json.dumps({"status": "completed", "output": out["output"], "headline_metrics": out["headline"]["delta_multi_minus_single"]}))
        return 0
    if not args.root:
        print(json.dumps({"error": "give a study directory, or --single and --multi5-permute (two finished formal stages)"}))
        return 2
    root = Path(args.root)
    report = {"probes": summarize_probe_results(root / "probes") if (root / "probes" / "training").is_dir() else None}
    for name in ("cloze", "recall", "routes", "token_statistics"):
        path = root / f"{name}.json"
        report[name] = read_json(path) if path.is_file() else None
    write_json(args.output, report)
    print(json.dumps({k: v is not None for k, v in report.items()}))
    return 0


def cmd_audit(args) -> int:
    from experiments.synbios_moe.audit import audit_study, build_study_audit

    if args.single_data or args.multi_data:     # both conditions of the comparison: lineage files + summary under --output
        spec = {"single": {"data": args.single_data, "probe_cache": args.single_cache, "pipeline": args.single_pipeline, "model": args.single_model},
                "multi5_permute": {"data": args.multi_data, "probe_cache": args.multi_cache, "pipeline": args.multi_pipeline,
                                   "model": args.multi_model}}
        try:
            summary = build_study_audit(spec, args.output or "audit")
        except (ValueError, OSError, KeyError) as exc:
            print(json.dumps({"status": "failed", "error": str(exc)}))
            return 1
        print(json.dumps({"status": summary["status"], "checks": len(summary["checks"])}))
        return 0
    verdict = audit_study(data_root=args.data, probe_cache=args.probe_cache, pipeline_root=args.pipeline)
    print(json.dumps(verdict, indent=1))
    return 0 if verdict["ok"] else 1


def cmd_oracle_first_token(args) -> int:
    from experiments.synbios_moe.mechanisms.oracle_first_token import oracle_first_token_validation

    codec = _codec(args)
    sink = EventSink.from_args(args)
    model = load_backbone(args.model_config, args.checkpoint, args.device, codec_vocab=codec.vocab_size)
    attributes = tuple(args.attributes.split(",")) if args.attributes else (tuple(args.attribute) if getattr(args, "attribute", None) else None)
    kwargs = {"attributes": attributes} if attributes else {}
    summary = oracle_first_token_validation(model, data_root=args.data, cache_root=args.probe_cache, probe_dir=args.probe_dir,
                                            output_dir=args.output, device=args.device, batch_size=args.batch_size,
                                            max_examples=args.max_examples,
                                            progress=lambda name, done: sink({"event": "oracle_progress", "attribute": name, "done": done}),
                                            **kwargs)
    print(json.dumps(summary["overall"]))
    return 0


def cmd_bad_case_routes(args) -> int:
    from experiments.synbios_moe.mechanisms.token_routes import bad_case_route_validation

    codec = _codec(args)
    sink = EventSink.from_args(args)
    model = load_backbone(args.model_config, args.checkpoint, args.device, codec_vocab=codec.vocab_size)
    attributes = tuple(args.attributes.split(",")) if args.attributes else (tuple(args.attribute) if getattr(args, "attribute", None) else None)
    summary = bad_case_route_validation(model, codec, data_root=args.data, cache_root=args.probe_cache, probe_dir=args.probe_dir,
                                        output_dir=args.output, device=args.device, attributes=attributes,
                                        batch_size=args.batch_size, max_examples=args.max_examples, pair_limit=args.pair_limit,
                                        progress=lambda name, done: sink({"event": "route_progress", "attribute": name, "done": done}))
    print(json.dumps({k: summary[k] for k in ("protocol", "examples", "attributes", "layers")}))
    return 0


def cmd_ground_truth_first_whole(args) -> int:
    from experiments.synbios_moe.artifact_io import write_json
    from experiments.synbios_moe.mechanisms.first_token_intervention import train_ground_truth_first_whole_probe
    from experiments.synbios_moe.probes.model import _atomic_torch_save, CHECKPOINT_VERSION

    codec = _codec(args)
    sink = EventSink.from_args(args)
    model = load_backbone(args.model_config, args.checkpoint, args.device, codec_vocab=codec.vocab_size)
    result = train_ground_truth_first_whole_probe(
        model, cache_root=args.probe_cache, probe_dir=args.probe_dir, attribute=args.attribute, codec=codec, device=args.device,
        batch_size=args.batch_size, evaluation_batch_size=args.evaluation_batch_size, steps=args.steps, seed=args.seed,
        recovery_checkpoint=args.recovery_checkpoint, checkpoint_interval_steps=args.checkpoint_interval_steps,
        resume=args.resume_probe, max_validation_examples=args.max_validation_examples, on_event=sink)
    out = Path(args.output)
    state = result.pop("probe_state")
    _atomic_torch_save({"version": CHECKPOINT_VERSION, "identity": result["identity"], "probe": state}, out.with_suffix(".pt"))
    write_json(out, result)          # the marker is written last
    print(json.dumps({"attribute": args.attribute, "accuracy_by_position": result["whole_accuracy_validation_by_source_position"]}))
    return 0


def cmd_ground_truth_first_report(args) -> int:
    from experiments.synbios_moe.mechanisms.intervention_report import summarize_ground_truth_first_whole

    summary = summarize_ground_truth_first_whole(args.run_dir, args.probe_dir, args.output)
    print(json.dumps({k: summary[k] for k in ("attributes_reported", "attributes_missing", "mean_gain_points")}))
    return 0


def cmd_company_relation(args) -> int:
    from experiments.synbios_moe.mechanisms.company_relation import fit_company_pair, load_position_curves

    summary = fit_company_pair(load_position_curves(args.input_csv, condition=args.condition), args.output)
    print(json.dumps({k: summary[k] for k in ("pair_mean_gain", "unpaired_max_gain")}))
    return 0


def cmd_probe_batch_benchmark(args) -> int:
    from experiments.synbios_moe.artifact_io import write_json
    from experiments.synbios_moe.probes.batch_benchmark import benchmark_probe_batches, parse_batch_sizes
    from experiments.synbios_moe.probes.dataset import CachedProbeDataset
    from experiments.synbios_moe.probes.model import DEFAULT_RANK

    codec = _codec(args)
    sink = EventSink.from_args(args)
    model = load_backbone(args.model_config, args.checkpoint, args.device, codec_vocab=codec.vocab_size)
    runs = []
    if args.kind:
        args.kinds = args.kind
        if args.batch_sizes:
            setattr(args, f"{args.kind}_batch_sizes", args.batch_sizes)
    for kind in args.kinds.split(","):
        split = "train" if args.mode == "training" else "validation"
        data = CachedProbeDataset(args.probe_cache, kind=kind, attribute=args.attribute, target=args.target, split=split)
        if args.ground_truth_first:
            if kind != "p":
                continue
            from experiments.synbios_moe.mechanisms.first_token_intervention import prepare_ground_truth_first_whole_data

            prepared = prepare_ground_truth_first_whole_data(cache_root=args.probe_cache, probe_dir=args.probe_dir,
                                                             attribute=args.attribute, codec=codec)
            data = prepared.train_data if args.mode == "training" else prepared.validation_data
        sizes = parse_batch_sizes(args.p_batch_sizes if kind == "p" else args.q_batch_sizes)
        sizes = tuple(s for s in sizes if s <= len(data)) or (min(len(data), sizes[0]),)
        runs.append(benchmark_probe_batches(
            model, data, kind=kind, num_classes=len(data.class_names), rank=args.rank or DEFAULT_RANK[kind], batch_sizes=sizes,
            device=args.device, mode=args.mode, warmup_steps=args.warmup_steps, measure_steps=args.measure_steps,
            memory_limit_percent=args.memory_limit_percent, on_result=lambda rec, k=kind: sink({"event": "probe_batch", "kind": k, **rec})))
    write_json(args.output, {"attribute": args.attribute, "target": args.target, "ground_truth_first": bool(args.ground_truth_first),
                             "benchmarks": runs})
    print(json.dumps({r["kind"]: r["recommended_capacity_batch_size"] for r in runs}))
    return 0


def cmd_summarize_probe_batch_benchmarks(args) -> int:
    from experiments.synbios_moe.artifact_io import write_json
    from experiments.synbios_moe.probes.batch_benchmark import summarize_probe_benchmarks

    summary = summarize_probe_benchmarks([*args.results, *(args.run or [])])
    write_json(args.output, summary)
    print(json.dumps({**{k: v["recommended_batch_size"] for k, v in summary["recommendations"].items()},
                      "ready_for_formal": summary["completeness"]["ready_for_formal"]}))
    if args.env_output:
        from experiments.synbios_moe.artifact_io import write_text
        from experiments.synbios_moe.probes.batch_benchmark import probe_batch_environment

        write_text(args.env_output, probe_batch_environment(summary))          # raises unless the benchmark is complete
    if args.require_complete_search and not summary["completeness"]["ready_for_formal"]:
        print(json.dumps({"error": "benchmark incomplete", **summary["completeness"]}), file=sys.stderr)
        return 2
    return 0


def cmd_compare_formal_studies(args) -> int:
    from experiments.synbios_moe.probes.comparison_report import build_formal_report_artifacts

    out = build_formal_report_artifacts(args.single, args.multi, args.output, single_cache=args.single_cache, multi_cache=args.multi_cache)
    print(json.dumps(out["headline"]["delta_multi_minus_single"]))
    return 0


def cmd_diagnostic_report(args) -> int:
    from experiments.synbios_moe.mechanisms.comparison_report import build_diagnostic_report_artifacts

    single, multi = args.single, args.multi
    if args.diagnostics and not (single and multi):          # the reference's form: one root, a directory per condition
        single, multi = str(Path(args.diagnostics) / "single"), str(Path(args.diagnostics) / "multi5_permute")
    if not (single and multi):
        print(json.dumps({"error": "give --single and --multi (diagnostics directories), or --diagnostics with single/ and multi5_permute/ inside"}))
        return 2
    result = build_diagnostic_report_artifacts({"single": single, "multi5_permute": multi}, args.output)
    if args.single_formal or args.multi_formal:
        result["formal_stages"] = {"single": args.single_formal, "multi5_permute": args.multi_formal}
    print(json.dumps(result))
    return 0


# ---------------------------------------------------------------------------------------------------------
# argument tree
# ---------------------------------------------------------------------------------------------------------

def build_parser() -> argparse.ArgumentParser:
    import torch

    default_device = "cuda" if torch.cuda.is_available() else "cpu"
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)

    def common(p, *, model=True, monitoring=True):
        p.add_argument("--codec", type=codec_argument, default="gpt2", metavar="{gpt2,bytes,bpe:<tokenizer directory>}")
        if model:
            p.add_argument("--model-config", required=True)
            p.add_argument("--checkpoint", required=True, help="exported model.pt")
            p.add_argument("--device", default=default_device)
        if monitoring:
            p.add_argument("--log-dir")
            p.add_argument("--quiet", action="store_true")
            p.add_argument("--log-interval", type=int, default=1, help="console: show every N-th progress event (the event file keeps all)")
            p.add_argument("--tensorboard", action=argparse.BooleanOptionalAction, default=False,
                           help="also write numeric event fields as TensorBoard scalars under --log-dir")

    p = sub.add_parser("prepare"); common(p, model=False)
    p.add_argument("--output", required=True); p.add_argument("--variant", default="single", choices=VARIANTS)
    p.add_argument("--num-people", type=int, default=100_000); p.add_argument("--seed", type=int, default=1337)
    p.add_argument("--max-shard-tokens", type=int, default=10_000_000); p.set_defaults(func=cmd_prepare)
    p.add_argument("--bpe-vocab-size", type=int, default=8192, help="with --codec bpe:<dir>, when <dir> holds no tokenizer yet: train one of this size")

    p = sub.add_parser("token-statistics"); common(p, model=False, monitoring=False)
    p.add_argument("--data", required=True); p.add_argument("--output", required=True)
    p.add_argument("--distribution-dir", help="also write the value-token distribution per attribute (summary.json and three CSV tables)")
    p.set_defaults(func=cmd_token_statistics)

    p = sub.add_parser("cache-probes"); common(p, model=False, monitoring=False)
    p.add_argument("--data", required=True); p.add_argument("--output", required=True); p.add_argument("--force", action="store_true")
    p.add_argument("--require-coverage", action="store_true"); p.set_defaults(func=cmd_cache_probes)

    p = sub.add_parser("validate-probe-cache"); p.add_argument("--probe-cache", required=True); p.add_argument("--data")
    p.set_defaults(func=cmd_validate_probe_cache)

    for name, fn in (("evaluate", cmd_evaluate), ("cloze-evaluate", cmd_cloze), ("analyze", cmd_analyze)):
        p = sub.add_parser(name); common(p)
        p.add_argument("--data", required=True); p.add_argument("--output", required=True)
        p.add_argument("--batch-size", type=int, default=32); p.add_argument("--max-items", type=int); p.set_defaults(func=fn)
        if name != "cloze-evaluate":
            p.add_argument("--examples", type=int, dest="max_items", help="same as --max-items (the reference's name)")
        if name == "analyze":
            # the reference analyses one probe task per call; here every attribute is analysed in one pass and these select nothing
            p.add_argument("--attribute", choices=ATTRIBUTES); p.add_argument("--target", choices=("first", "whole"), default="first")
            p.add_argument("--probe-cache")
        if name == "cloze-evaluate":
            # independent: every value from its true prefix, fixed length; progressive: the six holes of a biography filled left
            # to right in one growing sequence, each value generated until the source's next full stop
            p.add_argument("--protocol", choices=("independent", "progressive"), default="independent")
            p.add_argument("--examples", type=int, default=1000); p.add_argument("--start-index", type=int, default=0)
            p.add_argument("--max-new-tokens", type=int, default=16); p.add_argument("--sample-biographies", type=int, default=12)

    p = sub.add_parser("summarize-cloze"); p.add_argument("reports", nargs="*"); p.add_argument("--output", required=True)
    p.add_argument("--run", action="append", default=[], help="a cloze report (repeatable; same as a positional argument)")
    p.set_defaults(func=cmd_summarize_cloze)

    p = sub.add_parser("probe"); common(p)
    p.add_argument("--data", required=True); p.add_argument("--probe-cache"); p.add_argument("--output", required=True)
    p.add_argument("--attribute", choices=ATTRIBUTES, required=True); p.add_argument("--target", choices=("first", "whole"), default="first")
    p.add_argument("--kind", choices=("p", "q"), required=True); p.add_argument("--rank", type=int)
    p.add_argument("--checkpoint-model-sha256", help=argparse.SUPPRESS)
    p.add_argument("--batch-size", type=int); p.add_argument("--evaluation-batch-size", type=int)
    p.add_argument("--steps", type=int, default=30_000); p.add_argument("--seed", type=int, default=1337)
    p.add_argument("--recovery-checkpoint"); p.add_argument("--checkpoint-interval-steps", type=int)
    p.add_argument("--resume-probe", action=argparse.BooleanOptionalAction, default=True)
    p.add_argument("--evaluate-train", action="store_true"); p.add_argument("--skip-final-validation", action="store_true")
    p.add_argument("--max-eval-items", type=int); p.set_defaults(func=cmd_probe)

    p = sub.add_parser("validate-probe"); common(p)
    p.add_argument("--probe-cache", required=True); p.add_argument("--probe-state", "--probe-checkpoint", dest="probe_state", required=True)
    p.add_argument("--output", required=True); p.add_argument("--data", help="accepted for the reference's command lines; the cache names its dataset")
    p.add_argument("--batch-size", type=int, default=200); p.add_argument("--checkpoint-model-sha256", help=argparse.SUPPRESS)
    p.add_argument("--allow-checkpoint-mismatch", action="store_true", help="evaluate although the probe was trained on another backbone checkpoint")
    p.add_argument("--max-eval-items", type=int); p.set_defaults(func=cmd_validate_probe)

    p = sub.add_parser("probe-pipeline"); common(p)
    p.add_argument("--data", required=True); p.add_argument("--probe-cache", required=True); p.add_argument("--output", required=True)
    p.add_argument("--stage", choices=("smoke", "pilot", "formal"), required=True); p.add_argument("--config", "--pipeline-config", dest="config")
    p.add_argument("--num-gpus", type=int, help="use cuda:0 .. cuda:N-1 (instead of --devices)")
    p.add_argument("--gate-threshold", type=float, help="override the cloze gate's threshold"); p.add_argument("--force-gate", action="store_true", help="run the cloze gate again although a cached verdict matches")
    p.add_argument("--require-coverage", action="store_true", help="refuse a probe cache whose validation half lacks a class")
    p.add_argument("--quiet-workers", action="store_true", help="accepted: workers always log to files here")
    for kind in ("p", "q"):
        p.add_argument(f"--{kind}-batch-size", type=int); p.add_argument(f"--{kind}-validation-batch-size", type=int)
    p.add_argument("--evaluate-train", action=argparse.BooleanOptionalAction, default=None)
    p.add_argument("--devices", default=default_device); p.add_argument("--kinds", default="p,q"); p.add_argument("--attributes")
    p.add_argument("--steps", type=int); p.add_argument("--seed", type=int, default=1337)
    p.add_argument("--checkpoint-interval-steps", type=int); p.add_argument("--heartbeat-seconds", type=float)
    p.add_argument("--p-rank", type=int); p.add_argument("--q-rank", type=int)
    p.add_argument("--skip-gate", action="store_true"); p.add_argument("--skip-requirements", "--ignore-prerequisite", dest="skip_requirements", action="store_true")
    p.add_argument("--max-eval-items", type=int); p.set_defaults(func=cmd_probe_pipeline)

    p = sub.add_parser("summarize-probes"); p.add_argument("root", nargs="?"); p.add_argument("--output"); p.set_defaults(func=cmd_summarize_probes)
    p.add_argument("--run", action="append", default=[], help="NAME=DIRECTORY of a finished pipeline stage (repeatable; the reference's form)")
    p = sub.add_parser("report-formal-study"); p.add_argument("root", nargs="?"); p.add_argument("--output", required=True); p.set_defaults(func=cmd_report)
    # the reference's form: two finished formal stages (and their cloze reports) -> the comparison artifacts of compare-formal-studies
    p.add_argument("--single"); p.add_argument("--multi5-permute", dest="multi"); p.add_argument("--single-cloze"); p.add_argument("--multi5-permute-cloze", dest="multi_cloze")
    p.add_argument("--single-cache", help="default: <single>/../cache"); p.add_argument("--multi-cache", help="default: <multi5-permute>/../cache")
    p = sub.add_parser("audit-synbios-repository"); p.add_argument("--data"); p.add_argument("--probe-cache"); p.add_argument("--pipeline")
    for side in ("single", "multi"):
        for what in ("data", "cache", "pipeline", "model"):
            p.add_argument(f"--{side}-{what}")
    p.add_argument("--repo-root", default=".", help="accepted for the reference's command lines; paths here are given explicitly")
    p.add_argument("--output"); p.set_defaults(func=cmd_audit)

    p = sub.add_parser("oracle-first-token", aliases=["validate-probe-oracle-first-token"]); common(p)
    p.add_argument("--data", required=True); p.add_argument("--probe-cache", required=True); p.add_argument("--probe-dir", required=True)
    p.add_argument("--output", required=True); p.add_argument("--attributes"); p.add_argument("--batch-size", type=int, default=256)
    p.add_argument("--attribute", action="append", choices=ATTRIBUTES, help="one attribute (repeatable; the reference's form of --attributes)")
    p.add_argument("--max-examples", type=int); p.set_defaults(func=cmd_oracle_first_token)

    p = sub.add_parser("ground-truth-first-whole", aliases=["train-ground-truth-first-whole"]); common(p)
    p.add_argument("--probe-cache", required=True); p.add_argument("--probe-dir", required=True); p.add_argument("--output", required=True)
    p.add_argument("--attribute", required=True); p.add_argument("--steps", type=int, default=3000); p.add_argument("--seed", type=int, default=1337)
    p.add_argument("--batch-size", type=int, default=50); p.add_argument("--evaluation-batch-size", type=int, default=256)
    p.add_argument("--recovery-checkpoint"); p.add_argument("--checkpoint-interval-steps", type=int)
    p.add_argument("--resume-probe", action=argparse.BooleanOptionalAction, default=True)
    p.add_argument("--data", help="accepted for the reference's command lines; the cache names its dataset")
    p.add_argument("--evaluate-train", action="store_true", help="accepted: the report of this command is validation accuracy by source position")
    p.add_argument("--max-validation-examples", type=int); p.set_defaults(func=cmd_ground_truth_first_whole)

    p = sub.add_parser("ground-truth-first-report", aliases=["summarize-ground-truth-first-whole"]); p.add_argument("--run-dir", "--run", dest="run_dir", required=True); p.add_argument("--probe-dir", required=True)
    p.add_argument("--output"); p.set_defaults(func=cmd_ground_truth_first_report)

    p = sub.add_parser("company-relation"); p.add_argument("--input-csv", required=True); p.add_argument("--output", required=True)
    p.add_argument("--condition", default="multi5_permute"); p.set_defaults(func=cmd_company_relation)

    for name, aliases, gtf in (("probe-batch-benchmark", ["benchmark-probe-batches"], False),
                               ("benchmark-ground-truth-first-whole-batches", [], True)):
        p = sub.add_parser(name, aliases=aliases); common(p)
        p.add_argument("--probe-cache", required=True); p.add_argument("--output", required=True); p.add_argument("--probe-dir")
        p.add_argument("--attribute", default="university"); p.add_argument("--target", choices=("first", "whole"), default="whole")
        p.add_argument("--kinds", default="p" if gtf else "p,q"); p.add_argument("--mode", choices=("training", "validation"), default="training")
        p.add_argument("--p-batch-sizes", default="25,50,100,200"); p.add_argument("--q-batch-sizes", default="100,200,400,800")
        p.add_argument("--rank", type=int); p.add_argument("--warmup-steps", type=int, default=3); p.add_argument("--measure-steps", type=int, default=10)
        p.add_argument("--memory-limit-percent", type=float, default=92.0)
        p.add_argument("--ground-truth-first", action=argparse.BooleanOptionalAction, default=gtf)
        p.add_argument("--data", help="accepted for the reference's command lines; the cache names its dataset")
        p.add_argument("--kind", choices=("p", "q"), help="one probe kind (the reference's form of --kinds)")
        p.add_argument("--batch-sizes", help="candidates for --kind (the reference's form of --p-batch-sizes / --q-batch-sizes)")
        p.set_defaults(func=cmd_probe_batch_benchmark)

    p = sub.add_parser("bad-case-routes", aliases=["validate-probe-bad-case-routes"]); common(p)
    p.add_argument("--data", required=True); p.add_argument("--probe-cache", required=True); p.add_argument("--probe-dir", required=True)
    p.add_argument("--output", required=True); p.add_argument("--attributes"); p.add_argument("--batch-size", type=int, default=512)
    p.add_argument("--attribute", action="append", choices=ATTRIBUTES, help="one attribute (repeatable; the reference's form of --attributes)")
    p.add_argument("--max-examples", type=int); p.add_argument("--pair-limit", type=int, default=2000)
    p.set_defaults(func=cmd_bad_case_routes)

    p = sub.add_parser("summarize-probe-batch-benchmarks", aliases=["summarize-probe-benchmarks"]); p.add_argument("results", nargs="*")
    p.add_argument("--run", action="append", help="a benchmark result (repeatable; same as a positional argument)")
    p.add_argument("--output", required=True); p.add_argument("--env-output", help="write sourceable export lines of the recommended batch sizes")
    p.add_argument("--require-complete-search", action="store_true", help="exit 2 unless every kind / mode was measured twice and bracketed")
    p.set_defaults(func=cmd_summarize_probe_batch_benchmarks)

    p = sub.add_parser("compare-formal-studies"); p.add_argument("--single", required=True); p.add_argument("--multi", required=True)
    p.add_argument("--single-cache", required=True); p.add_argument("--multi-cache", required=True); p.add_argument("--output", required=True)
    p.set_defaults(func=cmd_compare_formal_studies)

    p = sub.add_parser("diagnostic-report", aliases=["report-probe-diagnostics"]); p.add_argument("--single"); p.add_argument("--multi")
    # the reference's form: one diagnostics root with a directory per condition, and the two formal stages (recorded in the report)
    p.add_argument("--diagnostics"); p.add_argument("--single-formal"); p.add_argument("--multi5-permute-formal", dest="multi_formal")
    p.add_argument("--output", required=True); p.set_defaults(func=cmd_diagnostic_report)
    return ap


def exported_model_file(checkpoint: str) -> str:
    """``--checkpoint`` names an exported ``model.pt`` or, as in the reference's launchers, a committed checkpoint directory
    (``latest`` inside a run directory picks its newest committed one); the directory form resolves to the export inside it."""

    path = Path(checkpoint)
    if path.name == "latest" and not path.exists():
        committed = sorted(d.parent for d in path.parent.glob("*/COMMITTED"))
        if not committed:
            raise SystemExit(f"no committed checkpoint under {path.parent}")
        path = committed[-1]
    if path.is_dir():
        if not (path / "COMMITTED").exists():
            raise SystemExit(f"{path} is not a committed checkpoint")
        if not (path / "model.pt").exists():
            raise SystemExit(f"{path} holds no model export (a checkpoint saved inside an epoch): use one saved at the end of an epoch")
        path = path / "model.pt"
    return str(path)


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if isinstance(getattr(args, "checkpoint", None), str) and (Path(args.checkpoint).is_dir() or Path(args.checkpoint).name == "latest"):
        args.checkpoint = exported_model_file(args.checkpoint)
    return int(args.func(args) or 0)


if __name__ == "__main__":
    raise SystemExit(main())
