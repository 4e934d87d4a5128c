#!/usr/bin/env python
"""Distributed training benchmark CLI.

    python scripts/run_dist_bench.py inventory
    python scripts/run_dist_bench.py validate-backend
    python scripts/run_dist_bench.py run --suite weak --config configs/bench/synbios_moe_fsdp.yaml --world-sizes 1,2,4,8
    python scripts/run_dist_bench.py run --suite capacity --batch-sizes 32,64,96,128,192
    python scripts/run_dist_bench.py run --suite backend --ops-backends torch,native
    python scripts/run_dist_bench.py present-weak | present-capacity | present-backend  <output dir>

Sub-commands and result layout follow the reference's ``scripts/run_dist_bench.py`` (``_worker``, ``inventory``,
``run --suite``, ``present-backend``, ``present-capacity``, ``validate-backend``).
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

DEFAULT_CONFIG = "configs/bench/synbios_moe_fsdp.yaml"


def _ints(text: str) -> tuple[int, ...]:
    return tuple(int(t) for t in text.split(",") if t)




def _strs(text: str) -> tuple[str, ...]:
    return tuple(t for t in text.split(",") if t)


class _Flatten(argparse.Action):
    """List options take both spellings: ``--world-sizes 1,2,4`` (one comma-separated value) and the reference's
    ``--world-sizes 1 2 4`` (several values)."""

    def __call__(self, parser, namespace, values, option_string=None):
        flat = tuple(item for value in values for item in (value if isinstance(value, tuple) else (value,)))
        setattr(namespace, self.dest, "auto" if flat == ("auto",) else flat)


def _batch_list(text: str) -> tuple:
    return ("auto",) if text.strip() == "auto" else _ints(text)


def _parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)
    w = sub.add_parser("_worker")
    w.add_argument("--config", required=True)
    w.add_argument("--model-config", default=None)
    w.add_argument("--strategy", default="fsdp")
    w.add_argument("--ops", default="native")
    w.add_argument("--engine", default="fused")
    w.add_argument("--batch-size", type=int, required=True)
    w.add_argument("--warmup-steps", type=int, default=5)
    w.add_argument("--measure-steps", type=int, default=20)
    w.add_argument("--output", default=None)
    inv = sub.add_parser("inventory")
    inv.add_argument("--output", help="directory that receives inventory.json (default: print only)")
    vb = sub.add_parser("validate-backend")
    vb.add_argument("--device", default="cuda:0"); vb.add_argument("--batch-size", type=int, default=2)
    vb.add_argument("--sequence-length", type=int, default=512); vb.add_argument("--output", help="also write the verdict as JSON")
    r = sub.add_parser("run")
    r.add_argument("--suite", choices=("weak", "capacity", "backend"), required=True)
    r.add_argument("--config", "--case-config", dest="config", default=DEFAULT_CONFIG)
    r.add_argument("--model-config", default=None)
    r.add_argument("--output-dir", "--output", dest="output_dir", default="results/distributed")
    r.add_argument("--strategies", nargs="+", type=_strs, action=_Flatten, default=("fsdp",))
    r.add_argument("--world-sizes", nargs="+", type=_ints, action=_Flatten, default=(1, 2, 4, 8))
    r.add_argument("--ops-backends", nargs="+", type=_strs, action=_Flatten, default=("native",))
    r.add_argument("--engines", nargs="+", type=_strs, action=_Flatten, default=("fused",))
    r.add_argument("--batch-sizes", nargs="+", type=_batch_list, action=_Flatten, default=(96,), help="local batch sizes (comma- or "
                   "space-separated), or `auto`: fractions of the largest batch the memory plan admits for every case of the sweep "
                   "(see docs/memory_planning.md)")
    r.add_argument("--local-batch", type=int, help="weak and backend suites: the one local batch size (the reference's option)")
    r.add_argument("--device-gb", type=float, default=180.0, help="device memory in GiB for `--batch-sizes auto`")
    r.add_argument("--repeats", type=int, default=2)
    r.add_argument("--warmup-steps", type=int, default=5)
    r.add_argument("--measure-steps", type=int, default=20)
    r.add_argument("--timeout", "--case-timeout-seconds", dest="timeout", type=float, default=1800.0, help="limit per case (seconds)")
    r.add_argument("--rerun-existing", action="store_true", help="measure every case again although a stored result has the same identity")
    r.add_argument("--memory-limit-percent", type=float, default=92.0, help="capacity suite: share of device memory a candidate batch may reserve")
    r.add_argument("--min-repeats", type=int, default=2, help="capacity and backend suites: repeats a row needs to count")
    r.add_argument("--master-port", type=int, default=29541)
    r.add_argument("--reuse-stale-results", action="store_true")
    r.add_argument("--reuse-failures", action="store_true")
    for name in ("present-weak", "present-capacity", "present-backend"):
        p = sub.add_parser(name)
        p.add_argument("output_dir", nargs="?", default="results/distributed")
        p.add_argument("--input", help="a suite's summary.json or its directory (the reference's option; instead of the positional root)")
        p.add_argument("--output", help="also write the table and the gates to this file")
        if name == "present-capacity":
            p.add_argument("--memory-limit-percent", type=float); p.add_argument("--min-repeats", type=int)
            p.add_argument("--require-batch-one", action="store_true", help="refuse a sweep that did not measure local batch 1")
        if name == "present-backend":
            p.add_argument("--validation", help="verdict file of validate-backend: presenting requires that it passed")
    return ap


def _table(rows: list[dict], cols: list[str]) -> str:
    fmt = lambda v: "" if v is None else f"{v:,.4g}" if isinstance(v, float) else str(v)   # noqa: E731
    lines = ["| " + " | ".join(cols) + " |", "|" + "---|" * len(cols)]
    lines += ["| " + " | ".join(fmt(r.get(c)) for c in cols) + " |" for r in rows]
    return "\n".join(lines)


def main(argv=None) -> int:
    args = _parser().parse_args(argv)
    from mini_train_sys_b200.bench import distributed as db

    if args.command == "_worker":
        rec = db.worker(args.config, args.model_config, strategy=args.strategy, ops=args.ops, engine=args.engine,
                        batch_size=args.batch_size, warmup_steps=args.warmup_steps, measure_steps=args.measure_steps,
                        output=args.output)
        if int(__import__("os").environ.get("RANK", "0")) == 0:
            print(json.dumps(rec))
        return 0
    if args.command == "inventory":
        text = json.dumps(db.inventory(), indent=1, default=str)
        if args.output:
            Path(args.output).mkdir(parents=True, exist_ok=True)
            (Path(args.output) / "inventory.json").write_text(text + "\n")
        print(text)
        return 0
    if args.command == "validate-backend":
        index = int(args.device.split(":")[1]) if ":" in args.device else 0
        result = db.validate_backend(index, batch=args.batch_size, sequence_length=args.sequence_length)
        if args.output:
            Path(args.output).parent.mkdir(parents=True, exist_ok=True)
            Path(args.output).write_text(json.dumps(result, indent=1) + "\n")
        print(json.dumps(result, indent=1))
        return 0 if result["passed"] else 1
    if args.command == "run":
        if args.local_batch and args.suite != "capacity":
            args.batch_sizes = (args.local_batch,)
        if args.batch_sizes == "auto":
            args.batch_sizes = db.planned_batch_ladder(args.config, args.model_config, strategies=args.strategies,
                                                       world_sizes=args.world_sizes, device_gib=args.device_gb)
            print(json.dumps({"planned_batch_sizes": list(args.batch_sizes)}), flush=True)
        settings = db.BenchmarkSettings(
            config=args.config, model_config=args.model_config, output_dir=args.output_dir, strategies=args.strategies,
            world_sizes=args.world_sizes, ops_backends=args.ops_backends, engines=args.engines, batch_sizes=args.batch_sizes,
            repeats=args.repeats, warmup_steps=args.warmup_steps, measure_steps=args.measure_steps, timeout_s=args.timeout,
            master_port=args.master_port, reuse_stale_results=args.reuse_stale_results, reuse_failures=args.reuse_failures,
            rerun_existing=args.rerun_existing, memory_limit=args.memory_limit_percent / 100.0, min_repeats=args.min_repeats)
        summary = db.run_suite(settings, args.suite, Path(__file__).resolve())
        key = args.suite
        body = summary[key]["selected"] if key == "capacity" else summary[key]
        print(_table(body, list(body[0].keys())) if body else "(no successful rows)")
        print(json.dumps(summary["quality_gates"]))
        return 0 if summary["quality_gates"]["passed"] else 1
    suite = args.command.split("-", 1)[1]
    summary_path = Path(args.output_dir) / suite / "summary.json"
    if args.input:
        given = Path(args.input)
        summary_path = given if given.is_file() else (given / "summary.json" if (given / "summary.json").is_file() else given / suite / "summary.json")
    summary = json.loads(summary_path.read_text())
    lines: list[str] = []
    if suite == "backend":
        if args.validation and not json.loads(Path(args.validation).read_text()).get("passed"):
            print("refusing to present: the backend validation did not pass", file=sys.stderr)
            return 1
        if not all(r["valid"] for r in summary["backend"]):
            print("refusing to present: a native row shows fallbacks or too few repeats", file=sys.stderr)
            return 1
        body = summary["backend"]
    elif suite == "capacity":
        capacity = summary["capacity"]
        if args.memory_limit_percent is not None or args.min_repeats is not None:       # present the stored rows under other limits
            capacity = db.present_capacity(summary["rows"], memory_limit=(args.memory_limit_percent or 92.0) / 100.0,
                                           min_repeats=args.min_repeats or 2)
        if args.require_batch_one and not any(r.get("batch_size") == 1 and r.get("status") == "ok" for r in summary["rows"]):
            print("refusing to present: the sweep did not measure local batch 1", file=sys.stderr)
            return 1
        body = capacity["selected"]
        lines.append(f"common fixed batch: {capacity['common_fixed_batch']}")
    else:
        body = summary["weak"]
    lines.append(_table(body, list(body[0].keys())) if body else "(no rows)")
    lines.append(json.dumps(summary["quality_gates"]))
    print("\n".join(lines))
    if args.output:
        Path(args.output).parent.mkdir(parents=True, exist_ok=True)
        Path(args.output).write_text("\n".join(lines) + "\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
