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


def _batches(text: str):
    """``--batch-sizes``: a comma-separated list, or ``auto`` (a ladder derived from the memory plan of the sweep's model)."""

    return "auto" if text.strip() == "auto" else _ints(text)


def _strs(text: str) -> tuple[str, ...]:
    return tuple(t for t in text.split(",") if t)


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
    sub.add_parser("inventory")
    sub.add_parser("validate-backend")
    r = sub.add_parser("run")
    r.add_argument("--suite", choices=("weak", "capacity", "backend"), required=True)
    r.add_argument("--config", default=DEFAULT_CONFIG)
    r.add_argument("--model-config", default=None)
    r.add_argument("--output-dir", default="results/distributed")
    r.add_argument("--strategies", type=_strs, default=("fsdp",))
    r.add_argument("--world-sizes", type=_ints, default=(1, 2, 4, 8))
    r.add_argument("--ops-backends", type=_strs, default=("native",))
    r.add_argument("--engines", type=_strs, default=("fused",))
    r.add_argument("--batch-sizes", type=_batches, default=(96,), help="comma-separated local batch sizes, or `auto`: fractions of "
                   "the largest batch the memory plan admits for every case of the sweep (see docs/memory_planning.md)")
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
        print(json.dumps(db.inventory(), indent=1, default=str))
        return 0
    if args.command == "validate-backend":
        result = db.validate_backend()
        print(json.dumps(result, indent=1))
        return 0 if result["passed"] else 1
    if args.command == "run":
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
    summary = json.loads((Path(args.output_dir) / suite / "summary.json").read_text())
    if suite == "backend":
        if not all(r["valid"] for r in summary["backend"]):
            print("refusing to present: a native row shows fallbacks or too few repeats", file=sys.stderr)
            return 1
        body = summary["backend"]
    elif suite == "capacity":
        body = summary["capacity"]["selected"]
        print(f"common fixed batch: {summary['capacity']['common_fixed_batch']}")
    else:
        body = summary["weak"]
    print(_table(body, list(body[0].keys())) if body else "(no rows)")
    print(json.dumps(summary["quality_gates"]))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
