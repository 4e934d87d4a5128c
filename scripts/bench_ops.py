#!/usr/bin/env python
"""Operator benchmarks: sweeps, parity gates, headline table, Nsight Compute helpers.

    python scripts/bench_ops.py run --suite dense --profiles project_formal --out results/operators
    python scripts/bench_ops.py run --suite moe
    python scripts/bench_ops.py summarize results/operators
    python scripts/bench_ops.py ncu-command gemm --mode full --output gemm_prof
    python scripts/bench_ops.py ncu-summary gemm_prof.ncu-rep

Covers the reference's dense and MoE operator runners plus ``scripts/summarize_operator_bench.py``.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def _parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)
    w = sub.add_parser("_worker", help="one case in this process (used by `run` and as the profiling target)")
    w.add_argument("--kernel", required=True)
    w.add_argument("--profile", default="project_formal")
    w.add_argument("--tokens", type=int, required=True)
    w.add_argument("--providers", default="torch,native")
    w.add_argument("--warmup", type=int, default=5)
    w.add_argument("--iters", type=int, default=20)
    w.add_argument("--no-check", action="store_true")
    r = sub.add_parser("run", help="sweep a suite, one subprocess per case")
    r.add_argument("--suite", choices=("dense", "moe", "all"), default="dense")
    r.add_argument("--profiles", default="project_formal")
    r.add_argument("--kernels", default=None, help="comma list; default: every kernel of the suite")
    r.add_argument("--providers", default="torch,native")
    r.add_argument("--out", default="results/operators")
    r.add_argument("--warmup", type=int, default=5)
    r.add_argument("--iters", type=int, default=20)
    r.add_argument("--refresh", action="store_true")
    r.add_argument("--timeout", type=float, default=900.0)
    s = sub.add_parser("summarize", help="merge cached scans into the headline table")
    s.add_argument("directory")
    s.add_argument("--format", choices=("json", "markdown"), default="markdown")
    s.add_argument("--plots", default=None, help="directory for one SVG per kernel (latency and speed-up over the token sizes)")
    c = sub.add_parser("ncu-command", help="print the capture command of a registered kernel")
    c.add_argument("kernel")
    c.add_argument("--mode", choices=("launches", "roofline", "full"), default="full")
    c.add_argument("--output", default=None)
    n = sub.add_parser("ncu-summary", help="reduce a .ncu-rep (or a launch-list CSV) to a short text summary")
    n.add_argument("report")
    n.add_argument("--algorithmic-bytes", type=float, default=None)
    sub.add_parser("ncu-kernels", help="list registered kernels")
    return ap


def _markdown(table: list[dict]) -> str:
    cols = ["kernel", "profile", "tokens", "provider", "fwd_ms", "full_ms", "bwd_ms", "speedup_full", "frac_of_gemm_peak",
            "frac_of_copy_peak", "parity"]
    fmt = lambda v: "" if v is None else f"{v:.4g}" if isinstance(v, float) else str(v)   # noqa: E731
    lines = ["| " + " | ".join(cols) + " |", "|" + "---|" * len(cols)]
    lines += ["| " + " | ".join(fmt(row.get(c)) for c in cols) + " |" for row in table]
    return "\n".join(lines)


def main(argv=None) -> int:
    args = _parser().parse_args(argv)
    from mini_train_sys_b200.bench import nsight, operators

    if args.command == "_worker":
        out = operators.worker(args.kernel, args.profile, args.tokens, args.providers.split(","), warmup=args.warmup,
                               iters=args.iters, check=not args.no_check)
        print(json.dumps(out, default=str))
        return 0
    if args.command == "run":
        suites = {"dense": operators.DENSE_KERNELS, "moe": operators.MOE_KERNELS,
                  "all": operators.DENSE_KERNELS + operators.MOE_KERNELS}
        kernels = tuple(args.kernels.split(",")) if args.kernels else suites[args.suite]
        bench = operators.OperatorBenchmark(Path(__file__).resolve(), Path(args.out), providers=args.providers.split(","),
                                            warmup=args.warmup, iters=args.iters, timeout_s=args.timeout)
        results = bench.run(kernels, args.profiles.split(","), refresh=args.refresh)
        gate = operators.quality_gate(results)
        print(_markdown(operators.headline_table(results)))
        print(json.dumps(gate))
        return 0 if gate["quality_gate_passed"] else 1
    if args.command == "summarize":
        results = []
        for path in sorted(Path(args.directory).glob("*.json")):
            results += list(json.loads(path.read_text()).values())
        table = operators.headline_table(results)
        print(json.dumps(table, indent=1) if args.format == "json" else _markdown(table))
        print(json.dumps(operators.quality_gate(results)))
        if args.plots:
            from mini_train_sys_b200.bench.plots import write_kernel_plots

            print(json.dumps({"plots": write_kernel_plots(table, args.plots)}))
        return 0
    if args.command == "ncu-command":
        print(nsight.command_for(args.kernel, "scripts/bench_ops.py", mode=args.mode, output=args.output))
        return 0
    if args.command == "ncu-kernels":
        for k in nsight.registered().values():
            print(f"{k.name:16s} {k.regex}")
        return 0
    if args.command == "ncu-summary":
        path = Path(args.report)
        if path.suffix == ".csv":
            rows = nsight.parse_launch_list(path.read_text())
            for name, n, us, share in nsight.launch_shares(rows):
                print(f"{share * 100:6.2f}%  {us:12.1f} us  {n:5d}x  {name}")
        else:
            print(nsight.roofline_summary(nsight.parse_raw_csv(nsight.export_raw_csv(path)),
                                          algorithmic_bytes=args.algorithmic_bytes))
        return 0
    return 2


if __name__ == "__main__":
    raise SystemExit(main())
