#!/usr/bin/env python
"""Roofline of one training step: algorithmic work per operator and the time it takes at the machine's measured peaks.

    python scripts/step_roofline.py --model-config configs/synbios_moe/model.yaml --local-batch 96 --measured-ms 62.69
    python scripts/step_roofline.py --model-config configs/model_125m_dense.yaml --local-batch 32 --format json

The denominators are the measured copy bandwidth and cuBLAS bf16 rates of ``MEASURED_PEAKS.json`` (or the documented
fallback); the arithmetic is ``mini_train_sys_b200/runtime/step_model.py``.  With ``--measured-ms`` (a device-timed step,
e.g. ``ms_per_step`` of ``bench.py``) the last line gives the achieved fraction of the whole-step bound.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from mini_train_sys_b200.models.config import ModelConfig  # noqa: E402
from mini_train_sys_b200.runtime.config import load_yaml_dict  # noqa: E402
from mini_train_sys_b200.runtime.step_model import NVLINK_GBS_MEASURED, comm_work, step_roofline  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model-config", required=True)
    ap.add_argument("--local-batch", type=int, required=True)
    ap.add_argument("--measured-ms", type=float, default=None, help="device-timed milliseconds per step to compare with")
    ap.add_argument("--format", choices=("markdown", "json"), default="markdown")
    ap.add_argument("--strategy", choices=("single", "ddp", "fsdp", "ep"), default="single", help="with --world-size: also list the NVLink traffic")
    ap.add_argument("--world-size", type=int, default=1)
    ap.add_argument("--sharding", choices=("full_shard", "shard_grad_op"), default="full_shard")
    ap.add_argument("--multimem", action="store_true", help="gradient sums inside the switch (parallel.comm.use_multimem)")
    ap.add_argument("--link-gbs", type=float, default=NVLINK_GBS_MEASURED, help="NVLink GB/s per direction per GPU (measured peer copy here: 770)")
    args = ap.parse_args(argv)
    payload = load_yaml_dict(args.model_config)
    model = ModelConfig(**(payload.get("model") or payload))
    report = step_roofline(model, args.local_batch, measured_ms=args.measured_ms)
    report["nvlink_paths"] = comm_work(model, args.local_batch, strategy=args.strategy, world_size=args.world_size, sharding=args.sharding,
                                       multimem=args.multimem, link_gbs=args.link_gbs)
    if args.format == "json":
        print(json.dumps(report, indent=1))
        return 0
    peaks = report["peaks"]
    print(f"peaks ({peaks.get('source', 'measured')}): copy {peaks['hbm_gbs']:.0f} GB/s, bf16 GEMM {peaks['bf16_tflops_sustained']:.0f} TFLOP/s sustained, "
          f"{peaks['bf16_tflops']:.0f} burst; {report['tokens_per_step']} tokens per step\n")
    print("| operator | bound by | launches | TFLOP / step | GB / step | ms at the sustained peak |")
    print("|---|---|---:|---:|---:|---:|")
    for row in report["items"]:
        print(f"| {row['item']} | {row['kind']} | {row['launches']} | {row['tflop_per_step'] or ''} | {row['gb_per_step'] or ''} | {row['bound_ms_sustained']:.3f} |")
    kinds = report["bound_ms_by_kind"]
    print(f"\nbound: {report['bound_ms_sustained']:.2f} ms (GEMM {kinds['gemm']:.2f}, attention {kinds['attention']:.2f}, memory {kinds['memory']:.2f}); "
          f"{report['bound_ms_burst']:.2f} ms at the burst GEMM rate")
    if report["nvlink_paths"]:
        print(f"\nNVLink traffic per rank and step ({args.strategy}, {args.world_size} ranks, {args.link_gbs:.0f} GB/s per direction): time to hide, not to add")
        print("| path | launches | GB in | GB out | ms alone |")
        print("|---|---:|---:|---:|---:|")
        for row in report["nvlink_paths"]:
            print(f"| {row['path']} | {row['launches']} | {row['gb_in']} | {row['gb_out']} | {row['alone_ms']:.3f} |")
    if args.measured_ms:
        print(f"measured: {args.measured_ms:.2f} ms -> {report['achieved_fraction_of_sustained_bound']:.3f} of the sustained bound, "
              f"{report['achieved_fraction_of_burst_bound']:.3f} of the burst bound")
    return 0


if __name__ == "__main__":
    sys.exit(main())
