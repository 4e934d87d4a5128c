#!/usr/bin/env python
"""Device-memory plan of a run: resident buffers, activations per sample, peak at a batch, and the largest batch that fits.

    python scripts/plan_memory.py --model-config configs/synbios_moe/model.yaml --strategy fsdp --world-size 8 --local-batch 96
    python scripts/plan_memory.py --config configs/server/b200_180gb/runs/fsdp_8gpu.yaml --model-config configs/synbios_moe/model.yaml

With ``--config`` the strategy, sharding mode, world size, batch and activation checkpointing are read from the run file.
The arithmetic is that of ``mini_train_sys_b200/runtime/memory_plan.py`` (fused engine, native back end, bf16); ``total_gib``
is what the device holds, ``max_memory_allocated_gib`` what ``torch.cuda.max_memory_allocated`` will report (symmetric
buffers are outside the caching allocator when there is more than one rank).
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
from mini_train_sys_b200.runtime.config import load_experiment, load_yaml_dict  # noqa: E402
from mini_train_sys_b200.runtime.memory_plan import GIB, STRATEGIES, plan_memory  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", help="run file: strategy, sharding, expected world size, batch and checkpointing are taken from it")
    ap.add_argument("--model-config", help="model file (or the run file embeds `model:`)")
    ap.add_argument("--strategy", choices=STRATEGIES)
    ap.add_argument("--world-size", type=int)
    ap.add_argument("--sharding", choices=("full_shard", "shard_grad_op"))
    ap.add_argument("--local-batch", type=int)
    ap.add_argument("--activation-checkpointing", action="store_true")
    ap.add_argument("--device-gb", type=float, default=180.0, help="device memory in GiB (B200: 180)")
    ap.add_argument("--headroom", type=float, default=0.9, help="share of the device the peak may take")
    args = ap.parse_args(argv)

    strategy, world, sharding, batch, checkpointing = "single", 1, "full_shard", 1, args.activation_checkpointing
    model_payload = None
    if args.config:
        cfg = load_experiment(args.config, args.model_config)
        strategy, batch = cfg.parallel.strategy, cfg.train.batch_size
        world = cfg.parallel.expected_world_size or 1
        if cfg.parallel.fsdp.sharding_strategy in ("full_shard", "shard_grad_op"):
            sharding = cfg.parallel.fsdp.sharding_strategy
        checkpointing = checkpointing or bool(cfg.parallel.fsdp.activation_checkpointing and strategy == "fsdp")
        model_payload = cfg.model
    elif args.model_config:
        model_payload = load_yaml_dict(args.model_config).get("model")
    if not model_payload:
        ap.error("give --model-config, or a --config that embeds `model:`")
    strategy = args.strategy or strategy
    world = args.world_size or world
    sharding = args.sharding or sharding
    batch = args.local_batch or batch
    model = ModelConfig(**model_payload)
    plan = plan_memory(model, strategy=strategy, world_size=world, sharding=sharding, local_batch_hint=batch,
                       activation_checkpointing=checkpointing)
    report = {"model_parameters": model.param_count(), "seq_len": model.seq_len, **plan.summary(batch),
              "device_gib": args.device_gb, "headroom": args.headroom,
              "fits": plan.total_bytes(batch) <= args.headroom * args.device_gb * GIB,
              "max_local_batch": plan.max_local_batch(args.device_gb * GIB, headroom=args.headroom)}
    print(json.dumps(report, indent=1))
    return 0 if report["fits"] else 1


if __name__ == "__main__":
    sys.exit(main())
