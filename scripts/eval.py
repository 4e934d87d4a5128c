"""Evaluate a consolidated checkpoint: mean cross entropy / perplexity on a token-shard split or random tokens.

    python scripts/eval.py --checkpoint checkpoints/run/epoch_000001_step_000000100 --data path/to/shards --split validation

(The reference ships this entry point as an unimplemented scaffold: scripts/eval.py:2-3.)
"""

from __future__ import annotations

import argparse
import json
import sys
from dataclasses import replace
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

from mini_train_sys_b200.data.dataloader import build_training_dataloader  # noqa: E402
from mini_train_sys_b200.runtime.config import DataConfig, load_yaml_dict  # noqa: E402
from mini_train_sys_b200.runtime.device import resolve_device  # noqa: E402
from mini_train_sys_b200.runtime.inference import evaluate_loss, load_model_for_inference  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--model-config", default=None, help="model YAML (default: the config stored in the checkpoint)")
    ap.add_argument("--data", default=None, help="token-shard directory; omitted = seeded random tokens")
    ap.add_argument("--split", default="validation")
    ap.add_argument("--batch-size", type=int, default=8)
    ap.add_argument("--max-batches", type=int, default=None)
    ap.add_argument("--ops", default="torch")
    ap.add_argument("--device", choices=["auto", "cpu", "cuda"], default="auto")
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)

    device = resolve_device(args.device)
    payload = load_yaml_dict(args.model_config).get("model") if args.model_config else None
    dtype = torch.bfloat16 if (device.type == "cuda" and args.ops != "torch") else torch.float32
    model = load_model_for_inference(args.checkpoint, model_payload=payload, ops=args.ops, device=device, dtype=dtype)
    data = DataConfig(source="token_shards", path=args.data, shuffle=False, num_workers=0, persistent_workers=False,
                      drop_last=False) if args.data else DataConfig(source="random", shuffle=False, num_workers=0,
                                                                    persistent_workers=False, num_tokens=64 * model.cfg.seq_len + 1)
    loader = build_training_dataloader(replace(data, pin_memory=False), seq_len=model.cfg.seq_len, batch_size=args.batch_size,
                                       vocab_size=model.cfg.vocab_size, seed=args.seed, split=args.split if args.data else "train")
    result = evaluate_loss(model, loader, device, max_batches=args.max_batches,
                           autocast_dtype=torch.bfloat16 if dtype == torch.bfloat16 else None)
    print(json.dumps({"event": "evaluate", "checkpoint": args.checkpoint, "split": args.split, **result}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
