"""Generate tokens from a consolidated checkpoint (greedy or temperature / top-k sampling, no KV cache).

    python scripts/sample.py --checkpoint <dir> --prompt-ids 1,2,3 --max-new-tokens 32 --top-k 40
    python scripts/sample.py --checkpoint <dir> --tokenizer <tokenizer dir> --prompt "Once upon a time"

(The reference ships this entry point as an unimplemented scaffold: scripts/sample.py:2-3.)
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

from mini_train_sys_b200.runtime.config import load_yaml_dict  # noqa: E402
from mini_train_sys_b200.runtime.device import resolve_device  # noqa: E402
from mini_train_sys_b200.runtime.inference import generate, load_model_for_inference  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--model-config", default=None)
    ap.add_argument("--tokenizer", default=None, help="tokenizer directory (needed for --prompt and for decoded output)")
    ap.add_argument("--prompt", default=None)
    ap.add_argument("--prompt-ids", default=None, help="comma-separated token ids")
    ap.add_argument("--max-new-tokens", type=int, default=32)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=None)
    ap.add_argument("--greedy", action="store_true")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--ops", default="torch")
    ap.add_argument("--device", choices=["auto", "cpu", "cuda"], default="auto")
    args = ap.parse_args(argv)

    device = resolve_device(args.device)
    payload = load_yaml_dict(args.model_config).get("model") if args.model_config else None
    model = load_model_for_inference(args.checkpoint, model_payload=payload, ops=args.ops, device=device)
    tokenizer = None
    if args.tokenizer:
        from mini_train_sys_b200.data.tokenizer import load_tokenizer

        tokenizer = load_tokenizer(args.tokenizer)
    if args.prompt_ids:
        ids = [int(t) for t in args.prompt_ids.split(",") if t.strip()]
    elif args.prompt is not None:
        if tokenizer is None:
            raise SystemExit("--prompt needs --tokenizer")
        ids = [tokenizer.boundary_token_id, *tokenizer.encode(args.prompt)]
    else:
        ids = [0]
    if any(not 0 <= t < model.cfg.vocab_size for t in ids):
        raise SystemExit("prompt token id outside the model vocabulary")
    gen = torch.Generator(device=device.type if device.type == "cuda" else "cpu").manual_seed(args.seed)
    out = generate(model, torch.tensor([ids], device=device), max_new_tokens=args.max_new_tokens, temperature=args.temperature,
                   top_k=args.top_k, greedy=args.greedy, generator=gen)[0].tolist()
    record = {"event": "sample", "prompt_tokens": len(ids), "tokens": out}
    if tokenizer is not None:
        record["text"] = tokenizer.decode(out)
    print(json.dumps(record, ensure_ascii=False))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
