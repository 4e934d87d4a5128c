"""Helpers shared by evaluation and sampling: rebuild a model from a checkpoint, score a split, generate text.

Evaluation and probes load only the consolidated ``model.pt`` export into a plain (unwrapped) model, whatever
strategy trained it (the reference's experiment layer does the same: scripts/synbios_moe.py:141-168).
"""

from __future__ import annotations

import math
from pathlib import Path
from typing import Any

import torch

from mini_train_sys_b200.models import MiniTransformer, ModelConfig, get_ops_backend
from mini_train_sys_b200.train.checkpoint import load_model_state_dict_from_checkpoint


def model_config_from_checkpoint(path: str | Path) -> dict[str, Any] | None:
    runtime = Path(path) / "runtime.pt"
    if not runtime.is_file():
        return None
    blob = torch.load(runtime, map_location="cpu", weights_only=False)
    cfg = (blob.get("config") or {}).get("model")
    return dict(cfg) if cfg else None


def load_model_for_inference(checkpoint: str | Path, *, model_payload: dict[str, Any] | None = None, ops: str = "torch",
                             device: torch.device | str = "cpu", dtype: torch.dtype = torch.float32) -> MiniTransformer:
    payload = model_payload or model_config_from_checkpoint(checkpoint)
    if not payload:
        raise ValueError("no model config given and none recorded in the checkpoint")
    model = MiniTransformer(ModelConfig(**payload), get_ops_backend(ops), activation_dtype=dtype)
    state = load_model_state_dict_from_checkpoint(checkpoint)
    missing, unexpected = model.load_state_dict(state, strict=False)
    missing = [k for k in missing if not (k == "lm_head.weight" and model.cfg.tie_word_embeddings)]
    if missing or unexpected:
        raise ValueError(f"checkpoint does not match the model: missing={missing[:4]} unexpected={unexpected[:4]}")
    return model.to(device).eval()


@torch.no_grad()
def evaluate_loss(model: MiniTransformer, loader, device: torch.device, *, max_batches: int | None = None,
                  autocast_dtype: torch.dtype | None = None) -> dict[str, float]:
    """Token-weighted mean cross entropy and perplexity over ``loader``."""

    total, tokens, batches = 0.0, 0, 0
    for batch in loader:
        ids, tgt = batch["input_ids"].to(device), batch["targets"].to(device)
        with torch.autocast(device.type, dtype=autocast_dtype, enabled=autocast_dtype is not None):
            hidden = model.hidden_states(ids)
            loss = model.ops.fused_linear_cross_entropy(hidden.reshape(-1, hidden.shape[-1]), model.lm_head.weight, tgt.reshape(-1))
        n = int((tgt != -100).sum())
        total += float(loss) * n
        tokens += n
        batches += 1
        if max_batches is not None and batches >= max_batches:
            break
    mean = total / max(tokens, 1)
    return {"loss": mean, "perplexity": math.exp(min(mean, 50.0)), "tokens": tokens, "batches": batches}


@torch.no_grad()
def generate(model: MiniTransformer, prompt_ids: torch.Tensor, *, max_new_tokens: int, temperature: float = 1.0,
             top_k: int | None = None, greedy: bool = False, generator: torch.Generator | None = None) -> torch.Tensor:
    """Autoregressive decoding without a KV cache: the prefix (cropped to ``seq_len``) is re-encoded every step."""

    ids = prompt_ids.clone()
    limit = model.cfg.seq_len
    for _ in range(max_new_tokens):
        window = ids[:, -limit:]
        _, logits = model(window)
        step = logits[:, -1, :].float()
        if greedy or temperature <= 0:
            nxt = step.argmax(-1, keepdim=True)
        else:
            step = step / temperature
            if top_k is not None and top_k > 0:
                kth = step.topk(min(top_k, step.shape[-1]), -1).values[:, -1:]
                step = step.masked_fill(step < kth, float("-inf"))
            nxt = torch.multinomial(torch.softmax(step, -1), 1, generator=generator)
        ids = torch.cat((ids, nxt), dim=1)
    return ids
