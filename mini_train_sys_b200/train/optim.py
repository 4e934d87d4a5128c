"""AdamW construction: weight decay on tensors with ``ndim >= 2`` only.

On the torch-optimizer path ``fused=True`` is selected for CUDA parameters; the own
sharded engines (parallel/flat_engine.py) build their optimizer from the same config and
run the update inside their fused reduce kernels (reference: minitrain/train/optim.py:7-47).
"""

from __future__ import annotations

from dataclasses import replace

import torch

from mini_train_sys_b200.runtime.config import OptimizerConfig


def split_decay_groups(model: torch.nn.Module) -> tuple[list[torch.nn.Parameter], list[torch.nn.Parameter]]:
    decay, plain = [], []
    for p in model.parameters():
        if p.requires_grad:
            (decay if p.ndim >= 2 else plain).append(p)
    return decay, plain


def build_optimizer(model: torch.nn.Module, *, cfg: OptimizerConfig | None = None, lr: float | None = None,
                    weight_decay: float | None = None) -> torch.optim.Optimizer:
    cfg = cfg or OptimizerConfig()
    if lr is not None:
        cfg = replace(cfg, lr=lr)
    if weight_decay is not None:
        cfg = replace(cfg, weight_decay=weight_decay)
    own = getattr(model, "build_sharded_optimizer", None)
    if own is not None:  # strategies that own flat shards provide their optimizer
        return own(cfg)
    decay, plain = split_decay_groups(model)
    on_cuda = any(p.is_cuda for p in model.parameters())
    return torch.optim.AdamW(
        [{"params": decay, "weight_decay": cfg.weight_decay}, {"params": plain, "weight_decay": 0.0}],
        lr=cfg.lr, betas=(cfg.beta1, cfg.beta2), eps=cfg.eps,
        fused=on_cuda if cfg.fused is None else cfg.fused,
    )
