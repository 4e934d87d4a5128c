"""Router capture and route statistics.

``capture_routes`` attaches forward hooks to every ``block.ffn.router`` (the router is a module whose output carries
``expert_indices`` of shape ``[tokens, K]`` in token order, reference: experiments/synbios_moe/mechanisms/routing.py:13-30)
and returns, per MoE layer, the top-k experts of every token reshaped to ``[batch, seq, K]``.
"""

from __future__ import annotations

import math
from contextlib import contextmanager
from typing import Iterator

import torch


@contextmanager
def capture_routes(model) -> Iterator[dict[int, list[torch.Tensor]]]:
    captured: dict[int, list[torch.Tensor]] = {}
    handles = []
    inner = getattr(model, "module", model)
    for layer, block in enumerate(inner.blocks):
        router = getattr(getattr(block, "ffn", None), "router", None)
        if router is None:
            continue

        def hook(_module, _inputs, output, layer=layer):
            captured.setdefault(layer, []).append(output.expert_indices.detach().to("cpu", torch.int64))

        handles.append(router.register_forward_hook(hook))
    try:
        yield captured
    finally:
        for h in handles:
            h.remove()


@torch.no_grad()
def routes_for_batch(model, input_ids: torch.Tensor) -> dict[int, torch.Tensor]:
    """``{layer: [batch, seq, K]}`` for one batch of token ids."""

    with capture_routes(model) as captured:
        model.hidden_states(input_ids)
    b, s = input_ids.shape
    return {layer: chunks[-1].view(b, s, -1) for layer, chunks in captured.items()}


def expert_load(routes: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Fraction of routes that go to each expert."""

    counts = torch.bincount(routes.reshape(-1), minlength=num_experts).double()
    return counts / counts.sum().clamp_min(1)


def normalized_mutual_information(labels: torch.Tensor, experts: torch.Tensor, num_experts: int) -> float:
    """NMI between a categorical label of each token (e.g. which attribute it belongs to) and its top-1 expert."""

    labels, experts = labels.reshape(-1).long(), experts.reshape(-1).long()
    keep = labels >= 0
    labels, experts = labels[keep], experts[keep]
    if labels.numel() == 0:
        return 0.0
    n_labels = int(labels.max()) + 1
    joint = torch.zeros(n_labels, num_experts, dtype=torch.float64)
    joint.index_put_((labels, experts), torch.ones_like(labels, dtype=torch.float64), accumulate=True)
    joint /= joint.sum()
    pl, pe = joint.sum(1, keepdim=True), joint.sum(0, keepdim=True)
    nz = joint > 0
    mi = float((joint[nz] * (joint[nz] / (pl @ pe)[nz]).log()).sum())
    hl = -float((pl[pl > 0] * pl[pl > 0].log()).sum())
    he = -float((pe[pe > 0] * pe[pe > 0].log()).sum())
    denom = math.sqrt(hl * he)
    return mi / denom if denom > 0 else 0.0
