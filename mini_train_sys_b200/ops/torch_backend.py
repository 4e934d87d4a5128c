"""Library-op backend (cuBLAS GEMMs, SDPA attention): the measured baseline.

Numerical contract as in minitrain/kernels/torch_ops.py:13-150: reductions in fp32,
activations returned in the input dtype, dropless MoE that keeps zero-weight routes.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from mini_train_sys_b200.models.ops import RouterPostprocessOutput


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    lo, hi = x.chunk(2, dim=-1)
    return torch.cat((-hi, lo), dim=-1)


def check_router_args(logits: torch.Tensor, top_k: int) -> None:
    if logits.ndim != 2 or logits.dtype != torch.float32:
        raise ValueError("router logits must be a 2D fp32 tensor")
    if logits.shape[0] == 0:
        raise ValueError("router logits must contain at least one token")
    if not 1 <= top_k <= logits.shape[1]:
        raise ValueError(f"top_k must be in [1, {logits.shape[1]}], got {top_k}")


class TorchOpsBackend:
    name = "torch"

    def rmsnorm(self, x, weight, eps):
        xf = x.float()
        inv = torch.rsqrt(xf.square().mean(dim=-1, keepdim=True) + eps)
        return (xf * inv * weight.float()).to(x.dtype)

    def rope(self, q, k, cos, sin):
        c = cos[None, None].to(q.dtype)
        s = sin[None, None].to(q.dtype)
        return q * c + rotate_half(q) * s, k * c + rotate_half(k) * s

    def swiglu(self, gate, up):
        return F.silu(gate) * up

    def attention(self, q, k, v, *, is_causal, dropout_p):
        return F.scaled_dot_product_attention(q, k, v, is_causal=is_causal, dropout_p=dropout_p)

    def cross_entropy(self, logits, targets):
        return F.cross_entropy(logits.float(), targets)

    def fused_linear_cross_entropy(self, x, weight, targets):
        return F.cross_entropy(F.linear(x, weight).float(), targets)

    def router_postprocess(self, logits, top_k, *, normalize):
        check_router_args(logits, top_k)
        lse = torch.logsumexp(logits, dim=-1, keepdim=True)
        probs = (logits - lse).exp()
        w, idx = probs.topk(top_k, dim=-1)
        if normalize:
            w = w / w.sum(-1, keepdim=True).clamp_min(torch.finfo(w.dtype).eps)
        ent = -(probs * probs.clamp_min(1e-9).log()).sum(-1).mean().detach()
        return RouterPostprocessOutput(w, idx.to(torch.int32), probs.mean(0), lse.square().mean(), ent)

    def fused_moe(self, x, gate_up_proj, down_proj, top_k_index, top_k_weights):
        out = torch.zeros_like(x)
        for e in torch.unique(top_k_index).tolist():
            tok, slot = torch.where(top_k_index == e)  # zero-weight routes stay in the graph
            if tok.numel() == 0:
                continue
            g, u = F.linear(x[tok], gate_up_proj[e]).chunk(2, dim=-1)
            y = F.linear(F.silu(g) * u, down_proj[e]) * top_k_weights[tok, slot, None]
            out.index_add_(0, tok, y.to(out.dtype))
        return out
