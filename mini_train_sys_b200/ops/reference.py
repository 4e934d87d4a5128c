"""fp32 oracle backend: a plain restatement of each operator's math.

Every native kernel is tested against these functions.  Nothing here calls a fused
library kernel: attention builds the full score matrix, the MoE evaluates every
expert on every token and masks, cross entropy is an explicit log-softmax gather.
Inputs of any float dtype are promoted to fp32; outputs follow the operator contract
(activations in the input dtype, losses in fp32).
"""

from __future__ import annotations

import math

import torch

from mini_train_sys_b200.models.ops import RouterPostprocessOutput
from mini_train_sys_b200.ops.torch_backend import check_router_args

IGNORE_INDEX = -100


def rmsnorm_ref(x, weight, eps):
    xf = x.float()
    ms = (xf * xf).sum(-1, keepdim=True) / xf.shape[-1]
    return (xf / torch.sqrt(ms + eps) * weight.float()).to(x.dtype)


def rope_ref(x, cos, sin):
    """Half-split rotation: pairs are ``(d, d + D/2)``."""

    xf = x.float()
    half = xf.shape[-1] // 2
    c = cos.float()[None, None, :, :half]
    s = sin.float()[None, None, :, :half]
    a, b = xf[..., :half], xf[..., half:]
    return torch.cat((a * c - b * s, b * c + a * s), dim=-1).to(x.dtype)


def swiglu_ref(gate, up):
    g = gate.float()
    return (g / (1.0 + torch.exp(-g)) * up.float()).to(gate.dtype)


def attention_ref(q, k, v, *, is_causal, keep_mask=None, dropout_p=0.0):
    """Explicit softmax(QK^T/sqrt(D))V; ``keep_mask`` replays a dropout pattern."""

    qf, kf, vf = q.float(), k.float(), v.float()
    scores = qf @ kf.transpose(-1, -2) / math.sqrt(q.shape[-1])
    if is_causal:
        sq, sk = scores.shape[-2:]
        allowed = torch.ones(sq, sk, dtype=torch.bool, device=q.device).tril(sk - sq)
        scores = scores.masked_fill(~allowed, float("-inf"))
    p = torch.softmax(scores, dim=-1)
    if keep_mask is not None:
        p = p * keep_mask.to(p.dtype) / (1.0 - dropout_p)
    return (p @ vf).to(q.dtype)


def cross_entropy_ref(logits, targets):
    lf = logits.float()
    valid = targets != IGNORE_INDEX
    safe = targets.clamp_min(0)
    logp = lf - torch.logsumexp(lf, dim=-1, keepdim=True)
    picked = logp.gather(-1, safe[:, None]).squeeze(-1)
    return -(picked * valid).sum() / valid.sum()


def router_ref(logits, top_k, normalize):
    check_router_args(logits, top_k)
    lse = torch.logsumexp(logits, dim=-1, keepdim=True)
    probs = torch.exp(logits - lse)
    w, idx = torch.topk(probs, top_k, dim=-1)
    if normalize:
        w = w / w.sum(-1, keepdim=True).clamp_min(torch.finfo(torch.float32).eps)
    ent = -(probs * torch.log(probs.clamp_min(1e-9))).sum(-1).mean().detach()
    return RouterPostprocessOutput(w, idx.to(torch.int32), probs.mean(0), (lse * lse).mean(), ent)


def moe_ref(x, gate_up_proj, down_proj, top_k_index, top_k_weights):
    """Dense evaluation: every expert on every token, combined with a [T, E] weight matrix."""

    xf = x.float()
    n_exp, two_i, _ = gate_up_proj.shape
    combine = torch.zeros(x.shape[0], n_exp, dtype=torch.float32, device=x.device)
    combine = combine.scatter_add(1, top_k_index.long(), top_k_weights.float())
    out = torch.zeros_like(xf)
    for e in range(n_exp):
        gu = xf @ gate_up_proj[e].float().t()
        g, u = gu[:, : two_i // 2], gu[:, two_i // 2:]
        y = (g / (1.0 + torch.exp(-g)) * u) @ down_proj[e].float().t()
        out = out + y * combine[:, e:e + 1]
    return out.to(x.dtype)


class ReferenceOpsBackend:
    name = "reference"

    def rmsnorm(self, x, weight, eps):
        return rmsnorm_ref(x, weight, eps)

    def rope(self, q, k, cos, sin):
        return rope_ref(q, cos, sin), rope_ref(k, cos, sin)

    def swiglu(self, gate, up):
        return swiglu_ref(gate, up)

    def attention(self, q, k, v, *, is_causal, dropout_p):
        keep = None
        if dropout_p > 0.0:
            shape = (*q.shape[:-1], k.shape[-2])
            keep = torch.rand(shape, device=q.device) >= dropout_p
        return attention_ref(q, k, v, is_causal=is_causal, keep_mask=keep, dropout_p=dropout_p)

    def cross_entropy(self, logits, targets):
        return cross_entropy_ref(logits, targets)

    def fused_linear_cross_entropy(self, x, weight, targets):
        return cross_entropy_ref(x.float() @ weight.float().t(), targets)

    def router_postprocess(self, logits, top_k, *, normalize):
        return router_ref(logits, top_k, normalize)

    def fused_moe(self, x, gate_up_proj, down_proj, top_k_index, top_k_weights):
        return moe_ref(x, gate_up_proj, down_proj, top_k_index, top_k_weights)
