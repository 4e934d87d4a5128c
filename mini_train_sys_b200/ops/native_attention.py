"""Autograd bridge for the tcgen05 FlashAttention kernels (``csrc/attention.cu``).

Contract kept from the reference's CUDA attention bridge (minitrain/kernels/cuda_ext/flash_attention.py:110-300):
a no-load capability predicate that rejects unsupported inputs before any kernel runs (the same checks are
repeated at the C++ boundary), ``(B, H, S, D)`` inputs that only need a unit inner stride (so views of a fused
QKV projection are consumed without copies), a stride-0 ``dout`` is materialised, and only ``O`` plus the fp32
log-sum-exp are saved for backward.  The dropout pattern is a stateless function of (seed, head, query, key);
``keep_mask`` reproduces it for tests.
"""

from __future__ import annotations

import torch

HEAD_DIM = 64


def _rows_aligned(t: torch.Tensor) -> bool:
    return (t.stride(3) == 1 and t.data_ptr() % 16 == 0 and all(s % 8 == 0 for s in t.stride()[:3]))


def supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, is_causal: bool, dropout_p: float) -> bool:
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        return False
    if not (q.dtype == k.dtype == v.dtype == torch.bfloat16):
        return False
    if q.dim() != 4 or q.shape != k.shape or q.shape != v.shape or q.shape[-1] != HEAD_DIM:
        return False
    b, h, s, _ = q.shape
    if b * h == 0 or s == 0 or b * h > 65535 or s > 65535:
        return False
    if not 0.0 <= float(dropout_p) < 1.0:
        return False
    return all(_rows_aligned(t) for t in (q, k, v))


def effective_dropout(p: float) -> float:
    """Drop probability actually applied: ``p`` quantised to 1/256."""

    return round(p * 256.0) / 256.0 if p > 0 else 0.0


def keep_mask(batch_heads: int, seq: int, dropout_p: float, seed: int, device) -> torch.Tensor:
    from mini_train_sys_b200.ops.native_backend import ext

    like = torch.empty(0, device=device)
    return ext().dropout_keep_mask(batch_heads, seq, dropout_p, seed, like).bool()


class _FlashAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, is_causal, dropout_p, seed):
        from mini_train_sys_b200.ops.native_backend import ext

        status = ext().status_tensor(q.device.index or 0)
        o, lse = ext().flash_fwd(q, k, v, is_causal, dropout_p, seed, status)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.meta = (is_causal, dropout_p, seed)
        return o

    @staticmethod
    def backward(ctx, d_o):
        from mini_train_sys_b200.ops.native_backend import ext

        q, k, v, o, lse = ctx.saved_tensors
        is_causal, dropout_p, seed = ctx.meta
        if not _rows_aligned(d_o) or 0 in d_o.stride()[:3]:
            d_o = d_o.contiguous()   # expanded (stride-0) or misaligned upstream gradients
        status = ext().status_tensor(q.device.index or 0)
        dq, dk, dv = ext().flash_bwd(d_o, q, k, v, o, lse, is_causal, dropout_p, seed, status, None, None, None)
        return dq, dk, dv, None, None, None


def flash_attention(q, k, v, *, is_causal: bool, dropout_p: float, seed: int | None = None) -> torch.Tensor:
    """Returns ``[B, H, S, D]`` whose storage is ``[B, S, H, D]``-contiguous (a free transpose for the caller)."""

    if seed is None:
        seed = int(torch.randint(0, 2**62, (1,)).item()) if dropout_p > 0 else 0
    return _FlashAttentionFn.apply(q, k, v, bool(is_causal), float(dropout_p), int(seed))


class _QKVAttentionFn(torch.autograd.Function):
    """RoPE + causal attention on a fused ``[B, S, 3, H, D]`` projection, in one autograd node.

    Forward rotates the q / k views into contiguous buffers and runs the attention kernel on them and on the
    strided v view.  Backward lets the attention kernels write dV straight into slot 2 of one fused gradient
    buffer and dQ / dK, rotated back in the epilogues that produce them, into slots 0 and 1, so the three view
    gradients never exist as separate zero-filled tensors that autograd would have to add up.
    """

    @staticmethod
    def forward(ctx, fused, cos, sin, is_causal, dropout_p, seed):
        from mini_train_sys_b200.ops.native_backend import ext

        e = ext()
        q, k, v = (fused[:, :, j].transpose(1, 2) for j in range(3))
        qr = e.rope(q, cos, sin, False, None)
        kr = e.rope(k, cos, sin, False, None)
        status = e.status_tensor(fused.device.index or 0)
        o, lse = e.flash_fwd(qr, kr, v, is_causal, dropout_p, seed, status)
        ctx.save_for_backward(qr, kr, fused, o, lse, cos, sin)
        ctx.meta = (is_causal, dropout_p, seed)
        return o

    @staticmethod
    def backward(ctx, d_o):
        from mini_train_sys_b200.ops.native_backend import ext

        e = ext()
        qr, kr, fused, o, lse, cos, sin = ctx.saved_tensors
        is_causal, dropout_p, seed = ctx.meta
        if not _rows_aligned(d_o) or 0 in d_o.stride()[:3]:
            d_o = d_o.contiguous()
        d_fused = torch.empty_like(fused)
        dq_slot, dk_slot, dv_slot = (d_fused[:, :, j].transpose(1, 2) for j in range(3))
        v = fused[:, :, 2].transpose(1, 2)
        status = e.status_tensor(fused.device.index or 0)
        # the kernels that produce dQ and dK rotate them back while storing, straight into slots 0 and 1
        e.flash_bwd(d_o, qr, kr, v, o, lse, is_causal, dropout_p, seed, status, dq_slot, dk_slot, dv_slot, cos, sin)
        return d_fused, None, None, None, None, None


def qkv_supported(fused: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, dropout_p: float) -> bool:
    if not (fused.is_cuda and fused.dtype == torch.bfloat16 and fused.dim() == 5 and fused.shape[2] == 3):
        return False
    b, s, _, h, d = fused.shape
    if d != HEAD_DIM or not fused.is_contiguous() or b * h == 0 or s == 0 or b * h > 65535 or s > 65535:
        return False
    if cos.dtype != fused.dtype or not (cos.is_contiguous() and sin.is_contiguous()) or cos.shape[0] < s:
        return False
    if cos.dim() != 2 or cos.shape[1] != HEAD_DIM or sin.shape != cos.shape:
        return False
    return 0.0 <= float(dropout_p) < 1.0


def qkv_attention(fused, cos, sin, *, is_causal: bool, dropout_p: float, seed: int | None = None) -> torch.Tensor:
    """``fused``: ``[B, S, 3, H, D]``.  Returns the context as ``[B, H, S, D]`` over ``[B, S, H, D]`` storage."""

    if seed is None:
        seed = int(torch.randint(0, 2**62, (1,)).item()) if dropout_p > 0 else 0
    return _QKVAttentionFn.apply(fused, cos, sin, bool(is_causal), float(dropout_p), int(seed))
