"""sm_100a operator backend: every hot op runs a hand-written CUDA kernel from ``csrc``.

* GEMM-shaped work (projections, fused linear cross-entropy, the grouped expert GEMMs and all
  of their dgrad / wgrad passes) goes through the tcgen05 + TMA kernel in ``gemm_sm100.cu``;
  no cuBLAS call is made on these paths.
* RMSNorm, RoPE, SwiGLU, cross entropy, the router and the MoE permutation kernels are
  bandwidth-bound kernels with 128-bit accesses.
* Attention runs the tcgen05 FlashAttention kernels in ``attention.cu``.

Inputs the kernels do not cover (CPU tensors, fp16, odd alignments) take the library path of
``TorchOpsBackend`` and are counted in ``dispatch_summary()`` so that a silent fallback shows
up in tests and benchmark records (the reference keeps similar counters for its CUDA attention:
minitrain/kernels/cuda_ext/__init__.py:43-50).
"""

from __future__ import annotations

import math
import os
import weakref
from collections import Counter

import torch

from mini_train_sys_b200.models.ops import RouterPostprocessOutput
from mini_train_sys_b200.ops.build import load_extension
from mini_train_sys_b200.ops.torch_backend import TorchOpsBackend, check_router_args

GEMM_DENSE, GEMM_GROUPED_M, GEMM_GROUPED_K = 0, 1, 2
EPI_STORE, EPI_SWIGLU, EPI_SWIGLU_BWD = 0, 1, 2
# Two-CTA clusters on 256 x 256 tiles (one third less L2 traffic per FLOP); MTS_GEMM_PAIR=0 selects one CTA per 128 x 256 tile.
GEMM_PAIR = os.environ.get("MTS_GEMM_PAIR", "1") != "0"

_ext = None


def ext():
    global _ext
    if _ext is None:
        _ext = load_extension()
    return _ext


def check_kernel_status(device: torch.device | int | None = None) -> None:
    """Raise if any kernel on ``device`` reported a bounded-wait timeout (synchronises)."""

    index = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    word = int(ext().status_tensor(index)[0].item())
    if word != 0:
        raise RuntimeError(f"a native kernel reported status {word} (1 = wait timeout)")


# ---------------------------------------------------------------------------------------------
# GEMM wrappers
# ---------------------------------------------------------------------------------------------
_weight_cache: dict[int, tuple] = {}
_rows_cache: dict[tuple, torch.Tensor] = {}


def bf16_weight(weight: torch.Tensor) -> torch.Tensor:
    """bf16 copy of a (usually fp32) parameter, refreshed only when the parameter changes.

    Entries are keyed by storage address and validated with the version counter, the shape and a
    weak reference to the tensor object that created the entry: once that object is gone the
    address may have been recycled, so the entry is dropped instead of trusted.
    """

    if weight.dtype == torch.bfloat16:
        return weight if weight.is_contiguous() else weight.contiguous()
    key = weight.data_ptr()
    hit = _weight_cache.get(key)
    version = weight._version
    if hit is not None and hit[0]() is not None and hit[1] == version and hit[2] == weight.shape:
        return hit[3]
    src = weight.detach()
    if not src.is_contiguous():
        src = src.contiguous()
    out = ext().cast_bf16(src.float() if src.dtype != torch.float32 else src)
    if len(_weight_cache) > 4096:
        for k in [k for k, v in _weight_cache.items() if v[0]() is None]:
            del _weight_cache[k]
    _weight_cache[key] = (weakref.ref(weight), version, weight.shape, out)
    return out


def _gemm(a, b, out, M, N, K, *, a_mn=False, b_mn=False, mode=GEMM_DENSE, epilogue=EPI_STORE, accumulate=False,
          atomic_out=False, aux=None, tile_group=None, num_row_tiles=None, group_rows=None, num_groups=1,
          b_group_stride_rows=0, out_group_stride=0, ldo=None, sm_limit=0, pair=None, k_splits=1, gather_a=None, gather_b=None,
          row_scale=None, row_slot=None, row_grad=None) -> None:
    if pair is None:
        pair = GEMM_PAIR
    ext().gemm(a, b, out, M, N, K, a_mn, b_mn, mode, epilogue, accumulate, atomic_out, aux, tile_group, num_row_tiles,
               group_rows, num_groups, b_group_stride_rows, out_group_stride, out.stride(-2) if ldo is None else ldo,
               sm_limit, bool(pair), k_splits, gather_a, gather_b, row_scale, row_slot, row_grad)


def gemm_nt(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, *, out_dtype=torch.bfloat16
            ) -> torch.Tensor:
    """``a[M, K] @ b[N, K]^T`` (both K-major)."""

    M, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    _gemm(a, b, out, M, N, K)
    return out


def gemm_nn(a: torch.Tensor, b_kn: torch.Tensor, out: torch.Tensor | None = None, *, K: int | None = None,
            out_dtype=torch.bfloat16) -> torch.Tensor:
    """``a[M, K] @ b_kn[K, N]`` (B is MN-major: no transpose is materialised)."""

    M = a.shape[0]
    K = a.shape[1] if K is None else K
    N = b_kn.shape[1]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    _gemm(a, b_kn, out, M, N, K, b_mn=True)
    return out


def _split_rows(k_rows: int, tiles: int, device: torch.device) -> tuple[torch.Tensor, int]:
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    splits = max(1, min(round(2 * sms / max(tiles, 1)), k_rows // 512 if k_rows >= 512 else 1))
    key = (k_rows, splits, device.index)
    hit = _rows_cache.get(key)
    if hit is None:
        per = -(-k_rows // splits)
        per = -(-per // 64) * 64
        bounds = [min(i * per, k_rows) for i in range(splits)] + [k_rows]
        hit = torch.tensor(bounds, dtype=torch.int32, device=device)
        _rows_cache[key] = hit
    return hit, splits


def gemm_tn(a_km: torch.Tensor, b_kn: torch.Tensor, out: torch.Tensor | None = None, *, accumulate: bool = False,
            M: int | None = None) -> torch.Tensor:
    """``a_km[K, M]^T @ b_kn[K, N]`` -> fp32 ``[M, N]`` (weight gradients; split-K with fp32 atomics)."""

    k_rows = a_km.shape[0]
    M = a_km.shape[1] if M is None else M
    N = b_kn.shape[1]
    tiles = -(-M // (256 if GEMM_PAIR else 128)) * -(-N // 256) * (2 if GEMM_PAIR else 1)   # in SMs' worth of work
    rows, splits = _split_rows(k_rows, tiles, a_km.device)
    if out is None:
        out = (torch.zeros if splits > 1 else torch.empty)(M, N, dtype=torch.float32, device=a_km.device)
        accumulate = False
    elif splits > 1 and not accumulate:
        out.zero_()              # the splits add into the output
    atomic = splits > 1
    _gemm(a_km, b_kn, out, M, N, 0, a_mn=True, b_mn=True, mode=GEMM_GROUPED_K, group_rows=rows, num_groups=splits,
          accumulate=accumulate and not atomic, atomic_out=atomic, out_group_stride=0)
    return out


def expert_wgrad_splits(rows: int, groups: int, m: int, n: int, device: torch.device) -> int:
    """How many parts to cut every expert's rows into for a grouped weight-gradient GEMM.

    One expert's gradient is only ``ceil(m / 256) * ceil(n / 256)`` tiles (12 for a 768 x 1024 down projection), so eight
    experts fill 96 of the 74 CTA pairs' second wave and leave the machine two thirds idle for half of the kernel.  Cutting
    the contraction gives more, shorter work items that add into the (pre-zeroed) output with TMA reduce-adds; the count is
    the one that wastes the least of the last wave while every part keeps at least 1,024 rows."""

    pairs = max(torch.cuda.get_device_properties(device).multi_processor_count // 2, 1) if GEMM_PAIR else \
        torch.cuda.get_device_properties(device).multi_processor_count
    tiles = groups * -(-m // (256 if GEMM_PAIR else 128)) * -(-n // 256)
    per_group = max(rows // max(groups, 1), 1)
    best, best_eff = 1, 0.0
    for s in range(1, 9):
        if s > 1 and per_group // s < 1024:
            break
        items = tiles * s
        eff = items / (-(-items // pairs) * pairs)
        if eff > best_eff + 0.02:
            best, best_eff = s, eff
    return best


def grad_sink(param: torch.Tensor):
    """``(fp32 destination, done callback, accumulate)`` when a sharding engine wants this parameter's gradient written in place.

    The engine attaches ``_mts_grad_sink`` to parameters; a backward function that honours it writes the fp32 gradient there,
    calls ``done(param)`` and returns no gradient for the parameter, which saves the bf16 round trip (fp32 -> parameter
    dtype -> fp32 copy in the accumulate hook) and two passes over every weight-sized tensor.  ``accumulate`` is False for
    parameters used once per step (the writer overwrites the destination) and True for parameters with several uses, such
    as a tied embedding / output matrix: every writer ADDS to the destination, which the engine zeroes after each step."""

    return getattr(param, "_mts_grad_sink", None)


def _sink_accumulates(sink) -> bool:
    return len(sink) > 2 and bool(sink[2])


def _gemm_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.is_cuda and weight.dim() == 2
            and x.shape[-1] == weight.shape[1] and x.shape[-1] % 8 == 0 and x.numel() > 0)


class _LinearFn(torch.autograd.Function):
    """``y = x @ W^T`` with the weight kept in fp32 (bf16 copy cached) and fp32 weight gradients."""

    @staticmethod
    def forward(ctx, x, weight):
        w16 = bf16_weight(weight)
        n_out, k_in = w16.shape
        x2 = x.reshape(-1, k_in)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        ld = -(-n_out // 8) * 8   # padded row pitch keeps the epilogue on 16-byte stores
        buf = torch.empty(x2.shape[0], ld, dtype=torch.bfloat16, device=x.device)
        _gemm(x2, w16, buf, x2.shape[0], n_out, k_in, ldo=ld)
        ctx.save_for_backward(x2, weight)
        ctx.in_shape = x.shape
        y = buf if ld == n_out else buf[:, :n_out]
        return y.view(*x.shape[:-1], n_out) if ld == n_out else y.reshape(*x.shape[:-1], n_out)

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        w16 = bf16_weight(weight)
        n_out, k_in = w16.shape
        dy2 = dy.reshape(-1, n_out)
        if n_out % 8 != 0:   # operand pitch must be a multiple of 8 elements
            pad = torch.zeros(dy2.shape[0], -(-n_out // 8) * 8, dtype=dy2.dtype, device=dy2.device)
            pad[:, :n_out] = dy2
            dy2 = pad
        elif not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm_nn(dy2, w16, K=dy2.shape[1]).view(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            sink = grad_sink(weight)
            if sink is not None:
                # fp32, straight into the engine's flat gradient buffer
                gemm_tn(dy2, x2, out=sink[0], M=n_out, accumulate=_sink_accumulates(sink))
                sink[1](weight)
            else:
                dw = gemm_tn(dy2, x2, M=n_out).to(weight.dtype)
        return dx, dw


# ---------------------------------------------------------------------------------------------
# memory-bound operators
# ---------------------------------------------------------------------------------------------
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        xc = x if x.is_contiguous() else x.contiguous()
        w32 = weight if weight.dtype == torch.float32 else weight.float()
        y, rstd = ext().rmsnorm_fwd(xc, w32.contiguous(), eps)
        ctx.save_for_backward(xc, w32, rstd, weight)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w32, rstd, weight = ctx.saved_tensors
        dyc = dy if dy.is_contiguous() else dy.contiguous()
        return (*_rmsnorm_backward(dyc, x, w32, rstd, weight, ctx.needs_input_grad[1], None), None)


def _rmsnorm_backward(dy, x, w32, rstd, weight, need_dw, dres):
    """``(dx, dw)``; the weight gradient goes straight into the engine's flat fp32 buffer when the parameter has a sink."""

    sink = grad_sink(weight) if need_dw else None
    if sink is not None and sink[0].is_contiguous():
        dx, _ = ext().rmsnorm_bwd(dy, x, w32, rstd, True, dres, sink[0])
        sink[1](weight)
        return dx, None
    dx, dw = ext().rmsnorm_bwd(dy, x, w32, rstd, need_dw, dres)
    return dx, (dw.to(weight.dtype) if dw is not None and dw.numel() else None)


class _RMSNormResidualFn(torch.autograd.Function):
    """``(rmsnorm(x), x)``: the second output is x itself, handed to the residual branch.  Autograd then delivers the
    gradient of that branch to this backward, where the kernel adds it to the gradient of the norm, instead of summing
    the two paths in a pass of its own."""

    @staticmethod
    def forward(ctx, x, weight, eps):
        xc = x if x.is_contiguous() else x.contiguous()
        w32 = weight if weight.dtype == torch.float32 else weight.float()
        y, rstd = ext().rmsnorm_fwd(xc, w32.contiguous(), eps)
        ctx.save_for_backward(xc, w32, rstd, weight)
        return y, xc          # an input returned as an output: autograd gives it a node of its own

    @staticmethod
    def backward(ctx, dy, dres):
        x, w32, rstd, weight = ctx.saved_tensors
        if dy is None:
            return dres, None, None
        dyc = dy if dy.is_contiguous() else dy.contiguous()
        if dres is not None and not dres.is_contiguous():
            dres = dres.contiguous()
        return (*_rmsnorm_backward(dyc, x, w32, rstd, weight, ctx.needs_input_grad[1], dres), None)


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, cos, sin):
        ctx.save_for_backward(cos, sin)
        return ext().rope(q, cos, sin, False, None), ext().rope(k, cos, sin, False, None)

    @staticmethod
    def backward(ctx, dq, dk):
        cos, sin = ctx.saved_tensors
        fix = lambda t: t if t.stride(-1) == 1 else t.contiguous()  # noqa: E731
        return ext().rope(fix(dq), cos, sin, True, None), ext().rope(fix(dk), cos, sin, True, None), None, None


class _SwigluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up):
        g, u = gate.contiguous(), up.contiguous()
        ctx.save_for_backward(g, u)
        return ext().swiglu_fwd(g, u)

    @staticmethod
    def backward(ctx, dy):
        g, u = ctx.saved_tensors
        dg, du = ext().swiglu_bwd(dy.contiguous(), g, u)
        return dg, du


class _CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets):
        rows, vocab = logits.shape
        lg = logits if logits.stride(1) == 1 else logits.contiguous()
        tg = targets.contiguous()
        lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
        stats = torch.zeros(2, dtype=torch.float32, device=logits.device)
        ext().ce_forward(lg, tg, lse, stats, vocab)
        ctx.save_for_backward(lg, tg, lse, stats)
        return stats[0] / stats[1]

    @staticmethod
    def backward(ctx, g):
        lg, tg, lse, stats = ctx.saved_tensors
        grad = lg.clone()
        ext().ce_backward(grad, tg, lse, stats[1:2], g.reshape(1).float().contiguous(), lg.shape[1])
        return grad, None


def _ce_chunk_rows() -> int:
    # 65,536 rows x 50k vocabulary is a 6.6 GB bf16 logit buffer: small on a 180 GB part, and it gives the three GEMMs of a
    # chunk enough 256 x 256 tiles to fill all SMs for several waves
    return int(os.environ.get("MTS_FUSED_CE_CHUNK_ROWS", "65536"))


class _FusedLinearCEFn(torch.autograd.Function):
    """Linear + cross entropy without ever holding ``[tokens, vocab]``.

    Rows are processed in chunks: logits GEMM into a reused bf16 buffer, cross entropy with the
    gradient written in place, then ``dX = dZ W`` and ``dW += dZ^T X`` straight from that buffer.
    Gradients are produced during the forward pass (as the reference's chunk loop does,
    minitrain/kernels/triton/fused_linear_cross_entropy.py:52-170); backward only scales them.
    """

    @staticmethod
    def forward(ctx, x, weight, targets):
        e = ext()
        w16 = bf16_weight(weight)
        vocab, hidden = w16.shape
        rows = x.shape[0]
        vp = -(-vocab // 8) * 8
        chunk = min(_ce_chunk_rows(), rows)
        xc = x if x.is_contiguous() else x.contiguous()
        tg = targets.contiguous()
        dev = x.device
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        stats = torch.zeros(2, dtype=torch.float32, device=dev)
        valid = torch.zeros(1, dtype=torch.float32, device=dev)
        e.count_valid(tg, valid)
        lse = torch.empty(rows, dtype=torch.float32, device=dev)
        logits = torch.empty(chunk, vp, dtype=torch.bfloat16, device=dev)
        dx = torch.empty_like(xc) if need_dx else None
        dw = torch.zeros(vocab, hidden, dtype=torch.float32, device=dev) if need_dw else None
        for lo in range(0, rows, chunk):
            n = min(chunk, rows - lo)
            xs, ts, ls = xc[lo:lo + n], tg[lo:lo + n], lse[lo:lo + n]
            z = logits[:n]
            _gemm(xs, w16, z, n, vocab, hidden, ldo=vp)
            e.ce_forward(z, ts, ls, stats, vocab)
            if not (need_dx or need_dw):
                continue
            e.ce_backward(z, ts, ls, valid, None, vocab)
            if need_dx:
                _gemm(z, w16, dx[lo:lo + n], n, hidden, vp, b_mn=True, ldo=hidden)
            if need_dw:
                key = ("one_group", n, dev.index)       # cached across calls: no host-to-device copy in steady state
                if key not in _rows_cache:
                    _rows_cache[key] = torch.tensor([0, n], dtype=torch.int32, device=dev)
                _gemm(z, xs, dw, vocab, hidden, 0, a_mn=True, b_mn=True, mode=GEMM_GROUPED_K, group_rows=_rows_cache[key],
                      num_groups=1, accumulate=True, ldo=hidden)
        ctx.save_for_backward(dx, dw, weight)
        ctx.w_dtype = weight.dtype
        return stats[0] / stats[1]

    @staticmethod
    def backward(ctx, g):
        dx, dw, weight = ctx.saved_tensors
        gx = dx * g.to(dx.dtype) if dx is not None else None
        gw = None
        if dw is not None:
            sink = grad_sink(weight)
            if sink is not None:       # scale straight into the engine's fp32 buffer: no weight-sized temporaries, no dtype round trip
                if _sink_accumulates(sink):
                    sink[0].addcmul_(dw, g.to(dw.dtype))
                else:
                    torch.mul(dw, g.to(dw.dtype), out=sink[0])
                sink[1](weight)
            else:
                gw = (dw * g).to(ctx.w_dtype)
        return gx, gw, None


class _EmbeddingFn(torch.autograd.Function):
    """Token embedding by the own gather kernel; the gradient is scattered in fp32 (into the engine's buffer when there is one)."""

    @staticmethod
    def forward(ctx, ids, weight):
        w = weight.detach()
        w = w if w.is_contiguous() else w.contiguous()
        idc = ids if ids.is_contiguous() else ids.contiguous()
        ctx.save_for_backward(idc, weight)
        return ext().embedding_fwd(idc, w)

    @staticmethod
    def backward(ctx, dout):
        ids, weight = ctx.saved_tensors
        go = dout if dout.is_contiguous() else dout.contiguous()
        sink = grad_sink(weight)
        if sink is not None:
            if not _sink_accumulates(sink):
                sink[0].zero_()
            ext().embedding_bwd(ids, go, sink[0])
            sink[1](weight)
            return None, None
        dw = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
        ext().embedding_bwd(ids, go, dw)
        return None, dw.to(weight.dtype)


_dropout_calls = 0


def _next_dropout_seed() -> int:
    """Seed of the next fused dropout: a function of ``torch.initial_seed()`` and a call counter (no device sync, and two
    runs that seed torch identically and make the same calls get the same masks)."""

    global _dropout_calls
    _dropout_calls += 1
    return (torch.initial_seed() * 0x9E3779B97F4A7C15 + _dropout_calls * 0xD1B54A32D192ED03) & 0x7FFFFFFFFFFFFFFF


class _DropoutAddFn(torch.autograd.Function):
    """``residual + dropout(y)`` in one pass; the keep pattern is recomputed (not stored) in backward."""

    @staticmethod
    def forward(ctx, y, residual, p, seed):
        ctx.p, ctx.seed = p, seed
        return ext().dropout_add(y.contiguous(), residual.contiguous(), p, seed)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        gy = ext().dropout_add(g, None, ctx.p, ctx.seed) if ctx.needs_input_grad[0] else None
        return gy, (g if ctx.needs_input_grad[1] else None), None, None


def _split_bf16(t32: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    hi = t32.to(torch.bfloat16)
    lo = (t32 - hi.float()).to(torch.bfloat16)
    return hi, lo


class _RouterLogitsFn(torch.autograd.Function):
    """fp32 router logits ``x @ W^T`` on the tensor cores with fp32-grade accuracy.

    ``x`` is bf16 (exact); the fp32 weight is split into a bf16 high and low part stacked along the
    output dimension, so one GEMM with fp32 accumulation yields ``x W_hi^T`` and ``x W_lo^T`` whose sum
    matches the fp32 product to about 2^-17.  The weight gradient uses the same split on the incoming
    fp32 gradient.  (The reference runs this GEMM in fp32 through cuBLAS: minitrain/model/moe_router.py:64-73.)
    """

    @staticmethod
    def forward(ctx, x, weight):
        n_exp, hidden = weight.shape
        if weight.dtype == torch.bfloat16:
            # a bf16 replica of the parameter (sharded engines): it is its own high part and the low part is zero
            w_hi = weight.detach()
            w_hi = w_hi if w_hi.is_contiguous() else w_hi.contiguous()
            width = -(-n_exp // 4) * 4
            out = torch.empty(x.shape[0], width, dtype=torch.float32, device=x.device)
            _gemm(x, w_hi, out, x.shape[0], n_exp, hidden, ldo=width)
            ctx.save_for_backward(x, weight, None)
            return out if width == n_exp else out[:, :n_exp].contiguous()
        w_hi, w_lo = _split_bf16(weight.detach().float())
        stacked = torch.zeros(2 * n_exp, hidden, dtype=torch.bfloat16, device=x.device)
        stacked[:n_exp], stacked[n_exp:] = w_hi, w_lo
        width = -(-2 * n_exp // 4) * 4
        out = torch.empty(x.shape[0], width, dtype=torch.float32, device=x.device)
        _gemm(x, stacked, out, x.shape[0], 2 * n_exp, hidden, ldo=width)
        ctx.save_for_backward(x, weight, w_hi)
        return out[:, :n_exp] + out[:, n_exp:2 * n_exp]

    @staticmethod
    def backward(ctx, g):
        x, weight, w_hi = ctx.saved_tensors
        if w_hi is None:     # bf16 replica: read it through the parameter, whose storage may have moved since forward
            w_hi = weight.detach() if weight.is_contiguous() else weight.detach().contiguous()
        n_exp, hidden = weight.shape
        g32 = g.float()
        g_hi, g_lo = _split_bf16(g32)
        pad = -(-2 * n_exp // 8) * 8
        g2 = torch.zeros(x.shape[0], pad, dtype=torch.bfloat16, device=x.device)
        g2[:, :n_exp], g2[:, n_exp:2 * n_exp] = g_hi, g_lo
        dx = dw = None
        if ctx.needs_input_grad[0]:   # result is rounded to bf16 anyway: the high parts suffice
            if n_exp % 8 == 0:
                ga, wk = g2[:, :n_exp], w_hi
            else:
                kpad = -(-n_exp // 8) * 8
                ga = torch.zeros(x.shape[0], kpad, dtype=torch.bfloat16, device=x.device)
                ga[:, :n_exp] = g_hi
                wk = torch.cat([w_hi, w_hi.new_zeros(kpad - n_exp, hidden)])
            dx = gemm_nn(ga, wk, K=ga.shape[1])
        if ctx.needs_input_grad[1]:
            both = gemm_tn(g2, x, M=2 * n_exp)
            dw = (both[:n_exp] + both[n_exp:2 * n_exp]).to(weight.dtype)
        return dx, dw


class _RouterProjectionFn(torch.autograd.Function):
    """fp32 router logits by the skinny-GEMM kernels: ``x`` (bf16) is read once per pass, arithmetic is fp32 FMA.

    Replaces three launches of the 256-wide tcgen05 GEMM per layer (32-38 us each for 0.6 GFLOP) by kernels that take
    the time of reading ``x``.  The weight may be the fp32 parameter or a bf16 replica of it (sharded engines)."""

    @staticmethod
    def forward(ctx, x, weight):
        w = weight.detach()
        w = w if w.is_contiguous() else w.contiguous()
        ctx.save_for_backward(x, weight)
        return ext().router_logits_fwd(x, w)

    @staticmethod
    def backward(ctx, g):
        x, weight = ctx.saved_tensors       # the parameter itself: its storage may have moved since forward (staged units)
        w = weight.detach()
        w = w if w.is_contiguous() else w.contiguous()
        dx, dw = ext().router_logits_bwd(g.float().contiguous(), x, w, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        return dx, (dw.to(weight.dtype) if dw is not None else None)


class _RouterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, top_k, normalize):
        lg = logits.contiguous()
        w, idx, lse, sums, balance = ext().router_forward(lg, top_k, normalize)
        tokens, experts = lg.shape
        ctx.save_for_backward(lg, lse, idx, w)
        ctx.normalize = normalize
        counts = sums[experts + 2:]
        ctx.mark_non_differentiable(idx, counts, balance)
        scaled = sums[:experts + 2] * (1.0 / tokens)          # mean probability per expert, mean lse^2, mean entropy
        return w, idx, scaled[:experts], scaled[experts], scaled[experts + 1], counts, balance

    @staticmethod
    def backward(ctx, g_w, _g_idx, g_mp, g_z, _g_ent, _g_counts, _g_balance):
        lg, lse, idx, w = ctx.saved_tensors
        opt = lambda t: None if t is None else t.float().contiguous()  # noqa: E731
        gz = None if g_z is None else g_z.float().reshape(1).contiguous()
        return ext().router_backward(lg, lse, idx, w, opt(g_w), opt(g_mp), gz, ctx.normalize), None, None


# MTS_MOE_GATHER=1: the grouped GEMMs fetch the rows of the routed experts by index (TMA tile::gather4) instead of reading
# an expert-sorted copy, and fold the route weight into their SwiGLU epilogues.  Off by default: a gather4 copy moves four
# 128-byte rows per instruction against 16 KB for a tiled copy, and at the 293M model's shapes the gathered GEMMs ran 1.6x to
# 2.8x slower than the tiled ones (764 vs 298 us for the up projection), which costs far more than the copy kernels it removes.
MOE_GATHER = os.environ.get("MTS_MOE_GATHER", "0") == "1"


class _GatheredMoEFn(torch.autograd.Function):
    """Routed SwiGLU experts without an expert-sorted copy of the activations.

    forward    up projection: A rows gathered from ``x`` by the routing plan inside the GEMM; the epilogue applies SwiGLU AND the
               route weight (``post = w * silu(gate) * up``), so the down projection yields weighted rows and the combine is a
               plain sum over a token's routes
    backward   d(post) = dout[token] W_down with A gathered from ``dout``; the epilogue scales by the route weight, applies the
               SwiGLU derivative and accumulates the route-weight gradient ``<d(post), silu(gate) * up>`` per row; both weight
               gradients gather their activation operand (``dout`` rows, ``x`` rows) the same way
    Neither the sorted activations, the sorted output gradients nor the expert outputs are kept for backward."""

    @staticmethod
    def forward(ctx, x, gate_up_proj, down_proj, top_k_index, top_k_weights):
        e = ext()
        n_exp, two_i, hidden = gate_up_proj.shape
        inter = two_i // 2
        tokens, k = top_k_index.shape
        xc = x if x.is_contiguous() else x.contiguous()
        idx = top_k_index.to(torch.int32).contiguous()
        w16 = top_k_weights.to(torch.bfloat16).contiguous()
        gu16 = bf16_weight(gate_up_proj).view(n_exp * two_i, hidden)
        dn16 = bf16_weight(down_proj).view(n_exp * hidden, inter)
        row_token, token_rows, tile_group, group_rows, meta = e.moe_plan(idx, n_exp)
        row_weight, row_slot = e.moe_row_meta(row_token, token_rows, w16.view(-1), k)
        cap = row_token.numel()
        dev = x.device
        post = torch.empty(cap, inter, dtype=torch.bfloat16, device=dev)
        pre = torch.empty(cap, two_i, dtype=torch.bfloat16, device=dev)
        tiles = meta[0:1]
        _gemm(xc, gu16, post, cap, two_i, hidden, mode=GEMM_GROUPED_M, epilogue=EPI_SWIGLU, aux=pre, tile_group=tile_group,
              num_row_tiles=tiles, b_group_stride_rows=two_i, ldo=inter, gather_a=row_token, row_scale=row_weight, pair=True)
        y = torch.empty(cap, hidden, dtype=torch.bfloat16, device=dev)
        _gemm(post, dn16, y, cap, hidden, inter, mode=GEMM_GROUPED_M, tile_group=tile_group, num_row_tiles=tiles,
              b_group_stride_rows=hidden, ldo=hidden, pair=True)
        out = torch.empty(tokens, hidden, dtype=torch.bfloat16, device=dev)
        e.moe_combine(y, token_rows, None, out, k)            # rows are already weighted
        ctx.save_for_backward(xc, pre, post, row_token, token_rows, tile_group, group_rows, meta, row_weight, row_slot,
                              gate_up_proj, down_proj)
        ctx.dims = (n_exp, inter, hidden, tokens, k)
        ctx.w_dtype = top_k_weights.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        e = ext()
        (xc, pre, post, row_token, token_rows, tile_group, group_rows, meta, row_weight, row_slot, gate_up_proj,
         down_proj) = ctx.saved_tensors
        n_exp, inter, hidden, tokens, k = ctx.dims
        two_i = 2 * inter
        cap = row_token.numel()
        dev = dout.device
        gu16 = bf16_weight(gate_up_proj).view(n_exp * two_i, hidden)
        dn16 = bf16_weight(down_proj).view(n_exp * hidden, inter)
        tiles = meta[0:1]
        go = dout if dout.is_contiguous() else dout.contiguous()
        dwts = torch.zeros(tokens * k, dtype=torch.float32, device=dev)
        d_pre = torch.empty(cap, two_i, dtype=torch.bfloat16, device=dev)
        _gemm(go, dn16, d_pre, cap, inter, hidden, b_mn=True, mode=GEMM_GROUPED_M, epilogue=EPI_SWIGLU_BWD, aux=pre,
              tile_group=tile_group, num_row_tiles=tiles, b_group_stride_rows=hidden, ldo=two_i, gather_a=row_token,
              row_scale=row_weight, row_slot=row_slot, row_grad=dwts, pair=True)
        dx = dgu = ddn = None
        if ctx.needs_input_grad[0]:
            dxs = torch.empty(cap, hidden, dtype=torch.bfloat16, device=dev)
            _gemm(d_pre, gu16, dxs, cap, hidden, two_i, b_mn=True, mode=GEMM_GROUPED_M, tile_group=tile_group,
                  num_row_tiles=tiles, b_group_stride_rows=two_i, ldo=hidden, pair=True)
            dx = torch.empty(tokens, hidden, dtype=torch.bfloat16, device=dev)
            e.moe_combine(dxs, token_rows, None, dx, k)
        for which, param in ((1, gate_up_proj), (2, down_proj)):
            if not ctx.needs_input_grad[which]:
                continue
            rows_out, cols_out = (two_i, hidden) if which == 1 else (hidden, inter)
            sink = grad_sink(param)
            grad = sink[0] if sink is not None else torch.empty(n_exp, rows_out, cols_out, dtype=torch.float32, device=dev)
            splits = expert_wgrad_splits(cap, n_exp, rows_out, cols_out, dev)
            adds = splits > 1 or (sink is not None and _sink_accumulates(sink))
            if splits > 1 and not (sink is not None and _sink_accumulates(sink)):
                grad.zero_()
            common = dict(a_mn=True, b_mn=True, mode=GEMM_GROUPED_K, group_rows=group_rows, num_groups=n_exp,
                          out_group_stride=rows_out * cols_out, ldo=cols_out, k_splits=splits, atomic_out=adds, pair=True)
            if which == 1:      # d W_up[e] = sum_r d_pre[r]^T x[token(r)]
                _gemm(d_pre, xc, grad, two_i, hidden, 0, gather_b=row_token, **common)
            else:               # d W_down[e] = sum_r dout[token(r)]^T post[r]   (post carries the route weight)
                _gemm(go, post, grad, hidden, inter, 0, gather_a=row_token, **common)
            if sink is not None:
                sink[1](param)
            elif which == 1:
                dgu = grad.to(param.dtype)
            else:
                ddn = grad.to(param.dtype)
        dw = dwts.view(tokens, k).to(ctx.w_dtype) if ctx.needs_input_grad[4] else None
        return dx, dgu, ddn, None, dw


class _FusedMoEFn(torch.autograd.Function):
    """Routed SwiGLU experts as four grouped tcgen05 GEMMs around an expert-sorted, 128-row padded layout."""

    @staticmethod
    def forward(ctx, x, gate_up_proj, down_proj, top_k_index, top_k_weights):
        e = ext()
        n_exp, two_i, hidden = gate_up_proj.shape
        inter = two_i // 2
        tokens, k = top_k_index.shape
        xc = x if x.is_contiguous() else x.contiguous()
        idx = top_k_index.to(torch.int32).contiguous()
        w16 = top_k_weights.to(torch.bfloat16).contiguous()
        gu16 = bf16_weight(gate_up_proj).view(n_exp * two_i, hidden)
        dn16 = bf16_weight(down_proj).view(n_exp * hidden, inter)
        row_token, token_rows, tile_group, group_rows, meta = e.moe_plan(idx, n_exp)
        cap = row_token.numel()
        dev = x.device
        xs = torch.empty(cap, hidden, dtype=torch.bfloat16, device=dev)
        e.moe_gather(xc, row_token, xs, meta)
        post = torch.empty(cap, inter, dtype=torch.bfloat16, device=dev)
        pre = torch.empty(cap, two_i, dtype=torch.bfloat16, device=dev)
        tiles = meta[0:1]
        _gemm(xs, gu16, post, cap, two_i, hidden, mode=GEMM_GROUPED_M, epilogue=EPI_SWIGLU, aux=pre,
              tile_group=tile_group, num_row_tiles=tiles, b_group_stride_rows=two_i, ldo=inter)
        y = torch.empty(cap, hidden, dtype=torch.bfloat16, device=dev)
        _gemm(post, dn16, y, cap, hidden, inter, mode=GEMM_GROUPED_M, tile_group=tile_group, num_row_tiles=tiles,
              b_group_stride_rows=hidden, ldo=hidden)
        out = torch.empty(tokens, hidden, dtype=torch.bfloat16, device=dev)
        e.moe_combine(y, token_rows, w16, out, k)
        ctx.save_for_backward(xs, pre, post, y, w16, row_token, token_rows, tile_group, group_rows, meta,
                              gate_up_proj, down_proj)
        ctx.dims = (n_exp, inter, hidden, tokens, k)
        ctx.w_dtype = top_k_weights.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        e = ext()
        (xs, pre, post, y, w16, row_token, token_rows, tile_group, group_rows, meta, gate_up_proj,
         down_proj) = ctx.saved_tensors
        n_exp, inter, hidden, tokens, k = ctx.dims
        two_i = 2 * inter
        cap = row_token.numel()
        dev = dout.device
        gu16 = bf16_weight(gate_up_proj).view(n_exp * two_i, hidden)
        dn16 = bf16_weight(down_proj).view(n_exp * hidden, inter)
        tiles = meta[0:1]
        go = dout.contiguous()
        dys = torch.empty(cap, hidden, dtype=torch.bfloat16, device=dev)
        dwts = torch.zeros(tokens * k, dtype=torch.float32, device=dev)
        e.moe_combine_bwd(go, y, row_token, token_rows, w16, dys, dwts, meta, k)
        # d(post) = dys @ W_down, fused with the SwiGLU derivative -> d(pre) = [d gate | d up]
        d_pre = torch.empty(cap, two_i, dtype=torch.bfloat16, device=dev)
        _gemm(dys, dn16, d_pre, cap, inter, hidden, b_mn=True, mode=GEMM_GROUPED_M, epilogue=EPI_SWIGLU_BWD, aux=pre,
              tile_group=tile_group, num_row_tiles=tiles, b_group_stride_rows=hidden, ldo=two_i)
        dx = dgu = ddn = None
        if ctx.needs_input_grad[0]:
            dxs = torch.empty(cap, hidden, dtype=torch.bfloat16, device=dev)
            _gemm(d_pre, gu16, dxs, cap, hidden, two_i, b_mn=True, mode=GEMM_GROUPED_M, tile_group=tile_group,
                  num_row_tiles=tiles, b_group_stride_rows=two_i, ldo=hidden)
            dx = torch.empty(tokens, hidden, dtype=torch.bfloat16, device=dev)
            e.moe_combine(dxs, token_rows, None, dx, k)
        if ctx.needs_input_grad[1]:
            sink = grad_sink(gate_up_proj)
            dgu = sink[0] if sink is not None else torch.empty(n_exp, two_i, hidden, dtype=torch.float32, device=dev)
            splits = expert_wgrad_splits(cap, n_exp, two_i, hidden, dev)
            if splits > 1:
                dgu.zero_()
            _gemm(d_pre, xs, dgu, two_i, hidden, 0, a_mn=True, b_mn=True, mode=GEMM_GROUPED_K, group_rows=group_rows,
                  num_groups=n_exp, out_group_stride=two_i * hidden, ldo=hidden, k_splits=splits, atomic_out=splits > 1)
            if sink is not None:
                sink[1](gate_up_proj)
                dgu = None
            else:
                dgu = dgu.to(gate_up_proj.dtype)
        if ctx.needs_input_grad[2]:
            sink = grad_sink(down_proj)
            ddn = sink[0] if sink is not None else torch.empty(n_exp, hidden, inter, dtype=torch.float32, device=dev)
            splits = expert_wgrad_splits(cap, n_exp, hidden, inter, dev)
            if splits > 1:
                ddn.zero_()
            _gemm(dys, post, ddn, hidden, inter, 0, a_mn=True, b_mn=True, mode=GEMM_GROUPED_K, group_rows=group_rows,
                  num_groups=n_exp, out_group_stride=hidden * inter, ldo=inter, k_splits=splits, atomic_out=splits > 1)
            if sink is not None:
                sink[1](down_proj)
                ddn = None
            else:
                ddn = ddn.to(down_proj.dtype)
        dw = dwts.view(tokens, k).to(ctx.w_dtype) if ctx.needs_input_grad[4] else None
        return dx, dgu, ddn, None, dw


# ---------------------------------------------------------------------------------------------
# backend
# ---------------------------------------------------------------------------------------------
def _native_act(*tensors: torch.Tensor) -> bool:
    return all(t.is_cuda and t.dtype in (torch.bfloat16, torch.float32) for t in tensors)


class NativeOpsBackend(TorchOpsBackend):
    name = "native"

    def __init__(self) -> None:
        ext()
        self.dispatch = Counter()

    def _count(self, op: str, native: bool) -> bool:
        self.dispatch[f"{op}:{'native' if native else 'fallback'}"] += 1
        return native

    def dispatch_summary(self) -> dict[str, int]:
        return dict(self.dispatch)

    # -- embedding (optional hook outside the 8-op protocol; the model uses it when present) -----
    def embedding(self, input_ids, weight):
        """bf16 rows of ``weight`` for every id, or ``None`` when the inputs are not covered (the caller falls back)."""

        ok = (input_ids.is_cuda and input_ids.dtype == torch.long and weight.is_cuda and weight.dim() == 2
              and weight.shape[1] % 8 == 0 and weight.dtype in (torch.float32, torch.bfloat16))
        if not self._count("embedding", ok):
            return None
        return _EmbeddingFn.apply(input_ids, weight)

    # -- projections ------------------------------------------------------------------------
    def linear(self, x, weight):
        if self._count("linear", _gemm_ok(x, weight)):
            return _LinearFn.apply(x, weight)
        return torch.nn.functional.linear(x, weight.to(x.dtype) if weight.dtype != x.dtype and not torch.is_autocast_enabled() else weight)

    # -- memory-bound ops ---------------------------------------------------------------------
    def rmsnorm(self, x, weight, eps):
        ok = _native_act(x) and weight.is_cuda and x.shape[-1] % 8 == 0 and x.shape[-1] <= 1024
        if self._count("rmsnorm", ok):
            return _RMSNormFn.apply(x, weight, eps)
        return super().rmsnorm(x, weight, eps)

    def rmsnorm_residual(self, x, weight, eps):
        """``(rmsnorm(x), x)`` for a pre-norm block: the backward sums the norm's and the residual's gradient in one kernel."""

        ok = _native_act(x) and weight.is_cuda and x.shape[-1] % 8 == 0 and x.shape[-1] <= 1024
        if self._count("rmsnorm", ok):
            if torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad):
                return _RMSNormResidualFn.apply(x, weight, eps)
            return _RMSNormFn.apply(x, weight, eps), x
        return super().rmsnorm(x, weight, eps), x

    def rope(self, q, k, cos, sin):
        def aligned(t):
            vec = 8 if t.dtype == torch.bfloat16 else 4
            return (t.dim() == 4 and t.stride(3) == 1 and t.shape[3] % 16 == 0 and t.data_ptr() % 16 == 0
                    and all(s % vec == 0 for s in t.stride()[:3]))
        ok = (_native_act(q, k) and q.dtype == k.dtype and cos.dtype == q.dtype and cos.is_contiguous()
              and sin.is_contiguous() and aligned(q) and aligned(k))
        if self._count("rope", ok):
            return _RopeFn.apply(q, k, cos, sin)
        return super().rope(q, k, cos, sin)

    def swiglu(self, gate, up):
        ok = _native_act(gate, up) and gate.dtype == up.dtype and gate.shape == up.shape and gate.numel() % 8 == 0
        if self._count("swiglu", ok):
            return _SwigluFn.apply(gate, up)
        return super().swiglu(gate, up)

    def dropout_add(self, y, residual, p: float):
        """``residual + dropout(y, p)`` (optional hook outside the 8-op protocol; the blocks use it when present)."""

        ok = (_native_act(y, residual) and y.dtype == residual.dtype and y.shape == residual.shape and y.numel() % 8 == 0
              and 0.0 <= p < 1.0)
        if self._count("dropout_add", ok):
            if p == 0.0:
                return residual + y
            return _DropoutAddFn.apply(y, residual, float(p), _next_dropout_seed())
        return residual + torch.nn.functional.dropout(y, p, training=p > 0.0)

    def cross_entropy(self, logits, targets):
        ok = _native_act(logits) and logits.dim() == 2 and targets.is_cuda and targets.dtype == torch.long
        if self._count("cross_entropy", ok):
            return _CrossEntropyFn.apply(logits, targets)
        return super().cross_entropy(logits, targets)

    def fused_linear_cross_entropy(self, x, weight, targets):
        ok = _gemm_ok(x, weight) and x.dim() == 2 and targets.is_cuda and targets.dtype == torch.long
        if self._count("fused_linear_cross_entropy", ok):
            return _FusedLinearCEFn.apply(x, weight, targets)
        return super().fused_linear_cross_entropy(x, weight, targets)

    def router_logits(self, hidden_states, weight):
        ok = (hidden_states.is_cuda and hidden_states.dtype == torch.bfloat16 and hidden_states.dim() == 2
              and hidden_states.is_contiguous() and hidden_states.shape[1] % 8 == 0 and weight.shape[0] <= 64)
        if self._count("router_logits", ok):
            if ext().router_logits_ok(weight.shape[0], weight.shape[1]) and weight.dtype in (torch.float32, torch.bfloat16):
                return _RouterProjectionFn.apply(hidden_states, weight)
            return _RouterLogitsFn.apply(hidden_states, weight)
        return torch.nn.functional.linear(hidden_states.float(), weight.float())

    def router_postprocess(self, logits, top_k, *, normalize):
        check_router_args(logits, top_k)
        ok = logits.is_cuda and logits.shape[1] <= 64 and top_k <= 8
        if self._count("router_postprocess", ok):
            w, idx, mean_prob, z, ent, counts, balance = _RouterFn.apply(logits, top_k, normalize)
            return RouterPostprocessOutput(w, idx, mean_prob, z, ent.detach(), expert_counts=counts, balance_stats=balance)
        return super().router_postprocess(logits, top_k, normalize=normalize)

    def fused_moe(self, x, gate_up_proj, down_proj, top_k_index, top_k_weights):
        n_exp, two_i, hidden = gate_up_proj.shape
        ok = (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and hidden % 8 == 0 and two_i % 256 == 0
              and n_exp <= 64 and gate_up_proj.is_cuda)
        if self._count("fused_moe", ok):
            fn = _GatheredMoEFn if (MOE_GATHER and GEMM_PAIR and hidden % 64 == 0 and (two_i // 2) % 64 == 0) else _FusedMoEFn
            return fn.apply(x, gate_up_proj, down_proj, top_k_index, top_k_weights)
        return super().fused_moe(x, gate_up_proj, down_proj, top_k_index, top_k_weights)

    def attention_qkv(self, fused, cos, sin, *, is_causal, dropout_p):
        """Fused RoPE + attention on a ``[B, S, 3, H, D]`` projection; ``None`` when the inputs are not covered."""

        from mini_train_sys_b200.ops import native_attention

        if not self._count("attention_qkv", native_attention.qkv_supported(fused, cos, sin, dropout_p)):
            return None
        return native_attention.qkv_attention(fused, cos, sin, is_causal=is_causal, dropout_p=dropout_p)

    def attention(self, q, k, v, *, is_causal, dropout_p):
        from mini_train_sys_b200.ops import native_attention

        if self._count("attention", native_attention.supported(q, k, v, is_causal=is_causal, dropout_p=dropout_p)):
            return native_attention.flash_attention(q, k, v, is_causal=is_causal, dropout_p=dropout_p)
        return super().attention(q, k, v, is_causal=is_causal, dropout_p=dropout_p)


def scaled_dot_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)
