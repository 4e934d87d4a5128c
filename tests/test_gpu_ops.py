"""sm_100a kernels against the fp32 oracle (``ops/reference.py``).  All tests need a GPU."""

import math

import pytest
import torch

from mini_train_sys_b200.ops import reference as ref

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.fixture(scope="module")
def nb():
    from mini_train_sys_b200.ops import native_backend

    return native_backend


@pytest.fixture(scope="module")
def ops(nb):
    return nb.NativeOpsBackend()


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.float(), want.float()
    return float((got - want).norm() / want.norm().clamp_min(1e-12))


def assert_close(got, want, tol, what="", floor=0.0):
    """Relative L2 error; ``floor`` is an absolute norm below which the expected value counts as zero."""

    got, want = got.detach().float(), want.detach().float()
    diff = float((got - want).norm())
    scale = max(float(want.norm()), floor)
    err = diff / max(scale, 1e-30)
    assert math.isfinite(err) and err <= tol, f"{what}: relative L2 error {err:.3e} > {tol:.1e}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,hidden", [(1000, 768), (37, 128), (513, 1024)])
def test_rmsnorm(ops, dtype, rows, hidden):
    torch.manual_seed(0)
    x = torch.randn(rows, hidden, device=DEV, dtype=dtype, requires_grad=True)
    w = (1 + 0.1 * torch.randn(hidden, device=DEV)).requires_grad_()
    dy = torch.randn(rows, hidden, device=DEV, dtype=dtype)
    y = ops.rmsnorm(x, w, 1e-5)
    gx, gw = torch.autograd.grad(y, (x, w), dy)
    x64 = x.detach().double().requires_grad_()
    w64 = w.detach().double().requires_grad_()
    y64 = x64 * torch.rsqrt(x64.pow(2).mean(-1, keepdim=True) + 1e-5) * w64
    rx, rw = torch.autograd.grad(y64, (x64, w64), dy.double())
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
    assert_close(y, y64, tol, "y")
    assert_close(gx, rx, tol, "dx")
    assert_close(gw, rw, 5e-3 if dtype == torch.bfloat16 else 1e-4, "dw")
    assert ops.dispatch["rmsnorm:native"] > 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_rmsnorm_residual_sums_both_gradient_paths_in_the_kernel(ops, dtype):
    torch.manual_seed(3)
    rows, hidden = 777, 768
    x = torch.randn(rows, hidden, device=DEV, dtype=dtype, requires_grad=True)
    w = (1 + 0.1 * torch.randn(hidden, device=DEV)).requires_grad_()
    dy = torch.randn(rows, hidden, device=DEV, dtype=dtype)
    dres = torch.randn(rows, hidden, device=DEV, dtype=dtype)
    y, res = ops.rmsnorm_residual(x, w, 1e-5)
    assert res.data_ptr() == x.data_ptr()
    gx, gw = torch.autograd.grad((y, res), (x, w), (dy, dres))
    x64 = x.detach().double().requires_grad_()
    w64 = w.detach().double().requires_grad_()
    y64 = x64 * torch.rsqrt(x64.pow(2).mean(-1, keepdim=True) + 1e-5) * w64
    rx, rw = torch.autograd.grad((y64, x64 * 1.0), (x64, w64), (dy.double(), dres.double()))
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
    assert_close(gx, rx, tol, "dx")
    assert_close(gw, rw, 5e-3 if dtype == torch.bfloat16 else 1e-4, "dw")
    # only the residual branch used: the gradient passes through unchanged
    y2, res2 = ops.rmsnorm_residual(x, w, 1e-5)
    (gx2,) = torch.autograd.grad(res2, x, dres, allow_unused=True)
    assert torch.equal(gx2, dres)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_rope_strided(ops, dtype):
    from mini_train_sys_b200.models.rotary import rope_tables

    torch.manual_seed(1)
    b, s, h, d = 3, 130, 4, 64
    fused = torch.randn(b, s, 3, h, d, device=DEV, dtype=dtype, requires_grad=True)
    q, k = fused[:, :, 0].transpose(1, 2), fused[:, :, 1].transpose(1, 2)
    cos, sin = (t.to(DEV).to(dtype) for t in rope_tables(d, 256, 10000.0))
    qo, ko = ops.rope(q, k, cos[:s], sin[:s])
    assert qo.is_contiguous() and qo.shape == (b, h, s, d)
    dq, dk = torch.randn_like(qo), torch.randn_like(ko)
    (g,) = torch.autograd.grad((qo, ko), fused, (dq, dk))
    f64 = fused.detach().double().requires_grad_()
    q64, k64 = f64[:, :, 0].transpose(1, 2), f64[:, :, 1].transpose(1, 2)
    rq, rk = ref.rope_ref(q64, cos[:s].double(), sin[:s].double()), ref.rope_ref(k64, cos[:s].double(), sin[:s].double())
    (rg,) = torch.autograd.grad((rq.double(), rk.double()), f64, (dq.double(), dk.double()))
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
    assert_close(qo, rq, tol, "q")
    assert_close(ko, rk, tol, "k")
    assert_close(g, rg, tol, "grad")


def test_swiglu(ops):
    torch.manual_seed(2)
    g = torch.randn(777, 1024, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    u = torch.randn(777, 1024, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    dy = torch.randn_like(g)
    y = ops.swiglu(g, u)
    gg, gu = torch.autograd.grad(y, (g, u), dy)
    g64, u64 = g.detach().double().requires_grad_(), u.detach().double().requires_grad_()
    y64 = torch.nn.functional.silu(g64) * u64
    rg, ru = torch.autograd.grad(y64, (g64, u64), dy.double())
    assert_close(y, y64, 1e-2, "y")
    assert_close(gg, rg, 1e-2, "dgate")
    assert_close(gu, ru, 1e-2, "dup")


@pytest.mark.parametrize("rows,vocab,dtype", [(64, 50257, torch.bfloat16), (33, 1000, torch.float32), (8, 7, torch.float32)])
def test_cross_entropy(ops, rows, vocab, dtype):
    torch.manual_seed(3)
    logits = (2 * torch.randn(rows, vocab, device=DEV)).to(dtype).requires_grad_()
    targets = torch.randint(0, vocab, (rows,), device=DEV)
    targets[::5] = -100
    loss = ops.cross_entropy(logits, targets)
    (g,) = torch.autograd.grad(loss, logits)
    l64 = logits.detach().double().requires_grad_()
    want = torch.nn.functional.cross_entropy(l64, targets)
    (rg,) = torch.autograd.grad(want, l64)
    assert abs(float(loss) - float(want)) < 2e-3 * max(1.0, abs(float(want)))
    assert_close(g, rg, 2e-2 if dtype == torch.bfloat16 else 1e-4, "dlogits")


@pytest.mark.parametrize("tokens,experts,k,normalize", [(257, 64, 2, True), (4096, 8, 2, True), (100, 4, 1, False), (50, 8, 3, False)])
def test_router(ops, tokens, experts, k, normalize):
    torch.manual_seed(4)
    logits = torch.randn(tokens, experts, device=DEV, requires_grad=True)
    out = ops.router_postprocess(logits, k, normalize=normalize)
    want = ref.router_ref(logits.detach().double().float().requires_grad_(), k, normalize)
    assert torch.equal(out.expert_indices.sort(-1).values, want.expert_indices.sort(-1).values)
    assert_close(out.expert_weights, want.expert_weights, 1e-5, "weights")
    assert_close(out.probability_per_expert, want.probability_per_expert, 1e-5, "mean prob")
    assert abs(float(out.z_loss) - float(want.z_loss)) < 1e-4 * max(1.0, float(want.z_loss))
    assert abs(float(out.entropy) - float(want.entropy)) < 1e-4
    # route counts and load-balance figures come from the routing kernels themselves
    counts = torch.bincount(out.expert_indices.reshape(-1).long(), minlength=experts).float()
    assert torch.equal(out.expert_counts, counts)
    load = counts / (tokens * k)
    want_stats = torch.stack([counts.max(), counts.min(), load.std(unbiased=False) * experts, load.max() * experts,
                              (counts == 0).sum().float()])
    assert_close(out.balance_stats[:5], want_stats, 1e-5, "balance figures")
    assert_close(out.balance_stats[5:], load, 1e-6, "load fractions")
    # combined gradient through all three differentiable outputs
    gw = torch.randn_like(out.expert_weights)
    gp = torch.randn(experts, device=DEV)
    l32 = logits.detach().clone().requires_grad_()
    w2 = ref.router_ref(l32, k, normalize)
    obj_ref = (w2.expert_weights * gw).sum() + (w2.probability_per_expert * gp).sum() + 0.7 * w2.z_loss
    (rg,) = torch.autograd.grad(obj_ref, l32)
    obj = (out.expert_weights * gw).sum() + (out.probability_per_expert * gp).sum() + 0.7 * out.z_loss
    (g,) = torch.autograd.grad(obj, logits)
    assert_close(g, rg, 1e-4, "dlogits")


GEMM_SHAPES = [(128, 256, 64), (256, 512, 128), (300, 520, 136), (1024, 768, 768), (4096, 2304, 768), (77, 8, 8),
               (129, 257, 72)]


@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
def test_gemm_nt(nb, m, n, k):
    torch.manual_seed(5)
    a = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(n, k, device=DEV, dtype=torch.bfloat16)
    n_pad = -(-n // 8) * 8
    out = torch.full((m, n_pad), 7.0, device=DEV, dtype=torch.bfloat16)
    nb._gemm(a, b, out, m, n, k, ldo=n_pad)
    want = a.float() @ b.float().t()
    assert_close(out[:, :n], want, 1e-2, f"nt {m}x{n}x{k}")
    pad = out[:, n:]     # inside the row pitch up to the next 16-byte boundary: left alone or zeroed, never garbage
    assert bool(((pad == 7.0) | (pad == 0.0)).all()), "columns beyond N hold garbage"
    nb.check_kernel_status()


@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
def test_gemm_nn(nb, m, n, k):
    torch.manual_seed(6)
    n8 = -(-n // 8) * 8
    a = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(k, n8, device=DEV, dtype=torch.bfloat16)
    out = nb.gemm_nn(a, b)
    assert_close(out, a.float() @ b.float(), 1e-2, f"nn {m}x{n8}x{k}")
    nb.check_kernel_status()


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (768, 2304, 4096), (200, 136, 1000), (2304, 768, 20000), (50, 72, 130)])
def test_gemm_tn(nb, m, n, k):
    torch.manual_seed(7)
    m8, n8 = -(-m // 8) * 8, -(-n // 8) * 8
    a = torch.randn(k, m8, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(k, n8, device=DEV, dtype=torch.bfloat16)
    out = nb.gemm_tn(a, b)
    assert out.dtype == torch.float32
    assert_close(out, a.float().t() @ b.float(), 1e-2, f"tn {m8}x{n8}x{k}")
    nb.check_kernel_status()


def test_linear_autograd(ops):
    torch.manual_seed(8)
    x = torch.randn(4, 130, 768, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (0.02 * torch.randn(2304, 768, device=DEV)).requires_grad_()
    dy = torch.randn(4, 130, 2304, device=DEV, dtype=torch.bfloat16)
    y = ops.linear(x, w)
    gx, gw = torch.autograd.grad(y, (x, w), dy)
    x64, w64 = x.detach().double().requires_grad_(), w.detach().double().requires_grad_()
    y64 = x64 @ w64.t()
    rx, rw = torch.autograd.grad(y64, (x64, w64), dy.double())
    assert gw.dtype == torch.float32
    assert_close(y, y64, 1e-2, "y")
    assert_close(gx, rx, 1.5e-2, "dx")
    assert_close(gw, rw, 1e-2, "dw")
    assert ops.dispatch["linear:native"] > 0


@pytest.mark.parametrize("rows,vocab,hidden,chunk", [(300, 1000, 128, 128), (1024, 50257, 768, 512)])
def test_fused_linear_cross_entropy(ops, monkeypatch, rows, vocab, hidden, chunk):
    monkeypatch.setenv("MTS_FUSED_CE_CHUNK_ROWS", str(chunk))
    torch.manual_seed(9)
    x = torch.randn(rows, hidden, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (0.05 * torch.randn(vocab, hidden, device=DEV)).requires_grad_()
    t = torch.randint(0, vocab, (rows,), device=DEV)
    t[::7] = -100
    loss = ops.fused_linear_cross_entropy(x, w, t)
    gx, gw = torch.autograd.grad(loss * 1.5, (x, w))
    x64, w64 = x.detach().double().requires_grad_(), w.detach().to(torch.bfloat16).double().requires_grad_()
    want = torch.nn.functional.cross_entropy(x64 @ w64.t(), t)
    rx, rw = torch.autograd.grad(want * 1.5, (x64, w64))
    assert abs(float(loss) - float(want)) < 5e-3 * max(1.0, abs(float(want)))
    assert_close(gx, rx, 3e-2, "dx")
    assert_close(gw, rw, 3e-2, "dw")


def _skewed_routes(tokens, experts, k, mode):
    if mode == "uniform":
        scores = torch.rand(tokens, experts, device=DEV)
    elif mode == "one_expert":
        scores = torch.rand(tokens, experts, device=DEV)
        scores[:, 1] += 10
    else:  # "empty": experts 0 and 3 never chosen
        scores = torch.rand(tokens, experts, device=DEV)
        scores[:, 0] -= 10
        scores[:, 3] -= 10
    idx = scores.topk(k, -1).indices.to(torch.int32)
    w = torch.rand(tokens, k, device=DEV)
    return idx, w / w.sum(-1, keepdim=True)


@pytest.mark.parametrize("mode", ["uniform", "one_expert", "empty"])
def test_moe_plan(nb, mode):
    torch.manual_seed(10)
    tokens, experts, k = 1500, 8, 2
    idx, _ = _skewed_routes(tokens, experts, k, mode)
    row_token, token_rows, tile_group, group_rows, meta = nb.ext().moe_plan(idx.contiguous(), experts)
    rt, tr, tg, gr, mt = (t.cpu() for t in (row_token, token_rows, tile_group, group_rows, meta))
    counts = torch.bincount(idx.flatten().long().cpu(), minlength=experts)
    assert int(mt[2]) == 0
    padded = (counts + 255) // 256 * 256     # two 128-row tiles: a 256-row work item of the paired GEMM stays inside one expert
    assert gr.tolist() == [0, *padded.cumsum(0).tolist()]
    assert int(mt[1]) == int(padded.sum()) and int(mt[0]) == int(padded.sum()) // 128
    flat = idx.flatten().cpu()
    assert tr.min() >= 0 and tr.unique().numel() == tokens * k
    for route in range(0, tokens * k, 97):
        row = int(tr[route])
        e = int(flat[route])
        assert gr[e] <= row < gr[e] + counts[e]
        assert int(rt[row]) == route // k
        assert int(tg[row // 128]) == e
    live = rt[: int(mt[1])]
    assert int((live >= 0).sum()) == tokens * k
    # token order is preserved inside every expert
    for e in range(experts):
        seg = rt[int(gr[e]): int(gr[e]) + int(counts[e])]
        assert bool((seg[1:] >= seg[:-1]).all())


@pytest.mark.parametrize("gathered", [True, False])
@pytest.mark.parametrize("mode", ["uniform", "one_expert", "empty"])
@pytest.mark.parametrize("tokens,hidden,inter,experts", [(1000, 128, 128, 4), (2048, 768, 1024, 8), (12288, 768, 1024, 8)])
def test_fused_moe(nb, ops, monkeypatch, mode, tokens, hidden, inter, experts, gathered):
    """Both forms of the routed experts: activations gathered by index inside the grouped GEMMs, and through a sorted copy."""

    monkeypatch.setattr(nb, "MOE_GATHER", gathered)
    torch.manual_seed(11)
    k = 2
    x = torch.randn(tokens, hidden, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    gu = (0.05 * torch.randn(experts, 2 * inter, hidden, device=DEV)).requires_grad_()
    dn = (0.05 * torch.randn(experts, hidden, inter, device=DEV)).requires_grad_()
    idx, w = _skewed_routes(tokens, experts, k, mode)
    w = w.to(torch.bfloat16).requires_grad_()
    dout = torch.randn(tokens, hidden, device=DEV, dtype=torch.bfloat16)
    out = ops.fused_moe(x, gu, dn, idx, w)
    gx, ggu, gdn, gw = torch.autograd.grad(out, (x, gu, dn, w), dout)
    leaves = [t.detach().float().requires_grad_() for t in (x, gu.to(torch.bfloat16), dn.to(torch.bfloat16), w)]
    want = ref.moe_ref(*leaves[:3], idx, leaves[3])
    rx, rgu, rdn, rw = torch.autograd.grad(want, leaves, dout.float())
    assert_close(out, want, 2e-2, "out")
    assert_close(gx, rx, 3e-2, "dx")
    assert_close(ggu, rgu, 3e-2, "d gate_up")
    assert_close(gdn, rdn, 3e-2, "d down")
    assert_close(gw, rw, 3e-2, "d route weights")
    assert ops.dispatch["fused_moe:native"] > 0


@pytest.mark.parametrize("splits", [2, 3, 5])
def test_grouped_k_gemm_with_split_groups(nb, splits):
    """Per-expert weight gradients with every expert's rows cut into parts that add into the expert's output."""

    torch.manual_seed(21)
    groups, m, n = 4, 768, 512
    sizes = [1280, 256, 0, 2048]                 # rows per group (multiples of 256, one of them empty)
    bounds = torch.tensor([0, *torch.tensor(sizes).cumsum(0).tolist()], dtype=torch.int32, device=DEV)
    rows = int(bounds[-1])
    a = torch.randn(rows, m, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(rows, n, device=DEV, dtype=torch.bfloat16)
    canary = 7.0
    buf = torch.full((groups * m * n + 2 * 1024,), canary, device=DEV)
    out = buf[1024:1024 + groups * m * n].view(groups, m, n)
    out.zero_()
    nb._gemm(a, b, out, m, n, 0, a_mn=True, b_mn=True, mode=nb.GEMM_GROUPED_K, group_rows=bounds, num_groups=groups,
             out_group_stride=m * n, ldo=n, k_splits=splits, atomic_out=True)
    torch.cuda.synchronize()
    assert bool((buf[:1024] == canary).all()) and bool((buf[-1024:] == canary).all()), "wrote outside the output"
    for gi in range(groups):
        lo, hi = int(bounds[gi]), int(bounds[gi + 1])
        want = a[lo:hi].float().t() @ b[lo:hi].float()
        assert_close(out[gi], want, 5e-3, f"group {gi}", floor=1e-3)
    nb.check_kernel_status()


def test_adamw_matches_torch(nb):
    torch.manual_seed(12)
    n = 100_003
    p = torch.randn(n + 1, device=DEV)[:n].clone()
    g = torch.randn(n, device=DEV)
    ref_p = p.clone().requires_grad_()
    opt = torch.optim.AdamW([ref_p], lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    shadow = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    for step in (1, 2, 3):
        ref_p.grad = g.clone() * 0.5
        opt.step()
        nb.ext().adamw_step(p, g, m, v, shadow, 1e-3, 0.9, 0.95, 1e-8, 0.1, step, None, 0.5)
    assert_close(p, ref_p.detach(), 1e-5, "adamw params")
    assert_close(shadow, ref_p.detach(), 1e-2, "bf16 shadow")


def test_tiny_model_matches_torch_backend():
    from mini_train_sys_b200.models import MiniTransformer, ModelConfig, get_ops_backend

    cfg = ModelConfig(vocab_size=1000, seq_len=128, n_layers=2, n_heads=4, hidden_size=256, intermediate_size=256,
                      ffn_type="moe", num_experts=4, experts_per_token=2, tie_word_embeddings=True)
    tokens = torch.randint(0, 1000, (4, 129), device=DEV)
    losses, grads = {}, {}
    for name in ("torch", "native"):
        torch.manual_seed(0)
        model = MiniTransformer(cfg, get_ops_backend(name), activation_dtype=torch.bfloat16).to(DEV)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss, _ = model(tokens[:, :-1], targets=tokens[:, 1:], use_fused_loss=True)
        loss.backward()
        losses[name] = float(loss)
        grads[name] = {n: p.grad.float().clone() for n, p in model.named_parameters()}
    assert abs(losses["torch"] - losses["native"]) < 2e-2, losses
    errors = {n: rel_err(grads["native"][n], g) for n, g in grads["torch"].items()}
    # router gradients are differences of nearly equal bf16 terms in both back ends, hence the wider band
    bad = {n: round(e, 4) for n, e in errors.items() if not e < (0.25 if "router" in n else 0.1)}
    assert not bad, f"gradient mismatch: {bad}"


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("b,h,s", [(2, 3, 128), (2, 2, 512), (1, 2, 130), (1, 1, 67), (2, 2, 1), (1, 2, 333)])
def test_flash_attention(causal, b, h, s):
    from mini_train_sys_b200.ops import native_attention as na

    torch.manual_seed(13)
    fused = torch.randn(b, s, 3, h, 64, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    q, k, v = (fused[:, :, j].transpose(1, 2) for j in range(3))
    assert na.supported(q, k, v, is_causal=causal, dropout_p=0.0)
    out = na.flash_attention(q, k, v, is_causal=causal, dropout_p=0.0)
    d_o = torch.randn(b, h, s, 64, device=DEV, dtype=torch.bfloat16)
    (g,) = torch.autograd.grad(out, fused, d_o)
    f32 = fused.detach().float().requires_grad_()
    q32, k32, v32 = (f32[:, :, j].transpose(1, 2) for j in range(3))
    want = ref.attention_ref(q32, k32, v32, is_causal=causal)
    (rg,) = torch.autograd.grad(want, f32, d_o.float())
    assert_close(out, want, 2e-2, "out")
    floor = 1e-3 * float(d_o.float().norm())   # with one key the softmax is constant and dq, dk vanish
    for j, name in enumerate("qkv"):
        assert_close(g[:, :, j], rg[:, :, j], 3e-2, f"d{name}", floor=floor)
    from mini_train_sys_b200.ops.native_backend import check_kernel_status

    check_kernel_status()


def _attention_against_fp32(b, h, s, causal, tol_out=2e-2, tol_grad=3e-2):
    from mini_train_sys_b200.ops import native_attention as na

    fused = torch.randn(b, s, 3, h, 64, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    q, k, v = (fused[:, :, j].transpose(1, 2) for j in range(3))
    out = na.flash_attention(q, k, v, is_causal=causal, dropout_p=0.0)
    d_o = torch.randn(b, h, s, 64, device=DEV, dtype=torch.bfloat16)
    (g,) = torch.autograd.grad(out, fused, d_o)
    f32 = fused.detach().float().requires_grad_()
    q32, k32, v32 = (f32[:, :, j].transpose(1, 2) for j in range(3))
    want = ref.attention_ref(q32, k32, v32, is_causal=causal)
    (rg,) = torch.autograd.grad(want, f32, d_o.float())
    assert_close(out, want, tol_out, f"out s={s}")
    floor = 1e-3 * float(d_o.float().norm())
    for j, name in enumerate("qkv"):
        assert_close(g[:, :, j], rg[:, :, j], tol_grad, f"d{name} s={s}", floor=floor)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("b,h,s", [(24, 12, 512), (2, 12, 2048), (32, 12, 384), (40, 8, 200)])
def test_flash_attention_many_items_per_cta(causal, b, h, s):
    """Shapes with more work items than resident CTAs: the persistent forward walks several (query tile, batch x head) items per
    CTA (barrier phases, the K / V buffers and the two O buffers in tensor memory wrap around), with an even and an odd number of
    query tiles, a ragged last tile, and 16 key tiles per item."""

    from mini_train_sys_b200.ops.native_backend import check_kernel_status

    torch.manual_seed(31)
    _attention_against_fp32(b, h, s, causal)
    check_kernel_status()


def test_flash_attention_every_length_up_to_130():
    """Every sequence length from 1 to 130: all ragged-edge positions of the first and the second 128-row tile."""

    from mini_train_sys_b200.ops.native_backend import check_kernel_status

    torch.manual_seed(32)
    for s in range(1, 131):
        _attention_against_fp32(1, 2, s, True)
    for s in (1, 2, 63, 64, 65, 127, 128, 129, 130):
        _attention_against_fp32(1, 2, s, False)
    check_kernel_status()


@pytest.mark.parametrize("b,h,s,p", [(2, 2, 200, 0.1), (1, 3, 512, 0.1), (3, 2, 1000, 0.25)])
def test_flash_attention_dropout_replay(b, h, s, p):
    from mini_train_sys_b200.ops import native_attention as na

    torch.manual_seed(14)
    seed = 1234567
    q, k, v = (torch.randn(b, h, s, 64, device=DEV, dtype=torch.bfloat16, requires_grad=True) for _ in range(3))
    out = na.flash_attention(q, k, v, is_causal=True, dropout_p=p, seed=seed)
    d_o = torch.randn_like(out)
    gq, gk, gv = torch.autograd.grad(out, (q, k, v), d_o)
    keep = na.keep_mask(b * h, s, p, seed, DEV).view(b, h, s, s)
    p_eff = na.effective_dropout(p)
    rate = 1.0 - keep.float().mean().item()
    assert abs(rate - p_eff) < 0.01, rate
    leaves = [t.detach().float().requires_grad_() for t in (q, k, v)]
    want = ref.attention_ref(*leaves, is_causal=True, keep_mask=keep, dropout_p=p_eff)
    rq, rk, rv = torch.autograd.grad(want, leaves, d_o.float())
    assert_close(out, want, 2e-2, "out")
    assert_close(gq, rq, 3e-2, "dq")
    assert_close(gk, rk, 3e-2, "dk")
    assert_close(gv, rv, 3e-2, "dv")
    # the same seed reproduces the pattern, a different seed changes it
    again = na.flash_attention(q, k, v, is_causal=True, dropout_p=p, seed=seed)
    other = na.flash_attention(q, k, v, is_causal=True, dropout_p=p, seed=seed + 1)
    assert torch.equal(again, out) and not torch.equal(other, out)


def test_attention_capability_contract():
    from mini_train_sys_b200.ops import native_attention as na

    ok = torch.randn(1, 2, 16, 64, device=DEV, dtype=torch.bfloat16)
    assert na.supported(ok, ok, ok, is_causal=True, dropout_p=0.0)
    assert not na.supported(ok.float(), ok.float(), ok.float(), is_causal=True, dropout_p=0.0)
    d128 = torch.randn(1, 2, 16, 128, device=DEV, dtype=torch.bfloat16)
    assert not na.supported(d128, d128, d128, is_causal=True, dropout_p=0.0)
    assert not na.supported(ok, ok[:, :, :8], ok, is_causal=True, dropout_p=0.0)
    assert not na.supported(ok, ok, ok, is_causal=True, dropout_p=1.0)
    assert not na.supported(ok.cpu(), ok.cpu(), ok.cpu(), is_causal=True, dropout_p=0.0)
    odd = torch.randn(1, 2, 16, 65, device=DEV, dtype=torch.bfloat16)[..., 1:]
    assert not na.supported(odd, odd, odd, is_causal=True, dropout_p=0.0)


@pytest.mark.parametrize("w_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,experts,hidden", [(3000, 8, 768), (777, 4, 256), (1025, 16, 384), (513, 6, 768)])
def test_router_logits_split_gemm(ops, w_dtype, tokens, experts, hidden):
    """Router projection: the skinny fp32 kernels for 4 / 8 / 16 experts, the split-bf16 tensor-core GEMM otherwise."""

    torch.manual_seed(15)
    x = torch.randn(tokens, hidden, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (0.02 * torch.randn(experts, hidden, device=DEV)).to(w_dtype).requires_grad_()
    g = torch.randn(tokens, experts, device=DEV)
    logits = ops.router_logits(x, w)
    gx, gw = torch.autograd.grad(logits, (x, w), g)
    x64, w64 = x.detach().double().requires_grad_(), w.detach().double().requires_grad_()
    want = x64 @ w64.t()
    rx, rw = torch.autograd.grad(want, (x64, w64), g.double())
    assert logits.dtype == torch.float32
    assert_close(logits, want, 2e-5, "logits")
    assert_close(gw, rw, 2e-5 if w_dtype == torch.float32 else 1e-2, "dW")     # a bf16 weight gets a bf16 gradient
    assert_close(gx, rx, 1e-2, "dx")


def test_qkv_attention_fused_path(ops):
    from mini_train_sys_b200.models.rotary import rope_tables

    torch.manual_seed(16)
    b, s, h = 2, 300, 4
    fused = torch.randn(b, s, 3, h, 64, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    cos, sin = (t[:s].to(DEV).to(torch.bfloat16).contiguous() for t in rope_tables(64, 512, 10000.0))
    out = ops.attention_qkv(fused, cos, sin, is_causal=True, dropout_p=0.0)
    assert out is not None and out.shape == (b, h, s, 64)
    d_o = torch.randn_like(out)
    (g,) = torch.autograd.grad(out, fused, d_o)
    f32 = fused.detach().float().requires_grad_()
    q, k, v = (f32[:, :, j].transpose(1, 2) for j in range(3))
    want = ref.attention_ref(ref.rope_ref(q, cos, sin), ref.rope_ref(k, cos, sin), v, is_causal=True)
    (rg,) = torch.autograd.grad(want, f32, d_o.float())
    assert_close(out, want, 2e-2, "out")
    assert_close(g, rg, 3e-2, "d fused qkv")


def test_dropout_add_masks_agree_between_passes(ops):
    torch.manual_seed(21)
    # |y| in [1, 2) and |res| < 1: a kept element always changes the sum visibly in bf16, so the mask can be read off the output
    y = ((1 + torch.rand(4096, 768, device=DEV)) * torch.where(torch.rand(4096, 768, device=DEV) < 0.5, -1.0, 1.0)).to(torch.bfloat16).requires_grad_()
    res = (torch.rand(4096, 768, device=DEV) * 1.8 - 0.9).to(torch.bfloat16).requires_grad_()
    p = 0.1
    out = ops.dropout_add(y, res, p)
    g = torch.randn_like(out)
    out.backward(g)
    kept = (out.detach().float() - res.detach().float()).abs() > 0          # y is never exactly zero
    rate = 1.0 - kept.float().mean().item()
    p_eff = round(p * 256) / 256
    assert abs(rate - p_eff) < 2e-3, rate
    scale = 1.0 / (1.0 - p_eff)
    want = torch.where(kept, y.detach().float() * scale, torch.zeros_like(y, dtype=torch.float32)) + res.detach().float()
    assert_close(out, want, 1e-2, "dropout_add forward")
    assert_close(y.grad, torch.where(kept, g.float() * scale, torch.zeros_like(g, dtype=torch.float32)), 1e-2, "dropout_add dy")
    assert torch.equal(res.grad, g)
    out2 = ops.dropout_add(y.detach(), res.detach(), p)                      # a new call draws a new mask
    assert not torch.equal(out2, out.detach())
    assert torch.equal(ops.dropout_add(y.detach(), res.detach(), 0.0), res.detach() + y.detach())


def test_moe_plan_and_fused_moe_skip_dropped_routes(nb, ops):
    """Expert id -1 marks a dropped route (capacity overflow, empty exchange slot): it gets no row and contributes nothing."""

    torch.manual_seed(12)
    tokens, experts, k, hidden, inter = 3000, 8, 2, 256, 256
    idx, w = _skewed_routes(tokens, experts, k, "uniform")
    drop = torch.rand(tokens, k, device=DEV) < 0.3
    dropped = torch.where(drop, torch.full_like(idx, -1), idx)
    row_token, token_rows, tile_group, group_rows, meta = nb.ext().moe_plan(dropped.contiguous(), experts)
    tr = token_rows.view(tokens, k)
    assert bool((tr[drop] == -1).all()) and bool((tr[~drop] >= 0).all())
    counts = torch.bincount(idx[~drop].long(), minlength=experts)
    assert int(meta[1]) == int(((counts + 255) // 256 * 256).sum())
    x = torch.randn(tokens, hidden, device=DEV, dtype=torch.bfloat16)
    gu = (torch.randn(experts, 2 * inter, hidden, device=DEV) * 0.05).requires_grad_()
    dn = (torch.randn(experts, hidden, inter, device=DEV) * 0.05).requires_grad_()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        got = ops.fused_moe(x, gu, dn, dropped, w)
        want = ops.fused_moe(x, gu, dn, idx, torch.where(drop, torch.zeros_like(w), w))
    assert_close(got, want, 2e-2, "fused_moe with dropped routes")
    nb.check_kernel_status()


@pytest.mark.parametrize("w_dtype", [torch.float32, torch.bfloat16])
def test_embedding_gather_and_scatter_add(ops, w_dtype):
    torch.manual_seed(31)
    vocab, hidden = 1003, 264
    w = torch.randn(vocab, hidden, device=DEV).to(w_dtype).requires_grad_()
    ids = torch.randint(0, vocab, (7, 129), device=DEV)
    ids[0, :40] = 5                                        # many tokens on one row: the reductions must not lose updates
    out = ops.embedding(ids, w)
    assert out.dtype == torch.bfloat16 and out.shape == (7, 129, hidden)
    assert torch.equal(out, w.detach().to(torch.bfloat16)[ids])
    g = torch.randn_like(out)
    (gw,) = torch.autograd.grad(out, w, g)
    want = torch.zeros(vocab, hidden, device=DEV, dtype=torch.float64)
    want.index_add_(0, ids.reshape(-1), g.reshape(-1, hidden).double())
    assert_close(gw, want, 1e-6 if w_dtype == torch.float32 else 5e-3, "dW")
    # the engine protocol: gradients ADDED into a flat fp32 buffer that already holds another contribution
    sink = torch.ones(vocab, hidden, device=DEV)
    calls = []
    w._mts_grad_sink = (sink, calls.append, True)
    out2 = ops.embedding(ids, w)
    assert torch.autograd.grad(out2, w, g, allow_unused=True)[0] is None and len(calls) == 1
    assert_close(sink, want + 1.0, 1e-6, "sink")


def test_embedding_refuses_ids_outside_the_vocabulary_without_touching_memory(nb, ops):
    w = torch.randn(64, 128, device=DEV)
    ids = torch.tensor([[1, 70, -3, 2]], device=DEV)
    out = ops.embedding(ids, w)
    torch.cuda.synchronize()
    assert torch.equal(out[0, 1], torch.zeros(128, device=DEV, dtype=torch.bfloat16)) and float(out[0, 0].float().abs().sum()) > 0
    with pytest.raises(RuntimeError, match="status 2"):
        nb.check_kernel_status()
    nb.ext().status_tensor(0).zero_()
    nb.check_kernel_status()


# ---- determinism and out-of-bounds guards (what a memory checker would otherwise report) -------------------------------

def _twice(fn):
    a = fn()
    torch.cuda.synchronize()
    b = fn()
    torch.cuda.synchronize()
    a, b = (a if isinstance(a, (tuple, list)) else (a,)), (b if isinstance(b, (tuple, list)) else (b,))
    for i, (x, y) in enumerate(zip(a, b)):
        assert torch.equal(x, y), f"output {i} differs between two identical launches"


def test_kernels_documented_as_deterministic_repeat_bit_for_bit(nb, ops):
    """Attention (forward and both backward sweeps), RMSNorm, the router, its projection and the routing plan have no
    atomics on their result paths: two launches on the same inputs must agree exactly."""

    from mini_train_sys_b200.ops import native_attention

    torch.manual_seed(41)
    e = nb.ext()
    x = torch.randn(4096, 768, device=DEV, dtype=torch.bfloat16)
    w = torch.rand(768, device=DEV) + 0.5
    _twice(lambda: e.rmsnorm_fwd(x, w, 1e-5))
    y, rstd = e.rmsnorm_fwd(x, w, 1e-5)
    dy = torch.randn_like(x)
    _twice(lambda: e.rmsnorm_bwd(dy, x, w, rstd, False, None)[0])
    wr = 0.02 * torch.randn(8, 768, device=DEV)
    _twice(lambda: e.router_logits_fwd(x, wr))
    g = torch.randn(4096, 8, device=DEV)
    _twice(lambda: tuple(e.router_logits_bwd(g, x, wr, True, True)))
    logits = torch.randn(4096, 8, device=DEV)
    _twice(lambda: tuple(e.router_forward(logits, 2, True)[:3]))
    idx = torch.randint(0, 8, (4096, 2), device=DEV, dtype=torch.int32)
    _twice(lambda: tuple(e.moe_plan(idx, 8)))
    q, k, v = (torch.randn(2, 4, 300, 64, device=DEV, dtype=torch.bfloat16).requires_grad_() for _ in range(3))
    go = torch.randn(2, 4, 300, 64, device=DEV, dtype=torch.bfloat16)

    def attention():
        out = native_attention.flash_attention(q, k, v, is_causal=True, dropout_p=0.0)
        return (out.detach(), *torch.autograd.grad(out, (q, k, v), go))

    _twice(attention)
    nb.check_kernel_status()


def test_outputs_stay_inside_their_buffers(nb):
    """Canary rows around the outputs of the kernels that compute their own addresses (gathers, scatters, tile stores with
    tails): anything written outside the requested extent shows up as a changed canary."""

    torch.manual_seed(42)
    e = nb.ext()
    canary = -123.0

    def framed(rows, cols, dtype):
        buf = torch.full((rows + 16, cols), canary, device=DEV, dtype=dtype)
        return buf, buf[8:8 + rows]

    def intact(buf, rows):
        return bool((buf[:8] == canary).all()) and bool((buf[8 + rows:] == canary).all())

    # GEMM with ragged M / N: 300 x 200 output inside a wider allocation, pitch 208
    a = torch.randn(300, 136, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(200, 136, device=DEV, dtype=torch.bfloat16)
    buf, out = framed(300, 208, torch.bfloat16)
    nb._gemm(a, b, out, 300, 200, 136, ldo=208)
    torch.cuda.synchronize()
    assert intact(buf, 300) and bool((out[:, 200:] == canary).all() | (out[:, 200:] == 0).all())
    assert_close(out[:, :200], a.float() @ b.float().t(), 5e-3, "gemm inside a frame")
    # expert permutation: gather into a framed buffer, then the weighted combine back
    tokens, k, experts, hidden = 777, 2, 8, 256
    idx = torch.randint(0, experts, (tokens, k), device=DEV, dtype=torch.int32)
    row_token, token_rows, tile_group, group_rows, meta = e.moe_plan(idx, experts)
    cap = row_token.numel()
    x = torch.randn(tokens, hidden, device=DEV, dtype=torch.bfloat16)
    buf, xs = framed(cap, hidden, torch.bfloat16)
    e.moe_gather(x, row_token, xs, meta)
    torch.cuda.synchronize()
    assert intact(buf, cap)
    live = row_token >= 0
    assert torch.equal(xs[live], x[row_token[live].long()])
    wts = torch.rand(tokens, k, device=DEV).to(torch.bfloat16)
    buf, mixed = framed(tokens, hidden, torch.bfloat16)
    e.moe_combine(xs, token_rows, wts, mixed, k)
    torch.cuda.synchronize()
    assert intact(buf, tokens)
    # embedding scatter-add into a framed fp32 table
    ids = torch.randint(0, 100, (5, 33), device=DEV)
    dout = torch.randn(5, 33, hidden, device=DEV, dtype=torch.bfloat16)
    buf, table = framed(100, hidden, torch.float32)
    table.zero_()
    e.embedding_bwd(ids, dout, table)
    torch.cuda.synchronize()
    assert intact(buf, 100)
    nb.check_kernel_status()


def test_release_build_reports_no_bounds_records(nb):
    e = nb.ext()
    assert e.debug_bounds_enabled() is False and e.debug_bounds_report() == []
