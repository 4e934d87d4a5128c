"""Operator benchmark runners: dense ops and MoE ops, one fresh process per (kernel, profile, size).

Same role as the reference's ``benchmarks/operators/dense_runner.py`` (profiles :52-73, kernel list :74-81, one
subprocess per case :456-499, tolerances :263-264, quality gate :528-556) and ``moe_runner.py`` (router sizes :55,
fused-MoE profiles :45-54, tolerances and the relative gate for expert-weight gradients :179-193).  A case that
runs out of memory or faults is recorded as data (``status``), it does not end the sweep.
"""

from __future__ import annotations

import json
import os
import subprocess
import sys
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch

from mini_train_sys_b200.bench.measurement import BenchCase, ResultCache, bench_sweep, case_key, gpu_tag


@dataclass(frozen=True)
class OperatorProfile:
    name: str
    hidden: int
    intermediate: int
    heads: int
    head_dim: int
    vocab: int
    seq_len: int
    experts: int = 8
    top_k: int = 2
    token_sizes: tuple[int, ...] = (512, 2048, 8192, 24576, 57344)


PROFILES = {
    # the 293M model of the headline benchmark: H768 / I1024 / 12 heads of 64 / GPT-2 vocabulary / S512
    "project_formal": OperatorProfile("project_formal", 768, 1024, 12, 64, 50257, 512),
    "mixtral_dense": OperatorProfile("mixtral_dense", 4096, 14336, 32, 128, 32000, 2048, token_sizes=(2048, 8192, 16384)),
    "mixtral_7b": OperatorProfile("mixtral_7b", 4096, 14336, 32, 128, 32000, 2048, token_sizes=(2048, 8192, 16384)),
}

DENSE_KERNELS = ("embedding", "rmsnorm", "rope", "swiglu", "attention", "cross_entropy", "fused_linear_cross_entropy", "linear")
MOE_KERNELS = ("router", "router_logits", "fused_moe")
ROUTER_TOKEN_SIZES = (1024, 4096, 16384, 65536, 262144, 524288)

_ACT = torch.bfloat16


def _randn(shape, device, *, grad=True, dtype=_ACT, scale=1.0):
    t = (torch.randn(shape, device=device, dtype=torch.float32) * scale).to(dtype)
    return t.requires_grad_(grad)


def build_case(kernel: str, profile: OperatorProfile, tokens: int) -> BenchCase:
    p = profile
    h, i, v = p.hidden, p.intermediate, p.vocab
    s = min(p.seq_len, tokens)
    b = max(tokens // s, 1)
    t = b * s
    label = f"{p.name}/{kernel}/T{t}"
    meta = {"profile": p.name, "batch": b, "seq_len": s}
    if kernel == "rmsnorm":
        return BenchCase(kernel, label, lambda d: {"x": _randn((t, h), d), "w": _randn((h,), d, dtype=torch.float32)},
                         lambda ops, a: ops.rmsnorm(a["x"], a["w"], 1e-5), t, bytes_moved=2 * t * h * 2, meta=meta)
    if kernel == "swiglu":
        return BenchCase(kernel, label, lambda d: {"g": _randn((t, i), d), "u": _randn((t, i), d)},
                         lambda ops, a: ops.swiglu(a["g"], a["u"]), t, bytes_moved=3 * t * i * 2, meta=meta)
    if kernel == "rope":
        def make(d):
            from mini_train_sys_b200.models.rotary import RotaryEmbedding

            rot = RotaryEmbedding(p.head_dim, s, 10000.0, cache_dtype=_ACT).to(d)
            cos, sin = rot(s)
            return {"q": _randn((b, p.heads, s, p.head_dim), d), "k": _randn((b, p.heads, s, p.head_dim), d), "cos": cos, "sin": sin}
        return BenchCase(kernel, label, make, lambda ops, a: ops.rope(a["q"], a["k"], a["cos"], a["sin"]), t,
                         bytes_moved=4 * t * p.heads * p.head_dim * 2, meta=meta)
    if kernel == "attention":
        def make(d):
            return {n: _randn((b, p.heads, s, p.head_dim), d) for n in ("q", "k", "v")}
        flops = 4.0 * b * p.heads * s * s * p.head_dim / 2       # causal: half the score grid
        return BenchCase(kernel, label, make, lambda ops, a: ops.attention(a["q"], a["k"], a["v"], is_causal=True, dropout_p=0.0),
                         t, flops=flops, atol=5e-2, rtol=8e-2, meta=meta)
    if kernel == "cross_entropy":
        return BenchCase(kernel, label, lambda d: {"logits": _randn((t, v), d), "y": torch.randint(0, v, (t,), device=d)},
                         lambda ops, a: ops.cross_entropy(a["logits"], a["y"]), t, bytes_moved=t * v * 2, meta=meta)
    if kernel == "fused_linear_cross_entropy":
        return BenchCase(kernel, label,
                         lambda d: {"x": _randn((t, h), d), "w": _randn((v, h), d, dtype=torch.float32, scale=0.02),
                                    "y": torch.randint(0, v, (t,), device=d)},
                         lambda ops, a: ops.fused_linear_cross_entropy(a["x"], a["w"], a["y"]), t, flops=2.0 * t * h * v,
                         atol=5e-2, rtol=8e-2, meta=meta)
    if kernel == "linear":
        def run(ops, a):
            if hasattr(ops, "linear"):
                return ops.linear(a["x"], a["w"])
            return torch.nn.functional.linear(a["x"], a["w"].to(a["x"].dtype))
        return BenchCase(kernel, label, lambda d: {"x": _randn((t, h), d), "w": _randn((3 * h, h), d, dtype=torch.float32, scale=0.02)},
                         run, t, flops=2.0 * t * h * 3 * h, atol=5e-2, rtol=8e-2, meta=meta)
    if kernel == "embedding":
        def run(ops, a):
            out = ops.embedding(a["ids"], a["w"]) if hasattr(ops, "embedding") else None
            return out if out is not None else torch.nn.functional.embedding(a["ids"], a["w"]).to(_ACT)
        return BenchCase(kernel, label, lambda d: {"ids": torch.randint(0, v, (t,), device=d), "w": _randn((v, h), d, dtype=torch.float32, scale=0.02)},
                         run, t, bytes_moved=t * h * (4 + 2), atol=1e-2, rtol=1e-2, meta=meta)
    if kernel == "router_logits":
        def run(ops, a):
            if hasattr(ops, "router_logits"):
                return ops.router_logits(a["x"], a["w"])
            with torch.autocast(a["x"].device.type, enabled=False):      # the router's logits are an fp32 product in every back end
                return torch.nn.functional.linear(a["x"].float(), a["w"].float())
        return BenchCase(kernel, label, lambda d: {"x": _randn((t, h), d), "w": _randn((p.experts, h), d, dtype=torch.float32, scale=0.02)},
                         run, t, bytes_moved=t * h * 2 + t * p.experts * 4, atol=2e-2, rtol=2e-2, meta=meta)
    if kernel == "router":
        return BenchCase(kernel, label, lambda d: {"logits": _randn((t, p.experts), d, dtype=torch.float32)},
                         lambda ops, a: ops.router_postprocess(a["logits"], p.top_k, normalize=True), t,
                         bytes_moved=t * p.experts * 4 + t * p.top_k * 8, atol=5e-5, rtol=5e-5, meta=meta)
    if kernel == "fused_moe":
        def make(d):
            idx = torch.stack([torch.randperm(p.experts, device=d)[:p.top_k] for _ in range(min(t, 4096))])
            idx = idx.repeat(-(-t // idx.shape[0]), 1)[:t].to(torch.int32)
            w = torch.rand(t, p.top_k, device=d).softmax(-1).requires_grad_()
            return {"x": _randn((t, h), d), "gu": _randn((p.experts, 2 * i, h), d, dtype=torch.float32, scale=0.02),
                    "dn": _randn((p.experts, h, i), d, dtype=torch.float32, scale=0.02), "idx": idx, "w": w}
        return BenchCase(kernel, label, make, lambda ops, a: ops.fused_moe(a["x"], a["gu"], a["dn"], a["idx"], a["w"]), t,
                         flops=2.0 * t * p.top_k * 3 * h * i, atol=5e-2, rtol=8e-2, meta=meta)
    raise ValueError(f"unknown kernel {kernel!r}")


def worker(kernel: str, profile_name: str, tokens: int, providers: list[str], *, warmup: int, iters: int, check: bool) -> dict[str, Any]:
    """Runs inside the per-case subprocess."""

    from mini_train_sys_b200.models import get_ops_backend

    torch.manual_seed(17)
    device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    case = build_case(kernel, PROFILES[profile_name], tokens)
    backends = {name: get_ops_backend(name) for name in providers}
    gate = (1e-2, 0.9999) if kernel == "fused_moe" else None
    with torch.autocast(device.type, dtype=_ACT):
        rows = bench_sweep([case], backends, device, warmup=warmup, iters=iters, check=check, relative_gate=gate)
    for row in rows:
        ops = backends[row["provider"]]
        if hasattr(ops, "dispatch_summary"):
            row["dispatch"] = ops.dispatch_summary()
    return {"status": "ok", "gpu": gpu_tag(), "rows": rows}


def run_case_subprocess(kernel: str, profile: str, tokens: int, providers: list[str], *, warmup: int, iters: int,
                        check: bool, timeout_s: float, script: Path) -> dict[str, Any]:
    cmd = [sys.executable, str(script), "_worker", "--kernel", kernel, "--profile", profile, "--tokens", str(tokens),
           "--providers", ",".join(providers), "--warmup", str(warmup), "--iters", str(iters)] + ([] if check else ["--no-check"])
    t0 = time.time()
    try:
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s, env=dict(os.environ))
    except subprocess.TimeoutExpired:
        return {"status": "timeout", "seconds": time.time() - t0}
    line = next((ln for ln in reversed(proc.stdout.splitlines()) if ln.startswith("{")), None)
    if proc.returncode != 0 or line is None:
        tail = (proc.stderr or proc.stdout)[-2000:]
        return {"status": "oom" if "out of memory" in tail.lower() else "failed", "returncode": proc.returncode, "log_tail": tail}
    return json.loads(line)


class OperatorBenchmark:
    """Sweep driver with a per-GPU result cache and the pass / fail summary the reports use."""

    def __init__(self, script: Path, cache_dir: Path, *, providers=("torch", "native"), warmup=5, iters=20, timeout_s=900.0) -> None:
        self.script, self.providers = Path(script), list(providers)
        self.warmup, self.iters, self.timeout_s = warmup, iters, timeout_s
        self.cache = ResultCache(cache_dir)

    def cases(self, kernels, profiles) -> list[tuple[str, str, int]]:
        out = []
        for prof in profiles:
            for kernel in kernels:
                sizes = ROUTER_TOKEN_SIZES if kernel == "router" else PROFILES[prof].token_sizes
                out += [(kernel, prof, n) for n in sizes]
        return out

    def run(self, kernels, profiles, *, refresh: bool = False, check: bool = True) -> list[dict[str, Any]]:
        results = []
        for kernel, prof, tokens in self.cases(kernels, profiles):
            key = case_key(kernel=kernel, profile=prof, tokens=tokens, providers=self.providers, iters=self.iters)
            hit = None if refresh else self.cache.get(key)
            if hit is None:
                hit = run_case_subprocess(kernel, prof, tokens, self.providers, warmup=self.warmup, iters=self.iters, check=check,
                                          timeout_s=self.timeout_s, script=self.script)
                hit.update(kernel=kernel, profile=prof, tokens=tokens)
                self.cache.put(key, hit)
            results.append(hit)
        return results


def quality_gate(results: list[dict[str, Any]]) -> dict[str, Any]:
    """``passed`` only if no case failed to run and no provider missed its parity check."""

    case_failures = [f"{r['profile']}/{r['kernel']}/T{r['tokens']}: {r['status']}" for r in results if r.get("status") != "ok"]
    wrong = []
    for r in results:
        for row in r.get("rows", []):
            c = row.get("correctness")
            if c is not None and not c["passed"]:
                wrong.append(f"{row['label']} [{row['provider']}]")
    return {"quality_gate_passed": not case_failures and not wrong, "case_failures": case_failures, "correctness_failures": wrong}


def headline_table(results: list[dict[str, Any]]) -> list[dict[str, Any]]:
    """One row per (kernel, profile, tokens, provider): p50 latencies, speed-up, roofline fraction."""

    table = []
    for r in results:
        for row in r.get("rows", []):
            full = row.get("full", {})
            table.append({"kernel": row["kernel"], "profile": r.get("profile"), "tokens": row["tokens"], "provider": row["provider"],
                          "fwd_ms": row.get("fwd", {}).get("p50_ms"), "full_ms": full.get("p50_ms"), "bwd_ms": row.get("bwd", {}).get("p50_ms"),
                          "speedup_full": row.get("speedup_vs_torch", {}).get("full"),
                          "frac_of_gemm_peak": full.get("frac_of_gemm_peak"), "frac_of_copy_peak": full.get("frac_of_copy_peak"),
                          "parity": (row.get("correctness") or {}).get("passed")})
    return table
