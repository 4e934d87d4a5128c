"""Measurement core of the operator benchmarks: cases, parity statistics, device timing, result cache.

Covers the role of the reference's ``benchmarks/operators/measurement.py`` (``BenchCase`` :221-318, streamed
``close_stats`` :320-414, ``correctness_stats`` :417-499, ``latency_ms`` :502-538, backward-only timing :552-586,
peak-memory deltas :541-603, ``bench_provider`` / ``bench_sweep`` :663-808, per-GPU JSON cache :63-160) with two
deliberate differences: latencies are always taken with CUDA events on the launching stream with an L2 flush
between iterations (no ``triton.testing``), and every record carries the roofline fraction against the measured
copy bandwidth and GEMM rate of the machine.
"""

from __future__ import annotations

import hashlib
import json
import math
import os
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Callable

import torch

_CHUNK = 4 * 1024 * 1024       # parity statistics stream over 4M-element chunks, so a [57344, 50257] logit grid never doubles
_L2_FLUSH_BYTES = 256 << 20    # larger than the 126 MB L2


@dataclass
class BenchCase:
    """One operator at one size: how to make inputs, how to call the op, and its algorithmic cost."""

    kernel: str
    label: str
    make_inputs: Callable[[torch.device], dict[str, Any]]          # tensors (leaf, requires_grad where differentiable)
    run: Callable[[Any, dict[str, Any]], Any]                      # (ops backend, inputs) -> tensor or tuple of tensors
    tokens: int = 0
    flops: float = 0.0                                             # forward FLOPs (backward counted as 2x)
    bytes_moved: float = 0.0                                       # forward algorithmic bytes
    atol: float = 2e-2
    rtol: float = 2e-2
    meta: dict[str, Any] = field(default_factory=dict)


def _flat_outputs(out: Any) -> list[torch.Tensor]:
    if isinstance(out, torch.Tensor):
        return [out]
    if isinstance(out, (tuple, list)):
        return [t for o in out for t in _flat_outputs(o)]
    if hasattr(out, "__dataclass_fields__"):
        return [getattr(out, k) for k in out.__dataclass_fields__ if isinstance(getattr(out, k), torch.Tensor)]
    return []


def close_stats(actual: torch.Tensor, expected: torch.Tensor, *, atol: float, rtol: float) -> dict[str, float]:
    """max_abs, max_rel, relative L2, cosine and the allclose verdict, streamed over chunks in fp64 accumulators."""

    a, e = actual.detach().reshape(-1), expected.detach().reshape(-1)
    if a.numel() != e.numel():
        return {"max_abs": math.inf, "max_rel": math.inf, "relative_l2": math.inf, "cosine": 0.0, "passed": False,
                "shape_mismatch": True}
    max_abs = max_rel = 0.0
    dot = na = ne = nd = 0.0
    violations = 0
    for lo in range(0, max(a.numel(), 1), _CHUNK):
        x, y = a[lo:lo + _CHUNK].double(), e[lo:lo + _CHUNK].double()
        if x.numel() == 0:
            break
        d = (x - y).abs()
        max_abs = max(max_abs, float(d.max()))
        max_rel = max(max_rel, float((d / y.abs().clamp_min(1e-12)).where(y.abs() > atol, torch.zeros_like(d)).max()))
        violations += int((d > atol + rtol * y.abs()).sum())
        dot += float((x * y).sum()); na += float((x * x).sum()); ne += float((y * y).sum()); nd += float((d * d).sum())
    finite = bool(torch.isfinite(a).all())
    rel_l2 = math.sqrt(nd / ne) if ne > 0 else math.sqrt(nd)
    cosine = dot / math.sqrt(na * ne) if na > 0 and ne > 0 else float(na == ne)
    return {"max_abs": max_abs, "max_rel": max_rel, "relative_l2": rel_l2, "cosine": cosine,
            "violations": violations, "finite": finite, "passed": finite and violations == 0}


def _differentiable(inputs: dict[str, Any]) -> list[tuple[str, torch.Tensor]]:
    return [(k, v) for k, v in inputs.items() if isinstance(v, torch.Tensor) and v.requires_grad]


def _clone_inputs(inputs: dict[str, Any]) -> dict[str, Any]:
    out = {}
    for k, v in inputs.items():
        if isinstance(v, torch.Tensor):
            c = v.detach().clone()
            c.requires_grad_(v.requires_grad)
            out[k] = c
        else:
            out[k] = v
    return out


def correctness_stats(case: BenchCase, provider, oracle, device: torch.device, *, seed: int = 17,
                      relative_gate: tuple[float, float] | None = None) -> dict[str, Any]:
    """Forward outputs and every input gradient of ``provider`` against ``oracle`` under the same random upstream grads.

    ``relative_gate=(max_rel_l2, min_cosine)`` replaces the element-wise check for gradients whose bf16 rounding
    makes ``allclose`` meaningless (expert-weight gradients; reference moe_runner.py:179-193).
    """

    torch.manual_seed(seed)
    base = case.make_inputs(device)
    results: dict[str, Any] = {"outputs": [], "grads": {}, "passed": True}
    runs = {}
    for name, ops in (("provider", provider), ("oracle", oracle)):
        inputs = _clone_inputs(base)
        outs = [o for o in _flat_outputs(case.run(ops, inputs)) if o.is_floating_point()]
        runs[name] = (inputs, outs)
    gen = torch.Generator(device=device).manual_seed(seed + 1)
    ups = [torch.randn(o.shape, device=device, dtype=torch.float32, generator=gen) for o in runs["oracle"][1]]
    for name in runs:
        inputs, outs = runs[name]
        diff = [o for o in outs if o.requires_grad]
        if diff:
            torch.autograd.backward(diff, [u.to(o.dtype) for o, u in zip(outs, ups) if o.requires_grad])
    for a, e in zip(runs["provider"][1], runs["oracle"][1]):
        s = close_stats(a.float(), e.float(), atol=case.atol, rtol=case.rtol)
        results["outputs"].append(s)
        results["passed"] &= bool(s["passed"])
    for (k, pa), (_, pe) in zip(_differentiable(runs["provider"][0]), _differentiable(runs["oracle"][0])):
        if pa.grad is None or pe.grad is None:
            results["grads"][k] = {"passed": pa.grad is None and pe.grad is None, "missing": True}
        else:
            s = close_stats(pa.grad.float(), pe.grad.float(), atol=case.atol, rtol=case.rtol)
            if relative_gate is not None and not s["passed"]:
                s["passed"] = s["finite"] and s["relative_l2"] <= relative_gate[0] and s["cosine"] >= relative_gate[1]
                s["gate"] = "relative"
            results["grads"][k] = s
        results["passed"] &= bool(results["grads"][k]["passed"])
    return results


class _L2Flusher:
    def __init__(self, device: torch.device) -> None:
        self.buf = torch.empty(_L2_FLUSH_BYTES, dtype=torch.uint8, device=device) if device.type == "cuda" else None

    def __call__(self) -> None:
        if self.buf is not None:
            self.buf.zero_()


def latency_ms(fn: Callable[[], Any], device: torch.device, *, warmup: int = 5, iters: int = 20,
               flush_l2: bool = True) -> dict[str, float]:
    """p50 / p95 / mean of ``fn`` in milliseconds: CUDA events on the current stream, L2 flushed before each timed call."""

    for _ in range(max(warmup, 3)):
        fn()
    if device.type != "cuda":
        times = []
        for _ in range(iters):
            t0 = time.perf_counter(); fn(); times.append((time.perf_counter() - t0) * 1e3)
    else:
        flush = _L2Flusher(device) if flush_l2 else (lambda: None)
        torch.cuda.synchronize(device)
        pairs = []
        for _ in range(iters):
            flush()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record()
            pairs.append((a, b))
        torch.cuda.synchronize(device)
        times = [a.elapsed_time(b) for a, b in pairs]
    times.sort()
    pick = lambda q: times[min(len(times) - 1, int(q * len(times)))]   # noqa: E731
    return {"p50_ms": pick(0.5), "p95_ms": pick(0.95), "mean_ms": sum(times) / len(times), "min_ms": times[0], "iters": len(times)}


def peak_memory_delta_mb(fn: Callable[[], Any], device: torch.device) -> float:
    if device.type != "cuda":
        return 0.0
    torch.cuda.synchronize(device)
    torch.cuda.reset_peak_memory_stats(device)
    before = torch.cuda.memory_allocated(device)
    fn()
    torch.cuda.synchronize(device)
    return (torch.cuda.max_memory_allocated(device) - before) / 2**20


def benchmark_step(case: BenchCase, ops, device: torch.device, mode: str, *, warmup: int, iters: int) -> dict[str, float]:
    """``mode`` is ``fwd`` (no grad), ``full`` (forward + backward) or ``bwd`` (backward only, graph retained)."""

    inputs = case.make_inputs(device)
    if mode == "fwd":
        def fn():
            with torch.no_grad():
                return case.run(ops, inputs)
    else:
        def forward():
            outs = [o for o in _flat_outputs(case.run(ops, inputs)) if o.is_floating_point() and o.requires_grad]
            return outs, [torch.ones_like(o) for o in outs]

        if mode == "full":
            def fn():
                outs, ups = forward()
                torch.autograd.backward(outs, ups)
                for _, t in _differentiable(inputs):
                    t.grad = None
        else:
            outs, ups = forward()

            def fn():
                torch.autograd.backward(outs, ups, retain_graph=True)
                for _, t in _differentiable(inputs):
                    t.grad = None
    stats = latency_ms(fn, device, warmup=warmup, iters=iters)
    stats["peak_delta_mb"] = peak_memory_delta_mb(fn, device)
    return stats


def measured_peaks(root: Path | None = None) -> dict[str, float]:
    """Copy bandwidth (GB/s) and bf16 GEMM rate (TFLOP/s) used as roofline denominators, with their provenance."""

    from mini_train_sys_b200.train.metrics import measured_peaks as load

    return load(root)


def roofline(case: BenchCase, ms: float, mode: str, peaks: dict[str, float]) -> dict[str, float]:
    scale = {"fwd": 1.0, "bwd": 2.0, "full": 3.0}[mode]
    out: dict[str, float] = {}
    if case.flops and ms > 0:
        out["tflops"] = case.flops * scale / ms / 1e9
        out["frac_of_gemm_peak"] = out["tflops"] / peaks["bf16_tflops"]
    if case.bytes_moved and ms > 0:
        out["gbs"] = case.bytes_moved * scale / ms / 1e6
        out["frac_of_copy_peak"] = out["gbs"] / peaks["hbm_gbs"]
    out["peaks"] = peaks.get("source", "measured")
    return out


def bench_provider(case: BenchCase, name: str, ops, oracle, device: torch.device, *, warmup: int = 5, iters: int = 20,
                   modes: tuple[str, ...] = ("fwd", "full", "bwd"), check: bool = True,
                   relative_gate: tuple[float, float] | None = None) -> dict[str, Any]:
    record: dict[str, Any] = {"kernel": case.kernel, "label": case.label, "provider": name, "tokens": case.tokens,
                              "meta": case.meta}
    if check and oracle is not None and name != "torch":
        record["correctness"] = correctness_stats(case, ops, oracle, device, relative_gate=relative_gate)
    peaks = measured_peaks()
    for mode in modes:
        stats = benchmark_step(case, ops, device, mode, warmup=warmup, iters=iters)
        stats.update(roofline(case, stats["p50_ms"], mode, peaks))
        record[mode] = stats
    return record


def bench_sweep(cases: list[BenchCase], providers: dict[str, Any], device: torch.device, **kw) -> list[dict[str, Any]]:
    """Every case under every provider; speed-ups are p50 ratios against the ``torch`` provider."""

    oracle = providers.get("torch")
    rows = []
    for case in cases:
        per_case = {name: bench_provider(case, name, ops, oracle, device, **kw) for name, ops in providers.items()}
        base = per_case.get("torch")
        for name, rec in per_case.items():
            if base is not None and name != "torch":
                rec["speedup_vs_torch"] = {m: base[m]["p50_ms"] / rec[m]["p50_ms"] for m in ("fwd", "full", "bwd")
                                           if m in rec and m in base and rec[m]["p50_ms"] > 0}
            rows.append(rec)
    return rows


# ---------------------------------------------------------------------------------------------------------
# result cache: one JSON file per (compute capability, GPU name), keyed by a digest of the case parameters
# ---------------------------------------------------------------------------------------------------------

def gpu_tag(device: torch.device | None = None) -> str:
    if not torch.cuda.is_available():
        return "cpu"
    props = torch.cuda.get_device_properties(device or 0)
    name = "".join(c if c.isalnum() else "-" for c in props.name.lower()).strip("-")
    return f"sm{props.major}{props.minor}-{name}"


def case_key(**params: Any) -> str:
    return hashlib.sha256(json.dumps(params, sort_keys=True, default=str).encode()).hexdigest()[:20]


class ResultCache:
    def __init__(self, directory: Path, tag: str | None = None) -> None:
        self.path = Path(directory) / f"{tag or gpu_tag()}.json"
        self.data: dict[str, Any] = json.loads(self.path.read_text()) if self.path.exists() else {}

    def get(self, key: str) -> Any:
        return self.data.get(key)

    def put(self, key: str, value: Any) -> None:
        self.data[key] = value
        self.path.parent.mkdir(parents=True, exist_ok=True)
        tmp = self.path.with_suffix(".json.tmp")
        tmp.write_text(json.dumps(self.data, indent=1, sort_keys=True, default=str))
        os.replace(tmp, self.path)


def case_to_json(case: BenchCase) -> dict[str, Any]:
    d = asdict(case)
    d.pop("make_inputs"); d.pop("run")
    return d
