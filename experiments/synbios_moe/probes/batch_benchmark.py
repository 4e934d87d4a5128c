"""Batch-size benchmark of probe training / validation steps under a memory cap.

For every candidate batch size the benchmark runs real steps (collate on the host, host-to-device copy, forward, and in
training mode backward + AdamW) on the LONGEST examples of the dataset, records step time, throughput and peak memory, and
recommends the fastest size whose peak reserved memory stays under the cap.  Several runs (one per GPU of a server) are
merged by keeping only sizes that were safe everywhere (reference: experiments/synbios_moe/probes/batch_benchmark.py:21-373).
"""

from __future__ import annotations

import json
import time
from pathlib import Path
from typing import Callable, Sequence

import torch
from torch import nn

from experiments.synbios_moe.probes.model import ADAM_EPS, DEFAULT_BATCH, LEARNING_RATE, WEIGHT_DECAY, AttributeProbe, collate


def parse_batch_sizes(value: str) -> tuple[int, ...]:
    sizes = tuple(dict.fromkeys(int(v.strip()) for v in value.split(",") if v.strip()))
    if not sizes or any(s <= 0 for s in sizes):
        raise ValueError("batch sizes must be a comma-separated list of positive integers")
    return tuple(sorted(sizes))


def _longest_items(dataset, count: int) -> list:
    longest = getattr(dataset, "longest", None)
    if callable(longest):
        return longest(count)
    return [dataset[i] for i in range(min(count, len(dataset)))]


def benchmark_probe_batches(backbone, dataset, *, kind: str, num_classes: int, rank: int, batch_sizes: Sequence[int], device="cpu",
                            mode: str = "training", warmup_steps: int = 3, measure_steps: int = 10, memory_limit_percent: float = 92.0,
                            on_result: Callable[[dict], None] | None = None) -> dict:
    if kind not in DEFAULT_BATCH:
        raise ValueError("kind must be 'p' or 'q'")
    if mode not in ("training", "validation"):
        raise ValueError("mode must be 'training' or 'validation'")
    if warmup_steps < 0 or measure_steps <= 0 or not 0 < memory_limit_percent <= 100:
        raise ValueError("invalid warm-up / measurement / memory-limit settings")
    candidates = tuple(sorted({int(s) for s in batch_sizes}))
    if not candidates or candidates[0] <= 0:
        raise ValueError("batch_sizes must contain positive integers")
    device = torch.device(device)
    # two distinct batches of the largest size when the dataset allows: reusing one device-resident batch would understate
    # allocator pressure at the capacity boundary
    items = _longest_items(dataset, min(len(dataset), 2 * candidates[-1]))
    if len(items) < candidates[-1]:
        raise ValueError("the dataset is smaller than the largest benchmark batch")
    eos = dataset.eos
    backbone.to(device)
    on_cuda = device.type == "cuda"
    results = []
    for size in candidates:
        record: dict = {"batch_size": size, "status": "completed"}
        probe = optimizer = None
        try:
            probe = AttributeProbe(backbone, num_classes, rank=rank, kind=kind).to(device)
            probe.train(mode == "training")
            if mode == "training":
                optimizer = torch.optim.AdamW([p for p in probe.parameters() if p.requires_grad], lr=LEARNING_RATE,
                                              weight_decay=WEIGHT_DECAY, eps=ADAM_EPS)
            if on_cuda:
                torch.cuda.empty_cache()
                torch.cuda.reset_peak_memory_stats(device)
            batches = [items[lo:lo + size] for lo in range(0, len(items) - size + 1, size)]
            timings, width, last = [], None, None
            for step in range(warmup_steps + measure_steps):
                started = time.perf_counter()
                ids, pos, labels = collate(batches[step % len(batches)], eos)
                ids, pos, labels = ids.to(device, non_blocking=True), pos.to(device, non_blocking=True), labels.to(device, non_blocking=True)
                if optimizer is not None:
                    optimizer.zero_grad(set_to_none=True)
                with torch.set_grad_enabled(mode == "training"):
                    logits = probe(ids, pos)
                    loss = nn.functional.cross_entropy(logits.flatten(0, 1), labels[:, None].expand(-1, logits.shape[1]).reshape(-1))
                if optimizer is not None:
                    loss.backward()
                    optimizer.step()
                if on_cuda:
                    torch.cuda.synchronize(device)
                width, last = int(ids.shape[1]), float(loss.detach())
                if step >= warmup_steps:
                    timings.append(time.perf_counter() - started)
                del logits, loss
            mean = sum(timings) / len(timings)
            if on_cuda:
                reserved, allocated = torch.cuda.max_memory_reserved(device), torch.cuda.max_memory_allocated(device)
                capacity = torch.cuda.get_device_properties(device).total_memory
                record.update({"peak_memory_reserved_mb": round(reserved / 2**20, 2), "peak_memory_allocated_mb": round(allocated / 2**20, 2),
                               "memory_capacity_mb": round(capacity / 2**20, 2), "peak_memory_percent": round(100 * reserved / capacity, 2)})
            record.update({"step_time_ms": round(1e3 * mean, 3), "examples_per_second": round(size / mean, 3), "sequence_length": width,
                           "loss": last, "batch_lifecycle": "fresh_host_batch_per_step"})
        except torch.OutOfMemoryError as exc:
            record.update({"status": "oom", "error": str(exc)[:300]})
        finally:
            del probe, optimizer
            if on_cuda:
                torch.cuda.empty_cache()
        results.append(record)
        if on_result is not None:
            on_result(dict(record))
    safe = [r for r in results if r["status"] == "completed" and float(r.get("peak_memory_percent", 0.0)) <= memory_limit_percent]
    best = max(safe, key=lambda r: float(r["examples_per_second"])) if safe else None
    paper = DEFAULT_BATCH[kind]
    paper_row = next((r for r in results if r["batch_size"] == paper), None)
    return {"kind": kind, "mode": mode, "device": str(device), "paper_training_batch_size": paper,
            "paper_batch_safe": bool(paper_row is not None and paper_row in safe), "memory_limit_percent": memory_limit_percent,
            "recommended_capacity_batch_size": int(best["batch_size"]) if best else None,
            "recommendation_scope": f"{mode}_capacity_profile", "results": results}


_IDENTITY_KEYS = ("attribute", "target", "rank", "checkpoint", "probe_cache", "ground_truth_first")


def summarize_probe_benchmarks(paths: Sequence[str | Path]) -> dict:
    """Merge runs (e.g. one per GPU): per (kind, mode) keep batch sizes measured and safe in EVERY run, pick the one with the
    best worst-case throughput.

    Replicas of one (kind, mode) must have measured the same candidates under the same memory limit on the same task,
    otherwise their intersection would silently mean something else.  ``completeness`` says whether the result may be used
    for a formal run: all four (kind, mode) cells measured, each at least twice, each with a recommendation that is not the
    largest candidate tried (a recommendation at the edge of the search says the search stopped too early)."""

    payloads = [json.loads(Path(p).read_text(encoding="utf-8")) for p in paths]
    if not payloads:
        raise ValueError("at least one benchmark result is required")
    groups: dict[tuple[str, str], list[dict]] = {}
    for payload in payloads:
        for run in payload.get("benchmarks", [payload]):
            groups.setdefault((run["kind"], run["mode"]), []).append({**{k: payload[k] for k in _IDENTITY_KEYS if k in payload}, **run})
    summary: dict = {"runs": [str(Path(p).resolve()) for p in paths], "recommendations": {}}
    for (kind, mode), runs in sorted(groups.items()):
        candidates = [tuple(sorted(int(x["batch_size"]) for x in r["results"])) for r in runs]
        if any(c != candidates[0] for c in candidates[1:]):
            raise ValueError(f"{kind}/{mode}: benchmark replicas used different batch-size candidates")
        if len({float(r["memory_limit_percent"]) for r in runs}) != 1:
            raise ValueError(f"{kind}/{mode}: benchmark replicas used different memory limits")
        for key in _IDENTITY_KEYS:
            seen = {json.dumps(r.get(key)) for r in runs if key in r}
            if len(seen) > 1 or (seen and any(key not in r for r in runs)):
                raise ValueError(f"{kind}/{mode}: benchmark replicas disagree on {key}")
        limit = float(runs[0]["memory_limit_percent"])
        rows = []
        for size in candidates[0]:
            cells = [next(x for x in r["results"] if int(x["batch_size"]) == size) for r in runs]
            ok = all(c["status"] == "completed" and float(c.get("peak_memory_percent", 0.0)) <= limit for c in cells)
            rows.append({"batch_size": size, "safe_everywhere": ok,
                         "min_examples_per_second": min(float(c.get("examples_per_second", 0.0)) for c in cells) if ok else None,
                         "max_peak_memory_percent": max(float(c.get("peak_memory_percent", 0.0)) for c in cells)})
        safe = [r for r in rows if r["safe_everywhere"]]
        best = max(safe, key=lambda r: r["min_examples_per_second"]) if safe else None
        summary["recommendations"][f"{kind}_{mode}"] = {
            "replicas": len(runs), "memory_limit_percent": limit, "candidates": rows,
            "largest_tested_batch_size": max(candidates[0]) if candidates[0] else None,
            "recommended_batch_size": best["batch_size"] if best else None,
            "recommended_is_search_boundary": bool(best and candidates[0] and best["batch_size"] == max(candidates[0]))}
    cells = [f"{kind}_{mode}" for kind in ("p", "q") for mode in ("training", "validation")]
    rec = summary["recommendations"]
    completeness = {"missing": [c for c in cells if c not in rec],
                    "single_replica": [c for c in cells if c in rec and rec[c]["replicas"] < 2],
                    "no_recommendation": [c for c in cells if c in rec and rec[c]["recommended_batch_size"] is None],
                    "at_search_boundary": [c for c in cells if c in rec and rec[c]["recommended_is_search_boundary"]]}
    completeness["ready_for_formal"] = not any(completeness.values())
    summary["completeness"] = completeness
    return summary


def probe_batch_environment(summary: dict) -> str:
    """Shell lines (``export P_BATCH_SIZE=...``) a launcher can source; only for a complete, bracketed benchmark
    (reference: experiments/synbios_moe/probes/batch_benchmark.py:361-373)."""

    if not summary.get("completeness", {}).get("ready_for_formal"):
        raise ValueError("the probe batch benchmark is not complete enough for formal use: " + json.dumps(summary.get("completeness")))
    rec = summary["recommendations"]
    values = {"P_BATCH_SIZE": rec["p_training"], "Q_BATCH_SIZE": rec["q_training"], "P_VALIDATION_BATCH_SIZE": rec["p_validation"],
              "Q_VALIDATION_BATCH_SIZE": rec["q_validation"]}
    return "".join(f"export {name}={int(cell['recommended_batch_size'])}\n" for name, cell in values.items())
