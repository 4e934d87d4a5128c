"""Throughput-derived metrics."""

from __future__ import annotations

import json
from pathlib import Path


def estimate_mfu(tokens_per_sec: float, flops_per_token: float, peak_flops: float) -> float:
    """Model FLOPs utilisation in [0, 1]: achieved training FLOP/s over ``peak_flops``."""

    if peak_flops <= 0:
        return 0.0
    return tokens_per_sec * flops_per_token / peak_flops


def measured_peaks(search_from: str | Path | None = None) -> dict[str, float]:
    """Measured roofline denominators (``MEASURED_PEAKS.json`` at the repository root) or the fallback."""

    here = Path(search_from or __file__).resolve()
    for parent in (here, *here.parents):
        candidate = parent / "MEASURED_PEAKS.json"
        if candidate.is_file():
            data = json.loads(candidate.read_text())
            return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]),
                    "bf16_tflops_sustained": float(data.get("bf16_tflops_sustained", data["bf16_tflops"])),
                    "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
