"""Benchmark harness: operator sweeps with parity gates, Nsight Compute helpers, distributed training suites."""
