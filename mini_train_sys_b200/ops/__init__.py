"""Operator backends: fp32 oracle, library baseline, and the sm_100a native kernels."""
