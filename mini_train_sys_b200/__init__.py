"""B200-native training system for Dense and top-k MoE decoder-only Transformers."""

__version__ = "0.1.0"
