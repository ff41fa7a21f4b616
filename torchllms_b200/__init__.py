"""A small, whole, single-GPU inference engine for NVIDIA B200 (sm_100a)."""

__version__ = "0.1.0"
