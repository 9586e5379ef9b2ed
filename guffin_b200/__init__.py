"""guffin_b200: B200 (sm_100a) backend for the Gemma speculative-decode hot path.

The product is the CUDA shared library (csrc/, C ABI in include/guffin_b200.h); this package
is its ctypes binding plus the seeded synthetic workloads the benchmarks use.
"""
from . import synthetic  # noqa: F401

__all__ = ["synthetic"]
