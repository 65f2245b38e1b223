"""B200-native decode engine for grad.cpp models (KV-cached token loop).

The product is the C-ABI shared library built from ``csrc/`` (declared in
``include/gradb.h``); this Python package is a thin ctypes mirror of it for
tests and benchmarks. There is no CPU fallback: loading fails if the CUDA
library has not been built.
"""
from . import checkpoint  # noqa: F401

__all__ = ["checkpoint"]
