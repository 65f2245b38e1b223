"""B200-native decode engine for grad.cpp models (KV-cached token loop).

The product is the C-ABI shared library built from ``csrc/`` (declared in
``include/gradb.h``); this Python package is a thin ctypes mirror of it for
tests and benchmarks. There is no CPU fallback: using the bindings fails
loudly if the CUDA library has not been built.
"""
from . import checkpoint  # noqa: F401
from . import binding  # noqa: F401
from . import sharding  # noqa: F401
from .binding import (BF16, FP32, BatchSession, GPTModel, InferenceSession, Sampling, TextGen,  # noqa: F401
                      lib)

__all__ = ["checkpoint", "binding", "GPTModel", "InferenceSession", "TextGen", "BatchSession", "Sampling",
           "FP32", "BF16", "lib"]
