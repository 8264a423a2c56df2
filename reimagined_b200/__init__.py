"""reimagined_b200 — B200 (sm_100a) implementation of the NSOS BitNet b1.58 ternary linear path.

The product is the C-ABI shared library ``libternary_b200.so`` (hand-written CUDA, see
``include/ternary_b200.h``).  This package only loads it and exposes thin ctypes wrappers that take
raw device pointers; PyTorch, where used by callers, merely owns device memory and streams.

There is no CPU fallback: importing :mod:`reimagined_b200.capi` raises if the library is absent.
"""
from .capi import LIB_PATH, TernaryB200Error, lib, check  # noqa: F401

__all__ = ["lib", "check", "LIB_PATH", "TernaryB200Error"]
