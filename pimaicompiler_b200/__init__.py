"""pimaicompiler_b200 — B200 (sm_100a) device back end for PimAiCompiler's fp16 recurrent/decode hot path.

The kernels live in ``csrc/`` and are reached only through the C ABI declared in
``include/pimb200.h`` (``libpimb200.so``); ``ops`` wraps that ABI for torch tensors.
"""
from . import _lib  # noqa: F401

__all__ = ["_lib"]
