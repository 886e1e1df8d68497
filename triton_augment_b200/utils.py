"""Utilities kept for source compatibility with triton_augment/utils.py."""
from __future__ import annotations

from . import _lib

__all__ = ["warmup_cache", "library_path", "debug_counters"]


def warmup_cache(*args, **kwargs) -> None:
    """The reference compiles its Triton kernels here ahead of the first batch
    (triton_augment/utils.py:138-216).  These kernels are compiled when the package is
    built, so the only thing left to warm is loading the shared library."""
    _lib.load()


def library_path() -> str:
    return _lib.LIB_PATH


def debug_counters(reset: bool = False):
    """(tiles staged through shared memory, tiles gathered directly, staging violations,
    barrier time-outs) on the current CUDA device since the last reset."""
    return _lib.debug_counters(reset)
