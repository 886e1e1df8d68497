"""Utilities kept for source compatibility with triton_augment/utils.py."""
from __future__ import annotations

from . import _lib

__all__ = ["warmup_cache", "library_path", "debug_counters", "check_status", "release_host_buffers"]


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


def check_status(device=None) -> None:
    """Raise if a kernel of the library gave up a bounded barrier wait on ``device`` since the last
    check (its launch then left part of the output unwritten).  The kernels are asynchronous, so
    call this after a synchronisation point; it reads one host word and synchronises nothing.
    ``forward_host`` does the check itself before it returns."""
    _lib.check_status(device)


def release_host_buffers(device=None) -> None:
    """Free the staging buffers, streams and events ``forward_host`` keeps on ``device``."""
    _lib.host_release(device)
