"""Autotune switches kept for source compatibility with triton_augment/config.py.

The reference tunes Triton block sizes at run time.  The CUDA kernels here are compiled
ahead of time with fixed launch shapes (persistent grids sized from the SM count and the
measured occupancy of each kernel), so there is nothing to tune: the functions record the
flag and do nothing else.
"""
import os

ENABLE_AUTOTUNE = os.getenv("TRITON_AUGMENT_ENABLE_AUTOTUNE", "0") == "1"

__all__ = ["ENABLE_AUTOTUNE", "enable_autotune", "disable_autotune", "is_autotune_enabled"]


def enable_autotune():
    """Accepted and ignored (see module docstring)."""
    global ENABLE_AUTOTUNE
    ENABLE_AUTOTUNE = True


def disable_autotune():
    """Accepted and ignored (see module docstring)."""
    global ENABLE_AUTOTUNE
    ENABLE_AUTOTUNE = False


def is_autotune_enabled() -> bool:
    return ENABLE_AUTOTUNE
