"""ctypes front end of the CPU oracle (oracle/fused_oracle.c).

TEST INFRASTRUCTURE ONLY.  The shipped package never imports this module; the
tests, the smoke check and the benchmark's CPU legs do.  It takes and returns
numpy arrays so that it has no dependency on the package under test.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libta_oracle.so")
_lib = None

CONTRAST_FAST = 0
CONTRAST_MEAN = 1


class _Params(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32),
        ("n", C.c_int32), ("c", C.c_int32), ("h", C.c_int32), ("w", C.c_int32),
        ("oh", C.c_int32), ("ow", C.c_int32),
        ("inp", C.c_void_p), ("out", C.c_void_p),
        ("top", C.c_void_p), ("left", C.c_void_p), ("flip", C.c_void_p),
        ("matrix", C.c_void_p),
        ("fill", C.c_float), ("interp", C.c_int32),
        ("apply_brightness", C.c_int32), ("apply_contrast", C.c_int32),
        ("apply_saturation", C.c_int32), ("apply_grayscale", C.c_int32),
        ("apply_normalize", C.c_int32),
        ("brightness", C.c_void_p), ("contrast", C.c_void_p), ("saturation", C.c_void_p),
        ("gray", C.c_void_p), ("mean", C.c_void_p), ("std", C.c_void_p),
        ("fma_coords", C.c_int32), ("contrast_mode", C.c_int32),
        ("gray_mean", C.c_void_p), ("src_index", C.c_void_p),
        ("threads", C.c_int32),
    ]


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile next to it (gcc only)."""
    src = os.path.join(_HERE, "fused_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        env = dict(os.environ)
        env.pop("CC", None)
        subprocess.run(["make", "-C", _HERE, "CC=gcc"], check=True, env=env,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.ta_oracle_fused_augment.argtypes = [C.POINTER(_Params)]
        _lib.ta_oracle_fused_augment.restype = C.c_int
        _lib.ta_oracle_gray_mean.argtypes = [C.POINTER(_Params), C.c_void_p]
        _lib.ta_oracle_gray_mean.restype = C.c_int
        _lib.ta_oracle_inverse_affine_matrix.argtypes = [C.c_int] + [C.c_void_p] * 6
        _lib.ta_oracle_inverse_affine_matrix.restype = None
        _lib.ta_oracle_max_threads.restype = C.c_int
    return _lib


def max_threads() -> int:
    return int(lib().ta_oracle_max_threads())


def coord_recipe(fma_coords) -> int:
    """How ``a*xc + b*yc`` of the coordinate map is contracted, per axis.

    ``False`` / ``0``: not at all (the CPU interpreter).  ``True``: ``fma(xc, a, b*yc)`` for both
    axes, what the reference's GPU build does in its nearest-sampling kernels.
    ``(rx, ry)`` or ``(rx, ry, k)``: explicit, 0 none / 1 ``fma(xc,a,b*yc)`` / 2 ``fma(yc,b,a*xc)``;
    ``k``: the last k of a reference thread's 8 pixels use recipe 1 for x (see gpu_recipe).
    """
    if isinstance(fma_coords, str):
        raise ValueError("resolve 'gpu' with gpu_recipe(...) first")
    if isinstance(fma_coords, (tuple, list)):
        k = int(fma_coords[2]) if len(fma_coords) > 2 else 0
        return int(fma_coords[0]) | (int(fma_coords[1]) << 2) | (k << 4)
    if isinstance(fma_coords, (bool, np.bool_)):
        return 5 if fma_coords else 0
    return int(fma_coords)


# gpu_recipe(): k per colour-flag combination (bit 0 brightness, 1 contrast, 2 saturation,
# 3 grayscale, 4 normalize) of the variants whose x and y recipes are swapped.
_LATE_X = {5: 1, 6: 1, 7: 3, 9: 2, 10: 1, 11: 3, 13: 2, 14: 2, 15: 3,
           21: 1, 22: 2, 23: 3, 25: 2, 26: 1, 27: 3, 29: 2, 30: 2, 31: 3}


def gpu_recipe(interpolation, flags, normalize=False, out_size=None, dtype=np.float32) -> tuple:
    """Contraction the reference's kernel shows when Triton 3.6 compiles it for sm_100.

    Measured on a B200 by comparing the reference's output with every recipe, for all 32
    combinations of the colour flags in fp32 (the sweep is described in
    tests/golden/make_gpu_golden.py):
      * nearest sampling: x and y are fma(xc, a, b*yc) in every variant;
      * bilinear sampling: x = fma(xc, a, b*yc), y = fma(yc, e, d*xc), except in the variants
        that take the RGB-triplet path (saturation or grayscale on) AND have brightness or
        contrast on, where it is the other way round: x = fma(yc, b, a*xc), y = fma(xc, d, e*yc);
      * in those swapped variants, when neither output dimension is divisible by 16 (Triton
        then specialises the kernel without vectorised stores and a thread's 8 pixels lie 128
        apart), the last k of a thread's 8 pixels use fma(xc, a, b*yc) for x after all; k is
        1, 2 or 3 depending on the flag combination (``_LATE_X``).  ``out_size`` = (oh, ow)
        enables this rule; it is known for fp32 only.
    Each compiled variant is a different LLVM module, hence the different choices.
    """
    if str(interpolation).lower() != "bilinear":
        return (1, 1)
    spatial = flags["saturation"] or flags["grayscale"]
    if not (spatial and (flags["brightness"] or flags["contrast"])):
        return (1, 2)
    k = 0
    if out_size is not None and np.dtype(dtype) == np.float32 and out_size[0] % 16 and out_size[1] % 16:
        bits = (int(bool(flags["brightness"])) | int(bool(flags["contrast"])) << 1 | int(bool(flags["saturation"])) << 2
                | int(bool(flags["grayscale"])) << 3 | int(bool(normalize)) << 4)
        k = _LATE_X[bits]
    return (2, 1, k)


def _vec(x, n, dtype):
    a = np.asarray(x)
    if a.ndim == 0:
        a = np.full((n,), a)
    a = np.ascontiguousarray(a.astype(dtype, copy=False))
    if a.shape != (n,):
        raise ValueError(f"expected shape ({n},), got {a.shape}")
    return a


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _prepare(image, top, left, height, width, flip, matrix, interpolation, fill, brightness,
             contrast, saturation, grayscale, mean, std, flags, fma_coords, contrast_mode,
             gray_mean, want_index, threads):
    image = np.ascontiguousarray(image)
    if image.dtype not in (np.float32, np.float16):
        raise TypeError("image must be float32 or float16")
    n, c, h, w = image.shape
    dt = image.dtype
    keep = {}
    keep["image"] = image
    keep["top"] = _vec(top, n, np.float32)
    keep["left"] = _vec(left, n, np.float32)
    keep["flip"] = _vec(flip, n, np.uint8)
    keep["matrix"] = None if matrix is None else np.ascontiguousarray(np.asarray(matrix, np.float32).reshape(n, 6))
    keep["b"] = _vec(brightness, n, dt)
    keep["c"] = _vec(contrast, n, dt)
    keep["s"] = _vec(saturation, n, dt)
    keep["g"] = _vec(grayscale, n, np.uint8)
    apply_norm = mean is not None and std is not None
    keep["mean"] = np.asarray(mean if apply_norm else (0, 0, 0), dtype=dt)
    keep["std"] = np.asarray(std if apply_norm else (1, 1, 1), dtype=dt)
    if flags is None:
        # Same value-based decisions as triton_augment/functional.py:1341-1344, 1356.
        flags = dict(brightness=bool(np.any(keep["b"] != 1)), contrast=bool(np.any(keep["c"] != 1)),
                     saturation=bool(np.any(keep["s"] != 1)), grayscale=bool(np.any(keep["g"])))
    keep["out"] = np.empty((n, c, height, width), dtype=dt)
    keep["gm"] = None if gray_mean is None else _vec(gray_mean, n, np.float32)
    keep["idx"] = np.empty((n, height, width), dtype=np.int32) if want_index else None
    p = _Params()
    p.dtype = 1 if dt == np.float16 else 0
    p.n, p.c, p.h, p.w, p.oh, p.ow = n, c, h, w, height, width
    p.inp, p.out = _ptr(image), _ptr(keep["out"])
    p.top, p.left, p.flip = _ptr(keep["top"]), _ptr(keep["left"]), _ptr(keep["flip"])
    p.matrix = _ptr(keep["matrix"])
    p.fill = float(fill)
    p.interp = 1 if str(interpolation).lower() == "bilinear" else 0
    p.apply_brightness = int(flags["brightness"])
    p.apply_contrast = int(flags["contrast"])
    p.apply_saturation = int(flags["saturation"])
    p.apply_grayscale = int(flags["grayscale"])
    p.apply_normalize = int(apply_norm)
    p.brightness, p.contrast, p.saturation = _ptr(keep["b"]), _ptr(keep["c"]), _ptr(keep["s"])
    p.gray, p.mean, p.std = _ptr(keep["g"]), _ptr(keep["mean"]), _ptr(keep["std"])
    if isinstance(fma_coords, str) and fma_coords == "gpu":
        fma_coords = gpu_recipe(interpolation, flags, apply_norm, (height, width), dt)
    p.fma_coords = coord_recipe(fma_coords)
    p.contrast_mode = int(contrast_mode)
    p.gray_mean = _ptr(keep["gm"])
    p.src_index = _ptr(keep["idx"])
    p.threads = int(threads)
    return p, keep


def fused_augment(image, top, left, height, width, flip=0, matrix=None, interpolation="nearest",
                  fill=0.0, brightness=1.0, contrast=1.0, saturation=1.0, grayscale=0,
                  mean=None, std=None, *, flags=None, fma_coords="gpu",
                  contrast_mode=CONTRAST_FAST, gray_mean=None, want_index=False, threads=0):
    """The reference's fused pass on the CPU.

    Arguments follow the kernel launch at triton_augment/functional.py:1399-1431:
    per-image vectors (or scalars, broadcast) and an already-built inverse
    affine matrix ``[n, 6]`` (``None`` means the crop/flip-only path).  ``flags``
    overrides the value-based apply_* decisions with a dict of four booleans.
    Returns the output array, or ``(output, src_index)`` with ``want_index``.
    """
    p, keep = _prepare(image, top, left, height, width, flip, matrix, interpolation, fill,
                       brightness, contrast, saturation, grayscale, mean, std, flags,
                       fma_coords, contrast_mode, gray_mean, want_index, threads)
    if contrast_mode == CONTRAST_MEAN and p.apply_contrast and gray_mean is None:
        gm = np.empty((p.n,), np.float32)
        rc = lib().ta_oracle_gray_mean(C.byref(p), _ptr(gm))
        if rc != 0:
            raise RuntimeError(f"ta_oracle_gray_mean failed: {rc}")
        keep["gm"] = gm
        p.gray_mean = _ptr(gm)
    rc = lib().ta_oracle_fused_augment(C.byref(p))
    if rc != 0:
        raise RuntimeError(f"ta_oracle_fused_augment failed: {rc}")
    return (keep["out"], keep["idx"]) if want_index else keep["out"]


def gray_mean(image, top, left, height, width, flip=0, matrix=None, interpolation="nearest",
              fill=0.0, brightness=1.0, *, apply_brightness=None, fma_coords="gpu"):
    """Per-image grayscale mean of the geometry+brightness result (exact contrast)."""
    n = np.asarray(image).shape[0]
    b = _vec(brightness, n, np.asarray(image).dtype)
    flags = dict(brightness=bool(np.any(b != 1)) if apply_brightness is None else bool(apply_brightness),
                 contrast=False, saturation=False, grayscale=False)
    p, keep = _prepare(image, top, left, height, width, flip, matrix, interpolation, fill,
                       brightness, 1.0, 1.0, 0, None, None, flags, fma_coords, CONTRAST_FAST,
                       None, False, 0)
    gm = np.empty((p.n,), np.float32)
    rc = lib().ta_oracle_gray_mean(C.byref(p), _ptr(gm))
    if rc != 0:
        raise RuntimeError(f"ta_oracle_gray_mean failed: {rc}")
    return gm


def inverse_affine_matrix(center, angle, translate, scale, shear):
    """fp32/libm evaluation of triton_augment/functional.py:824-892; returns [n, 6]."""
    angle = np.ascontiguousarray(angle, np.float32)
    n = angle.shape[0]
    center = np.ascontiguousarray(center, np.float32).reshape(n, 2)
    translate = np.ascontiguousarray(translate, np.float32).reshape(n, 2)
    scale = np.ascontiguousarray(scale, np.float32).reshape(n)
    shear = np.ascontiguousarray(shear, np.float32).reshape(n, 2)
    out = np.empty((n, 6), np.float32)
    lib().ta_oracle_inverse_affine_matrix(n, _ptr(center), _ptr(angle), _ptr(translate), _ptr(scale),
                                          _ptr(shear), _ptr(out))
    return out
