"""Functional API: the host side of the fused augmentation pass.

Same names, arguments and error behaviour as triton_augment/functional.py of
yuhezhang-ai/triton-augment v0.3.0; every function ends in one call into
libta_b200.so (hand-written sm_100a CUDA) instead of a Triton launch.  The
stand-alone functionals are the fused kernel with no-op arguments.
"""
from __future__ import annotations

import os
from typing import Sequence

import torch

from . import _lib

__all__ = [
    "adjust_brightness", "adjust_contrast", "adjust_contrast_fast", "adjust_saturation", "normalize",
    "apply_brightness", "apply_contrast", "apply_saturation", "apply_normalize", "rgb_to_grayscale",
    "crop", "center_crop", "horizontal_flip", "affine", "rotate", "fused_augment",
]

_DEG2RAD = 3.141592653589793 / 180.0
# TA_B200_TORCH_MATRIX=1 builds the affine matrices with the reference's torch expressions
# instead of the library's single kernel (same bits either way; kept for cross-checking).
_MATRIX_KERNEL = os.environ.get("TA_B200_TORCH_MATRIX", "0") != "1"


class InterpolationMode:
    """Interpolation names accepted by the geometric functions (reference: functional.py:41-47)."""
    NEAREST = "nearest"
    BILINEAR = "bilinear"


# ----------------------------------------------------------------------------- checks and conversions
def _validate_image_tensor(tensor, name: str = "tensor", allow_uint8: bool = False) -> None:
    """Reference: functional.py:50-81 (same exception types).  ``allow_uint8``: the fused entry
    points also take bytes (an extension, see fused_augment)."""
    if not isinstance(tensor, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor, got {type(tensor)}")
    if not tensor.is_cuda:
        raise ValueError(f"{name} must be on CUDA device")
    if tensor.ndim != 4:
        raise ValueError(f"{name} must be a 4D tensor with shape (N, C, H, W), got shape {tensor.shape}")
    if tensor.shape[1] not in (1, 3):
        raise TypeError(f"Input image tensor permitted channel values are 1 or 3, but found {tensor.shape[1]}")
    if tensor.dtype not in (torch.float32, torch.float16) and not (allow_uint8 and tensor.dtype == torch.uint8):
        raise TypeError(f"{name} must be float32 or float16, got {tensor.dtype}")


def _work_dtype(image: torch.Tensor, out_dtype=None):
    """dtype of the result and of the per-image factors: the image's; for bytes float32, or
    float16 when ``out_dtype`` asks for it."""
    if image.dtype == torch.uint8:
        if out_dtype not in (None, torch.float32, torch.float16):
            raise TypeError(f"out_dtype must be torch.float32 or torch.float16, got {out_dtype}")
        return torch.float32 if out_dtype is None else out_dtype
    if out_dtype is not None and out_dtype != image.dtype:
        raise ValueError(f"out_dtype applies to uint8 images; a {image.dtype} image gives a {image.dtype} result")
    return image.dtype


def _convert_to_tensor(value, batch_size: int, dtype, device, name: str = "parameter") -> torch.Tensor:
    """Scalar -> filled ``(N,)`` tensor; tensor -> checked and cast (reference: functional.py:88-135)."""
    if isinstance(value, torch.Tensor):
        if value.shape != (batch_size,):
            raise ValueError(f"{name} tensor must have shape ({batch_size},), got {value.shape}")
        # dense: the library reads [n] vectors by pointer, so a strided view (params[:, 0], x[::2]) is copied
        return value.to(device=device, dtype=dtype).contiguous()
    return torch.full((batch_size,), value, dtype=dtype, device=device)


def _sample_uniform_tensor(size: int, min_val: float, max_val: float, device) -> torch.Tensor:
    """One ``uniform_`` draw of ``size`` values from the device's default generator (functional.py:162)."""
    return torch.empty(size, device=device).uniform_(min_val, max_val)


def _sample_bernoulli_tensor(size: int, p: float, device) -> torch.Tensor:
    """``rand(size) < p`` (functional.py:187)."""
    return torch.rand(size, device=device) < p


def _pair_tensor(value, batch_size: int, device, name: str) -> torch.Tensor:
    """``[a, b]`` / ``(2,)`` / ``(N, 2)`` -> fp32 ``(N, 2)`` (reference: functional.py:996-1021)."""
    if isinstance(value, torch.Tensor):
        if value.ndim == 1 and value.shape[0] == 2:
            return value.unsqueeze(0).repeat(batch_size, 1).to(device=device, dtype=torch.float32)
        if value.ndim == 2 and value.shape == (batch_size, 2):
            return value.to(device=device, dtype=torch.float32).contiguous()
        raise ValueError(f"{name} tensor must be shape (2,) or ({batch_size}, 2), got {value.shape}")
    if len(value) != 2:
        raise ValueError(f"{name} must have 2 values, got {len(value)}")
    return torch.tensor([value], device=device, dtype=torch.float32).repeat(batch_size, 1)


def _prepare_affine_params_to_tensor(angle, translate, scale, shear, center, batch_size, height, width, device):
    """Reference: functional.py:978-1038.  ``center`` in pixels becomes an offset from the image centre."""
    angle_t = _convert_to_tensor(angle, batch_size, torch.float32, device, "angle")
    translate_t = _pair_tensor(translate, batch_size, device, "translate")
    scale_t = _convert_to_tensor(scale, batch_size, torch.float32, device, "scale")
    shear_t = _pair_tensor(shear, batch_size, device, "shear")
    if center is None:
        center_t = torch.zeros(batch_size, 2, device=device, dtype=torch.float32)
    else:
        if len(center) != 2:
            raise ValueError(f"center must have 2 values, got {len(center)}")
        center_t = torch.tensor([[center[0] - width * 0.5, center[1] - height * 0.5]], device=device,
                                dtype=torch.float32).repeat(batch_size, 1)
    return angle_t, translate_t, scale_t, shear_t, center_t


def _get_inverse_affine_matrix(center, angle, translate, scale, shear) -> torch.Tensor:
    """Inverse of translate * centre * rotate-scale-shear * centre^-1 as ``[N, 6]`` rows.

    The formula is torchvision's; the order of the elementwise torch operations is the
    reference's (functional.py:853-890) on purpose: the matrix is an input of the kernel,
    and both kernels must see bit-identical inputs for their outputs to be comparable.
    """
    if _MATRIX_KERNEL and angle.is_cuda and all(t.dtype == torch.float32 and t.device == angle.device
                                               for t in (center, angle, translate, scale, shear)):
        # One launch instead of ~30 elementwise ones.  The kernel rounds every operation
        # individually in the order below and returns the same bits as the torch expressions
        # (tests/test_gpu_api.py::test_matrix_kernel_is_bit_identical_to_torch_ops).
        return _lib.inverse_affine_matrix(center, angle, translate, scale, shear)
    rot = angle * _DEG2RAD
    sx = shear[:, 0] * _DEG2RAD
    sy = shear[:, 1] * _DEG2RAD
    cx, cy = center[:, 0], center[:, 1]
    tx, ty = translate[:, 0], translate[:, 1]
    cos_sy = torch.cos(sy)
    a = torch.cos(rot - sy) / cos_sy
    b = -torch.cos(rot - sy) * torch.tan(sx) / cos_sy - torch.sin(rot)
    c = torch.sin(rot - sy) / cos_sy
    d = -torch.sin(rot - sy) * torch.tan(sx) / cos_sy + torch.cos(rot)
    m0, m1, m3, m4 = d / scale, -b / scale, -c / scale, a / scale
    m2 = m0 * (-cx - tx) + m1 * (-cy - ty)
    m5 = m3 * (-cx - tx) + m4 * (-cy - ty)
    return torch.stack([m0, m1, m2 + cx, m3, m4, m5 + cy], dim=1)


def _prepare_affine_matrix_only(batch_size, device, img_height, img_width, angle, translate, scale, shear, center):
    """Reference: functional.py:1185-1215."""
    a, t, s, sh, c = _prepare_affine_params_to_tensor(angle, translate, scale, shear, center, batch_size,
                                                      img_height, img_width, device)
    return _get_inverse_affine_matrix(c, a, t, s, sh)


def _fill_arg(fill, channels: int = 3):
    """``fill`` as the library takes it: a float, or a list of per-channel floats.

    A number or None (= 0) fills every channel alike.  A sequence gives one value per channel,
    as in torchvision (one value: all channels); the reference reads only the first value of a
    sequence and marks per-channel values as to do (functional.py:942-945)."""
    if fill is None:
        return 0.0
    if isinstance(fill, (list, tuple)):
        vals = [float(v) for v in fill]
        if len(vals) == 1:
            return vals[0]
        if len(vals) != channels:
            raise ValueError(f"fill has {len(vals)} values but the image has {channels} channels")
        return vals if channels == 3 else vals[0]
    return float(fill)


def _is_bilinear(interpolation) -> bool:
    return str(interpolation).lower() == "bilinear"


def _check_interpolation(interpolation) -> None:
    if str(interpolation).lower() not in ("nearest", "bilinear"):
        raise ValueError(f"Only 'nearest' and 'bilinear' interpolation are supported, got {interpolation}")


_TRIPLE_CACHE = {}


def _rounded_triple(values, dtype):
    """mean/std as Python floats holding image-dtype-rounded values (functional.py:1350-1351)."""
    key = (tuple(float(v) for v in values), dtype)
    hit = _TRIPLE_CACHE.get(key)
    if hit is None:
        hit = [float(v) for v in torch.tensor(key[0], dtype=dtype).to(torch.float32)]
        if len(_TRIPLE_CACHE) < 64:
            _TRIPLE_CACHE[key] = hit
    return hit


def _contrast_mode(mode) -> int:
    m = str(mode).lower()
    if m == "fast":
        return _lib.CONTRAST_FAST
    if m in ("torchvision", "mean", "exact"):
        return _lib.CONTRAST_MEAN
    raise ValueError(f"contrast_mode must be 'fast' or 'torchvision', got {mode}")


# ----------------------------------------------------------------------------- the one launch
def _run_fused(image, height, width, top, left, flip, matrix, bilinear, fill, brightness, contrast,
               saturation, gray, mean, std, apply_bits, contrast_mode=_lib.CONTRAST_FAST, out_dtype=None, first_image=0):
    """Allocate the output and enqueue the kernel(s) on torch's current stream."""
    image = image.contiguous()
    n, c = image.shape[0], image.shape[1]
    if c == 1 and apply_bits & (_lib.APPLY_SATURATION | _lib.APPLY_GRAYSCALE):
        raise ValueError("saturation and grayscale need a 3-channel image")
    work = _work_dtype(image, out_dtype)
    mean_mode = bool(apply_bits & _lib.APPLY_CONTRAST) and contrast_mode == _lib.CONTRAST_MEAN
    if mean_mode and image.dtype == torch.uint8 and work == torch.float16:
        raise ValueError('contrast_mode="torchvision" reads uint8 images into float32 results only')
    out = torch.empty(n, c, height, width, dtype=work, device=image.device)
    if n == 0:
        return out
    params = _lib.make_params(image, out, top, left, flip, matrix, fill, bilinear, apply_bits, brightness,
                              contrast, saturation, gray, mean, std, contrast_mode)
    if mean_mode and not first_image:
        _lib.launch_fused_mean(params, image.device)      # reduction + fused pass, one launch where possible
        return out
    keep = None
    if mean_mode:
        keep = _lib.launch_gray_mean(params, image.device)
        params.gray_mean = keep.data_ptr()
    _lib.launch_fused(params, image.device, first_image=first_image)
    return out


def fused_augment(image, top, left, height: int, width: int, flip_horizontal=False, angle=0.0,
                  translate=[0.0, 0.0], scale=1.0, shear=[0.0, 0.0], interpolation="nearest", fill=0.0,
                  center=None, brightness_factor=1.0, contrast_factor=1.0, saturation_factor=1.0,
                  grayscale=False, mean=None, std=None, *, contrast_mode="fast", out_dtype=None, _flags=None,
                  _matrix=None, _first_image=0) -> torch.Tensor:
    """Affine + crop + flip + brightness + contrast + saturation + grayscale + normalize, one pass.

    Drop-in for the reference's ``fused_augment`` (functional.py:1218-1433): per-image
    arguments are Python scalars or ``(N,)`` tensors (translate/shear: 2-lists, ``(2,)`` or
    ``(N, 2)``), operations whose arguments are all neutral are skipped, any non-identity
    affine argument selects the affine path.  Returns a new ``(N, C, height, width)`` tensor.

    Extra: ``fill`` may be a sequence of one value per channel (torchvision's meaning; the
    reference uses the first value for every channel).

    Extra, keyword only: ``contrast_mode="torchvision"`` blends towards the per-image
    grayscale mean (torchvision's adjust_contrast) instead of 0.5; ``_flags`` lets the
    transform classes state which operations are on, which saves the device-to-host reads
    that deciding it from tensor values needs.

    Extra: a ``torch.uint8`` image is read as ``value / 255`` (torchvision's ToTensor scaling)
    inside the kernel and gives a float32 result equal, within float32 tolerance, to the call on
    ``image.float() / 255`` - without that tensor ever existing, and with a quarter of the input
    traffic.  The reference takes float images only.  The classes that are one call of this
    function (TritonFusedAugment, TritonColorJitterNormalize, TritonColorJitter,
    TritonRandomCropFlip, ...) therefore take bytes too; the stand-alone functionals do not.
    ``contrast_mode="torchvision"`` on bytes needs a width that is a multiple of 16 (the mean
    pre-pass stages whole 16-byte units of a row) and raises otherwise.
    ``out_dtype=torch.float16`` (uint8 images only) rounds ``value / 255`` to half and continues
    like a float16 image: half the output bytes of the float32 result, equal to the call on
    ``(image.float() / 255).half()`` within the float16 tolerance; not with
    ``contrast_mode="torchvision"``.
    """
    _validate_image_tensor(image, "image", allow_uint8=True)
    n, _, img_h, img_w = image.shape
    if height <= 0 or width <= 0:
        raise ValueError(f"Crop size must be positive, got height={height}, width={width}")
    dev, dt = image.device, _work_dtype(image, out_dtype)

    brightness = _convert_to_tensor(brightness_factor, n, dt, dev, "brightness_factor")
    contrast = _convert_to_tensor(contrast_factor, n, dt, dev, "contrast_factor")
    saturation = _convert_to_tensor(saturation_factor, n, dt, dev, "saturation_factor")
    gray = _convert_to_tensor(grayscale, n, torch.bool, dev, "grayscale")
    apply_norm = mean is not None and std is not None
    if apply_norm and (len(mean) != 3 or len(std) != 3):
        raise ValueError("mean and std must have 3 values for RGB channels")

    if _flags is None:
        _flags = _flags_from_values(angle, translate, scale, shear, brightness_factor, contrast_factor,
                                    saturation_factor, grayscale, brightness, contrast, saturation, gray)
    bits = ((_lib.APPLY_BRIGHTNESS if _flags["brightness"] else 0) | (_lib.APPLY_CONTRAST if _flags["contrast"] else 0)
            | (_lib.APPLY_SATURATION if _flags["saturation"] else 0) | (_lib.APPLY_GRAYSCALE if _flags["grayscale"] else 0)
            | (_lib.APPLY_NORMALIZE if apply_norm else 0))

    top_t = _convert_to_tensor(top, n, torch.float32, dev, "top")
    left_t = _convert_to_tensor(left, n, torch.float32, dev, "left")
    flip_t = _convert_to_tensor(flip_horizontal, n, torch.bool, dev, "flip_horizontal")
    matrix = None
    if _flags["affine"] and _matrix is not None:
        matrix = _matrix                 # built by the caller from these same parameters
    elif _flags["affine"]:
        matrix = _prepare_affine_matrix_only(n, dev, img_h, img_w, angle, translate, scale, shear, center).contiguous()
    return _run_fused(image, height, width, top_t, left_t, flip_t, matrix, _flags["affine"] and _is_bilinear(interpolation),
                      _fill_arg(fill, image.shape[1]), brightness, contrast, saturation, gray,
                      _rounded_triple(mean, dt) if apply_norm else None, _rounded_triple(std, dt) if apply_norm else None,
                      bits, _contrast_mode(contrast_mode), out_dtype, _first_image)


def _flags_from_values(angle, translate, scale, shear, bf_arg, cf_arg, sf_arg, gray_arg, bf, cf, sf, gray):
    """Which operations are on, decided from argument VALUES exactly like the reference
    (functional.py:1308-1332, 1341-1344, 1356).  Python scalars are decided on the host;
    all tensor arguments are decided together with a single device-to-host read."""
    host = {"affine": False, "brightness": None, "contrast": None, "saturation": None, "grayscale": None}
    pending = {}

    def scalar_or_tensor(key, arg, tensor_test, scalar_test):
        if isinstance(arg, torch.Tensor):
            pending.setdefault(key, []).append(tensor_test)
        elif scalar_test(arg):
            host[key] = True

    scalar_or_tensor("affine", angle, lambda: torch.any(angle != 0), lambda v: v != 0)
    scalar_or_tensor("affine", translate, lambda: torch.any(translate != 0), lambda v: v[0] != 0 or v[1] != 0)
    scalar_or_tensor("affine", scale, lambda: torch.any(scale != 1.0), lambda v: v != 1.0)
    scalar_or_tensor("affine", shear, lambda: torch.any(shear != 0), lambda v: v[0] != 0 or v[1] != 0)
    for key, arg, t in (("brightness", bf_arg, bf), ("contrast", cf_arg, cf), ("saturation", sf_arg, sf)):
        if isinstance(arg, torch.Tensor):
            pending[key] = [lambda t=t: torch.any(t != 1.0)]
        else:
            # the reference compares the image-dtype tensor it filled with the scalar
            host[key] = bool(torch.tensor(arg, dtype=t.dtype) != 1.0)
    if isinstance(gray_arg, torch.Tensor):
        pending["grayscale"] = [lambda: torch.any(gray)]
    else:
        host["grayscale"] = bool(gray_arg)
    if pending:
        keys = [k for k in pending if not host.get(k)]
        if keys:
            dev = bf.device
            stacked = torch.stack([torch.stack([f().to(dev) for f in pending[k]]).any() for k in keys])
            for k, v in zip(keys, stacked.tolist()):
                host[k] = bool(v) or bool(host.get(k))
    return {k: bool(v) for k, v in host.items()}


from ._functional_ops import *  # noqa: E402,F401,F403  (stand-alone functionals built on _run_fused)
from ._functional_ops import apply_brightness, apply_contrast, apply_normalize, apply_saturation  # noqa: E402,F401
