"""Stand-alone functionals.  Each is the fused kernel with neutral arguments for
everything it does not do, so there is one CUDA code path to verify.  Names,
arguments and exceptions follow triton_augment/functional.py (cited per function).
"""
from __future__ import annotations

from typing import Sequence

import torch

from . import _lib
from . import functional as _F

__all__ = [
    "adjust_brightness", "adjust_contrast", "adjust_contrast_fast", "adjust_saturation", "normalize",
    "rgb_to_grayscale", "crop", "center_crop", "horizontal_flip", "affine", "rotate", "_apply_affine_matrix",
]


def _identity_geometry(image):
    n, _, h, w = image.shape
    return dict(height=h, width=w, top=None, left=None, flip=None, matrix=None, bilinear=False, fill=0.0)


def _colour_only(image, bits, *, brightness=None, contrast=None, saturation=None, gray=None, mean=None, std=None,
                 contrast_mode=_lib.CONTRAST_FAST):
    g = _identity_geometry(image)
    return _F._run_fused(image, g["height"], g["width"], None, None, None, None, False, 0.0, brightness, contrast,
                         saturation, gray, mean, std, bits, contrast_mode)


def _factor(image, value):
    return torch.full((image.shape[0],), value, dtype=image.dtype, device=image.device)


def adjust_brightness(image, brightness_factor: float):
    """clamp(x * factor, 0, 1).  Reference: functional.py:273-326."""
    _F._validate_image_tensor(image, "image")
    if brightness_factor < 0:
        raise ValueError(f"brightness_factor ({brightness_factor}) is not non-negative.")
    return _colour_only(image, _lib.APPLY_BRIGHTNESS, brightness=_factor(image, brightness_factor))


def adjust_contrast(image, contrast_factor: float):
    """torchvision-exact contrast: clamp(x * f + mean_n * (1 - f)) with mean_n the image's grayscale
    mean.  Reference: functional.py:329-403 (three passes there; a reduction pre-pass and the fused
    kernel here)."""
    _F._validate_image_tensor(image, "image")
    if contrast_factor < 0:
        raise ValueError(f"contrast_factor ({contrast_factor}) is not non-negative.")
    return _colour_only(image, _lib.APPLY_CONTRAST, contrast=_factor(image, contrast_factor),
                        contrast_mode=_lib.CONTRAST_MEAN)


def adjust_contrast_fast(image, contrast_factor: float):
    """clamp((x - 0.5) * f + 0.5).  Reference: functional.py:406-470."""
    _F._validate_image_tensor(image, "image")
    if contrast_factor < 0:
        raise ValueError(f"contrast_factor ({contrast_factor}) is not non-negative.")
    return _colour_only(image, _lib.APPLY_CONTRAST, contrast=_factor(image, contrast_factor))


def adjust_saturation(image, saturation_factor: float):
    """Blend with the pixel's own grayscale.  1-channel images are returned as a copy.
    Reference: functional.py:473-541."""
    _F._validate_image_tensor(image, "image")
    if saturation_factor < 0:
        raise ValueError(f"saturation_factor ({saturation_factor}) is not non-negative.")
    if image.shape[1] == 1:
        return image.clone()
    return _colour_only(image, _lib.APPLY_SATURATION, saturation=_factor(image, saturation_factor))


def normalize(image, mean, std):
    """(x - mean_c) / std_c.  Reference: functional.py:544-602."""
    _F._validate_image_tensor(image, "image")
    if len(mean) != 3 or len(std) != 3:
        raise ValueError("mean and std must have 3 values for RGB channels")
    return _colour_only(image, _lib.APPLY_NORMALIZE, mean=_F._rounded_triple(mean, image.dtype),
                        std=_F._rounded_triple(std, image.dtype))


def rgb_to_grayscale(image, num_output_channels: int = 1, grayscale_mask=None):
    """0.2989 R + 0.587 G + 0.114 B, replicated to 3 channels; optional per-image mask.  With
    ``num_output_channels=1`` the result is channel 0 of the 3-channel buffer, as in the
    reference (functional.py:190-270)."""
    _F._validate_image_tensor(image, "image")
    if num_output_channels not in (1, 3):
        raise ValueError(f"num_output_channels must be 1 or 3, got {num_output_channels}")
    if image.shape[1] != 3:
        raise ValueError(f"Expected 3 channels (RGB), got {image.shape[1]}")
    n = image.shape[0]
    if grayscale_mask is None:
        mask = torch.ones(n, dtype=torch.bool, device=image.device)
    else:
        mask = _F._convert_to_tensor(grayscale_mask, n, torch.bool, image.device, "grayscale_mask")
    out = _colour_only(image, _lib.APPLY_GRAYSCALE, gray=mask)
    return out[:, 0:1, :, :] if num_output_channels == 1 else out


def crop(image, top, left, height: int, width: int, fill=0.0):
    """Copy a window; ``top`` / ``left`` are ints or int tensors of shape ``(N,)``.
    Reference: functional.py:610-690.

    The window may leave the image (negative offsets, or a window larger than the image): the
    part outside reads ``fill`` (a number, or one value per channel; default 0, which is what
    torchvision's ``crop`` pads with).  The reference notes this as future work
    (functional.py:644-646) and reads out of bounds."""
    _F._validate_image_tensor(image, "image")
    n, c, h, w = image.shape
    if height <= 0 or width <= 0:
        raise ValueError(f"Crop size must be positive, got height={height}, width={width}")
    top_t = _F._convert_to_tensor(top, n, torch.int32, image.device, "top").to(torch.float32)
    left_t = _F._convert_to_tensor(left, n, torch.int32, image.device, "left").to(torch.float32)
    fill = _F._fill_arg(fill, c)
    if fill == 0.0 or fill == [0.0, 0.0, 0.0]:
        return _F._run_fused(image, height, width, top_t, left_t, None, None, False, 0.0, None, None, None, None,
                             None, None, 0)
    # A fill value other than zero: the same window through the nearest-neighbour affine kernel with
    # the identity matrix, which reads exactly the texels a crop reads and knows about fill values.
    identity = torch.tensor([1.0, 0.0, 0.0, 0.0, 1.0, 0.0], device=image.device).repeat(n, 1)
    return _F._run_fused(image, height, width, top_t, left_t, None, identity, False, fill, None, None, None, None,
                         None, None, 0)


def center_crop(image, output_size):
    """Reference: functional.py:693-747.  Offsets are (size - crop) // 2 as there; torchvision
    rounds (size - crop) / 2 instead, which differs by one pixel when the difference is odd."""
    _F._validate_image_tensor(image, "image")
    if isinstance(output_size, int):
        ch = cw = output_size
    elif isinstance(output_size, (tuple, list)) and len(output_size) == 1:
        ch = cw = output_size[0]
    else:
        ch, cw = output_size
    h, w = image.shape[2], image.shape[3]
    if ch > h or cw > w:
        raise ValueError(f"Crop size ({ch}, {cw}) larger than image size ({h}, {w}). "
                         f"Padding not yet supported in MVP.")
    return crop(image, (h - ch) // 2, (w - cw) // 2, ch, cw)


def horizontal_flip(image, flip_mask=None):
    """Mirror left-right, all images or those selected by ``flip_mask``.  Reference:
    functional.py:750-821 (which returns a copy early when nothing is selected; the kernel
    produces the same copy without the device-to-host read)."""
    _F._validate_image_tensor(image, "image")
    n, _, h, w = image.shape
    if flip_mask is None:
        mask = torch.ones(n, dtype=torch.bool, device=image.device)
    else:
        mask = _F._convert_to_tensor(flip_mask, n, torch.bool, image.device, "flip_mask")
    return _F._run_fused(image, h, w, None, None, mask, None, False, 0.0, None, None, None, None, None, None, 0)


def _apply_affine_matrix(image, matrix, interpolation="bilinear", fill=0.0):
    """Resample with a given inverse matrix ``(6,)`` or ``(N, 6)``.  Reference: functional.py:895-975."""
    _F._validate_image_tensor(image, "image")
    _F._check_interpolation(interpolation)
    n, _, h, w = image.shape
    if matrix.ndim == 1 and matrix.shape[0] == 6:
        matrix = matrix.unsqueeze(0).repeat(n, 1)
    elif not (matrix.ndim == 2 and matrix.shape == (n, 6)):
        raise ValueError(f"matrix must be shape (6,) or ({n}, 6), got {matrix.shape}")
    matrix = matrix.to(dtype=torch.float32, device=image.device).contiguous()
    fill_val = _F._fill_arg(fill, image.shape[1])     # a sequence: one value per channel (the reference takes fill[0])
    return _F._run_fused(image, h, w, None, None, None, matrix, _F._is_bilinear(interpolation), fill_val, None,
                         None, None, None, None, None, 0)


def affine(image, angle, translate, scale, shear, interpolation=_F.InterpolationMode.NEAREST, fill=0.0, center=None):
    """Rotate / translate / scale / shear about the image centre (or ``center`` in pixels);
    scalars or per-image tensors.  Reference: functional.py:1041-1114."""
    _F._validate_image_tensor(image, "image")
    n, _, h, w = image.shape
    a, t, s, sh, c = _F._prepare_affine_params_to_tensor(angle, translate, scale, shear, center, n, h, w, image.device)
    return _apply_affine_matrix(image, _F._get_inverse_affine_matrix(c, a, t, s, sh), interpolation, fill)


def _expanded_size(matrix6, width: int, height: int):
    """Size of the canvas that holds a whole ``width x height`` image after the transform whose
    inverse is ``matrix6``: torchvision's rule (the corners' extent, snapped with a tolerance of
    1e-4, evaluated in float32 like torchvision's _compute_affine_output_size)."""
    m = torch.tensor(matrix6, dtype=torch.float32).view(2, 3)
    half_w, half_h = 0.5 * width, 0.5 * height
    pts = torch.tensor([[-half_w, -half_h, 1.0], [-half_w, half_h, 1.0], [half_w, half_h, 1.0], [half_w, -half_h, 1.0]])
    new_pts = torch.matmul(pts, m.T)
    half = torch.tensor([half_w, half_h])
    lo, hi = new_pts.min(dim=0).values + half, new_pts.max(dim=0).values + half
    tol = 1e-4
    size = torch.ceil((hi / tol).trunc_() * tol) - torch.floor((lo / tol).trunc_() * tol)
    return int(size[0]), int(size[1])


def rotate(image, angle, interpolation=_F.InterpolationMode.NEAREST, expand: bool = False, center=None, fill=0.0):
    """Rotate by ``angle`` degrees about the image centre (or ``center``).  Reference:
    functional.py:1117-1181, which raises NotImplementedError for ``expand=True``.

    ``expand=True`` (built here): the result is large enough to hold the whole rotated image -
    torchvision's size rule - and is the same resampling on that larger canvas: the kernel
    already takes an output size and a (possibly negative, possibly half-pixel) window offset, so
    the expanded image is the window centred on the input's centre.  One size per call, so the
    angle must be a number (or a tensor holding one value for all images); ``center`` must be None."""
    _F._validate_image_tensor(image, "image")
    if not expand:
        return affine(image, -angle, [0.0, 0.0], 1.0, [0.0, 0.0], interpolation, fill, center)
    if center is not None:
        raise ValueError("expand=True rotates about the image centre; center must be None")
    if isinstance(angle, torch.Tensor):
        if angle.numel() != 1 and not bool((angle == angle.reshape(-1)[0]).all()):
            raise ValueError("expand=True needs one angle for the whole batch: every image gets the same output size")
        angle = float(angle.reshape(-1)[0])
    _F._check_interpolation(interpolation)
    n, c, h, w = image.shape
    # the matrix on the host for the size rule, in torchvision's float64 formula for a pure rotation
    import math
    rot = math.radians(-float(angle))
    quarter = float(angle) % 360.0
    if quarter in (0.0, 180.0):
        ow, oh = w, h
    elif quarter in (90.0, 270.0):               # exact quarter turns swap the sides (torchvision takes its rot90 path)
        ow, oh = h, w
    else:
        ow, oh = _expanded_size([math.cos(rot), math.sin(rot), 0.0, -math.sin(rot), math.cos(rot), 0.0], w, h)
    a, t, s, sh, ctr = _F._prepare_affine_params_to_tensor(-float(angle), [0.0, 0.0], 1.0, [0.0, 0.0], None, n, h, w, image.device)
    matrix = _F._get_inverse_affine_matrix(ctr, a, t, s, sh).contiguous()
    top = torch.full((n,), (h - oh) * 0.5, dtype=torch.float32, device=image.device)
    left = torch.full((n,), (w - ow) * 0.5, dtype=torch.float32, device=image.device)
    return _F._run_fused(image, oh, ow, top, left, None, matrix, _F._is_bilinear(interpolation), _F._fill_arg(fill, c),
                         None, None, None, None, None, None, 0)


apply_brightness = adjust_brightness
apply_contrast = adjust_contrast
apply_saturation = adjust_saturation
apply_normalize = normalize
