"""Geometric transform classes (re-exported by transforms.py)."""
from __future__ import annotations

import torch
import torch.nn as nn

from . import functional as F
from . import transforms as T
from .functional import InterpolationMode

__all__ = ["TritonRandomCrop", "TritonCenterCrop", "TritonRandomHorizontalFlip", "TritonRandomCropFlip",
           "TritonRandomAffine", "TritonRandomRotation"]

_NO_COLOUR = dict(brightness=False, contrast=False, saturation=False, grayscale=False)


def _draw_offsets(lay, h, w, th, tw, dtype):
    """Two ``randint`` draws, top then left (transforms.py:972-973, 1210-1211, 1464-1465)."""
    dev = lay.param_device
    top = torch.randint(0, h - th + 1, (lay.count,), device=dev, dtype=dtype)
    left = torch.randint(0, w - tw + 1, (lay.count,), device=dev, dtype=dtype)
    return top, left


def _padding_ltrb(padding):
    """torchvision's padding argument -> (left, top, right, bottom)."""
    if padding is None:
        return 0, 0, 0, 0
    if isinstance(padding, int):
        return padding, padding, padding, padding
    p = [int(v) for v in padding]
    if len(p) == 1:
        return p[0], p[0], p[0], p[0]
    if len(p) == 2:
        return p[0], p[1], p[0], p[1]
    if len(p) == 4:
        return tuple(p)
    raise ValueError(f"Padding must be an int or a 1, 2, or 4 element sequence, got {len(p)} elements")


class TritonRandomCrop(T._BatchAware):
    """Random ``size`` window per image.  Reference: transforms.py:899-989.

    ``padding``, ``pad_if_needed`` and ``fill`` (keyword arguments after the reference's; constant
    padding only) follow torchvision's RandomCrop: the window is drawn from the image padded by
    ``padding`` (and, with ``pad_if_needed``, by whatever a too-small side lacks, on both ends),
    and whatever part of it lies outside the image reads ``fill``.  Nothing is padded in memory:
    the kernel takes the window's offset, which may be negative.  Without them an image smaller
    than the window raises, as in the reference (which has no padding yet: functional.py:644-646)."""

    def __init__(self, size, same_on_batch: bool = False, same_on_frame: bool = True, padding=None,
                 pad_if_needed: bool = False, fill=0.0):
        super().__init__(same_on_batch, same_on_frame)
        self.size = T._size_pair(size)
        self.padding = _padding_ltrb(padding)
        if min(self.padding) < 0:
            raise ValueError("padding must not be negative")
        self.pad_if_needed = bool(pad_if_needed)
        self.fill = fill

    def forward(self, image: torch.Tensor) -> torch.Tensor:
        lay = self._layout(image)
        h, w = lay.image.shape[2:]
        th, tw = self.size
        left_pad, top_pad, right_pad, bottom_pad = self.padding
        if self.pad_if_needed:                    # torchvision pads a short side by the missing amount at both ends
            if h + top_pad + bottom_pad < th:
                d = th - (h + top_pad + bottom_pad)
                top_pad, bottom_pad = top_pad + d, bottom_pad + d
            if w + left_pad + right_pad < tw:
                d = tw - (w + left_pad + right_pad)
                left_pad, right_pad = left_pad + d, right_pad + d
        ph, pw = h + top_pad + bottom_pad, w + left_pad + right_pad
        if ph < th or pw < tw:
            raise ValueError(f"Image size ({h}, {w}) is smaller than crop size ({th}, {tw}). "
                             f"Padding not yet supported in MVP." if (ph, pw) == (h, w) else
                             f"Padded image size ({ph}, {pw}) is smaller than crop size ({th}, {tw}).")
        if (ph, pw) == (h, w) and self.fill in (0, 0.0):
            out = self._through_fused(image, self._twin)           # top and left from the one-launch sampler
            if out is not None:
                return out
        top, left = _draw_offsets(lay, ph, pw, th, tw, torch.int32)
        if top_pad or left_pad:
            top, left = top - top_pad, left - left_pad
        return lay.restore(F.crop(lay.image, lay.spread(top), lay.spread(left), th, tw, fill=self.fill))

    def _twin(self):
        from ._transforms_fused import TritonFusedAugment
        t = TritonFusedAugment(crop_size=self.size, same_on_batch=self.same_on_batch, same_on_frame=self.same_on_frame)
        t._draw_gray = False                     # this class draws top and left only
        return t

    def __repr__(self):
        return f"{self.__class__.__name__}(size={self.size}, " + self._tail()


class TritonCenterCrop(nn.Module):
    """Central ``size`` window.  Reference: transforms.py:992-1041 (no upload of host tensors)."""

    def __init__(self, size):
        super().__init__()
        self.size = T._size_pair(size)

    def forward(self, image: torch.Tensor) -> torch.Tensor:
        lay = T._Layout(image, False, True, upload=False)
        return lay.restore(F.center_crop(lay.image, self.size))

    def __repr__(self):
        return f"{self.__class__.__name__}(size={self.size})"


class TritonRandomHorizontalFlip(T._BatchAware):
    """Mirror with probability ``p`` per image; ``p == 0`` returns the input object without
    drawing.  Reference: transforms.py:1044-1114."""

    def __init__(self, p: float = 0.5, same_on_batch: bool = False, same_on_frame: bool = True):
        super().__init__(same_on_batch, same_on_frame)
        if not (0.0 <= p <= 1.0):
            raise ValueError(f"p ({p}) must be in [0, 1]")
        self.p = p

    def forward(self, image: torch.Tensor) -> torch.Tensor:
        if self.p == 0:
            return image
        out = self._through_fused(image, self._twin)
        if out is not None:
            return out
        lay = self._layout(image)
        mask = lay.spread(F._sample_bernoulli_tensor(lay.count, self.p, lay.param_device))
        return lay.restore(F.horizontal_flip(lay.image, flip_mask=mask))

    def _twin(self):
        from ._transforms_fused import TritonFusedAugment
        t = TritonFusedAugment(horizontal_flip_p=self.p, same_on_batch=self.same_on_batch, same_on_frame=self.same_on_frame)
        t._draw_gray = False                     # this class draws the flip mask only
        return t

    def __repr__(self):
        return f"{self.__class__.__name__}(p={self.p}, " + self._tail()


class TritonRandomCropFlip(T._BatchAware):
    """Random crop + random mirror in one launch.  Draws: int32 top, int32 left, then the
    flip mask - always, also for ``horizontal_flip_p == 0``.  Reference: transforms.py:1117-1249."""

    def __init__(self, size, horizontal_flip_p: float = 0.5, same_on_batch: bool = False, same_on_frame: bool = True):
        super().__init__(same_on_batch, same_on_frame)
        self.size = T._size_pair(size)
        if not (0.0 <= horizontal_flip_p <= 1.0):
            raise ValueError(f"horizontal_flip_p ({horizontal_flip_p}) must be in [0, 1]")
        self.horizontal_flip_p = horizontal_flip_p

    def forward(self, image: torch.Tensor) -> torch.Tensor:
        lay = self._layout(image)
        h, w = lay.image.shape[2:]
        th, tw = self.size
        if th > h or tw > w:
            raise ValueError(f"Crop size ({th}, {tw}) is larger than image size ({h}, {w})")
        out = self._through_fused(image, self._twin)
        if out is not None:
            return out
        top, left = _draw_offsets(lay, h, w, th, tw, torch.int32)
        flip = F._sample_bernoulli_tensor(lay.count, self.horizontal_flip_p, lay.param_device)
        out = F.fused_augment(lay.image, top=lay.spread(top), left=lay.spread(left), height=th, width=tw,
                              flip_horizontal=lay.spread(flip), brightness_factor=1.0, contrast_factor=1.0,
                              saturation_factor=1.0, grayscale=False, mean=None, std=None,
                              _flags=dict(affine=False, **_NO_COLOUR))
        return lay.restore(out)

    def _twin(self):
        from ._transforms_fused import TritonFusedAugment
        t = TritonFusedAugment(crop_size=self.size, horizontal_flip_p=self.horizontal_flip_p,
                               same_on_batch=self.same_on_batch, same_on_frame=self.same_on_frame)
        t._draw_flip_always, t._draw_gray = True, False      # this class draws top, left and - always - the flip mask
        return t

    def __repr__(self):
        return (f"{self.__class__.__name__}(size={self.size}, horizontal_flip_p={self.horizontal_flip_p}, "
                + self._tail())


class TritonRandomAffine(T._BatchAware):
    """Random rotation / translation / scale / shear with a constant-size output.

    Ranges follow torchvision's RandomAffine; unlike torchvision the sampled translation is
    not rounded to whole pixels (reference: transforms.py:1722-1727).  Draw order: angle
    (always), tx, ty (if translate), scale (if scale), shear x, shear y (if shear, the y draw
    happens even for a zero-width range).  Reference: transforms.py:1582-1817.
    """

    def __init__(self, degrees, translate=None, scale=None, shear=None, interpolation=InterpolationMode.NEAREST,
                 fill: float = 0.0, center=None, same_on_batch: bool = False, same_on_frame: bool = True):
        super().__init__(same_on_batch, same_on_frame)
        if isinstance(degrees, (int, float)):
            if degrees < 0:
                raise ValueError("If degrees is a single number, it must be positive.")
            self.degrees = (-float(degrees), float(degrees))
        else:
            if len(degrees) != 2:
                raise ValueError("If degrees is a sequence, it must be of length 2.")
            self.degrees = (float(degrees[0]), float(degrees[1]))
        self.translate = None
        if translate is not None:
            if len(translate) != 2:
                raise ValueError("translate should be a sequence of length 2.")
            if not (0.0 <= translate[0] <= 1.0 and 0.0 <= translate[1] <= 1.0):
                raise ValueError("translation values should be between 0 and 1")
            self.translate = (float(translate[0]), float(translate[1]))
        self.scale = None
        if scale is not None:
            if len(scale) != 2:
                raise ValueError("scale should be a sequence of length 2.")
            if scale[0] > scale[1]:
                raise ValueError("scale should be (min, max)")
            self.scale = (float(scale[0]), float(scale[1]))
        self.shear = None
        if shear is not None:
            if isinstance(shear, (int, float)):
                if shear < 0:
                    raise ValueError("If shear is a single number, it must be positive.")
                self.shear = (-float(shear), float(shear), 0.0, 0.0)
            elif len(shear) == 2:
                self.shear = (float(shear[0]), float(shear[1]), 0.0, 0.0)
            elif len(shear) == 4:
                self.shear = tuple(float(v) for v in shear)
            else:
                raise ValueError("shear should be a single number or a sequence of length 2 or 4.")
        self.interpolation = interpolation
        self.fill = [float(v) for v in fill] if isinstance(fill, (list, tuple)) else float(fill)   # number, or one per channel
        self.center = center

    def _get_params(self, param_count: int, device, img_size):
        height, width = img_size
        u = F._sample_uniform_tensor
        angle = u(param_count, self.degrees[0], self.degrees[1], device)
        if self.translate is not None:
            max_dx, max_dy = float(self.translate[0] * width), float(self.translate[1] * height)
            tx = u(param_count, -max_dx, max_dx, device)
            ty = u(param_count, -max_dy, max_dy, device)
            translate = torch.stack([tx, ty], dim=1)
        else:
            translate = torch.zeros((param_count, 2), device=device)
        scale = u(param_count, self.scale[0], self.scale[1], device) if self.scale is not None \
            else torch.ones(param_count, device=device)
        if self.shear is not None:
            sx = u(param_count, self.shear[0], self.shear[1], device)
            sy = u(param_count, self.shear[2], self.shear[3], device)
            shear = torch.stack([sx, sy], dim=1)
        else:
            shear = torch.zeros((param_count, 2), device=device)
        return angle, translate, scale, shear

    def _twin(self):
        from ._transforms_fused import TritonFusedAugment
        t = TritonFusedAugment(degrees=self.degrees, translate=self.translate, scale=self.scale, shear=self.shear,
                               interpolation=self.interpolation, fill=self.fill, same_on_batch=self.same_on_batch,
                               same_on_frame=self.same_on_frame)
        t._draw_gray = False                     # this class draws the affine parameters only
        return t

    def forward(self, img: torch.Tensor) -> torch.Tensor:
        # (a rotation centre other than the image's goes into the matrix, which the sampler builds for the
        #  image centre; a zero-width angle range with nothing else set would make the twin skip the angle draw)
        if self.center is None and (self.degrees != (0.0, 0.0) or self.translate is not None or self.scale is not None
                                    or self.shear is not None):
            twin = self.__dict__.get("_fused_twin")
            if twin is not None:                 # attributes that tests and users change after construction
                twin.interpolation, twin.fill = self.interpolation, self.fill
            out = self._through_fused(img, self._twin)
            if out is not None:
                return out
        lay = self._layout(img)
        h, w = lay.image.shape[2:]
        angle, translate, scale, shear = self._get_params(lay.count, lay.param_device, (h, w))
        out = F.affine(lay.image, angle=lay.spread(angle), translate=lay.spread2(translate), scale=lay.spread(scale),
                       shear=lay.spread2(shear), interpolation=self.interpolation, fill=self.fill, center=self.center)
        return lay.restore(out)

    def __repr__(self):
        return (f"{self.__class__.__name__}(degrees={self.degrees}, translate={self.translate}, scale={self.scale}, "
                f"shear={self.shear}, interpolation={self.interpolation}, fill={self.fill}, center={self.center}, "
                + self._tail())


class TritonRandomRotation(TritonRandomAffine):
    """Random rotation only.  Reference: transforms.py:1822-1902.

    ``expand=True`` (the reference raises NotImplementedError) enlarges the result to hold the
    whole rotated image.  All images of a call then need one output size, i.e. one angle: it
    works when a call draws a single parameter set (``same_on_batch=True`` with
    ``same_on_frame=True``, or a single image) and raises ValueError otherwise.  The angle is read
    back to the host to size the output (one device-to-host read per call)."""

    def __init__(self, degrees, interpolation=InterpolationMode.NEAREST, expand: bool = False, center=None,
                 fill: float = 0.0, same_on_batch: bool = False, same_on_frame: bool = True):
        if expand and center is not None:
            raise ValueError("expand=True rotates about the image centre; center must be None")
        self.expand = bool(expand)
        super().__init__(degrees=degrees, translate=None, scale=None, shear=None, interpolation=interpolation,
                         fill=fill, center=center, same_on_batch=same_on_batch, same_on_frame=same_on_frame)

    def forward(self, img: torch.Tensor) -> torch.Tensor:
        if not self.expand:
            return super().forward(img)
        lay = self._layout(img)
        if lay.count != 1:
            raise ValueError("expand=True gives every image of a call the same output size, so the call must draw ONE "
                             f"angle (same_on_batch=True and same_on_frame=True, or a single image); this call draws {lay.count}")
        h, w = lay.image.shape[2:]
        angle = float(self._get_params(1, lay.param_device, (h, w))[0][0])
        # affine(angle) is rotate(-angle): the class applies the drawn angle the way its parent does
        out = F.rotate(lay.image, -angle, interpolation=self.interpolation, expand=True, fill=self.fill)
        if lay.was_3d:
            return out.squeeze(0)
        return out.reshape(*lay.shape[:-2], *out.shape[-2:]) if len(lay.shape) == 5 else out

    def __repr__(self):
        return (f"{self.__class__.__name__}(degrees={self.degrees}, interpolation={self.interpolation}, "
                f"fill={self.fill}, " + self._tail())
