"""Colour transform classes (re-exported by transforms.py)."""
from __future__ import annotations

import torch
import torch.nn as nn

from . import functional as F
from . import transforms as T

__all__ = ["TritonColorJitter", "TritonNormalize", "TritonColorJitterNormalize", "TritonGrayscale",
           "TritonRandomGrayscale"]


def _draw_factor(rng_range, count, device):
    """One ``uniform_`` draw if the range can change the image, else ones and NO draw."""
    if rng_range is None:
        return torch.ones(count, device=device)
    return F._sample_uniform_tensor(count, rng_range[0], rng_range[1], device)


class _JitterBase(T._BatchAware):
    """brightness / contrast / saturation ranges and their sampling, shared by the three
    jittering classes.  Draw order: brightness, contrast, saturation (transforms.py:356-387)."""

    def __init__(self, brightness, contrast, saturation, same_on_batch, same_on_frame, contrast_mode="fast"):
        super().__init__(same_on_batch, same_on_frame)
        self.brightness = T._check_range(brightness, "brightness")
        self.contrast = T._check_range(contrast, "contrast")
        self.saturation = T._check_range(saturation, "saturation")
        F._contrast_mode(contrast_mode)
        self.contrast_mode = contrast_mode

    def _check_input(self, value, name, center=1.0, bound=(0, float("inf")), clip_first_on_zero=True):
        return T._check_range(value, name, center, bound, clip_first_on_zero)

    def _draw_jitter(self, count, device):
        return (_draw_factor(self.brightness, count, device), _draw_factor(self.contrast, count, device),
                _draw_factor(self.saturation, count, device))

    def _jitter_flags(self):
        return dict(affine=False, brightness=self.brightness is not None, contrast=self.contrast is not None,
                    saturation=self.saturation is not None, grayscale=False)


class TritonColorJitter(_JitterBase):
    """Random brightness, contrast (fast formula unless ``contrast_mode="torchvision"``) and
    saturation, per image or shared (``same_on_batch`` / ``same_on_frame``).
    Reference: transforms.py:251-455."""

    def __init__(self, brightness=None, contrast=None, saturation=None, same_on_batch: bool = False,
                 same_on_frame: bool = True, contrast_mode: str = "fast"):
        super().__init__(brightness, contrast, saturation, same_on_batch, same_on_frame, contrast_mode)

    def _get_params(self, param_count: int, device):
        return self._draw_jitter(param_count, device)

    def _twin(self):
        from ._transforms_fused import TritonFusedAugment
        t = TritonFusedAugment(brightness=self.brightness or 0, contrast=self.contrast or 0, saturation=self.saturation or 0,
                               same_on_batch=self.same_on_batch, same_on_frame=self.same_on_frame,
                               contrast_mode=self.contrast_mode)
        t._draw_gray = False                     # this class draws brightness, contrast, saturation only
        return t

    def forward(self, img: torch.Tensor) -> torch.Tensor:
        out = self._through_fused(img, self._twin)
        if out is not None:
            return out
        lay = self._layout(img)
        b, c, s = (lay.spread(p) for p in self._get_params(lay.count, lay.param_device))
        h, w = lay.image.shape[2:]
        out = F.fused_augment(lay.image, top=0, left=0, height=h, width=w, flip_horizontal=False,
                              brightness_factor=b, contrast_factor=c, saturation_factor=s, grayscale=False,
                              mean=None, std=None, contrast_mode=self.contrast_mode, _flags=self._jitter_flags())
        return lay.restore(out)

    def __repr__(self):
        return (f"{self.__class__.__name__}(brightness={self.brightness}, contrast={self.contrast}, "
                f"saturation={self.saturation}, " + self._tail())


class TritonNormalize(nn.Module):
    """(x - mean) / std per channel.  Reference: transforms.py:458-526."""

    def __init__(self, mean, std):
        super().__init__()
        self.mean, self.std = tuple(mean), tuple(std)
        if len(self.mean) != 3 or len(self.std) != 3:
            raise ValueError("mean and std must have 3 values for RGB channels")

    def forward(self, img: torch.Tensor) -> torch.Tensor:
        lay = T._Layout(img, False, True)
        return lay.restore(F.normalize(lay.image, mean=self.mean, std=self.std))

    def __repr__(self):
        return f"{self.__class__.__name__}(mean={self.mean}, std={self.std})"


class TritonColorJitterNormalize(_JitterBase):
    """Colour jitter + random grayscale + normalize in one kernel launch.
    Reference: transforms.py:529-746.  The grayscale mask is drawn on every call, also
    when ``grayscale_p == 0`` (transforms.py:664-666)."""

    def __init__(self, brightness=None, contrast=None, saturation=None, grayscale_p: float = 0.0, mean=None,
                 std=None, same_on_batch: bool = False, same_on_frame: bool = True, contrast_mode: str = "fast"):
        super().__init__(brightness, contrast, saturation, same_on_batch, same_on_frame, contrast_mode)
        self.grayscale_p = grayscale_p
        if not (0.0 <= grayscale_p <= 1.0):
            raise ValueError(f"grayscale_p must be in [0, 1], got {grayscale_p}")
        if (mean is None) != (std is None):
            raise ValueError("mean and std must both be provided or both be None")
        if mean is not None:
            mean = tuple(mean)
            if len(mean) != 3:
                raise ValueError("mean must have 3 values for RGB channels")
        if std is not None:
            std = tuple(std)
            if len(std) != 3:
                raise ValueError("std must have 3 values for RGB channels")
        self.mean, self.std = mean, std

    def _get_params(self, param_count: int, device):
        b, c, s = self._draw_jitter(param_count, device)
        return b, c, s, F._sample_bernoulli_tensor(param_count, self.grayscale_p, device)

    def _colour_flags(self, affine=False):
        flags = self._jitter_flags()
        flags.update(affine=affine, grayscale=self.grayscale_p > 0)
        return flags

    def _twin(self):
        from ._transforms_fused import TritonFusedAugment
        return TritonFusedAugment(brightness=self.brightness or 0, contrast=self.contrast or 0, saturation=self.saturation or 0,
                                  grayscale_p=self.grayscale_p, mean=self.mean, std=self.std, same_on_batch=self.same_on_batch,
                                  same_on_frame=self.same_on_frame, contrast_mode=self.contrast_mode)

    def forward(self, img: torch.Tensor) -> torch.Tensor:
        out = self._through_fused(img, self._twin)
        if out is not None:
            return out
        lay = self._layout(img)
        b, c, s, g = (lay.spread(p) for p in self._get_params(lay.count, lay.param_device))
        h, w = lay.image.shape[2:]
        out = F.fused_augment(lay.image, top=0, left=0, height=h, width=w, flip_horizontal=False,
                              brightness_factor=b, contrast_factor=c, saturation_factor=s, grayscale=g,
                              mean=self.mean, std=self.std, contrast_mode=self.contrast_mode,
                              _flags=self._colour_flags())
        return lay.restore(out)

    def __repr__(self):
        return (f"{self.__class__.__name__}(brightness={self.brightness}, contrast={self.contrast}, "
                f"saturation={self.saturation}, grayscale_p={self.grayscale_p}, mean={self.mean}, "
                f"std={self.std}, " + self._tail())


class TritonGrayscale(nn.Module):
    """RGB -> grayscale with 1 or 3 output channels.  Does not upload host tensors (the
    reference does not either: transforms.py:775-790)."""

    def __init__(self, num_output_channels: int = 1):
        super().__init__()
        if num_output_channels not in (1, 3):
            raise ValueError(f"num_output_channels must be 1 or 3, got {num_output_channels}")
        self.num_output_channels = num_output_channels

    def forward(self, image: torch.Tensor) -> torch.Tensor:
        lay = T._Layout(image, False, True, upload=False)
        return lay.restore(F.rgb_to_grayscale(lay.image, num_output_channels=self.num_output_channels))

    def __repr__(self):
        return f"{self.__class__.__name__}(num_output_channels={self.num_output_channels})"


class TritonRandomGrayscale(T._BatchAware):
    """Grayscale with probability ``p`` per image.  As in the reference (transforms.py:842-882)
    the INPUT OBJECT is returned when ``p == 0`` (no draw) or when no image was selected."""

    def __init__(self, p: float = 0.1, num_output_channels: int = 3, same_on_batch: bool = False,
                 same_on_frame: bool = True):
        super().__init__(same_on_batch, same_on_frame)
        if not (0.0 <= p <= 1.0):
            raise ValueError(f"p ({p}) must be in [0, 1]")
        if num_output_channels not in (1, 3):
            raise ValueError(f"num_output_channels must be 1 or 3, got {num_output_channels}")
        self.p, self.num_output_channels = p, num_output_channels

    def forward(self, image: torch.Tensor) -> torch.Tensor:
        if self.p == 0:
            return image
        lay = self._layout(image, upload=False)
        mask = lay.spread(F._sample_bernoulli_tensor(lay.count, self.p, lay.param_device))
        if not torch.any(mask).item():
            return image
        out = F.rgb_to_grayscale(lay.image, num_output_channels=self.num_output_channels, grayscale_mask=mask)
        return lay.restore(out)

    def __repr__(self):
        return (f"{self.__class__.__name__}(p={self.p}, num_output_channels={self.num_output_channels}, "
                + self._tail())
