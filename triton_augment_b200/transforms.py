"""Transform classes: the `nn.Module` face of the fused augmentation pass.

Same class names, constructor arguments, defaults, exceptions and - above all - the
same order and size of random draws as triton_augment/transforms.py of
yuhezhang-ai/triton-augment v0.3.0, so a seed gives the same parameters.  The
structure is not the reference's: shape handling and parameter broadcasting live in
one base class and one layout object instead of being repeated per class.
"""
from __future__ import annotations

import collections.abc
from typing import Optional, Sequence, Tuple, Union

import torch
import torch.nn as nn

from . import functional as F
from .functional import InterpolationMode

__all__ = [
    "TritonColorJitter", "TritonNormalize", "TritonColorJitterNormalize", "TritonGrayscale",
    "TritonRandomGrayscale", "TritonRandomCrop", "TritonCenterCrop", "TritonRandomHorizontalFlip",
    "TritonRandomCropFlip", "TritonRandomRotation", "TritonRandomAffine", "TritonFusedAugment",
]


# ----------------------------------------------------------------------------- shapes and broadcasting
def _normalize_video_shape(image: torch.Tensor):
    """(C,H,W) / (N,C,H,W) / (N,T,C,H,W) -> (N*,C,H,W) plus what is needed to undo it.
    Reference: transforms.py:26-68."""
    shape, was_3d = image.shape, image.ndim == 3
    if was_3d:
        return image.unsqueeze(0), None, None, shape, True
    if image.ndim == 4:
        return image, image.shape[0], None, shape, False
    if image.ndim == 5:
        return image.reshape(-1, *image.shape[2:]), image.shape[0], image.shape[1], shape, False
    raise ValueError(f"Expected 3D, 4D, or 5D tensor, got {image.ndim}D tensor with shape {image.shape}")


def _compute_param_count(batch_size, num_frames, same_on_batch: bool, same_on_frame: bool) -> int:
    """How many independent parameter sets to draw: 1, N, T or N*T.  Reference: transforms.py:71-114."""
    if batch_size is None:
        return 1
    if num_frames is None:
        return 1 if same_on_batch else batch_size
    n = 1 if same_on_batch else batch_size
    t = 1 if same_on_frame else num_frames
    return n * t


def _broadcast_params_to_all_samples(params, batch_size, num_frames, total_samples, same_on_batch, same_on_frame):
    """Spread ``[P]`` drawn values over the ``N*T`` flattened samples (video-major).
    Reference: transforms.py:117-197, including its rule that a vector which already has
    ``total_samples`` entries is returned untouched."""
    count = params.shape[0]
    if count == total_samples:
        return params
    if count == 1:
        return params.expand(total_samples).contiguous()
    if batch_size is None or num_frames is None:
        return params
    n, t = batch_size, num_frames
    if same_on_frame and not same_on_batch:
        if count != n:
            raise ValueError(f"Expected {n} params for same_on_frame=True, got {count}")
        return params.unsqueeze(1).expand(n, t).reshape(-1).contiguous()
    if same_on_batch and not same_on_frame:
        if count != t:
            raise ValueError(f"Expected {t} params for same_on_batch=True, got {count}")
        return params.unsqueeze(0).expand(n, t).reshape(-1).contiguous()
    raise ValueError(f"Unexpected param shape {params.shape} for video with batch_size={batch_size}, "
                     f"num_frames={num_frames}, total_samples={total_samples}, "
                     f"same_on_batch={same_on_batch}, same_on_frame={same_on_frame}")


def _broadcast_2d_params(params, batch_size, num_frames, total_samples, same_on_batch, same_on_frame):
    """``[P, 2]`` version of the above.  Reference: transforms.py:200-218."""
    if params.shape[0] == total_samples:
        return params
    cols = [_broadcast_params_to_all_samples(params[:, i], batch_size, num_frames, total_samples,
                                             same_on_batch, same_on_frame) for i in (0, 1)]
    return torch.stack(cols, dim=1)


def _reshape_to_original(output, original_shape, was_3d: bool):
    """Reference: transforms.py:222-248."""
    if was_3d:
        return output.squeeze(0)
    if len(original_shape) == 5:
        return output.reshape(original_shape[0], original_shape[1], *output.shape[1:])
    return output


def _ensure_cuda(img: torch.Tensor) -> torch.Tensor:
    """Host tensors are uploaded; the result stays on the GPU (reference: transforms.py:1498-1504)."""
    if img.is_cuda:
        return img
    if not torch.cuda.is_available():
        raise RuntimeError("Triton-Augment requires CUDA, but CUDA is not available. "
                           "Please ensure you have a CUDA-capable GPU and PyTorch with CUDA support.")
    return img.cuda()


def _check_range(value, name, center=1.0, bound=(0, float("inf")), clip_first_on_zero=True):
    """Jitter argument -> ``(lo, hi)`` or None when it cannot change anything.  torchvision's
    ColorJitter rule as used by the reference (transforms.py:325-354)."""
    if value is None:
        return None
    if isinstance(value, (int, float)):
        if value < 0:
            raise ValueError(f"If {name} is a single number, it must be non negative.")
        value = [center - float(value), center + float(value)]
        if clip_first_on_zero:
            value[0] = max(value[0], 0.0)
    elif isinstance(value, collections.abc.Sequence) and len(value) == 2:
        value = [float(v) for v in value]
    else:
        raise TypeError(f"{name}={value} should be a single number or a sequence with length 2.")
    if not bound[0] <= value[0] <= value[1] <= bound[1]:
        raise ValueError(f"{name} values should be between {bound} and increasing, but got {value}.")
    return None if value[0] == value[1] == center else (float(value[0]), float(value[1]))


def _size_pair(size):
    if isinstance(size, int):
        pair = (size, size)
    elif isinstance(size, (tuple, list)) and len(size) == 1:
        pair = (size[0], size[0])
    else:
        pair = tuple(size)
    if len(pair) != 2:
        raise ValueError(f"size must have 2 elements, got {len(pair)}")
    return pair


class _Layout:
    """Shape bookkeeping of one forward call."""

    def __init__(self, image: torch.Tensor, same_on_batch: bool, same_on_frame: bool, upload: bool = True,
                 param_device=None):
        flat, self.batch, self.frames, self.shape, self.was_3d = _normalize_video_shape(image)
        self.image = _ensure_cuda(flat) if upload else flat
        # where the random parameters are drawn: the image's device, like the reference
        self.param_device = self.image.device if param_device is None else torch.device(param_device)
        self.sob, self.sof = same_on_batch, same_on_frame
        self.total = self.image.shape[0]
        self.count = _compute_param_count(self.batch, self.frames, same_on_batch, same_on_frame)

    def spread(self, p):
        return _broadcast_params_to_all_samples(p, self.batch, self.frames, self.total, self.sob, self.sof)

    def spread2(self, p):
        return _broadcast_2d_params(p, self.batch, self.frames, self.total, self.sob, self.sof)

    def restore(self, out):
        return _reshape_to_original(out, self.shape, self.was_3d)


class _BatchAware(nn.Module):
    # Set to torch.device("cpu") to draw parameters from the CPU generator instead of the
    # image's device (reproducible across machines; the tests use it).  None = reference behaviour.
    _param_device = None

    def __init__(self, same_on_batch: bool = False, same_on_frame: bool = True):
        super().__init__()
        self.same_on_batch = same_on_batch
        self.same_on_frame = same_on_frame

    def _layout(self, image, upload=True) -> _Layout:
        return _Layout(image, self.same_on_batch, self.same_on_frame, upload, self._param_device)

    # True (default): where PyTorch's CUDA generator can be reproduced inside the library's sampler
    # kernel, a forward draws all its parameters with one launch - the same values, the generator
    # left where the reference's separate draws would leave it.  False: draw with PyTorch itself.
    one_launch_draws = True

    def _through_fused(self, image, make):
        """forward() of a class whose draws are a subset of TritonFusedAugment's, through a private
        TritonFusedAugment (built once by ``make``) and its one-launch sampler.  Returns None when
        that path is not available for this call (the caller then draws with PyTorch)."""
        if not self.one_launch_draws or self._param_device is not None:
            return None
        d = self.__dict__.get("_fused_twin")
        if d is None:
            d = make()
            self.__dict__["_fused_twin"] = d          # (not a registered sub-module: it has no state of its own)
        lay = d._layout(image)
        flags = d._torch_flags(lay, lay.param_device)
        if not flags:
            return None
        return lay.restore(d._forward_fast(lay, flags))

    def _tail(self):
        return f"same_on_batch={self.same_on_batch}, same_on_frame={self.same_on_frame})"


from ._transforms_color import *      # noqa: E402,F401,F403
from ._transforms_geometric import *  # noqa: E402,F401,F403
from ._transforms_fused import *      # noqa: E402,F401,F403
