"""B200-native fused image / video augmentation behind the API of yuhezhang-ai/triton-augment.

    import triton_augment_b200 as ta
    aug = ta.TritonFusedAugment(crop_size=224, horizontal_flip_p=0.5, degrees=15,
                                brightness=0.2, contrast=0.2, saturation=0.2, grayscale_p=0.1,
                                mean=(0.485, 0.456, 0.406), std=(0.229, 0.224, 0.225))
    out = aug(batch)            # batch: (N,3,H,W), (N,T,3,H,W) or (3,H,W), float32/float16

The kernels are hand-written CUDA for sm_100a in a C-ABI shared library (include/ta_b200.h);
there is no CPU or other-GPU fallback.
"""
from . import config, functional, transforms, utils
from .config import disable_autotune, enable_autotune, is_autotune_enabled
from .functional import (InterpolationMode, adjust_brightness, adjust_contrast, adjust_contrast_fast,
                         adjust_saturation, affine, apply_brightness, apply_contrast, apply_normalize,
                         apply_saturation, center_crop, crop, fused_augment, horizontal_flip, normalize,
                         rgb_to_grayscale, rotate)
from .graphs import GraphedTransform
from .multi_gpu import ShardedAugment, ShardError, shard_bounds
from .transforms import (TritonCenterCrop, TritonColorJitter, TritonColorJitterNormalize, TritonFusedAugment,
                         TritonGrayscale, TritonNormalize, TritonRandomAffine, TritonRandomCrop,
                         TritonRandomCropFlip, TritonRandomGrayscale, TritonRandomHorizontalFlip,
                         TritonRandomRotation)
from .utils import warmup_cache

__version__ = "0.3.0+b200"

__all__ = [
    "functional", "transforms", "utils", "config", "InterpolationMode", "warmup_cache", "enable_autotune",
    "disable_autotune", "is_autotune_enabled", "TritonColorJitter", "TritonNormalize",
    "TritonColorJitterNormalize", "TritonGrayscale", "TritonRandomGrayscale", "TritonRandomCrop",
    "TritonCenterCrop", "TritonRandomHorizontalFlip", "TritonRandomCropFlip", "TritonRandomAffine",
    "TritonRandomRotation", "TritonFusedAugment", "adjust_brightness", "adjust_contrast",
    "adjust_contrast_fast", "adjust_saturation", "normalize", "rgb_to_grayscale", "apply_brightness",
    "apply_contrast", "apply_saturation", "apply_normalize", "crop", "center_crop", "horizontal_flip",
    "affine", "rotate", "fused_augment", "ShardedAugment", "ShardError", "shard_bounds", "GraphedTransform",
]
