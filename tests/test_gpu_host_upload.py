"""Host-buffer entry point on large images: only the box of source pixels that a call reads is
uploaded.  The device staging buffers are first filled with NaN (float) or 255 (bytes) through a
whole-image upload, so that any texel read outside the uploaded box would show; the result must
equal the device path's bit for bit, and the whole-image upload's.  The cases cover the three
forms an upload takes: whole image, a run of whole rows per channel, a strided box per channel."""
import pytest
import torch

from conftest import MEAN, STD

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _poison(ta, shape, dtype, crop):
    from triton_augment_b200 import _lib
    bad = (torch.full(shape, 255, dtype=torch.uint8) if dtype == torch.uint8
           else torch.full(shape, float("nan"), dtype=dtype)).pin_memory()
    _lib.host_upload(0)
    try:
        ta.TritonFusedAugment(crop_size=crop).forward_host(bad, device=DEV)
    finally:
        _lib.host_upload(1)


CASES = [
    # (dtype, n, h, w, crop, transform arguments)
    (torch.float32, 7, 600, 520, (256, 320), dict(degrees=25, translate=(0.1, 0.1), scale=(0.8, 1.2), shear=8,
                                                   interpolation="bilinear", fill=0.25)),
    (torch.float32, 5, 520, 600, (301, 277), dict(degrees=40, interpolation="nearest")),
    (torch.float32, 6, 640, 512, (128, 200), dict()),                                       # crop + flip only
    (torch.float16, 5, 768, 800, (500, 333), dict(degrees=15, scale=(0.9, 1.1), interpolation="bilinear")),
    (torch.uint8, 6, 1100, 1008, (640, 512), dict(degrees=20, translate=(0.2, 0.2), interpolation="bilinear")),
    (torch.uint8, 4, 1100, 1008, (333, 222), dict()),
    # boxes much narrower than the image with rows of 2 KiB and more: strided copies
    (torch.float32, 3, 700, 1536, (300, 600), dict()),
    (torch.float32, 3, 640, 1800, (200, 640), dict(degrees=5, interpolation="bilinear")),
    (torch.uint8, 3, 600, 4096, (500, 2100), dict(degrees=3, interpolation="nearest")),
]


@pytest.mark.parametrize("case", range(len(CASES)))
def test_trimmed_upload_equals_device_path(case):
    import triton_augment_b200 as ta
    from triton_augment_b200 import _lib
    dtype, n, h, w, crop, kw = CASES[case]
    aug = ta.TritonFusedAugment(crop_size=crop, horizontal_flip_p=0.5, brightness=0.2, contrast=0.2, saturation=0.2,
                                grayscale_p=0.3, mean=MEAN, std=STD, **kw)
    g = torch.Generator().manual_seed(case)
    host = (torch.randint(0, 256, (n, 3, h, w), generator=g, dtype=torch.uint8) if dtype == torch.uint8
            else torch.rand(n, 3, h, w, generator=g).to(dtype)).pin_memory()
    torch.manual_seed(100 + case); want = aug(host.to(DEV)).cpu()
    _poison(ta, (n, 3, h, w), dtype, crop)
    _lib.host_upload(2)                    # boxes whatever the copy plan costs
    try:
        torch.manual_seed(100 + case); got = aug.forward_host(host, device=DEV)
    finally:
        _lib.host_upload(1)
    assert torch.isfinite(got.float()).all()
    assert got.equal(want)
    _poison(ta, (n, 3, h, w), dtype, crop)
    torch.manual_seed(100 + case); auto = aug.forward_host(host, device=DEV)      # default: by cost
    assert auto.equal(want)
    _lib.host_upload(0)
    try:
        torch.manual_seed(100 + case); whole = aug.forward_host(host, device=DEV)
    finally:
        _lib.host_upload(1)
    assert whole.equal(want)


def test_trimmed_upload_with_mean_contrast_and_windows_off_the_image():
    import triton_augment_b200 as ta
    n, h, w = 6, 560, 512
    host = torch.rand(n, 3, h, w).pin_memory()
    # exact contrast: the mean pre-pass reads the same box
    aug = ta.TritonFusedAugment(crop_size=(300, 256), degrees=20, interpolation="bilinear", brightness=0.2, contrast=0.3,
                                contrast_mode="torchvision", mean=MEAN, std=STD)
    torch.manual_seed(5); want = aug(host.to(DEV)).cpu()
    from triton_augment_b200 import _lib
    _poison(ta, (n, 3, h, w), torch.float32, (300, 256))
    _lib.host_upload(2)
    try:
        torch.manual_seed(5); got = aug.forward_host(host, device=DEV)
    finally:
        _lib.host_upload(1)
    assert got.equal(want)
    # translations that push most (or all) of the window off the image: fill, no stale texel
    far = ta.TritonFusedAugment(crop_size=(256, 256), degrees=10, translate=(0.9, 0.9), interpolation="bilinear", fill=0.5)
    torch.manual_seed(6); want = far(host.to(DEV)).cpu()
    _poison(ta, (n, 3, h, w), torch.float32, (256, 256))
    _lib.host_upload(2)
    try:
        torch.manual_seed(6); got = far.forward_host(host, device=DEV)
    finally:
        _lib.host_upload(1)
    assert torch.isfinite(got).all() and got.equal(want)
