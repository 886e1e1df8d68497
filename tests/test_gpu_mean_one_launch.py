"""Mean-mode (torchvision-exact) contrast in one launch.

ta_b200_fused_augment_mean() can run the grayscale-mean reduction and the fused pass as one
cooperative launch of the two-phase kernel (ta_b200_mean_path(1) or (2)): thread blocks alternate
between reduction tiles of one image and fused-pass tiles of the image one or two before it, and
a dedicated warp of block n % grid finishes image n's mean once all partial sums are counted.  The
partial sums and the order they are added in are those of the default two-launch sequence, so the
paths must agree bit for bit - output and means - for every sampling mode, flag combination,
channel count and batch size, including batches smaller than the lag and images of a single tile."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
MEAN, STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)


def _case(_lib, F, n, c, h, w, oh, ow, mode, bits, seed):
    g = torch.Generator().manual_seed(seed)
    img = torch.rand(n, c, h, w, generator=g).to(DEV)
    top = torch.randint(0, h - oh + 1, (n,), generator=g).float().to(DEV)
    left = torch.randint(0, w - ow + 1, (n,), generator=g).float().to(DEV)
    flip = (torch.rand(n, generator=g) < 0.5).to(DEV)
    u = lambda: (torch.rand(n, generator=g) * 0.6 + 0.7).to(DEV)
    bf, cf, sf = u(), u(), u()
    gray = (torch.rand(n, generator=g) < 0.3).to(DEV)
    matrix = None
    if mode != "none":
        angle = (torch.rand(n, generator=g) * 30 - 15).to(DEV)
        matrix = F._prepare_affine_matrix_only(n, DEV, h, w, angle, [2.5, -3.0], 1.07, [4.0, 0.0], None).contiguous()
    keep = (img, top, left, flip, bf, cf, sf, gray, matrix)

    def run(path):
        out = torch.full((n, c, oh, ow), -3.0, device=DEV)
        p = _lib.make_params(img, out, top, left, flip, matrix, 0.0, mode == "bilinear", bits, bf, cf, sf, gray,
                             F._rounded_triple(MEAN, torch.float32), F._rounded_triple(STD, torch.float32),
                             contrast_mode=_lib.CONTRAST_MEAN)
        _lib.mean_path(path)
        try:
            means = _lib.launch_fused_mean(p, DEV)
            torch.cuda.synchronize()
        finally:
            _lib.mean_path(0)
        return out, means
    return run, keep


@pytest.mark.parametrize("mode", ["none", "nearest", "bilinear"])
def test_one_launch_equals_two_launches(mode):
    from triton_augment_b200 import _lib, functional as F
    _lib.debug_counters(reset=True)
    B, Cn, S, G, N = _lib.APPLY_BRIGHTNESS, _lib.APPLY_CONTRAST, _lib.APPLY_SATURATION, _lib.APPLY_GRAYSCALE, _lib.APPLY_NORMALIZE
    shapes = [(1, 3, 96, 128, 64, 64),           # one image, one tile
              (2, 3, 160, 192, 130, 150),
              (7, 3, 200, 208, 161, 177),        # sizes that are not multiples of the tile
              (5, 1, 160, 192, 130, 150),        # one channel
              (3, 3, 640, 640, 512, 512)]        # more tiles per image than thread blocks
    for i, (n, c, h, w, oh, ow) in enumerate(shapes):
        for bits in ((Cn, B | Cn, B | Cn | N) if c == 1 else (Cn, B | Cn | S | G | N, Cn | S, B | Cn | G)):
            run, _ = _case(_lib, F, n, c, h, w, oh, ow, mode, bits, seed=10 * i + bits)
            two, m2 = run(0)
            for lag in (1, 2):
                one, m1 = run(lag)
                assert torch.equal(m1, m2), (mode, n, c, bits, lag)
                assert torch.equal(one, two), (mode, n, c, bits, lag, float((one - two).abs().max()))
            assert bool((m1 > 0.2).all()) and bool((m1 < 0.8).all())
    staged, direct, viol, timeouts = _lib.debug_counters()
    assert timeouts == 0 and not _lib.status(DEV)


def test_one_launch_through_the_class_and_against_torchvision_contrast():
    """The public path: TritonFusedAugment(contrast_mode='torchvision') makes one library call."""
    import triton_augment_b200 as ta
    from triton_augment_b200 import _lib
    aug = ta.TritonFusedAugment(crop_size=200, horizontal_flip_p=0.5, degrees=12, interpolation="bilinear", brightness=0.3,
                                contrast=0.4, saturation=0.2, grayscale_p=0.2, mean=MEAN, std=STD, contrast_mode="torchvision")
    x = torch.rand(9, 3, 256, 256, device=DEV)
    torch.manual_seed(6); a = aug(x)
    _lib.mean_path(2)
    try:
        torch.manual_seed(6); b = aug(x)
    finally:
        _lib.mean_path(0)
    assert torch.equal(a, b)
    # no affine, no crop: torchvision's adjust_contrast on the whole image is the same operation
    import torchvision.transforms.v2.functional as tvF
    y = torch.rand(4, 3, 224, 224, device=DEV)
    got = ta.adjust_contrast(y, 1.3)
    want = torch.stack([tvF.adjust_contrast(y[i], 1.3) for i in range(4)])
    assert float((got - want).abs().max()) <= 1e-5


def test_scratch_too_small_falls_back_to_two_launches():
    """With less scratch than the one-launch path needs (but enough for the reduction kernel) the
    entry point takes the two-launch sequence and still returns the same bits."""
    from triton_augment_b200 import _lib, functional as F
    lib = _lib.load()
    run, keep = _case(_lib, F, 4, 3, 160, 192, 130, 150, "bilinear", _lib.APPLY_BRIGHTNESS | _lib.APPLY_CONTRAST, seed=3)
    want, want_means = run(0)
    img, top, left, flip, bf, cf, sf, gray, matrix = keep
    out = torch.empty_like(want)
    p = _lib.make_params(img, out, top, left, flip, matrix, 0.0, True, _lib.APPLY_BRIGHTNESS | _lib.APPLY_CONTRAST, bf, cf,
                         sf, gray, None, None, contrast_mode=_lib.CONTRAST_MEAN)
    small = (4 * 4 + 255) // 256 * 256 + 4 * 4 * min(128, (130 * 150 + 4095) // 4096)       # the gather kernel's need
    scratch = torch.empty(small, dtype=torch.uint8, device=DEV)
    means = torch.empty(4, device=DEV)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.ta_b200_fused_augment_mean(C.byref(p), C.c_void_p(means.data_ptr()), C.c_void_p(scratch.data_ptr()), small, stream)
    assert rc == 0, lib.ta_b200_last_error().decode()
    torch.cuda.synchronize()
    assert float((means - want_means).abs().max()) <= 2e-6          # the gather kernel adds in another order
    assert float((out - want).abs().max()) <= 1e-5
