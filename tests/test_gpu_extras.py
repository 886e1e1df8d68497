"""The geometric extras the reference lists as future work: per-channel fill values
(triton_augment/functional.py:942-945), rotate(expand=True) (functional.py:1164-1165) and crop
windows that leave the image, with padding (functional.py:644-646).  Each is the same fused
kernel with other arguments; torchvision's v2 functionals on the GPU are the comparison."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _img(n=3, c=3, h=90, w=120, seed=0):
    return torch.rand(n, c, h, w, generator=torch.Generator().manual_seed(seed)).to(DEV)


@pytest.mark.parametrize("interp", ["nearest", "bilinear"])
def test_per_channel_fill_equals_three_scalar_fills(interp):
    """Channel c of the per-channel call is channel c of the call with the scalar fill[c]: exact."""
    import triton_augment_b200 as ta
    img = _img()
    fill = [0.25, -1.0, 0.7]
    kw = dict(angle=33.0, translate=[14.0, -9.0], scale=0.8, shear=[6.0, 2.0], interpolation=interp)
    got = ta.affine(img, fill=fill, **kw)
    for c in range(3):
        assert torch.equal(got[:, c], ta.affine(img, fill=fill[c], **kw)[:, c])
    assert float((got[:, 1] == -1.0).float().mean()) > 0.05          # the fill value is actually visible
    one = ta.affine(img[:, :1].contiguous(), fill=[0.3], **kw)       # 1-channel images take a single value
    assert torch.equal(one, ta.affine(img[:, :1].contiguous(), fill=0.3, **kw))
    with pytest.raises(ValueError):
        ta.affine(img, fill=[0.1, 0.2], **kw)
    # through the fused entry point and the class as well
    fused = ta.fused_augment(img, 5, 7, 64, 80, angle=33.0, scale=0.8, interpolation=interp, fill=fill, brightness_factor=1.1)
    for c in range(3):
        ref = ta.fused_augment(img, 5, 7, 64, 80, angle=33.0, scale=0.8, interpolation=interp, fill=fill[c], brightness_factor=1.1)
        assert torch.equal(fused[:, c], ref[:, c])
    aug = ta.TritonRandomAffine(degrees=40, scale=(0.6, 0.7), fill=fill, interpolation=interp)
    out = aug(img)
    assert float((out[:, 1] == -1.0).float().mean()) > 0.05


def test_per_channel_fill_vs_torchvision():
    import torchvision.transforms.v2.functional as tvF
    from torchvision.transforms import InterpolationMode as IM
    import triton_augment_b200 as ta
    img = _img(2, 3, 101, 77, seed=3)
    fill = [0.9, 0.1, 0.5]
    got = ta.affine(img, 20.0, [5.0, 3.0], 0.9, [4.0, 0.0], interpolation="bilinear", fill=fill)
    want = tvF.affine(img, 20.0, [5.0, 3.0], 0.9, [4.0, 0.0], interpolation=IM.BILINEAR, fill=fill)
    d = (got - want).abs()
    # torchvision blends the border through a mask channel, so the one-pixel rim may differ; the rest agrees
    assert float(d.median()) <= 1e-5 and float((d <= 1e-3).float().mean()) >= 0.97


@pytest.mark.parametrize("interp", ["nearest", "bilinear"])
@pytest.mark.parametrize("angle", [17.0, -42.5, 90.0, 135.0, 180.0, 270.0])
def test_rotate_expand_matches_torchvision(interp, angle):
    import torchvision.transforms.v2.functional as tvF
    from torchvision.transforms import InterpolationMode as IM
    import triton_augment_b200 as ta
    img = _img(2, 3, 64, 97, seed=int(abs(angle)))
    got = ta.rotate(img, angle, interpolation=interp, expand=True)
    want = tvF.rotate(img, angle, interpolation=IM.BILINEAR if interp == "bilinear" else IM.NEAREST, expand=True)
    assert got.shape == want.shape, (tuple(got.shape), tuple(want.shape))
    d = (got - want).abs()
    if angle % 90 == 0:
        assert float(d.max()) <= (1e-5 if interp == "bilinear" else 0.0)   # quarter turns: a permutation (cos 90 deg is 6e-17 in the matrix, not 0)
    elif interp == "bilinear":
        assert float(d.median()) <= 1e-5 and float((d <= 1e-3).float().mean()) >= 0.98
    else:
        assert float((d == 0).float().mean()) >= 0.75                  # the reference's own criterion for nearest
    # nothing of the source is lost: the expanded canvas holds (about) all of its mass
    assert abs(float(got.sum()) / float(img.sum()) - 1.0) < 0.02


def test_rotate_expand_argument_rules_and_class():
    import triton_augment_b200 as ta
    img = _img(4)
    with pytest.raises(ValueError):
        ta.rotate(img, torch.tensor([10.0, 20.0, 30.0, 40.0], device=DEV), expand=True)      # four sizes in one batch
    same = ta.rotate(img, torch.full((4,), 25.0, device=DEV), expand=True)
    assert torch.equal(same, ta.rotate(img, 25.0, expand=True))
    aug = ta.TritonRandomRotation(30, expand=True, same_on_batch=True, interpolation="bilinear")
    torch.manual_seed(4)
    out = aug(img)
    torch.manual_seed(4)
    angle = float(aug._get_params(1, DEV, (90, 120))[0][0])
    assert torch.equal(out, ta.rotate(img, -angle, interpolation="bilinear", expand=True))
    assert out.shape[-2] > 90 and out.shape[-1] > 120
    video = torch.rand(2, 3, 3, 40, 50, device=DEV)
    assert aug(video).shape[:3] == (2, 3, 3)
    with pytest.raises(ValueError):
        ta.TritonRandomRotation(30, expand=True)(img)                                        # one angle per image


def test_crop_outside_the_image_pads():
    import torch.nn.functional as nnF
    import torchvision.transforms.v2.functional as tvF
    import triton_augment_b200 as ta
    img = _img(3, 3, 40, 52, seed=9)
    # zero padding: torchvision's crop does the same
    for top, left, ch, cw in ((-5, -7, 30, 40), (20, 30, 40, 40), (-10, -10, 60, 72), (35, 50, 16, 16)):
        assert torch.equal(ta.crop(img, top, left, ch, cw), tvF.crop(img, top, left, ch, cw)), (top, left, ch, cw)
    # a fill value, scalar and per channel: pad first, then crop
    for fill in (0.5, [0.2, 0.4, 0.6]):
        padded = torch.stack([nnF.pad(img[:, c], (8, 8, 8, 8), value=(fill if isinstance(fill, float) else fill[c]))
                              for c in range(3)], dim=1)
        tops = torch.tensor([-8, 3, 20], device=DEV, dtype=torch.int32)
        lefts = torch.tensor([-8, -2, 30], device=DEV, dtype=torch.int32)
        got = ta.crop(img, tops, lefts, 28, 30, fill=fill)
        for i in range(3):
            t, l = int(tops[i]) + 8, int(lefts[i]) + 8
            assert torch.equal(got[i], padded[i, :, t:t + 28, l:l + 30])


def test_random_crop_with_padding_follows_torchvision_rules():
    import triton_augment_b200 as ta
    img = _img(6, 3, 32, 32, seed=2)
    aug = ta.TritonRandomCrop(32, padding=4, fill=[1.5, 2.5, 3.5])
    torch.manual_seed(0)
    out = aug(img)
    assert out.shape == (6, 3, 32, 32)
    # the same draws by hand: offsets over the padded size, shifted back by the padding
    torch.manual_seed(0)
    top = torch.randint(0, 40 - 32 + 1, (6,), device=DEV, dtype=torch.int32) - 4
    left = torch.randint(0, 40 - 32 + 1, (6,), device=DEV, dtype=torch.int32) - 4
    assert torch.equal(out, ta.crop(img, top, left, 32, 32, fill=[1.5, 2.5, 3.5]))
    assert bool((out[:, 0] == 1.5).any()) and bool((out[:, 2] == 3.5).any())
    # pad_if_needed: an image smaller than the window
    small = ta.TritonRandomCrop((48, 40), pad_if_needed=True)(img)
    assert small.shape == (6, 3, 48, 40)
    with pytest.raises(ValueError):
        ta.TritonRandomCrop(48)(img)                                   # no padding asked for: the reference's error


def test_the_layout_without_fill_rgb_is_still_accepted():
    """A caller compiled against the parameter block that ended at gray_mean passes that smaller
    struct_size; the library must not read past it and must give the scalar-fill result."""
    from triton_augment_b200 import _lib, functional as F
    lib = _lib.load()
    img = _img(2, 3, 48, 64, seed=5)
    out_new, out_old = torch.empty(2, 3, 40, 48, device=DEV), torch.empty(2, 3, 40, 48, device=DEV)
    matrix = F._prepare_affine_matrix_only(2, DEV, 48, 64, 30.0, [0.0, 0.0], 0.7, [0.0, 0.0], None).contiguous()
    for out, size in ((out_new, C.sizeof(_lib.FusedParams)), (out_old, _lib.FusedParams.fill_rgb.offset)):
        p = _lib.make_params(img, out, None, None, None, matrix, 0.4, True, 0, None, None, None, None, None, None)
        p.struct_size = size
        p.fill_rgb[0] = p.fill_rgb[1] = p.fill_rgb[2] = 9.0          # garbage past the old layout's end: must be ignored
        p.fill_per_channel = 0 if size == C.sizeof(_lib.FusedParams) else 1
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        assert lib.ta_b200_fused_augment(C.byref(p), stream) == 0, lib.ta_b200_last_error()
    torch.cuda.synchronize()
    assert torch.equal(out_new, out_old) and bool((out_new == 0.4).any())
    p.struct_size = 100
    assert lib.ta_b200_fused_augment(C.byref(p), None) == -2
