"""uint8 images (an extension: the reference takes float tensors only).  A byte b enters the
pipeline as b / 255 inside the kernel; the float32 result must equal the float32 call on
image.float() / 255 within the float32 tolerance of the task (1e-5), and plain crop + flip must
equal indexing of image * (1/255) bit for bit."""
import numpy as np
import pytest
import torch

from conftest import MEAN, STD
from oracle import fused_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-5


def _dev():
    return torch.device("cuda:0")


def _case(seed, n, h, w, oh, ow):
    g = torch.Generator().manual_seed(seed)
    img = torch.randint(0, 256, (n, 3, h, w), generator=g, dtype=torch.uint8)
    u = lambda lo, hi, *s: torch.rand(*s, generator=g) * (hi - lo) + lo
    return dict(
        img=img, top=torch.randint(0, h - oh + 1, (n,), generator=g).float(),
        left=torch.randint(0, w - ow + 1, (n,), generator=g).float(), flip=torch.rand(n, generator=g) < 0.5,
        angle=u(-15, 15, n), translate=torch.stack([u(-0.1 * w, 0.1 * w, n), u(-0.1 * h, 0.1 * h, n)], 1),
        scale=u(0.9, 1.1, n), shear=torch.stack([u(-5, 5, n), torch.zeros(n)], 1),
        b=u(0.8, 1.2, n), c=u(0.8, 1.2, n), s=u(0.8, 1.2, n), g=torch.rand(n, generator=g) < 0.4)


def _call(ta, image, p, oh, ow, interp, bits):
    dev = _dev()
    d = lambda t: t.to(dev)
    kw = {}
    if interp != "none":
        kw.update(angle=d(p["angle"]), translate=d(p["translate"]), scale=d(p["scale"]), shear=d(p["shear"]),
                  interpolation=interp)
    if bits & 1: kw["brightness_factor"] = d(p["b"])
    if bits & 2: kw["contrast_factor"] = d(p["c"])
    if bits & 4: kw["saturation_factor"] = d(p["s"])
    if bits & 8: kw["grayscale"] = d(p["g"])
    if bits & 16: kw.update(mean=MEAN, std=STD)
    return ta.fused_augment(d(image), d(p["top"]), d(p["left"]), oh, ow, d(p["flip"]), **kw)


@pytest.mark.parametrize("interp", ["none", "nearest", "bilinear"])
@pytest.mark.parametrize("shape", [(3, 160, 192, 120, 144), (2, 97, 131, 61, 77), (4, 256, 256, 224, 224)])
def test_bytes_equal_the_float_call_on_scaled_image(interp, shape):
    """Staged rows (width a multiple of 16) and the gather fallback (width 131), odd output sizes."""
    import triton_augment_b200 as ta
    n, h, w, oh, ow = shape
    p = _case(7, n, h, w, oh, ow)
    scaled = p["img"].float() * (1.0 / 255.0)
    for bits in (0, 5, 14, 31):
        got = _call(ta, p["img"], p, oh, ow, interp, bits)
        want = _call(ta, scaled, p, oh, ow, interp, bits)
        assert got.dtype == torch.float32 and got.shape == want.shape
        err = float((got - want).abs().max())
        assert err <= TOL, (interp, shape, bits, err)


def test_bytes_against_the_oracle():
    import triton_augment_b200 as ta
    n, h, w, oh, ow = 3, 128, 160, 100, 112
    p = _case(11, n, h, w, oh, ow)
    scaled = (p["img"].float() * (1.0 / 255.0)).numpy()
    matrix = ta.functional._prepare_affine_matrix_only(n, _dev(), h, w, p["angle"].to(_dev()), p["translate"].to(_dev()),
                                                       p["scale"].to(_dev()), p["shear"].to(_dev()), None).cpu().numpy()
    for interp in ("nearest", "bilinear"):
        got = _call(ta, p["img"], p, oh, ow, interp, 31).cpu().numpy()
        want = O.fused_augment(scaled, p["top"].numpy(), p["left"].numpy(), oh, ow, p["flip"].numpy(), matrix=matrix,
                               interpolation=interp, brightness=p["b"].numpy(), contrast=p["c"].numpy(),
                               saturation=p["s"].numpy(), grayscale=p["g"].numpy(), mean=MEAN, std=STD)
        assert float(np.abs(got - want).max()) <= TOL, interp


def test_crop_flip_of_bytes_is_exact():
    import triton_augment_b200 as ta
    from triton_augment_b200 import _lib
    dev = _dev()
    n, h, w, oh, ow = 3, 96, 128, 70, 90
    p = _case(3, n, h, w, oh, ow)
    _lib.debug_counters(reset=True)
    got = _call(ta, p["img"], p, oh, ow, "none", 0)
    staged = _lib.debug_counters()[0]
    scaled = (p["img"].float() * (1.0 / 255.0)).to(dev)
    want = torch.stack([
        (scaled[i, :, int(p["top"][i]):int(p["top"][i]) + oh, int(p["left"][i]):int(p["left"][i]) + ow].flip(-1) if p["flip"][i]
         else scaled[i, :, int(p["top"][i]):int(p["top"][i]) + oh, int(p["left"][i]):int(p["left"][i]) + ow]) for i in range(n)])
    assert torch.equal(got, want)
    assert staged > 0


def test_staging_assertions_hold_for_bytes():
    """The checked build counts shared-memory taps outside what was staged (128-byte row pitch,
    copies aligned to 16 columns): none, on random geometry."""
    import triton_augment_b200 as ta
    from triton_augment_b200 import _lib
    dev = _dev()
    _lib.debug_counters(reset=True)
    for seed, (n, h, w, oh, ow) in enumerate([(2, 200, 256, 150, 200), (2, 144, 176, 144, 176), (3, 300, 320, 96, 300)]):
        p = _case(20 + seed, n, h, w, oh, ow)
        d = lambda t: t.to(dev)
        matrix = ta.functional._prepare_affine_matrix_only(n, dev, h, w, d(p["angle"]), d(p["translate"]), d(p["scale"]),
                                                           d(p["shear"]), None).contiguous()
        for bilinear in (False, True):
            out = torch.empty(n, 3, oh, ow, device=dev)
            prm = _lib.make_params(d(p["img"]), out, d(p["top"]), d(p["left"]), d(p["flip"]).to(torch.uint8), matrix, 0.0,
                                   bilinear, 0, None, None, None, None, None, None)
            _lib.launch_fused(prm, dev, checked=True)
            torch.cuda.synchronize()
            ref = ta.fused_augment(d(p["img"]).float() * (1.0 / 255.0), d(p["top"]), d(p["left"]), oh, ow, d(p["flip"]),
                                   angle=d(p["angle"]), translate=d(p["translate"]), scale=d(p["scale"]), shear=d(p["shear"]),
                                   interpolation="bilinear" if bilinear else "nearest")
            assert float((out - ref).abs().max()) <= (2e-6 if bilinear else 0.0)
    staged, direct, violations, timeouts = _lib.debug_counters()
    assert violations == 0 and timeouts == 0 and staged > 50


def test_bytes_single_channel_fill_and_large_rotation():
    """One channel, a non-zero fill (border tiles are gathered, not staged) and rotations large
    enough that some tiles need per-group windows or the gather fallback."""
    import triton_augment_b200 as ta
    dev = _dev()
    g = torch.Generator().manual_seed(17)
    n, h, w, oh, ow = 4, 176, 208, 150, 163
    img = torch.randint(0, 256, (n, 1, h, w), generator=g, dtype=torch.uint8).to(dev)
    angle = torch.tensor([40.0, -75.0, 10.0, 0.0], device=dev)
    scale = torch.tensor([0.6, 1.4, 1.0, 2.0], device=dev)
    top = torch.tensor([3.0, 0.0, 26.0, 11.0], device=dev)
    left = torch.tensor([0.0, 45.0, 7.0, 20.0], device=dev)
    flip = torch.tensor([True, False, True, False], device=dev)
    bf = torch.tensor([0.9, 1.1, 1.2, 0.8], device=dev)
    for interp in ("nearest", "bilinear"):
        kw = dict(angle=angle, scale=scale, interpolation=interp, fill=0.5, brightness_factor=bf, contrast_factor=1.15)
        got = ta.fused_augment(img, top, left, oh, ow, flip, **kw)
        want = ta.fused_augment(img.float() * (1.0 / 255.0), top, left, oh, ow, flip, **kw)
        assert float((got - want).abs().max()) <= TOL, interp


def test_transform_class_and_host_path_take_bytes():
    import triton_augment_b200 as ta
    dev = _dev()
    aug = ta.TritonFusedAugment(crop_size=96, horizontal_flip_p=0.5, degrees=10, scale=(0.9, 1.1), interpolation="bilinear",
                                brightness=0.2, contrast=0.2, saturation=0.2, grayscale_p=0.2, mean=MEAN, std=STD)
    g = torch.Generator().manual_seed(5)
    img = torch.randint(0, 256, (6, 3, 128, 144), generator=g, dtype=torch.uint8)
    torch.manual_seed(42)
    a = aug(img.to(dev))
    torch.manual_seed(42)
    b = aug(img.to(dev).float() * (1.0 / 255.0))
    assert a.dtype == torch.float32 and float((a - b).abs().max()) <= TOL
    torch.manual_seed(42)
    c = aug.forward_host(img.pin_memory(), device=dev)
    assert c.dtype == torch.float32 and not c.is_cuda
    assert torch.equal(c, a.cpu())
    # the other classes that are one fused call take bytes as well
    for t in (ta.TritonColorJitterNormalize(brightness=0.2, contrast=0.2, saturation=0.2, grayscale_p=0.3, mean=MEAN, std=STD),
              ta.TritonRandomCropFlip(size=(100, 120), horizontal_flip_p=0.5)):
        torch.manual_seed(8)
        u = t(img.to(dev))
        torch.manual_seed(8)
        f = t(img.to(dev).float() * (1.0 / 255.0))
        assert u.dtype == torch.float32 and float((u - f).abs().max()) <= TOL, type(t).__name__
    # torchvision-exact contrast: its mean pre-pass reads bytes through the staged kernel
    kw = dict(brightness_factor=1.1, contrast_factor=torch.tensor([0.7, 1.3, 1.1, 0.9, 1.2, 0.8], device=dev),
              contrast_mode="torchvision", angle=7.0, interpolation="bilinear")
    u = ta.fused_augment(img.to(dev), 3, 5, 100, 120, **kw)
    f = ta.fused_augment(img.to(dev).float() * (1.0 / 255.0), 3, 5, 100, 120, **kw)
    assert float((u - f).abs().max()) <= TOL
    odd = torch.randint(0, 256, (2, 3, 50, 70), dtype=torch.uint8, device=dev)      # rows of 70 bytes cannot be staged
    with pytest.raises(Exception, match="16-byte"):
        ta.fused_augment(odd, 0, 0, 40, 40, contrast_factor=1.1, contrast_mode="torchvision")
    with pytest.raises(TypeError):
        ta.functional.crop(img.to(dev), 0, 0, 64, 64)      # the stand-alone functionals stay float-only


@pytest.mark.parametrize("interp", ["none", "nearest", "bilinear"])
@pytest.mark.parametrize("shape", [(3, 160, 192, 120, 144), (2, 97, 131, 61, 77), (4, 256, 256, 224, 224)])
def test_bytes_to_half_equal_the_half_call_on_scaled_image(interp, shape):
    """out_dtype=float16: within the float16 tolerance of the task (1e-2) of the float16 call on
    (image / 255).half(); plain crop + flip is that image indexed, bit for bit."""
    import triton_augment_b200 as ta
    n, h, w, oh, ow = shape
    p = _case(9, n, h, w, oh, ow)
    scaled = (p["img"].float() * (1.0 / 255.0)).half()
    dev = _dev()
    for bits in (0, 5, 14, 31):
        kw = {}
        d = lambda t: t.to(dev)
        if interp != "none":
            kw.update(angle=d(p["angle"]), translate=d(p["translate"]), scale=d(p["scale"]), shear=d(p["shear"]),
                      interpolation=interp)
        if bits & 1: kw["brightness_factor"] = d(p["b"])
        if bits & 2: kw["contrast_factor"] = d(p["c"])
        if bits & 4: kw["saturation_factor"] = d(p["s"])
        if bits & 8: kw["grayscale"] = d(p["g"])
        if bits & 16: kw.update(mean=MEAN, std=STD)
        got = ta.fused_augment(d(p["img"]), d(p["top"]), d(p["left"]), oh, ow, d(p["flip"]), out_dtype=torch.float16, **kw)
        want = ta.fused_augment(d(scaled), d(p["top"]), d(p["left"]), oh, ow, d(p["flip"]), **kw)
        assert got.dtype == torch.float16 and got.shape == want.shape
        err = float((got.float() - want.float()).abs().max())
        assert err <= 1e-2, (interp, shape, bits, err)
        if bits == 0 and interp != "bilinear":
            assert torch.equal(got, want), (interp, shape)


def test_half_output_through_the_transform_and_its_limits():
    import triton_augment_b200 as ta
    dev = _dev()
    img = torch.randint(0, 256, (6, 3, 96, 128), dtype=torch.uint8, device=dev)
    kw = dict(crop_size=(64, 80), horizontal_flip_p=0.5, degrees=10, interpolation="bilinear", brightness=0.2,
              contrast=0.2, saturation=0.2, grayscale_p=0.2, mean=MEAN, std=STD)
    for fast in (False, True):
        torch.manual_seed(3)
        got = ta.TritonFusedAugment(out_dtype=torch.float16, fast_rng=fast, **kw)(img)
        torch.manual_seed(3)
        want = ta.TritonFusedAugment(fast_rng=fast, **kw)((img.float() * (1.0 / 255.0)).half())
        assert got.dtype == torch.float16
        assert float((got.float() - want.float()).abs().max()) <= 1e-2
    # a float batch keeps its dtype whatever the transform's out_dtype says
    assert ta.TritonFusedAugment(out_dtype=torch.float16, **kw)(img.float() / 255).dtype == torch.float32
    # host-buffer path
    torch.manual_seed(4)
    host = ta.TritonFusedAugment(out_dtype=torch.float16, **kw).forward_host(img.cpu())
    torch.manual_seed(4)
    want = ta.TritonFusedAugment(out_dtype=torch.float16, **kw)(img)
    assert host.dtype == torch.float16 and torch.equal(host, want.cpu())
    with pytest.raises(ValueError):
        ta.fused_augment(img, 0, 0, 64, 64, contrast_factor=1.1, contrast_mode="torchvision", out_dtype=torch.float16)
    with pytest.raises(ValueError):
        ta.fused_augment(img.float(), 0, 0, 64, 64, out_dtype=torch.float16)
    with pytest.raises(TypeError):
        ta.fused_augment(img, 0, 0, 64, 64, out_dtype=torch.float64)
