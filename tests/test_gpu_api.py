"""GPU tests of the API surface: stand-alone functionals and transform classes against vectors
produced by the reference (tests/golden), torchvision-exact contrast, 3D/4D/5D handling,
the host-buffer entry point and the batch-sharded wrapper."""
import numpy as np
import pytest
import torch

from conftest import MEAN, STD
from oracle import fused_oracle as O
from test_host_logic_cpu import SPECS

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ta():
    import triton_augment_b200 as ta
    return ta


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _close(got, want, atol):
    got = got.detach().cpu().numpy().astype(np.float32)
    want = np.asarray(want).astype(np.float32)
    assert got.shape == want.shape, (got.shape, want.shape)
    return float(np.abs(got - want).max()) <= atol, float(np.abs(got - want).max())


def test_standalone_functionals_vs_reference_vectors(functional_golden):
    ta, z = _ta(), functional_golden
    img, half = _t(z["image"]), _t(z["image"].astype(np.float16))
    mask = torch.tensor([True, False, True], device=DEV)
    cases = {
        "brightness_1.3": (ta.adjust_brightness(img, 1.3), 1e-6),
        "contrast_1.4": (ta.adjust_contrast(img, 1.4), 2e-6),
        "contrast_0.6": (ta.adjust_contrast(img, 0.6), 2e-6),
        "contrast_fast_1.4": (ta.adjust_contrast_fast(img, 1.4), 1e-6),
        "saturation_0.3": (ta.adjust_saturation(img, 0.3), 1e-6),
        "saturation_1.7": (ta.adjust_saturation(img, 1.7), 1e-6),
        "normalize": (ta.normalize(img, MEAN, STD), 2e-6),
        "gray3": (ta.rgb_to_grayscale(img, 3), 1e-6),
        "gray1": (ta.rgb_to_grayscale(img, 1), 1e-6),
        "gray3_masked": (ta.rgb_to_grayscale(img, 3, mask), 1e-6),
        "crop_2_3_9_11": (ta.crop(img, 2, 3, 9, 11), 0),
        "crop_per_image": (ta.crop(img, _t(z["crop_tops"]), _t(z["crop_lefts"]), 9, 11), 0),
        "center_crop_10_8": (ta.center_crop(img, (10, 8)), 0),
        "hflip": (ta.horizontal_flip(img), 0),
        "hflip_masked": (ta.horizontal_flip(img, mask), 0),
        "gray_contrast_1.5": (ta.adjust_contrast(_t(z["gray_image"]), 1.5), 2e-6),
        "f16_contrast_1.4": (ta.adjust_contrast(half, 1.4), 2e-3),
        "f16_normalize": (ta.normalize(half, MEAN, STD), 4e-3),
        "f16_saturation_0.3": (ta.adjust_saturation(half, 0.3), 2e-3),
        "f16_brightness_1.3": (ta.adjust_brightness(half, 1.3), 1e-3),
    }
    for key, (got, atol) in cases.items():
        ok, err = _close(got, z[key], atol)
        assert ok, (key, err)
    assert ta.rgb_to_grayscale(img, 1).shape == (3, 1, 18, 22)
    assert ta.adjust_saturation(_t(z["gray_image"]), 0.5).equal(_t(z["gray_image"]))     # 1 channel: copy


def test_affine_and_rotate_vs_reference_vectors(functional_golden):
    """The stored vectors come from the CPU interpreter (matrix from CPU libm, unfused
    coordinates), so a small share of pixels may land on the other side of a rounding."""
    ta, z = _ta(), functional_golden
    img = _t(z["image"])
    outs = {
        "affine_nearest": ta.affine(img, 20.0, [2.0, -1.5], 1.1, [5.0, 2.0], "nearest"),
        "affine_bilinear": ta.affine(img, 20.0, [2.0, -1.5], 1.1, [5.0, 2.0], "bilinear", fill=0.25),
        "affine_center": ta.affine(img, -12.0, [0.0, 0.0], 1.0, [0.0, 0.0], "bilinear", center=[4.0, 6.0]),
        "rotate_per_image": ta.rotate(img, _t(z["rotate_angles"]), "bilinear"),
        "rotate_30_nearest": ta.rotate(img, 30.0),
    }
    for key, got in outs.items():
        diff = np.abs(got.cpu().numpy() - z[key])
        if "nearest" in key:
            assert (diff > 1e-6).mean() < 0.02, key
        else:
            assert diff.max() < 2e-4, (key, float(diff.max()))
    with pytest.raises(ValueError):                   # expand=True is built here (tests/test_gpu_extras.py); it needs the centre
        ta.rotate(img, 10.0, expand=True, center=[3.0, 4.0])
    with pytest.raises(ValueError):
        ta.affine(img, 10.0, [0, 0], 1.0, [0, 0], interpolation="bicubic")


@pytest.mark.parametrize("key", sorted(SPECS))
def test_transform_classes_vs_reference_forward(class_golden, key):
    """Class forward for 3D / 4D / 5D inputs and every same_on_batch / same_on_frame setting:
    parameters are drawn from the CPU generator under the stored seed (so they are the
    reference's), the image is processed on the GPU, the result is compared with the
    reference's stored forward output."""
    ta = _ta()
    cls_name, kwargs = SPECS[key]
    affine = any(k in kwargs for k in ("degrees", "translate", "scale", "shear")) or "affine" in key or "rotation" in key
    for rank in ("3d", "4d", "5d"):
        img = _t(class_golden[f"image_{rank}"])
        for sob, sof in ((False, True), (True, True), (False, False), (True, False)):
            tag = f"{key}|{rank}|{int(sob)}{int(sof)}"
            if f"{tag}|out" not in class_golden.files:
                continue
            tr = getattr(ta, cls_name)(**dict(kwargs, same_on_batch=sob, same_on_frame=sof))
            tr._param_device = torch.device("cpu")
            torch.manual_seed(int(class_golden[f"{tag}|seed"]))
            got = tr(img).cpu().numpy()
            want = class_golden[f"{tag}|out"]
            assert got.shape == want.shape, tag
            diff = np.abs(got - want)
            if not affine:
                assert diff.max() <= 1e-5, (tag, float(diff.max()))
            elif str(kwargs.get("interpolation", "nearest")) == "bilinear":
                assert diff.max() <= 5e-4, (tag, float(diff.max()))
            else:
                assert (diff > 1e-5).mean() < 0.03, (tag, float((diff > 1e-5).mean()))


def test_shape_handling_and_seed_determinism():
    ta = _ta()
    aug = ta.TritonFusedAugment(crop_size=16, horizontal_flip_p=0.5, degrees=10, brightness=0.2, saturation=0.2,
                                grayscale_p=0.2, mean=MEAN, std=STD)
    x5 = torch.rand(2, 3, 3, 24, 28, device=DEV)
    assert aug(x5).shape == (2, 3, 3, 16, 16)
    assert aug(x5[0, 0]).shape == (3, 16, 16)
    assert aug(x5[0]).shape == (3, 3, 16, 16)
    torch.manual_seed(5); a = aug(x5)
    torch.manual_seed(5); b = aug(x5)
    assert a.equal(b)
    # same_on_frame: identical frames stay identical; independent frames do not
    video = torch.rand(2, 1, 3, 24, 28, device=DEV).expand(2, 4, 3, 24, 28).contiguous()
    out = aug(video)
    assert out[:, 0].equal(out[:, 3])
    free = ta.TritonFusedAugment(crop_size=16, degrees=10, brightness=0.2, same_on_frame=False)
    out = free(video)
    assert not out[:, 0].equal(out[:, 3])
    # 5D with independent frames == the flattened 4D batch under the same seed
    torch.manual_seed(9); o5 = free(video)
    torch.manual_seed(9); o4 = free(video.reshape(8, 3, 24, 28))
    assert o5.reshape(8, 3, 16, 16).equal(o4)
    # host tensors are uploaded, the result stays on the GPU; non-contiguous input is handled
    assert aug(torch.rand(2, 3, 24, 28)).is_cuda
    nc = torch.rand(2, 3, 28, 24, device=DEV).transpose(2, 3)
    torch.manual_seed(1); r1 = aug(nc)
    torch.manual_seed(1); r2 = aug(nc.contiguous())
    assert r1.equal(r2)


def test_exact_contrast_inside_the_fused_pipeline():
    """contrast_mode='torchvision': mean of the geometry+brightness image, then the blend."""
    ta = _ta()
    rng = np.random.default_rng(4)
    for dtype, tol in ((np.float32, 1e-5), (np.float16, 1e-2)):
        n, h, w, oh, ow = 3, 40, 48, 24, 32
        img = rng.random((n, 3, h, w), dtype=np.float32).astype(dtype)
        top, left = rng.integers(0, h - oh + 1, n).astype(np.float32), rng.integers(0, w - ow + 1, n).astype(np.float32)
        flip = np.array([True, False, True])
        b, c, s = (rng.uniform(0.8, 1.2, n).astype(np.float32) for _ in range(3))
        for interp in (None, "bilinear"):
            kw, matrix = {}, None
            if interp:
                angle = rng.uniform(-15, 15, n).astype(np.float32)
                kw = dict(angle=_t(angle), interpolation=interp)
                matrix = ta.functional._prepare_affine_matrix_only(n, torch.device(DEV), h, w, _t(angle), [0.0, 0.0],
                                                                   1.0, [0.0, 0.0], None).cpu().numpy()
            got = ta.fused_augment(_t(img), _t(top), _t(left), oh, ow, _t(flip), brightness_factor=_t(b),
                                   contrast_factor=_t(c), saturation_factor=_t(s), mean=MEAN, std=STD,
                                   contrast_mode="torchvision", **kw)
            want = O.fused_augment(img, top, left, oh, ow, flip, matrix=matrix, interpolation=interp or "nearest",
                                   brightness=b.astype(dtype), contrast=c.astype(dtype), saturation=s.astype(dtype),
                                   mean=MEAN, std=STD, contrast_mode=O.CONTRAST_MEAN)
            ok, err = _close(got, want, tol)
            assert ok, (dtype, interp, err)
    # class API and determinism of the reduction
    aug = ta.TritonColorJitterNormalize(contrast=0.3, contrast_mode="torchvision")
    x = torch.rand(4, 3, 64, 64, device=DEV)
    torch.manual_seed(0); a = aug(x)
    torch.manual_seed(0); b2 = aug(x)
    assert a.equal(b2)


def test_host_buffer_entry_point_matches_device_path():
    ta = _ta()
    aug = ta.TritonFusedAugment(crop_size=(40, 48), horizontal_flip_p=0.5, degrees=15, translate=(0.1, 0.1),
                                scale=(0.9, 1.1), shear=5, interpolation="bilinear", brightness=0.2, contrast=0.2,
                                saturation=0.2, grayscale_p=0.3, mean=MEAN, std=STD)
    for dtype in (torch.float32, torch.float16):
        host = torch.rand(37, 3, 64, 72).to(dtype).pin_memory()       # odd count: last slice is short
        torch.manual_seed(21); want = aug(host.to(DEV)).cpu()
        torch.manual_seed(21); got = aug.forward_host(host)
        assert not got.is_cuda and got.equal(want)
    # output sizes that are not multiples of 16: the reference's per-pixel coordinate recipe follows
    # the pixel's index in the whole batch, also when the batch goes through in slices
    odd = ta.TritonFusedAugment(crop_size=(41, 50), horizontal_flip_p=0.5, degrees=15, translate=(0.1, 0.1),
                                scale=(0.9, 1.1), shear=5, interpolation="bilinear", brightness=0.2, contrast=0.2,
                                saturation=0.2, grayscale_p=0.3, mean=MEAN, std=STD)
    host = torch.rand(37, 3, 64, 72).pin_memory()
    torch.manual_seed(22); want = odd(host.to(DEV)).cpu()
    torch.manual_seed(22); got = odd.forward_host(host)
    assert got.equal(want)
    mean_mode = ta.TritonFusedAugment(crop_size=32, contrast=0.3, brightness=0.2, contrast_mode="torchvision")
    host = torch.rand(9, 3, 48, 48).pin_memory()
    torch.manual_seed(3); want = mean_mode(host.to(DEV)).cpu()
    torch.manual_seed(3); got = mean_mode.forward_host(host)
    assert got.equal(want)


def test_sharded_wrapper_equals_single_device():
    """Parameters are drawn once for the whole batch and sliced, so any number of shards gives
    the bits a single launch gives.  With one GPU the shards all land on it."""
    ta = _ta()
    aug = ta.TritonFusedAugment(crop_size=24, horizontal_flip_p=0.5, degrees=12, scale=(0.9, 1.1), brightness=0.2,
                                saturation=0.2, grayscale_p=0.2, mean=MEAN, std=STD)
    ndev = torch.cuda.device_count()
    devices = list(range(ndev)) if ndev > 1 else [0, 0, 0]
    x = torch.rand(10, 3, 40, 44, device=DEV)
    torch.manual_seed(77); want = aug(x)
    torch.manual_seed(77); parts = ta.ShardedAugment(aug, devices)(x)
    assert [p.shape[0] for p in parts] == [b - a for a, b in ta.shard_bounds(10, len(devices))]
    assert torch.cat([p.to(DEV) for p in parts]).equal(want)
    video = torch.rand(4, 5, 3, 40, 44, device=DEV)
    torch.manual_seed(78); want = aug(video)
    torch.manual_seed(78); got = ta.ShardedAugment(aug, devices)(video, gather_to=DEV)
    assert got.equal(want)
    # per-rank flavour: every rank seeds alike and owns one slice
    outs = []
    for rank in range(3):
        torch.manual_seed(79)
        a, b = ta.shard_bounds(10, 3)[rank]
        outs.append(ta.ShardedAugment.for_rank(aug, rank, 3, device=DEV)((x[a:b], tuple(x.shape))))
    torch.manual_seed(79)
    assert torch.cat(outs).equal(aug(x))
    # bilinear float32 with an output whose sides are not multiples of 16: the per-pixel coordinate
    # recipe follows the pixel's index in the whole batch, so shards must be told where they start
    odd = ta.TritonFusedAugment(crop_size=(29, 37), horizontal_flip_p=0.5, degrees=12, scale=(0.9, 1.1), shear=4,
                                interpolation="bilinear", brightness=0.2, saturation=0.2, grayscale_p=0.2, mean=MEAN, std=STD)
    torch.manual_seed(80); want = odd(x)
    torch.manual_seed(80); parts = ta.ShardedAugment(odd, devices)(x)
    assert torch.cat([p.to(DEV) for p in parts]).equal(want)


def test_matrix_kernel_is_bit_identical_to_torch_ops():
    """The affine matrix is an INPUT of the fused kernel; the single-launch matrix kernel may
    replace the reference's ~30 elementwise torch operations only because it returns the same
    bits.  Checked over benchmark-like, extreme and near-identity parameter ranges."""
    from triton_augment_b200 import _lib, functional as F
    g = torch.Generator(device=DEV).manual_seed(0)
    u = lambda lo, hi, *s: torch.empty(*s, device=DEV).uniform_(lo, hi, generator=g)
    for n, a, t, s0, s1, sh, c in ((200_000, 15, 128, 0.9, 1.1, 5, 0), (200_000, 180, 500, 0.3, 3.0, 45, 100),
                                   (200_000, 1e-3, 0.1, 0.999, 1.001, 1e-3, 0), (7, 90, 10, 1.0, 1.0, 0, 0)):
        angle, tr, sc, shr, ce = u(-a, a, n), u(-t, t, n, 2), u(s0, s1, n), u(-sh, sh, n, 2), u(-c, c, n, 2)
        got = _lib.inverse_affine_matrix(ce, angle, tr, sc, shr)
        old = F._MATRIX_KERNEL
        F._MATRIX_KERNEL = False
        try:
            want = F._get_inverse_affine_matrix(ce, angle, tr, sc, shr)
        finally:
            F._MATRIX_KERNEL = old
        assert torch.equal(got.view(torch.int32), want.contiguous().view(torch.int32))


def test_null_offset_vectors_mean_zero():
    """C ABI: top, left and flip may be NULL (zero offsets, no flip), on the device entry point
    and on the host-buffer one (whose upload plan reads them too)."""
    from triton_augment_b200 import _lib
    for dtype in (torch.float32, torch.float16, torch.uint8):
        for (n, h, w, oh, ow) in ((3, 64, 96, 64, 96), (2, 70, 130, 33, 41), (2, 600, 1040, 300, 320)):
            img = (torch.randint(0, 256, (n, 3, h, w), dtype=torch.uint8, device=DEV) if dtype == torch.uint8
                   else torch.rand(n, 3, h, w, device=DEV).to(dtype))
            work = torch.float32 if dtype == torch.uint8 else dtype
            z, zf = torch.zeros(n, device=DEV), torch.zeros(n, dtype=torch.uint8, device=DEV)
            for matrix in (None, torch.tensor([[0.98, 0.1, 2.0, -0.1, 0.97, -1.5]] * n, device=DEV)):
                for bilinear in ((False, True) if matrix is not None else (False,)):
                    a = torch.empty(n, 3, oh, ow, dtype=work, device=DEV)
                    b = torch.empty_like(a)
                    rest = (0.0, bilinear, 0, None, None, None, None, None, None)
                    _lib.launch_fused(_lib.make_params(img, a, None, None, None, matrix, *rest), DEV)
                    _lib.launch_fused(_lib.make_params(img, b, z, z, zf, matrix, *rest), DEV)
                    assert torch.equal(a, b)
                    host_in, host_out = img.cpu().pin_memory(), torch.empty(n, 3, oh, ow, dtype=work).pin_memory()
                    host_matrix = matrix.cpu().contiguous() if matrix is not None else None
                    _lib.launch_fused_host(_lib.make_params(host_in, host_out, None, None, None, host_matrix, *rest), DEV)
                    assert torch.equal(host_out, b.cpu())
