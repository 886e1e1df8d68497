"""The five benchmark configurations at FULL size, through the class API, against the CPU oracle.

Parameters are drawn on the GPU by the transform itself (seeded), captured, and handed to the
oracle together with the matrix the GPU path used, so both sides see identical inputs.
fp32: max |diff| <= 1e-5, fp16: <= 1e-2; nearest-mode runs are additionally checked with an
index image so that every sampled texel is the oracle's.  Size-independent properties (flip
twice, identity affine == crop path, shard == whole) are checked on the same tensors.
"""
import numpy as np
import pytest
import torch

from conftest import MEAN, STD
from oracle import fused_oracle as O

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
JITTER = dict(brightness=0.2, contrast=0.2, saturation=0.2, grayscale_p=0.1, mean=MEAN, std=STD)
AFFINE = dict(degrees=15, translate=(0.1, 0.1), scale=(0.9, 1.1), shear=5)


def _ta():
    import triton_augment_b200 as ta
    return ta


def _pixels(shape, dtype, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return torch.rand(shape, device=DEV, generator=g).to(dtype)


def _run_and_check(aug, img, tol, chunk=64):
    """forward() with captured parameters vs the oracle, `chunk` images at a time on the CPU."""
    ta = _ta()
    from triton_augment_b200.transforms import _Layout
    lay = _Layout(img, aug.same_on_batch, aug.same_on_frame)
    h, w = lay.image.shape[2:]
    torch.manual_seed(1234)
    params = aug._spread_all(lay, aug._get_params(lay.count, DEV, (h, w)))
    got = aug._apply(lay.image, params)
    angle, translate, scale, shear, top, left, flip, b, c, s, g = params
    matrix = None
    if aug.has_affine:
        matrix = ta.functional._prepare_affine_matrix_only(lay.total, DEV, h, w, angle, translate, scale, shear, None)
    oh, ow = got.shape[2:]
    np_ = lambda t: t.detach().cpu().numpy()
    dt = np.float16 if img.dtype == torch.float16 else np.float32
    worst = 0.0
    for a in range(0, lay.total, chunk):
        z = slice(a, min(a + chunk, lay.total))
        want = O.fused_augment(np_(lay.image[z]), np_(top[z]), np_(left[z]), oh, ow, np_(flip[z]),
                               matrix=None if matrix is None else np_(matrix[z]),
                               interpolation=str(getattr(aug, "interpolation", "nearest")),
                               brightness=np_(b[z]).astype(dt), contrast=np_(c[z]).astype(dt),
                               saturation=np_(s[z]).astype(dt), grayscale=np_(g[z]), mean=MEAN, std=STD,
                               flags=dict(brightness=True, contrast=True, saturation=True, grayscale=True))
        worst = max(worst, float(np.abs(np_(got[z]).astype(np.float32) - want.astype(np.float32)).max()))
    assert worst <= tol, worst
    return lay, params, got


def test_c1_colour_gray_normalize():
    ta = _ta()
    aug = ta.TritonFusedAugment(**JITTER)                      # same kernel path as TritonColorJitterNormalize
    _run_and_check(aug, _pixels((32, 3, 224, 224), torch.float32), 1e-5)
    cj = ta.TritonColorJitterNormalize(**JITTER)
    x = _pixels((32, 3, 224, 224), torch.float32, 1)
    torch.manual_seed(3); a = cj(x)
    torch.manual_seed(3); b = aug(x)                            # no geometry configured: draws coincide
    assert a.shape == (32, 3, 224, 224) and torch.isfinite(a).all() and a.equal(b)


def test_c2_crop_flip_colour():
    ta = _ta()
    aug = ta.TritonFusedAugment(crop_size=112, horizontal_flip_p=0.5, **JITTER)
    lay, params, got = _run_and_check(aug, _pixels((256, 3, 224, 224), torch.float32), 1e-5)
    assert got.shape == (256, 3, 112, 112)


@pytest.mark.parametrize("interp", ["nearest", "bilinear"])
def test_c3_affine_full_size(interp):
    ta = _ta()
    aug = ta.TritonFusedAugment(crop_size=1024, horizontal_flip_p=0.5, interpolation=interp, **AFFINE, **JITTER)
    img = _pixels((64, 3, 1280, 1280), torch.float32)
    lay, params, got = _run_and_check(aug, img, 1e-5, chunk=16)
    assert got.shape == (64, 3, 1024, 1024)
    staged, direct, viol, timeouts = ta.utils.debug_counters()
    assert timeouts == 0 and viol == 0
    # sharding is invisible: any slice of the batch with its slice of the parameters gives the same bits
    from triton_augment_b200.multi_gpu import slice_params
    part = aug._apply(img[40:56], slice_params(params, 40, 56))
    assert part.equal(got[40:56])
    if interp == "nearest":
        # geometry alone, bit-exact: sampled source index of every output pixel of 4 images
        idx = torch.arange(1280 * 1280, device=DEV, dtype=torch.float32).reshape(1, 1, 1280, 1280).expand(4, 3, 1280, 1280).contiguous()
        angle, translate, scale, shear, top, left, flip = (p[:4] for p in params[:7])
        out = ta.fused_augment(idx, top, left, 1024, 1024, flip, angle=angle, translate=translate, scale=scale,
                               shear=shear, interpolation="nearest", fill=-1.0)
        matrix = ta.functional._prepare_affine_matrix_only(4, DEV, 1280, 1280, angle, translate, scale, shear, None)
        _, want = O.fused_augment(idx.cpu().numpy(), top.cpu().numpy(), left.cpu().numpy(), 1024, 1024,
                                  flip.cpu().numpy(), matrix=matrix.cpu().numpy(), fill=-1.0, want_index=True)
        assert np.array_equal(out[:, 0].cpu().numpy().astype(np.int64), want.astype(np.int64))


def test_c4_fp16_affine():
    ta = _ta()
    aug = ta.TritonFusedAugment(crop_size=448, horizontal_flip_p=0.5, **AFFINE, **JITTER)
    img = _pixels((512, 3, 512, 512), torch.float16)
    lay, params, got = _run_and_check(aug, img[:128], 1e-2, chunk=64)       # a quarter of the batch vs the oracle
    torch.manual_seed(1234)
    full = aug(img)
    assert full.shape == (512, 3, 448, 448) and full.dtype == torch.float16 and torch.isfinite(full).all()


def test_c5_video_and_large_batch():
    ta = _ta()
    aug = ta.TritonFusedAugment(crop_size=112, horizontal_flip_p=0.5, same_on_frame=True, same_on_batch=False, **JITTER)
    video = _pixels((8, 16, 3, 224, 224), torch.float32)
    lay, params, got = _run_and_check(aug, video, 1e-5)
    assert got.shape == (128, 3, 112, 112)
    assert params[4].reshape(8, 16).std(dim=1).max() == 0        # crop offsets shared by the frames of a video
    torch.manual_seed(5)
    out = aug(video)
    assert out.shape == (8, 16, 3, 112, 112)
    # 4096-image batch: whole == concatenation of 8 shards (what 8 GPUs would compute)
    big = _pixels((4096, 3, 224, 224), torch.float32, 2)
    flat = ta.TritonFusedAugment(crop_size=112, horizontal_flip_p=0.5, **JITTER)
    torch.manual_seed(6); whole = flat(big)
    torch.manual_seed(6); parts = ta.ShardedAugment(flat, [0] * 8)(big)
    assert [p.shape[0] for p in parts] == [512] * 8 and torch.cat(parts).equal(whole)


def test_size_independent_properties_at_full_size():
    ta = _ta()
    img = _pixels((16, 3, 1280, 1280), torch.float32, 7)
    n = img.shape[0]
    top = torch.randint(0, 257, (n,), device=DEV).float()
    left = torch.randint(0, 257, (n,), device=DEV).float()
    ones = torch.ones(n, device=DEV, dtype=torch.bool)
    # identity affine (nearest and bilinear) == the crop/flip path, bit for bit
    plain = ta.fused_augment(img, top, left, 1024, 1024, ones)
    for interp in ("nearest", "bilinear"):
        via_affine = ta.fused_augment(img, top, left, 1024, 1024, ones, interpolation=interp,
                                      _flags=dict(affine=True, brightness=False, contrast=False, saturation=False, grayscale=False))
        assert via_affine.equal(plain), interp
    # flipping twice is the identity; crop of a crop composes
    once = ta.horizontal_flip(img)
    assert ta.horizontal_flip(once).equal(img)
    assert ta.crop(ta.crop(img, 100, 60, 1000, 1100), 24, 40, 512, 768).equal(ta.crop(img, 124, 100, 512, 768))
    # normalize is affine in the pixels: normalize(a) - normalize(b) == (a - b) / std
    a, b = img[:4], img[4:8]
    lhs = ta.normalize(a, MEAN, STD) - ta.normalize(b, MEAN, STD)
    rhs = (a - b) / torch.tensor(STD, device=DEV).view(1, 3, 1, 1)
    assert (lhs - rhs).abs().max() < 2e-5
    # empty batch
    empty = ta.fused_augment(img[:0], 0, 0, 64, 64)
    assert empty.shape == (0, 3, 64, 64)
