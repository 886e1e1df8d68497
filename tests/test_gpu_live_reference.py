"""CUDA kernels against the reference's Triton kernels, both run HERE on the same tensors.

The unmodified reference package (yuhezhang-ai/triton-augment v0.3.0, installed into the
git-ignored baseline/_ref) is imported next to this package; every case builds one set of
inputs and parameters, calls `triton_augment.functional.fused_augment` (or a transform class)
and the same function of `triton_augment_b200`, and compares element by element:

    float32 <= 1e-5 absolute, float16 <= 1e-2, nearest-mode sampled indices identical.

The reference compiles one kernel per (colour-flag combination, sampling mode, dtype,
"are the output sizes multiples of 16") and its compiler picks the multiply-add contraction of
the coordinate arithmetic per compiled variant; `test_every_compiled_variant` therefore walks
all 32 x 2 x 2 x 2 of them.  The other tests follow the reference's own test grids
(tests/test_fused_affine.py:36-44, tests/test_fused_all.py:22-67 of the reference) and run the
transform classes from the same seed.

Skipped, with the reason, when the reference or Triton cannot be imported.
"""
import itertools
import os
import sys

import numpy as np
import pytest
import torch

from conftest import GOLDEN, MEAN, STD, ROOT

pytestmark = pytest.mark.gpu
sys.path.insert(0, GOLDEN)
DEV = torch.device("cuda:0")
TOL = {torch.float32: 1e-5, torch.float16: 1e-2}


@pytest.fixture(scope="module")
def ref():
    """The reference package, imported from baseline/_ref."""
    path = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(path, "triton_augment")):
        pytest.skip("the reference is not installed under baseline/_ref (pip install --no-index --no-deps --target "
                    "baseline/_ref <reference checkout>)")
    try:
        import triton  # noqa: F401
    except Exception as e:                                   # pragma: no cover - depends on the image
        pytest.skip(f"triton cannot be imported: {e}")
    os.environ["TRITON_AUGMENT_SUPPRESS_FIRST_RUN_MESSAGE"] = "1"
    if path not in sys.path:
        sys.path.insert(0, path)
    import triton_augment
    assert triton_augment.__version__ == "0.3.0"
    return triton_augment


@pytest.fixture(scope="module")
def ta():
    import triton_augment_b200
    return triton_augment_b200


def _err(a, b):
    return float((a.float() - b.float()).abs().max()) if a.numel() else 0.0


# ----------------------------------------------------------------------------- every compiled variant
SIZES = {"div16": (3, 272, 304, 208, 240),       # both output sizes multiples of 16: vectorised stores in the reference
         "odd": (3, 300, 340, 211, 203),          # neither: scalar stores, per-pixel contraction rule
         "rows320": (2, 400, 432, 320, 336)}      # whole 64-row tiles (the two sizes above take the 64 x 32 tile shape for float32)


@pytest.mark.parametrize("size", sorted(SIZES))
@pytest.mark.parametrize("interp", ["nearest", "bilinear"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["f32", "f16"])
def test_every_compiled_variant(ref, ta, dtype, interp, size):
    import make_gpu_golden as G
    n, h, w, oh, ow = SIZES[size]
    p = G.case_params(f"live_{size}", n, h, w, oh, ow)
    img = G.procedural_image(n, 3, h, w, dtype)
    bad = []
    for bits in range(32):
        want = G.run(ref.functional, img, p, oh, ow, interp, colour=True, bits=bits)
        got = G.run(ta.functional, img, p, oh, ow, interp, colour=True, bits=bits)
        assert got.shape == want.shape and got.dtype == want.dtype
        e = _err(got, want)
        if not e <= TOL[dtype]:
            bad.append((bits, e))
    assert not bad, f"{interp} {dtype} {size}: (flags, max |diff|) over tolerance {TOL[dtype]}: {bad}"


@pytest.mark.parametrize("size", sorted(SIZES))
def test_nearest_sampled_indices_are_identical(ref, ta, size):
    """Index image in, colour operations off: the output IS the sampled source index (or the
    fill value -1), so equality means the same texel was read for every output pixel."""
    import make_gpu_golden as G
    n, h, w, oh, ow = SIZES[size]
    p = G.case_params(f"live_{size}", n, h, w, oh, ow)
    idx = G.index_image(n, h, w)
    want = G.run(ref.functional, idx, p, oh, ow, "nearest", colour=False)
    got = G.run(ta.functional, idx, p, oh, ow, "nearest", colour=False)
    assert torch.equal(got, want)
    assert float((want >= 0).float().mean()) > 0.5            # the case samples inside the image mostly


# ----------------------------------------------------------------------------- the reference's affine grid
def _affine_grid():
    """The value sets of the reference's own fused-affine test (tests/test_fused_affine.py:36-44)."""
    return itertools.product([1, 4], ["nearest", "bilinear"], [(100, 111), (256, 256)], [[0.0, 0.0], [5, 1]],
                             [True, False], [0.0, 30.0], [[0.0, 0.0], [10.0, 5.0]], [[10, 10, 80, 80], [0, 0, 100, 111]])


def test_reference_affine_grid(ref, ta):
    g = torch.Generator(device=DEV).manual_seed(11)
    bad, count = [], 0
    for batch, interp, (h, w), shear, flip, angle, translate, (top, left, ch, cw) in _affine_grid():
        img = torch.rand(batch, 3, h, w, device=DEV, generator=g)
        kw = dict(top=top, left=left, height=ch, width=cw, flip_horizontal=flip, angle=angle, translate=translate,
                  scale=1.0, shear=shear, interpolation=interp)
        want = ref.functional.fused_augment(img, **kw)
        got = ta.functional.fused_augment(img, **kw)
        count += 1
        ok = torch.equal(got, want) if interp == "nearest" else _err(got, want) <= 1e-5
        if not ok:
            bad.append((batch, interp, h, w, shear, flip, angle, translate, top, left, ch, cw, _err(got, want)))
    assert count == 256 and not bad, bad[:8]


# ----------------------------------------------------------------------------- crop + flip + colour grid
def _fusion_cases():
    """Shape classes of the reference's complete-fusion test (tests/test_fused_all.py:22-67): square,
    wide, tall, odd and prime sizes, tiny and large images, large batches, whole-image and edge
    crops, extreme factors, with and without normalize.  (n, h, w), (top, left, ch, cw), flip,
    brightness, saturation, normalize."""
    cases = []
    rng = np.random.default_rng(2024)
    shapes = [(4, 224, 224), (2, 256, 256), (1, 480, 480),           # square
              (2, 208, 104), (3, 120, 232),                            # wide / tall
              (2, 221, 221), (1, 193, 199), (3, 225, 231),             # odd and prime sizes
              (8, 64, 64), (1, 16, 15), (2, 90, 90),                   # small and tiny
              (16, 128, 128), (32, 72, 72),                            # large batches
              (1, 1021, 1021)]                                         # one large odd image
    for n, h, w in shapes:
        ch = max(2, int(h * rng.uniform(0.4, 0.9)))
        cw = max(3, int(w * rng.uniform(0.4, 0.9)))
        if (h, w) == (16, 15):
            ch, cw = 2, 3
        top, left = int(rng.integers(0, h - ch + 1)), int(rng.integers(0, w - cw + 1))
        cases.append(((n, h, w), (top, left, ch, cw), bool(rng.random() < 0.5), float(np.round(rng.uniform(0.5, 1.5), 2)),
                      float(np.round(rng.uniform(0.5, 1.5), 2)), True))
    cases += [((2, 128, 128), (0, 0, 128, 128), True, 1.3, 0.8, True),        # whole image
              ((2, 224, 224), (112, 112, 112, 112), True, 1.15, 0.92, True),   # bottom-right corner
              ((1, 320, 320), (0, 160, 160, 160), False, 1.3, 0.7, True),      # right half
              ((1, 320, 320), (160, 0, 160, 160), True, 0.9, 1.2, True),       # bottom half
              ((1, 224, 224), (50, 50, 112, 112), False, 0.0, 0.0, True),      # factors at both extremes
              ((2, 224, 224), (50, 50, 112, 112), True, 2.0, 2.0, True),
              ((2, 224, 224), (20, 30, 112, 112), True, 1.2, 0.9, False),      # no normalize
              ((2, 256, 256), (0, 0, 128, 128), False, 1.0, 1.0, True)]        # identity colour factors
    return cases


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["f32", "f16"])
@pytest.mark.parametrize("contrast", [1.0, 0.8])
def test_reference_fusion_grid(ref, ta, dtype, contrast):
    g = torch.Generator(device=DEV).manual_seed(12)
    bad = []
    for (n, h, w), (top, left, ch, cw), flip, bright, sat, norm in _fusion_cases():
        img = torch.rand(n, 3, h, w, device=DEV, generator=g).to(dtype)
        kw = dict(top=top, left=left, height=ch, width=cw, flip_horizontal=flip, brightness_factor=bright,
                  contrast_factor=contrast, saturation_factor=sat, mean=MEAN if norm else None, std=STD if norm else None)
        want = ref.functional.fused_augment(img, **kw)
        got = ta.functional.fused_augment(img, **kw)
        e = _err(got, want)
        if not e <= TOL[dtype]:
            bad.append((n, h, w, top, left, ch, cw, flip, bright, sat, norm, e))
    assert not bad, bad


# ----------------------------------------------------------------------------- transform classes, same seed
CLASS_CASES = [
    ("TritonFusedAugment", dict(crop_size=(120, 136), horizontal_flip_p=0.5, degrees=15, translate=(0.1, 0.1),
                                scale=(0.9, 1.1), shear=5, interpolation="bilinear", brightness=0.2, contrast=0.2,
                                saturation=0.2, grayscale_p=0.5, mean=MEAN, std=STD)),
    ("TritonFusedAugment", dict(crop_size=112, horizontal_flip_p=0.5, degrees=20, interpolation="nearest",
                                brightness=0.3, grayscale_p=0.5, mean=MEAN, std=STD, same_on_batch=True)),
    ("TritonFusedAugment", dict(crop_size=96, horizontal_flip_p=0.5, brightness=0.2, contrast=0.2, saturation=0.2,
                                grayscale_p=0.5, mean=MEAN, std=STD, same_on_frame=False)),
    ("TritonColorJitterNormalize", dict(brightness=0.2, contrast=0.2, saturation=0.2, grayscale_p=0.5, mean=MEAN, std=STD)),
    ("TritonRandomCropFlip", dict(size=(100, 90), horizontal_flip_p=0.5)),
    ("TritonRandomAffine", dict(degrees=25, translate=(0.1, 0.2), scale=(0.8, 1.2), shear=(-5, 5, -3, 3),
                                interpolation="bilinear")),
    ("TritonColorJitter", dict(brightness=0.4, contrast=0.4, saturation=0.4)),
]


@pytest.mark.parametrize("case", range(len(CLASS_CASES)))
@pytest.mark.parametrize("ndim", [4, 5])
def test_transform_classes_from_the_same_seed(ref, ta, case, ndim):
    """Same constructor arguments, same seed, same input: the draws must come out in the
    reference's order and the kernels must agree, for image batches and for videos."""
    name, kw = CLASS_CASES[case]
    g = torch.Generator(device=DEV).manual_seed(100 + case)
    shape = (6, 3, 160, 176) if ndim == 4 else (3, 4, 3, 160, 176)
    x = torch.rand(shape, device=DEV, generator=g)
    theirs, ours = getattr(ref, name)(**kw), getattr(ta, name)(**kw)
    for seed in (1, 2):
        torch.manual_seed(seed)
        want = theirs(x)
        torch.manual_seed(seed)
        got = ours(x)
        assert got.shape == want.shape
        assert _err(got, want) <= 1e-5, (name, ndim, seed, _err(got, want))


def test_class_flags_when_no_image_draws_grayscale(ref, ta):
    """Known, bounded difference.  The classes here decide from their CONSTRUCTOR arguments
    which operations are compiled in (no device-to-host read, so a forward can be captured in
    a CUDA graph); the reference decides from the drawn VALUES.  When grayscale_p > 0 but no image
    of the batch draws grayscale, the reference runs its no-grayscale variant, whose compiler
    contracted the bilinear coordinate arithmetic the other way (brightness on, saturation off):
    the results then differ by one rounding of a source coordinate, <= 1e-3 on uniform-noise
    pixels.  Passing the same parameters through the functional entry point, which decides from
    the values like the reference, agrees to 1e-5."""
    kw = dict(crop_size=128, degrees=15, interpolation="bilinear", brightness=0.2, grayscale_p=1e-6, mean=MEAN, std=STD)
    x = torch.rand(4, 3, 160, 160, device=DEV, generator=torch.Generator(device=DEV).manual_seed(7))
    torch.manual_seed(5)
    want = ref.TritonFusedAugment(**kw)(x)
    ours = ta.TritonFusedAugment(**kw)
    torch.manual_seed(5)
    got = ours(x)
    assert _err(got, want) <= 1e-3
    torch.manual_seed(5)
    lay = ours._layout(x)
    angle, translate, scale, shear, top, left, flip, b, c, s, gmask = ours._spread_all(
        lay, ours._get_params(lay.count, lay.param_device, (160, 160)))
    assert not bool(gmask.any())
    exact = ta.functional.fused_augment(x, top, left, 128, 128, flip, angle=angle, translate=translate, scale=scale,
                                        shear=shear, interpolation="bilinear", brightness_factor=b, grayscale=gmask,
                                        mean=MEAN, std=STD)
    assert _err(exact, want) <= 1e-5
