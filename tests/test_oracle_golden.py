"""Pins the CPU oracle against vectors produced by the reference's own kernels.

tests/golden/fused_cases.npz holds outputs of the unmodified reference
(functional.fused_augment -> its Triton kernel under the CPU interpreter).  The
interpreter does not contract multiplies and adds, so the oracle is run with
fma_coords=0 and must then agree bit-for-bit in fp32.
"""
import numpy as np
import pytest

from conftest import MEAN, STD, fused_case
from oracle import fused_oracle as O


def _run(case, fma):
    kw = {}
    if "matrix" in case:
        kw = dict(matrix=case["matrix"], interpolation=str(case["interp"]), fill=float(case["fill"]))
    norm = bool(case["norm"])
    return O.fused_augment(case["image"], case["top"], case["left"], int(case["oh"]), int(case["ow"]),
                           case["flip"], brightness=case["brightness"], contrast=case["contrast"],
                           saturation=case["saturation"], grayscale=case["gray"],
                           mean=MEAN if norm else None, std=STD if norm else None, fma_coords=fma, **kw)


def test_every_case_is_covered(fused_golden):
    names = list(fused_golden["names"])
    assert len(names) >= 35
    assert any(n.startswith("f16_") for n in names) and any("bilinear" in n for n in names)


def test_oracle_matches_reference_fp32(fused_golden):
    checked = 0
    for name in fused_golden["names"]:
        case = fused_case(fused_golden, str(name))
        if case["image"].dtype != np.float32:
            continue
        got = _run(case, fma=False)
        want = case["out"]
        assert got.shape == want.shape, name
        assert np.array_equal(got, want), (name, float(np.abs(got - want).max()))
        checked += 1
    assert checked >= 25


def test_oracle_matches_reference_fp16(fused_golden):
    """fp16: the interpreter's type promotion is numpy's, not the GPU compiler's,
    so agreement is required to 2 fp16 ulp of the largest value (|x| < 4)."""
    checked = 0
    for name in fused_golden["names"]:
        case = fused_case(fused_golden, str(name))
        if case["image"].dtype != np.float16:
            continue
        got = _run(case, fma=False).astype(np.float32)
        want = case["out"].astype(np.float32)
        err = np.abs(got - want).max()
        assert err <= 2 * 2.0 ** -9, (name, float(err))
        checked += 1
    assert checked >= 8


def test_fma_recipe_differs_only_at_coordinate_ulp(fused_golden):
    """The GPU contraction can move a coordinate by one ulp; for nearest sampling that
    changes at most a handful of texels, never the bulk of the image."""
    case = fused_case(fused_golden, "affine_nearest_plain")
    a, b = _run(case, fma=False), _run(case, fma=True)
    assert (a != b).mean() < 0.01


def test_matrix_restatement(functional_golden):
    z = functional_golden
    got = O.inverse_affine_matrix(z["mat_center"], z["mat_angle"], z["mat_translate"], z["mat_scale"], z["mat_shear"])
    np.testing.assert_allclose(got, z["mat_out"], rtol=2e-5, atol=2e-5)


def test_exact_contrast_restatement(functional_golden):
    """adjust_contrast (torchvision-exact) = gray mean pre-pass + blend."""
    z = functional_golden
    img = z["image"]
    for key, f in (("contrast_1.4", 1.4), ("contrast_0.6", 0.6)):
        got = O.fused_augment(img, 0, 0, img.shape[2], img.shape[3], contrast=f,
                              contrast_mode=O.CONTRAST_MEAN, fma_coords=False)
        np.testing.assert_allclose(got, z[key], rtol=0, atol=2e-6)
    g = z["gray_image"]
    got = O.fused_augment(g, 0, 0, g.shape[2], g.shape[3], contrast=1.5, contrast_mode=O.CONTRAST_MEAN)
    np.testing.assert_allclose(got, z["gray_contrast_1.5"], rtol=0, atol=2e-6)


@pytest.mark.parametrize("key,kw", [
    ("brightness_1.3", dict(brightness=1.3)),
    ("contrast_fast_1.4", dict(contrast=1.4)),
    ("saturation_0.3", dict(saturation=0.3)),
    ("saturation_1.7", dict(saturation=1.7)),
    ("normalize", dict(mean=MEAN, std=STD)),
    ("gray3", dict(grayscale=1)),
    ("gray3_masked", dict(grayscale=[1, 0, 1])),
    ("hflip", dict(flip=1)),
    ("hflip_masked", dict(flip=[1, 0, 1])),
])
def test_standalone_functionals_are_the_fused_pass_with_noops(functional_golden, key, kw):
    z = functional_golden
    img = z["image"]
    got = O.fused_augment(img, 0, 0, img.shape[2], img.shape[3], fma_coords=False, **kw)
    if key.startswith("hflip"):
        assert np.array_equal(got, z[key]), key
    else:
        # Python-float factors stay double inside the interpreter ((1.0 - 1.7) is rounded
        # once, after the subtraction); the GPU build and the oracle take them as fp32.
        np.testing.assert_allclose(got, z[key], rtol=0, atol=5e-7)


def test_standalone_crop(functional_golden):
    z = functional_golden
    img = z["image"]
    assert np.array_equal(O.fused_augment(img, 2, 3, 9, 11), z["crop_2_3_9_11"])
    assert np.array_equal(O.fused_augment(img, z["crop_tops"], z["crop_lefts"], 9, 11), z["crop_per_image"])
    assert np.array_equal(O.fused_augment(img, 4, 7, 10, 8), z["center_crop_10_8"])
