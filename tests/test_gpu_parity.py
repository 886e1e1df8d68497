"""GPU parity: the CUDA path (through the C ABI) against the CPU oracle and against the
golden vectors produced by the reference's own kernels.

Tolerances (stated by the task): fp32 max |diff| <= 1e-5, fp16 <= 1e-2; nearest-mode
geometry (which source texel each output pixel reads) bit-exact.
"""
import numpy as np
import pytest
import torch

from conftest import MEAN, STD, fused_case
from oracle import fused_oracle as O

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5
FP16_TOL = 1e-2


def _dev():
    return torch.device("cuda:0")


def _ta():
    import triton_augment_b200 as ta
    return ta


def _run_cuda(case, **over):
    ta = _ta()
    dev = _dev()
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    img = t(case["image"])
    kw = dict(brightness_factor=t(case["brightness"].astype(np.float32)),
              contrast_factor=t(case["contrast"].astype(np.float32)),
              saturation_factor=t(case["saturation"].astype(np.float32)),
              grayscale=t(case["gray"]).bool())
    for k in ("brightness", "contrast", "saturation"):
        if case[k].ndim == 0:
            kw[k + "_factor"] = float(case[k])
    if case["gray"].ndim == 0:
        kw["grayscale"] = bool(case["gray"])
    if "matrix" in case:
        kw.update(angle=t(case["angle"]), translate=t(case["translate"]), scale=t(case["scale"]),
                  shear=t(case["shear"]), interpolation=str(case["interp"]), fill=float(case["fill"]))
    if bool(case["norm"]):
        kw.update(mean=MEAN, std=STD)
    kw.update(over)
    out = ta.fused_augment(img, t(case["top"]), t(case["left"]), int(case["oh"]), int(case["ow"]),
                           t(case["flip"]).bool(), **kw)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def _run_oracle(case, fma="gpu"):
    kw = {}
    if "matrix" in case:
        kw = dict(matrix=case["matrix"], interpolation=str(case["interp"]), fill=float(case["fill"]))
    norm = bool(case["norm"])
    return O.fused_augment(case["image"], case["top"], case["left"], int(case["oh"]), int(case["ow"]),
                           case["flip"], brightness=case["brightness"], contrast=case["contrast"],
                           saturation=case["saturation"], grayscale=case["gray"],
                           mean=MEAN if norm else None, std=STD if norm else None, fma_coords=fma, **kw)


def _names(z):
    return [str(n) for n in z["names"]]


def test_golden_cases_vs_oracle(fused_golden):
    """Every golden case: CUDA vs the oracle evaluated with the GPU coordinate recipe."""
    for name in _names(fused_golden):
        case = fused_case(fused_golden, name)
        got = _run_cuda(case).astype(np.float32)
        want = _run_oracle(case).astype(np.float32)
        tol = FP16_TOL if case["image"].dtype == np.float16 else FP32_TOL
        err = float(np.abs(got - want).max())
        assert err <= tol, (name, err)


def test_golden_cases_vs_reference_outputs(fused_golden):
    """Every golden case against the stored output of the reference's own kernel (CPU
    interpreter, which does not contract a*x+b*y).  Non-affine cases have exact integer
    coordinates, so they must agree to tolerance everywhere.  Affine cases may differ where
    the one-ulp coordinate difference flips a rounding: there the check is that pixels whose
    coordinates agree (oracle fma vs non-fma give the same value) match, and that they are
    the overwhelming majority."""
    for name in _names(fused_golden):
        case = fused_case(fused_golden, name)
        got = _run_cuda(case).astype(np.float32)
        want = case["out"].astype(np.float32)
        tol = FP16_TOL if case["image"].dtype == np.float16 else FP32_TOL
        if "matrix" not in case:
            assert float(np.abs(got - want).max()) <= tol, name
            continue
        a = _run_oracle(case).astype(np.float32)
        b = _run_oracle(case, fma=False).astype(np.float32)
        same = np.abs(a - b) <= 1e-7
        # nearest: a flipped rounding moves a few texels; bilinear: any coordinate ulp shows
        assert same.mean() > (0.80 if str(case["interp"]) == "bilinear" else 0.97), name
        assert float(np.abs(got - want)[same].max()) <= tol, name


def test_nearest_geometry_is_bit_exact():
    """Index image (pixel value = its own flat index, exact in fp32) through nearest sampling:
    the sampled index of every output pixel must equal the oracle's."""
    ta = _ta()
    dev = _dev()
    rng = np.random.default_rng(3)
    for (n, h, w, oh, ow) in [(3, 96, 128, 64, 96), (2, 257, 264, 130, 200), (2, 64, 64, 64, 64)]:
        idx = np.arange(h * w, dtype=np.float32).reshape(1, 1, h, w)
        img = np.broadcast_to(idx, (n, 3, h, w)).copy()
        angle = rng.uniform(-15, 15, n).astype(np.float32)
        translate = rng.uniform(-0.1 * w, 0.1 * w, (n, 2)).astype(np.float32)
        scale = rng.uniform(0.9, 1.1, n).astype(np.float32)
        shear = np.stack([rng.uniform(-5, 5, n), np.zeros(n)], 1).astype(np.float32)
        top = rng.integers(0, h - oh + 1, n).astype(np.float32)
        left = rng.integers(0, w - ow + 1, n).astype(np.float32)
        flip = rng.random(n) < 0.5
        t = lambda a: torch.from_numpy(a).to(dev)
        out = ta.fused_augment(t(img), t(top), t(left), oh, ow, t(flip), angle=t(angle), translate=t(translate),
                               scale=t(scale), shear=t(shear), interpolation="nearest", fill=-1.0)
        matrix = ta.functional._prepare_affine_matrix_only(n, dev, h, w, t(angle), t(translate), t(scale), t(shear),
                                                           None).cpu().numpy()
        _, want_idx = O.fused_augment(img, top, left, oh, ow, flip, matrix=matrix, fill=-1.0, want_index=True)
        got_idx = out[:, 0].cpu().numpy().astype(np.int64)
        assert np.array_equal(got_idx, want_idx.astype(np.int64)), (h, w)
        assert np.array_equal(out[:, 1].cpu().numpy(), out[:, 0].cpu().numpy())


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("interp", ["none", "nearest", "bilinear"])
def test_every_flag_combination(dtype, interp):
    """All 32 on/off combinations of the five colour operations, odd sizes, per-image parameters."""
    ta = _ta()
    dev = _dev()
    rng = np.random.default_rng(11)
    n, h, w, oh, ow = 3, 45, 56, 29, 41
    img = rng.random((n, 3, h, w), dtype=np.float32).astype(dtype)
    top = rng.integers(0, h - oh + 1, n).astype(np.float32)
    left = rng.integers(0, w - ow + 1, n).astype(np.float32)
    flip = np.array([True, False, True])
    angle = rng.uniform(-15, 15, n).astype(np.float32)
    translate = rng.uniform(-4, 4, (n, 2)).astype(np.float32)
    scale = rng.uniform(0.9, 1.1, n).astype(np.float32)
    shear = rng.uniform(-5, 5, (n, 2)).astype(np.float32)
    t = lambda a: torch.from_numpy(a).to(dev)
    matrix = None
    akw = {}
    if interp != "none":
        akw = dict(angle=t(angle), translate=t(translate), scale=t(scale), shear=t(shear), interpolation=interp)
        matrix = ta.functional._prepare_affine_matrix_only(n, dev, h, w, t(angle), t(translate), t(scale), t(shear),
                                                           None).cpu().numpy()
    tol = FP16_TOL if dtype == np.float16 else FP32_TOL
    for bits in range(32):
        b = rng.uniform(0.8, 1.2, n).astype(np.float32) if bits & 1 else np.ones(n, np.float32)
        c = rng.uniform(0.8, 1.2, n).astype(np.float32) if bits & 2 else np.ones(n, np.float32)
        s = rng.uniform(0.8, 1.2, n).astype(np.float32) if bits & 4 else np.ones(n, np.float32)
        g = np.array([True, False, True]) if bits & 8 else np.zeros(n, bool)
        norm = bool(bits & 16)
        got = ta.fused_augment(t(img), t(top), t(left), oh, ow, t(flip), brightness_factor=t(b), contrast_factor=t(c),
                               saturation_factor=t(s), grayscale=t(g), mean=MEAN if norm else None,
                               std=STD if norm else None, **akw).cpu().numpy().astype(np.float32)
        want = O.fused_augment(img, top, left, oh, ow, flip, matrix=matrix,
                               interpolation=interp if interp != "none" else "nearest",
                               brightness=b.astype(dtype), contrast=c.astype(dtype), saturation=s.astype(dtype),
                               grayscale=g, mean=MEAN if norm else None, std=STD if norm else None,
                               ).astype(np.float32)
        err = float(np.abs(got - want).max())
        assert err <= tol, (bits, err)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_vectorised_crop_flip_kernel_every_shift(dtype):
    """Crop/flip with whole-vector output rows runs on the 128-bit kernel, which shifts each
    lane's run out of two aligned vectors.  Every left offset 0..16, with and without flip,
    input widths that are and are not multiples of the vector (so the shift changes from row
    to row), odd heights, and windows that leave the image (read as 0): bit-exact vs the oracle."""
    ta = _ta()
    dev = _dev()
    rng = np.random.default_rng(8)
    for (h, w, oh, ow) in [(40, 200, 33, 136), (37, 203, 30, 144), (50, 178, 50, 160), (48, 172, 40, 152)]:
        n = 17
        img = rng.random((n, 3, h, w), dtype=np.float32).astype(dtype)
        left = np.arange(n, dtype=np.float32)
        top = (np.arange(n) % max(1, h - oh + 1)).astype(np.float32)
        for flip_all in (False, True):
            flip = np.full(n, flip_all)
            flip[3] = not flip_all
            t = lambda a: torch.from_numpy(a).to(dev)
            got = ta.fused_augment(t(img), t(top), t(left), oh, ow, t(flip)).cpu().numpy()
            want = O.fused_augment(img, top, left, oh, ow, flip)
            assert np.array_equal(got, want), (dtype, h, w, flip_all)
    # channel planes that are not whole vectors although the tensor is (51 * 394 elements, 4 images):
    # the channels of a strip then sit at different offsets within a vector
    img = rng.random((4, 3, 51, 394), dtype=np.float32).astype(dtype)
    top = np.array([5.0, 7.0, 0.0, 21.0], np.float32)
    left = np.array([31.0, 134.0, 0.0, 190.0], np.float32)
    for flip_all in (False, True):
        flip = np.array([flip_all, flip_all, not flip_all, flip_all])
        t = lambda a: torch.from_numpy(a).to(dev)
        got = ta.fused_augment(t(img), t(top), t(left), 30, 204, t(flip)).cpu().numpy()
        assert np.array_equal(got, O.fused_augment(img, top, left, 30, 204, flip)), (dtype, "odd planes", flip_all)
    # windows partly outside the image: left beyond w - ow, negative top
    img = rng.random((4, 3, 32, 64), dtype=np.float32).astype(dtype)
    top = np.array([-3.0, 0.0, 5.0, 30.0], np.float32)
    left = np.array([-8.0, 40.0, 0.0, 60.0], np.float32)
    flip = np.array([False, True, False, True])
    t = lambda a: torch.from_numpy(a).to(dev)
    got = ta.fused_augment(t(img), t(top), t(left), 16, 32, t(flip), brightness_factor=1.1, mean=MEAN, std=STD)
    want = O.fused_augment(img, top, left, 16, 32, flip, brightness=np.float32(1.1).astype(dtype), mean=MEAN, std=STD)
    tol = FP16_TOL if dtype == np.float16 else FP32_TOL
    assert float(np.abs(got.cpu().numpy().astype(np.float32) - want.astype(np.float32)).max()) <= tol


def test_staging_assertions_hold_on_random_geometry():
    """The checked build of the staged kernel counts every shared-memory tap that falls outside
    what was staged; over random matrices, sizes, offsets and flips there must be none, no
    barrier may time out, and the output must equal the oracle's bit for bit."""
    ta = _ta()
    from triton_augment_b200 import _lib
    dev = _dev()
    rng = np.random.default_rng(2024)
    _lib.debug_counters(reset=True)
    for trial in range(12):
        for dtype in (np.float32, np.float16):
            n = 2
            h = int(rng.integers(64, 300))
            w = int(rng.integers(8, 40)) * 8
            oh, ow = int(rng.integers(16, h + 1)), int(rng.integers(16, w + 1))
            img = rng.random((n, 3, h, w), dtype=np.float32).astype(dtype)
            lim = 15 if trial % 2 == 0 else 60
            angle = rng.uniform(-lim, lim, n).astype(np.float32)
            translate = rng.uniform(-0.2 * w, 0.2 * w, (n, 2)).astype(np.float32)
            scale = rng.uniform(0.7, 1.6, n).astype(np.float32)
            shear = rng.uniform(-10, 10, (n, 2)).astype(np.float32)
            top = rng.integers(0, h - oh + 1, n).astype(np.float32)
            left = rng.integers(0, w - ow + 1, n).astype(np.float32)
            flip = rng.random(n) < 0.5
            t = lambda a: torch.from_numpy(a).to(dev)
            matrix_t = ta.functional._prepare_affine_matrix_only(n, dev, h, w, t(angle), t(translate), t(scale),
                                                                 t(shear), None).contiguous()
            for bilinear in (False, True):
                out = torch.empty(n, 3, oh, ow, dtype=t(img).dtype, device=dev)
                p = _lib.make_params(t(img), out, t(top), t(left), t(flip.astype(np.uint8)), matrix_t, 0.25, bilinear,
                                     0, None, None, None, None, None, None)
                _lib.launch_fused(p, dev, checked=True)
                torch.cuda.synchronize()
                want = O.fused_augment(img, top, left, oh, ow, flip, matrix=matrix_t.cpu().numpy(), fill=0.25,
                                       interpolation="bilinear" if bilinear else "nearest",
                                       flags=dict(brightness=False, contrast=False, saturation=False, grayscale=False))
                got = out.cpu().numpy()
                if bilinear:
                    assert float(np.abs(got.astype(np.float32) - want.astype(np.float32)).max()) <= (
                        FP16_TOL if dtype == np.float16 else 2e-6)
                else:
                    assert np.array_equal(got, want)
    staged, direct, violations, timeouts = _lib.debug_counters()
    assert violations == 0 and timeouts == 0
    assert staged > 100


def test_one_large_image():
    """A single 2048x3072 image (coordinates in the thousands, thousands of tiles of one image,
    staged and gathered tiles side by side): nearest picks the oracle's texel for every pixel,
    bilinear stays within tolerance."""
    ta = _ta()
    dev = _dev()
    n, h, w, oh, ow = 1, 2048, 3072, 1900, 2900
    idx = np.arange(h * w, dtype=np.float32).reshape(1, 1, h, w)          # < 2^24: exact in fp32
    img = np.broadcast_to(idx, (n, 3, h, w)).copy()
    angle = np.array([9.0], np.float32)
    translate = np.array([[31.0, -17.0]], np.float32)
    scale = np.array([1.05], np.float32)
    shear = np.array([[3.0, 0.0]], np.float32)
    top, left, flip = np.array([70.0], np.float32), np.array([90.0], np.float32), np.array([True])
    t = lambda a: torch.from_numpy(a).to(dev)
    akw = dict(angle=t(angle), translate=t(translate), scale=t(scale), shear=t(shear))
    matrix = ta.functional._prepare_affine_matrix_only(n, dev, h, w, t(angle), t(translate), t(scale), t(shear),
                                                       None).cpu().numpy()
    out = ta.fused_augment(t(img), t(top), t(left), oh, ow, t(flip), interpolation="nearest", fill=-1.0, **akw)
    _, want_idx = O.fused_augment(img, top, left, oh, ow, flip, matrix=matrix, fill=-1.0, want_index=True)
    assert np.array_equal(out[:, 0].cpu().numpy().astype(np.int64), want_idx.astype(np.int64))
    pix = np.random.default_rng(5).random((n, 3, h, w), dtype=np.float32)
    got = ta.fused_augment(t(pix), t(top), t(left), oh, ow, t(flip), interpolation="bilinear",
                           brightness_factor=1.1, saturation_factor=0.9, mean=MEAN, std=STD, **akw).cpu().numpy()
    want = O.fused_augment(pix, top, left, oh, ow, flip, matrix=matrix, interpolation="bilinear",
                           brightness=np.float32(1.1), saturation=np.float32(0.9), mean=MEAN, std=STD)
    assert float(np.abs(got - want).max()) <= FP32_TOL
