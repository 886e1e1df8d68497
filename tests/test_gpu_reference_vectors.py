"""CUDA kernels against vectors produced by the reference's own Triton kernels ON A B200
(tests/golden/gpu_reference_cases.npz, written by tests/golden/make_gpu_golden.py).

This is the comparison the task names: same inputs and parameters through the reference's GPU
kernels and through ours; fp32 within 1e-5, fp16 within 1e-2, nearest-mode geometry bit-exact
(checked through a SHA-256 of the sampled-index image, 3 million pixels at 1280x1280)."""
import hashlib
import os
import sys

import numpy as np
import pytest
import torch

from conftest import GOLDEN, MEAN, STD

pytestmark = pytest.mark.gpu
sys.path.insert(0, GOLDEN)


@pytest.fixture(scope="module")
def vectors():
    return np.load(os.path.join(GOLDEN, "gpu_reference_cases.npz"))


def _inputs(z, name):
    import make_gpu_golden as G            # procedural inputs only; does not import the reference
    n, h, w, oh, ow = (int(v) for v in z[f"{name}|shape"])
    p = {k: z[f"{name}|{k}"] for k in ("angle", "translate", "scale", "shear", "top", "left", "flip",
                                        "brightness", "contrast", "saturation", "gray")}
    return G, (n, h, w, oh, ow), p, getattr(torch, str(z[f"{name}|dtype"]))


def test_parameters_regenerate(vectors):
    """The fixture's parameters come from a seeded generator in the script; make sure the
    script still produces them (otherwise the stored outputs would not belong to them)."""
    for name in vectors["names"]:
        G, (n, h, w, oh, ow), p, _ = _inputs(vectors, str(name))
        again = G.case_params(str(name), n, h, w, oh, ow)
        for k, v in p.items():
            assert np.array_equal(np.asarray(again[k]), v), (name, k)


def test_matrix_equals_the_reference_matrix(vectors):
    import triton_augment_b200 as ta
    for name in vectors["names"]:
        name = str(name)
        G, (n, h, w, oh, ow), p, _ = _inputs(vectors, name)
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(G.DEV)
        m = ta.functional._prepare_affine_matrix_only(n, G.DEV, h, w, t(p["angle"]), t(p["translate"]), t(p["scale"]),
                                                      t(p["shear"]), None)
        assert np.array_equal(m.cpu().numpy().view(np.int32), vectors[f"{name}|matrix"].view(np.int32)), name


def test_nearest_geometry_hash(vectors):
    import triton_augment_b200 as ta
    for name in vectors["names"]:
        name = str(name)
        G, (n, h, w, oh, ow), p, _ = _inputs(vectors, name)
        got = G.run(ta.functional, G.index_image(n, h, w), p, oh, ow, "nearest", colour=False)
        idx = got[:, 0].cpu().numpy().astype(np.int32)
        assert hashlib.sha256(idx.tobytes()).hexdigest() == str(vectors[f"{name}|nearest_index_sha256"]), name


@pytest.mark.parametrize("interp", ["nearest", "bilinear"])
def test_every_fp32_variant_against_stored_reference_values(vectors, interp):
    """All 32 colour-flag combinations of either sampling mode, on one case whose output sizes are
    multiples of 16 and one where neither is (the reference then compiles scalar stores and mixes
    two coordinate contractions inside one launch): values of the reference's kernels at seeded
    pixel positions.  Pins the per-variant contraction rule and the per-pixel one."""
    import triton_augment_b200 as ta
    import make_gpu_golden as G
    for name in G.ALL_VARIANT_CASES:
        if f"{name}|{interp}_variants" not in vectors.files:
            pytest.fail(f"{name}: fixture has no per-variant values; regenerate with tests/golden/make_gpu_golden.py")
        G_, (n, h, w, oh, ow), p, dtype = _inputs(vectors, name)
        img = G.procedural_image(n, 3, h, w, dtype)
        pn, py, px = (torch.from_numpy(v).to(G.DEV) for v in G.variant_points(name, n, oh, ow))
        want_all = vectors[f"{name}|{interp}_variants"]
        bad = []
        for bits in range(32):
            got = G.run(ta.functional, img, p, oh, ow, interp, colour=True, bits=bits)
            err = float(np.abs(got[pn, :, py, px].cpu().numpy() - want_all[bits]).max())
            if not err <= 1e-5:
                bad.append((bits, err))
        assert not bad, (name, interp, bad)


@pytest.mark.parametrize("interp", ["nearest", "bilinear"])
def test_full_pipeline_against_reference_output(vectors, interp):
    """All colour operations on; for the case whose output dimensions are not divisible by 16
    (the reference then mixes two coordinate contractions inside one launch) also three other
    flag combinations."""
    import triton_augment_b200 as ta
    for name in vectors["names"]:
        name = str(name)
        G, (n, h, w, oh, ow), p, dtype = _inputs(vectors, name)
        stride = int(vectors[f"{name}|stride"])
        img = G.procedural_image(n, 3, h, w, dtype)
        for bits in (31,) + (G.EXTRA_FLAGS.get(name, ()) if interp == "bilinear" else ()):
            got = G.run(ta.functional, img, p, oh, ow, interp, colour=True, bits=bits)
            sub = got[:, :, ::stride, ::stride].cpu().numpy().astype(np.float32)
            want = vectors[f"{name}|{interp}_sub" + ("" if bits == 31 else f"_flags{bits}")].astype(np.float32)
            tol = 1e-2 if dtype == torch.float16 else 1e-5
            err = float(np.abs(sub - want).max())
            assert err <= tol, (name, interp, bits, err)
