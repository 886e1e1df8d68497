"""The staged affine kernel copies, per output tile, only the source row segments it
expects to read.  If that expectation were ever too small the kernel would sample
uninitialised shared memory, so the footprint arithmetic (csrc/ta_footprint.h, compiled
for the host too) is checked here, without a GPU, against a brute-force walk over every
pixel of every tile with the reference's coordinate arithmetic."""
import numpy as np
import pytest

from triton_augment_b200 import _lib

f32 = np.float32


def _coords(h, w, oh, ow, top, left, flip, m, xs, ys):
    """x_in, y_in of triton_augment/kernels/geometric_kernel.py:386-415 for pixel grids xs, ys (fp32 steps)."""
    xf = (f32(ow - 1) - xs.astype(f32)) if flip else xs.astype(f32)
    x_img = (xf + f32(left)).astype(f32)
    y_img = (ys.astype(f32) + f32(top)).astype(f32)
    hw, hh = f32(w) * f32(0.5), f32(h) * f32(0.5)
    xc = ((x_img - hw).astype(f32) + f32(0.5)).astype(f32)
    yc = ((y_img - hh).astype(f32) + f32(0.5)).astype(f32)
    m = m.astype(f32)
    # fma(xc, a, b*yc): product exact in float64, one rounding to fp32
    ux = (xc.astype(np.float64) * np.float64(m[0]) + (m[1] * yc).astype(f32).astype(np.float64)).astype(f32)
    uy = (xc.astype(np.float64) * np.float64(m[3]) + (m[4] * yc).astype(f32).astype(np.float64)).astype(f32)
    sx = (((ux + m[2]).astype(f32) + hw).astype(f32) - f32(0.5)).astype(f32)
    sy = (((uy + m[5]).astype(f32) + hh).astype(f32) - f32(0.5)).astype(f32)
    return sx, sy


def _matrix(rng, deg, tr, sc, sh, h, w):
    ang = np.deg2rad(rng.uniform(-deg, deg))
    sx, sy = np.deg2rad(rng.uniform(-sh, sh)), np.deg2rad(rng.uniform(-sh / 2, sh / 2))
    s = rng.uniform(*sc)
    tx, ty = rng.uniform(-tr * w, tr * w), rng.uniform(-tr * h, tr * h)
    a = np.cos(ang - sy) / np.cos(sy)
    b = -np.cos(ang - sy) * np.tan(sx) / np.cos(sy) - np.sin(ang)
    c = np.sin(ang - sy) / np.cos(sy)
    d = -np.sin(ang - sy) * np.tan(sx) / np.cos(sy) + np.cos(ang)
    m0, m1, m3, m4 = d / s, -b / s, -c / s, a / s
    return np.array([m0, m1, m0 * -tx + m1 * -ty, m3, m4, m3 * -tx + m4 * -ty], f32)


def _check_image(bilinear, elem_bytes, h, w, oh, ow, top, left, flip, m):
    shape = _lib.tile_shape()
    tw, th, max_rows = shape[:3]
    pitch = shape[{4: 3, 2: 4, 1: 5}[elem_bytes]]
    chunk = 16 // elem_bytes
    staged = 0
    for ty in range((oh + th - 1) // th):
        for tx in range((ow + tw - 1) // tw):
            rows, row0, xs, xe = _lib.tile_footprint(bilinear, elem_bytes, h, w, oh, ow, top, left, flip, m, tx, ty)
            if rows == 0:
                continue
            staged += 1
            assert rows <= max_rows
            xs, xe = np.array(xs), np.array(xe)
            assert np.all(xs % chunk == 0) and np.all(xe % chunk == 0) and np.all(xe - xs <= pitch)
            px = np.arange(tx * tw, min((tx + 1) * tw, ow))
            py = np.arange(ty * th, min((ty + 1) * th, oh))
            gx, gy = np.meshgrid(px, py)
            sx, sy = _coords(h, w, oh, ow, top, left, flip, m, gx, gy)
            if bilinear:
                x0, y0 = np.floor(sx).astype(int), np.floor(sy).astype(int)
                taps = [(x0, y0), (x0 + 1, y0), (x0, y0 + 1), (x0 + 1, y0 + 1)]
            else:
                taps = [(np.rint(sx).astype(int), np.rint(sy).astype(int))]
            for txs, tys in taps:
                r = tys - row0
                assert r.min() >= 0 and r.max() < rows, (tx, ty, r.min(), r.max(), rows)
                assert np.all(txs >= xs[r]) and np.all(txs < xe[r]), (tx, ty)
    return staged


@pytest.mark.parametrize("bilinear", [False, True])
@pytest.mark.parametrize("elem_bytes", [4, 2])
def test_footprint_covers_every_tap(bilinear, elem_bytes):
    rng = np.random.default_rng(5 + int(bilinear) + elem_bytes)
    staged_total = 0
    for trial in range(24):
        h, w = int(rng.integers(40, 400)), int(rng.integers(40, 400)) // 8 * 8 + 8
        oh, ow = int(rng.integers(8, h + 1)), int(rng.integers(8, w + 1))
        top, left = float(rng.integers(0, h - oh + 1)), float(rng.integers(0, w - ow + 1))
        if trial % 3 == 0:
            m = _matrix(rng, 15, 0.1, (0.9, 1.1), 5, h, w)         # the benchmark's ranges
        elif trial % 3 == 1:
            m = _matrix(rng, 180, 0.3, (0.6, 2.5), 25, h, w)       # anything goes
        else:
            m = _matrix(rng, 3, 0.5, (0.95, 1.05), 0, h, w)        # nearly axis aligned, big shifts
        staged_total += _check_image(bilinear, elem_bytes, h, w, oh, ow, top, left, bool(trial & 1), m)
    assert staged_total > 50


def test_benchmark_geometry_is_always_staged():
    """1280x1280 -> 1024x1024 with the headline configuration's parameter ranges: every tile
    must fit the staging buffer (otherwise the fast path is not what gets measured)."""
    rng = np.random.default_rng(1)
    tw, th = _lib.tile_shape()[:2]
    for _ in range(12):
        m = _matrix(rng, 15, 0.1, (0.9, 1.1), 5, 1280, 1280)
        top, left = float(rng.integers(0, 257)), float(rng.integers(0, 257))
        nx, ny = (1024 + tw - 1) // tw, (1024 + th - 1) // th
        for tx, ty in [(0, 0), (nx - 1, ny - 1), (nx // 2, ny // 2), (nx - 1, 0), (0, ny - 1)]:
            rows, *_ = _lib.tile_footprint(True, 4, 1280, 1280, 1024, 1024, top, left, False, m, tx, ty)
            assert rows > 0


def test_degenerate_matrices_are_not_staged():
    for m in ([np.nan] * 6, [np.inf, 0, 0, 0, 1, 0], [1e9, 0, 0, 0, 1e9, 0], [0, 0, 0, 0, 0, 0]):
        rows, *_ = _lib.tile_footprint(True, 4, 64, 64, 64, 64, 0.0, 0.0, False, np.array(m, f32), 0, 0)
        if rows:   # the all-zero matrix maps the tile to one point, which does fit
            assert np.allclose(m, 0)


def test_half_pixel_benchmark_geometry_is_always_staged():
    """512x512 -> 448x448 half images with the benchmark's parameter ranges: every 64 x 64 tile
    (up to 96 source rows) must fit the staging buffer."""
    rng = np.random.default_rng(2)
    shape = _lib.tile_shape()
    tw, th = shape[:2]
    assert th == 64 and shape[2] == 96 and tuple(shape[6:8]) == (64, 96)
    for _ in range(40):
        m = _matrix(rng, 15, 0.1, (0.9, 1.1), 5, 512, 512)
        top, left = float(rng.integers(0, 65)), float(rng.integers(0, 65))
        nx, ny = (448 + tw - 1) // tw, (448 + th - 1) // th
        for tx in range(nx):
            for ty in range(ny):
                for flip in (False, True):
                    rows, *_ = _lib.tile_footprint(True, 2, 512, 512, 448, 448, top, left, flip, m, tx, ty)
                    assert 0 < rows <= 96
