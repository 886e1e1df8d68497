"""Vectors from the reference's Triton kernels compiled for, and run on, a real GPU.

    python tests/golden/make_gpu_golden.py --reference baseline/_ref

`--reference` is a directory that contains the reference package `triton_augment` (the
unmodified v0.3.0, e.g. installed with `pip install --target baseline/_ref`).  Unlike
make_golden.py (CPU interpreter) this pins what the GPU build of the reference computes,
including the multiply-add contraction in its coordinate arithmetic.

Inputs are procedural (an integer hash of the pixel position, exact on any device) so they are
regenerated instead of stored.  Stored per case: the per-image parameters, and
  * nearest: SHA-256 of the sampled-source-index image (index image in, colour ops off) and
  * a strided subsample of the full-colour output (nearest and bilinear).
The script also checks the CPU oracle against the reference on the spot and prints what it
finds, and times the reference's fused call on the 1280x1280 -> 1024x1024 configuration.

How the coordinate recipe in oracle.fused_oracle.gpu_recipe() was found: for each of the 32
colour-flag combinations, each sampling mode and fp32 / fp16, the reference's output on a
1280x1280 procedural image was compared with the oracle under all nine (x, y) contraction
recipes; exactly one recipe reproduces the fp32 output to <= 2e-6 everywhere (sizes divisible by
16; with other sizes some variants mix two forms across lanes and ~1-4 % of pixels keep a
one-ulp coordinate difference).  Those variants were then resolved pixel by pixel: with neither
output dimension divisible by 16 the last 1-3 of a reference thread's 8 pixels (128 apart in the
linear output index) use the x recipe of the unswapped variants; the case "scalar_stores"
pins this for three flag combinations.
"""
from __future__ import annotations

import argparse
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
MEAN, STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)
DEV = torch.device("cuda:0")
STRIDE = 8

CASES = [
    # name, n, h, w, oh, ow, dtype
    ("c3_like_1280", 3, 1280, 1280, 1024, 1024, "float32"),
    ("odd_sizes", 4, 517, 640, 401, 512, "float32"),
    ("c4_like_512_f16", 4, 512, 512, 448, 448, "float16"),
    ("scalar_stores", 3, 300, 340, 211, 203, "float32"),     # neither output dimension divisible by 16
    ("variants_div16", 3, 272, 304, 208, 240, "float32"),    # both divisible by 16
]
# Cases for which EVERY compiled fp32 variant of the reference kernel is pinned: 32 colour-flag
# combinations x {nearest, bilinear}, the values at VARIANT_POINTS seeded pixel positions each.
ALL_VARIANT_CASES = ("scalar_stores", "variants_div16")
VARIANT_POINTS = 768
# extra flag combinations (bit 0 brightness, 1 contrast, 2 saturation, 3 grayscale, 4 normalize) and
# the subsampling stride per case
EXTRA_FLAGS = {"scalar_stores": (5, 9, 14)}
STRIDES = {"scalar_stores": 3}


def procedural_image(n, c, h, w, dtype):
    """uniform-looking pixels in [0, 1) from an integer hash of (n, c, y, x): exact everywhere."""
    i64 = torch.int64
    ys = torch.arange(h, device=DEV, dtype=i64).view(1, 1, h, 1)
    xs = torch.arange(w, device=DEV, dtype=i64).view(1, 1, 1, w)
    cs = torch.arange(c, device=DEV, dtype=i64).view(1, c, 1, 1)
    ns = torch.arange(n, device=DEV, dtype=i64).view(n, 1, 1, 1)
    v = (xs * 73856093) ^ (ys * 19349663) ^ (cs * 83492791) ^ (ns * 2654435761)
    v = (v * 2246822519 + 3266489917) & 0xFFFFFFFF
    v = (v ^ (v >> 15)) & 0xFFFFFF
    return (v.to(torch.float32) / 16777216.0).to(dtype)


def index_image(n, h, w):
    return torch.arange(h * w, device=DEV, dtype=torch.float32).view(1, 1, h, w).expand(n, 3, h, w).contiguous()


def case_params(name, n, h, w, oh, ow):
    rng = np.random.default_rng(sum(map(ord, name)))
    f = lambda a: np.asarray(a, np.float32)
    return dict(angle=f(rng.uniform(-15, 15, n)), translate=f(np.stack([rng.uniform(-0.1 * w, 0.1 * w, n),
                                                                          rng.uniform(-0.1 * h, 0.1 * h, n)], 1)),
                scale=f(rng.uniform(0.9, 1.1, n)), shear=f(np.stack([rng.uniform(-5, 5, n), np.zeros(n)], 1)),
                top=f(rng.integers(0, h - oh + 1, n)), left=f(rng.integers(0, w - ow + 1, n)),
                flip=(np.arange(n) % 2 == 0), brightness=f(rng.uniform(0.8, 1.2, n)),
                contrast=f(rng.uniform(0.8, 1.2, n)), saturation=f(rng.uniform(0.8, 1.2, n)),
                gray=(np.arange(n) == 1))


def variant_points(name, n, oh, ow):
    """(image, row, column) of the pixels stored per variant of an ALL_VARIANT_CASES case."""
    rng = np.random.default_rng(7 + sum(map(ord, name)))
    return rng.integers(0, n, VARIANT_POINTS), rng.integers(0, oh, VARIANT_POINTS), rng.integers(0, ow, VARIANT_POINTS)


def run(F, img, p, oh, ow, interp, colour, bits=31):
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    kw = dict(angle=t(p["angle"]), translate=t(p["translate"]), scale=t(p["scale"]), shear=t(p["shear"]),
              interpolation=interp, fill=-1.0 if not colour else 0.0)
    if colour:
        if bits & 1: kw.update(brightness_factor=t(p["brightness"]))
        if bits & 2: kw.update(contrast_factor=t(p["contrast"]))
        if bits & 4: kw.update(saturation_factor=t(p["saturation"]))
        if bits & 8: kw.update(grayscale=t(p["gray"]))
        if bits & 16: kw.update(mean=MEAN, std=STD)
    return F.fused_augment(img, t(p["top"]), t(p["left"]), oh, ow, t(p["flip"]), **kw)


def oracle_kwargs(p, bits, dtype):
    kw = {}
    if bits & 1: kw["brightness"] = p["brightness"].astype(dtype)
    if bits & 2: kw["contrast"] = p["contrast"].astype(dtype)
    if bits & 4: kw["saturation"] = p["saturation"].astype(dtype)
    if bits & 8: kw["grayscale"] = p["gray"]
    if bits & 16: kw.update(mean=MEAN, std=STD)
    return kw


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.path.join(ROOT, "baseline", "_ref"))
    ap.add_argument("--out", default=os.path.join(HERE, "gpu_reference_cases.npz"))
    args = ap.parse_args()
    os.environ["TRITON_AUGMENT_SUPPRESS_FIRST_RUN_MESSAGE"] = "1"
    sys.path.insert(0, args.reference)
    sys.path.insert(0, ROOT)
    import triton_augment as ref
    assert ref.__version__ == "0.3.0"
    from oracle import fused_oracle as O
    RF = ref.functional
    out = {"names": np.array([c[0] for c in CASES]), "stride": np.int64(STRIDE)}
    for name, n, h, w, oh, ow, dtype in CASES:
        tdt = getattr(torch, dtype)
        p = case_params(name, n, h, w, oh, ow)
        for k, v in p.items():
            out[f"{name}|{k}"] = np.asarray(v)
        out[f"{name}|shape"] = np.array([n, h, w, oh, ow])
        out[f"{name}|dtype"] = np.array(dtype)
        matrix = RF._prepare_affine_matrix_only(n, DEV, h, w, *(torch.from_numpy(p[k]).to(DEV) for k in
                                                                ("angle", "translate", "scale", "shear")), None)
        out[f"{name}|matrix"] = matrix.cpu().numpy()
        # geometry: which texel does nearest sampling read?
        idx_out = run(RF, index_image(n, h, w), p, oh, ow, "nearest", colour=False)[:, 0].cpu().numpy().astype(np.int32)
        out[f"{name}|nearest_index_sha256"] = np.array(hashlib.sha256(idx_out.tobytes()).hexdigest())
        for fma in (1, 0):
            _, want = O.fused_augment(index_image(n, h, w).cpu().numpy(), p["top"], p["left"], oh, ow, p["flip"],
                                      matrix=out[f"{name}|matrix"], fill=-1.0, want_index=True, fma_coords=bool(fma))
            print(f"{name}: oracle(fma_coords={fma}) vs GPU reference, nearest indices: "
                  f"{int((want != idx_out).sum())} of {idx_out.size} differ")
        img = procedural_image(n, 3, h, w, tdt)
        stride = STRIDES.get(name, STRIDE)
        out[f"{name}|stride"] = np.int64(stride)
        for interp in ("nearest", "bilinear"):
            for bits in (31,) + (EXTRA_FLAGS.get(name, ()) if interp == "bilinear" else ()):
                res = run(RF, img, p, oh, ow, interp, colour=True, bits=bits)
                key = f"{name}|{interp}_sub" + ("" if bits == 31 else f"_flags{bits}")
                out[key] = res[:, :, ::stride, ::stride].cpu().numpy()
                want = O.fused_augment(img.cpu().numpy(), p["top"], p["left"], oh, ow, p["flip"], matrix=out[f"{name}|matrix"],
                                       interpolation=interp, **oracle_kwargs(p, bits, dtype))   # default: the measured GPU recipe
                d = np.abs(res.cpu().numpy().astype(np.float32) - want.astype(np.float32))
                print(f"{name}: oracle vs GPU reference, {interp} flags {bits}: max |diff| {d.max():.3e}, "
                      f"{int((d > 1e-5).sum())} of {d.size} above 1e-5")
        if name in ALL_VARIANT_CASES:
            pn, py, px = (torch.from_numpy(v).to(DEV) for v in variant_points(name, n, oh, ow))
            worst = 0.0
            for interp in ("nearest", "bilinear"):
                vals = []
                for bits in range(32):
                    res = run(RF, img, p, oh, ow, interp, colour=True, bits=bits)
                    vals.append(res[pn, :, py, px].cpu().numpy())                 # [points, 3]
                    want = O.fused_augment(img.cpu().numpy(), p["top"], p["left"], oh, ow, p["flip"],
                                           matrix=out[f"{name}|matrix"], interpolation=interp, **oracle_kwargs(p, bits, dtype))
                    worst = max(worst, float(np.abs(res.cpu().numpy() - want).max()))
                out[f"{name}|{interp}_variants"] = np.stack(vals)                 # [32, points, 3]
            print(f"{name}: oracle vs GPU reference over all 64 fp32 variants: max |diff| {worst:.3e}")
    np.savez_compressed(args.out, **out)
    print("wrote", args.out, os.path.getsize(args.out) // 1024, "KiB")

    # timing of the reference's own fused call on the headline configuration (kernel + its host code)
    tr = ref.TritonFusedAugment(crop_size=1024, horizontal_flip_p=0.5, degrees=15, translate=(0.1, 0.1), scale=(0.9, 1.1),
                                shear=5, brightness=0.2, contrast=0.2, saturation=0.2, grayscale_p=0.1, mean=MEAN, std=STD)
    big = torch.rand(64, 3, 1280, 1280, device=DEV)
    for interp in ("nearest", "bilinear"):
        tr.interpolation = interp
        for _ in range(5):
            tr(big)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(20):
            tr(big)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / 20
        print(f"reference TritonFusedAugment.forward, 64x3x1280x1280 -> 1024, {interp}: {ms:.3f} ms per call "
              f"({64 / ms * 1e3:.0f} images/s, {2 * 64 * 3 * 1024 * 1024 * 4 / ms / 1e6:.0f} GB/s algorithmic)")


if __name__ == "__main__":
    main()
