"""Generate the golden fixtures in this directory from the reference itself.

Run once, in a container that has the reference checked out, e.g.

    python tests/golden/make_golden.py --reference <checkout of triton-augment v0.3.0>

The reference (yuhezhang-ai/triton-augment v0.3.0) only has GPU kernels, so the
script executes its *unmodified* Python + Triton code on CPU tensors under
Triton's interpreter (TRITON_INTERPRET=1).  Two harness-side shims make that
possible; neither changes what the reference computes:

* the interpreter has no libdevice, so ``libdevice.rint`` is replaced by numpy's
  ``rint`` (same round-half-to-even rule);
* inputs are wrapped in a ``torch.Tensor`` subclass whose ``is_cuda`` reads True,
  so the reference's "must be on CUDA" checks pass while the data stays on the
  CPU.

Because numpy never contracts a*b+c into an fma, coordinates in these vectors
follow the unfused recipe (oracle ``fma_coords=0``).

Outputs (all small, committed):
  fused_cases.npz      functional.fused_augment: inputs, per-image parameters, outputs
  functional_cases.npz the stand-alone functionals (crop, flip, affine, rotate, colour ops)
  class_cases.npz      transform classes under torch.manual_seed on the CPU generator:
                       sampled parameters and forward outputs for 3D/4D/5D inputs
"""
from __future__ import annotations

import argparse
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
os.environ["TRITON_AUGMENT_SUPPRESS_FIRST_RUN_MESSAGE"] = "1"

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
MEAN = (0.485, 0.456, 0.406)
STD = (0.229, 0.224, 0.225)


def load_reference(path):
    sys.path.insert(0, path)
    import triton.language as tl
    from triton.language.extra.cuda import libdevice
    from triton.runtime.interpreter import TensorHandle

    def _rint(x, _semantic=None):
        return tl.tensor(TensorHandle(np.rint(x.handle.data), x.dtype.scalar), x.type)

    libdevice.rint = _rint
    import triton_augment as ta
    assert ta.__version__ == "0.3.0", ta.__version__
    return ta


class _FakeCuda(torch.Tensor):
    is_cuda = property(lambda self: True)


def fake(t):
    return torch.Tensor._make_subclass(_FakeCuda, t.contiguous())


def pixels(rng, shape, dtype=np.float32):
    return rng.random(shape, dtype=np.float32).astype(dtype)


def np_(t):
    return torch.as_tensor(t).detach().cpu().numpy()


# --------------------------------------------------------------------------- fused_augment
def fused_cases(ta):
    F = ta.functional
    rng = np.random.default_rng(20251125)
    cases = []

    def add(name, shape, oh, ow, *, dtype=np.float32, affine=None, interp="nearest", fill=0.0,
            crop=True, flip=True, b=None, c=None, s=None, g=None, norm=True, scalar_params=False,
            out_of_range_pixels=False):
        n, ch, h, w = shape
        img = pixels(rng, shape, dtype)
        if out_of_range_pixels:
            img = (img * 3.0 - 1.0).astype(dtype)
        top = rng.integers(0, h - oh + 1, n).astype(np.int32) if crop else np.zeros(n, np.int32)
        left = rng.integers(0, w - ow + 1, n).astype(np.int32) if crop else np.zeros(n, np.int32)
        fl = (rng.random(n) < 0.5) if flip else np.zeros(n, bool)
        if flip and n > 1:
            fl[0], fl[1] = True, False
        kw = {}
        if affine is not None:
            deg, tr, sc, sh = affine
            kw["angle"] = torch.tensor(rng.uniform(-deg, deg, n), dtype=torch.float32)
            kw["translate"] = torch.tensor(np.stack([rng.uniform(-tr * w, tr * w, n),
                                                     rng.uniform(-tr * h, tr * h, n)], 1), dtype=torch.float32)
            kw["scale"] = torch.tensor(rng.uniform(sc[0], sc[1], n), dtype=torch.float32)
            kw["shear"] = torch.tensor(np.stack([rng.uniform(-sh, sh, n), rng.uniform(-sh / 2, sh / 2, n)], 1),
                                       dtype=torch.float32)
            kw["interpolation"] = interp
            kw["fill"] = fill
        def factor(r):
            if r is None:
                return 1.0
            if scalar_params:
                return float(np.float32(rng.uniform(*r)))
            return torch.tensor(rng.uniform(r[0], r[1], n), dtype=torch.float32)
        bf, cf, sf = factor(b), factor(c), factor(s)
        gm = False if g is None else torch.tensor(rng.random(n) < g)
        if g is not None and n > 1:
            gm[0], gm[-1] = True, False
        out = F.fused_augment(
            fake(torch.from_numpy(img)),
            top=torch.from_numpy(top), left=torch.from_numpy(left), height=oh, width=ow,
            flip_horizontal=torch.from_numpy(fl),
            brightness_factor=bf, contrast_factor=cf, saturation_factor=sf, grayscale=gm,
            mean=MEAN if norm else None, std=STD if norm else None, **kw)
        rec = dict(name=name, image=img, top=top, left=left, flip=fl.astype(np.uint8), oh=oh, ow=ow,
                   brightness=np.float32(np_(bf)), contrast=np.float32(np_(cf)), saturation=np.float32(np_(sf)),
                   gray=np.uint8(np_(gm)), norm=norm, interp=interp, fill=np.float32(fill), out=np_(out))
        if affine is not None:
            rec.update(angle=np_(kw["angle"]), translate=np_(kw["translate"]), scale=np_(kw["scale"]),
                       shear=np_(kw["shear"]))
            mat = F._prepare_affine_matrix_only(n, torch.device("cpu"), h, w, kw["angle"], kw["translate"],
                                                kw["scale"], kw["shear"], None)
            rec["matrix"] = np_(mat)
        cases.append(rec)

    J = (0.8, 1.2)
    AFF = (15.0, 0.1, (0.9, 1.1), 5.0)
    # colour + grayscale + normalize, no geometry (first benchmark configuration in miniature)
    add("colour_all_32x32", (4, 3, 32, 32), 32, 32, crop=False, flip=False, b=J, c=J, s=J, g=0.3)
    add("colour_all_odd", (3, 3, 17, 23), 17, 23, crop=False, flip=False, b=J, c=J, s=J, g=0.3)
    add("colour_no_norm", (2, 3, 8, 8), 8, 8, crop=False, flip=False, b=J, c=J, s=J, g=0.5, norm=False)
    add("colour_scalar_factors", (2, 3, 9, 11), 9, 11, crop=False, flip=False, b=J, c=J, s=J, scalar_params=True)
    add("colour_unclamped_input", (2, 3, 12, 12), 12, 12, crop=False, flip=False, b=J, c=J, s=J, g=0.5,
        out_of_range_pixels=True)
    add("one_pixel", (2, 3, 1, 1), 1, 1, crop=False, flip=False, b=J, s=J)
    for nm, kw in [("only_b", dict(b=J)), ("only_c", dict(c=J)), ("only_s", dict(s=J)), ("only_g", dict(g=0.5)),
                   ("b_s", dict(b=J, s=J)), ("c_g", dict(c=J, g=0.5)), ("none", dict())]:
        add(f"flags_{nm}", (3, 3, 10, 12), 7, 9, norm=(nm != "none"), **kw)
    # crop + flip (+ colour): second configuration in miniature, odd and prime sizes
    add("crop_flip_colour", (6, 3, 40, 44), 20, 24, b=J, c=J, s=J, g=0.2)
    add("crop_flip_prime", (3, 3, 31, 37), 13, 29, b=J, s=J)
    add("crop_flip_only", (4, 3, 16, 15), 8, 7, norm=False)
    add("linear_path_rgb", (3, 3, 20, 18), 11, 10, b=J, c=J)
    add("linear_path_gray1", (3, 1, 20, 18), 11, 10, b=J, c=J, norm=False)
    # affine, nearest and bilinear: third configuration in miniature
    for interp in ("nearest", "bilinear"):
        add(f"affine_{interp}_all", (4, 3, 48, 56), 32, 40, affine=AFF, interp=interp, b=J, c=J, s=J, g=0.3)
        add(f"affine_{interp}_plain", (3, 3, 33, 29), 21, 17, affine=AFF, interp=interp, norm=False)
        add(f"affine_{interp}_fill", (2, 3, 24, 24), 24, 24, affine=(40.0, 0.3, (0.5, 0.8), 20.0), interp=interp,
            fill=0.5, crop=False, b=J)
        add(f"affine_{interp}_zoom", (2, 3, 20, 28), 20, 28, affine=(90.0, 0.0, (1.5, 2.5), 0.0), interp=interp,
            crop=False, flip=False, norm=False)
        add(f"affine_{interp}_gray1", (2, 1, 19, 23), 10, 12, affine=AFF, interp=interp, b=J, norm=False)
    # fp16: fourth configuration in miniature, one case per precision state of the colour tier
    H = np.float16
    add("f16_affine_nearest_all", (4, 3, 40, 48), 28, 32, dtype=H, affine=AFF, b=J, c=J, s=J, g=0.3)
    add("f16_affine_bilinear_all", (3, 3, 40, 48), 28, 32, dtype=H, affine=AFF, interp="bilinear", b=J, c=J, s=J, g=0.3)
    add("f16_colour_all", (3, 3, 16, 16), 16, 16, dtype=H, crop=False, flip=False, b=J, c=J, s=J, g=0.5)
    add("f16_only_c", (2, 3, 12, 10), 8, 6, dtype=H, c=J)
    add("f16_only_s", (2, 3, 12, 10), 8, 6, dtype=H, s=J)
    add("f16_only_g", (2, 3, 12, 10), 8, 6, dtype=H, g=0.5)
    add("f16_only_norm", (2, 3, 12, 10), 8, 6, dtype=H)
    add("f16_crop_flip_only", (2, 3, 12, 10), 8, 6, dtype=H, norm=False)
    return cases


# --------------------------------------------------------------------------- stand-alone functionals
def functional_cases(ta):
    F = ta.functional
    rng = np.random.default_rng(7)
    out = {}
    img = pixels(rng, (3, 3, 18, 22))
    t = fake(torch.from_numpy(img))
    out["image"] = img
    out["brightness_1.3"] = np_(F.adjust_brightness(t, 1.3))
    out["contrast_1.4"] = np_(F.adjust_contrast(t, 1.4))
    out["contrast_0.6"] = np_(F.adjust_contrast(t, 0.6))
    out["contrast_fast_1.4"] = np_(F.adjust_contrast_fast(t, 1.4))
    out["saturation_0.3"] = np_(F.adjust_saturation(t, 0.3))
    out["saturation_1.7"] = np_(F.adjust_saturation(t, 1.7))
    out["normalize"] = np_(F.normalize(t, MEAN, STD))
    out["gray3"] = np_(F.rgb_to_grayscale(t, 3))
    out["gray1"] = np_(F.rgb_to_grayscale(t, 1))
    mask = torch.tensor([True, False, True])
    out["gray3_masked"] = np_(F.rgb_to_grayscale(t, 3, mask))
    out["crop_2_3_9_11"] = np_(F.crop(t, 2, 3, 9, 11))
    tops = torch.tensor([0, 4, 9], dtype=torch.int32)
    lefts = torch.tensor([11, 0, 5], dtype=torch.int32)
    out["crop_per_image"] = np_(F.crop(t, tops, lefts, 9, 11))
    out["crop_tops"], out["crop_lefts"] = np_(tops), np_(lefts)
    out["center_crop_10_8"] = np_(F.center_crop(t, (10, 8)))
    out["hflip"] = np_(F.horizontal_flip(t))
    out["hflip_masked"] = np_(F.horizontal_flip(t, mask))
    out["affine_nearest"] = np_(F.affine(t, 20.0, [2.0, -1.5], 1.1, [5.0, 2.0], "nearest"))
    out["affine_bilinear"] = np_(F.affine(t, 20.0, [2.0, -1.5], 1.1, [5.0, 2.0], "bilinear", fill=0.25))
    out["affine_center"] = np_(F.affine(t, -12.0, [0.0, 0.0], 1.0, [0.0, 0.0], "bilinear", center=[4.0, 6.0]))
    angles = torch.tensor([10.0, -35.0, 90.0])
    out["rotate_per_image"] = np_(F.rotate(t, angles, "bilinear"))
    out["rotate_angles"] = np_(angles)
    out["rotate_30_nearest"] = np_(F.rotate(t, 30.0))
    gray = pixels(rng, (2, 1, 9, 7))
    out["gray_image"] = gray
    out["gray_contrast_1.5"] = np_(F.adjust_contrast(fake(torch.from_numpy(gray)), 1.5))
    half = img.astype(np.float16)
    th = fake(torch.from_numpy(half))
    out["f16_contrast_1.4"] = np_(F.adjust_contrast(th, 1.4))
    out["f16_normalize"] = np_(F.normalize(th, MEAN, STD))
    out["f16_saturation_0.3"] = np_(F.adjust_saturation(th, 0.3))
    out["f16_brightness_1.3"] = np_(F.adjust_brightness(th, 1.3))
    # inverse-matrix table: reference torch ops on the CPU
    n = 16
    ang = torch.tensor(rng.uniform(-180, 180, n), dtype=torch.float32)
    tr = torch.tensor(rng.uniform(-50, 50, (n, 2)), dtype=torch.float32)
    sc = torch.tensor(rng.uniform(0.5, 2.0, n), dtype=torch.float32)
    sh = torch.tensor(rng.uniform(-30, 30, (n, 2)), dtype=torch.float32)
    ce = torch.tensor(rng.uniform(-20, 20, (n, 2)), dtype=torch.float32)
    out["mat_angle"], out["mat_translate"], out["mat_scale"] = np_(ang), np_(tr), np_(sc)
    out["mat_shear"], out["mat_center"] = np_(sh), np_(ce)
    out["mat_out"] = np_(F._get_inverse_affine_matrix(ce, ang, tr, sc, sh))
    return out


# --------------------------------------------------------------------------- transform classes
CLASS_SPECS = {
    "fused_full": ("TritonFusedAugment", dict(crop_size=(12, 16), horizontal_flip_p=0.5, degrees=15,
                                               translate=(0.1, 0.1), scale=(0.9, 1.1), shear=5,
                                               interpolation="bilinear", brightness=0.2, contrast=0.2,
                                               saturation=0.2, grayscale_p=0.3, mean=MEAN, std=STD)),
    "fused_no_affine": ("TritonFusedAugment", dict(crop_size=10, horizontal_flip_p=0.5, brightness=0.2,
                                                    saturation=0.2, grayscale_p=0.2, mean=MEAN, std=STD)),
    "fused_rot_only": ("TritonFusedAugment", dict(degrees=(-30, 10), contrast=(0.5, 1.5))),
    "fused_shear4": ("TritonFusedAugment", dict(crop_size=8, shear=(-5, 5, -3, 3), scale=(0.8, 1.2),
                                                 horizontal_flip_p=1.0, fill=0.5)),
    "colour_jitter_norm": ("TritonColorJitterNormalize", dict(brightness=0.2, contrast=0.2, saturation=0.2,
                                                               grayscale_p=0.1, mean=MEAN, std=STD)),
    "colour_jitter": ("TritonColorJitter", dict(brightness=(0.5, 1.5), saturation=0.4)),
    "crop_flip": ("TritonRandomCropFlip", dict(size=(9, 13), horizontal_flip_p=0.5)),
    "random_crop": ("TritonRandomCrop", dict(size=7)),
    "random_flip": ("TritonRandomHorizontalFlip", dict(p=0.5)),
    "random_gray": ("TritonRandomGrayscale", dict(p=0.5)),
    "random_affine": ("TritonRandomAffine", dict(degrees=20, translate=(0.1, 0.2), scale=(0.8, 1.2), shear=10,
                                                  interpolation="bilinear")),
    "random_rotation": ("TritonRandomRotation", dict(degrees=45)),
}


def class_cases(ta):
    rng = np.random.default_rng(99)
    out = {}
    shapes = {"3d": (3, 20, 24), "4d": (5, 3, 20, 24), "5d": (2, 3, 3, 20, 24)}
    imgs = {k: pixels(rng, s) for k, s in shapes.items()}
    for k, v in imgs.items():
        out[f"image_{k}"] = v
    seed = 1000
    for key, (cls_name, kwargs) in CLASS_SPECS.items():
        for rank in ("3d", "4d", "5d"):
            for sob, sof in ((False, True), (True, True), (False, False), (True, False)):
                if rank != "5d" and not sof:
                    continue
                if rank == "3d" and sob:
                    continue
                seed += 1
                kw = dict(kwargs)
                kw.update(same_on_batch=sob, same_on_frame=sof)
                tr = getattr(ta, cls_name)(**kw)
                torch.manual_seed(seed)
                res = tr(fake(torch.from_numpy(imgs[rank])))
                tag = f"{key}|{rank}|{int(sob)}{int(sof)}"
                out[f"{tag}|seed"] = np.int64(seed)
                out[f"{tag}|out"] = np_(res)
    # sampled parameters alone (RNG consumption order), 7 parameter sets, 20x24 image
    for key, (cls_name, kwargs) in CLASS_SPECS.items():
        tr = getattr(ta, cls_name)(**kwargs)
        if not hasattr(tr, "_get_params"):
            continue
        seed += 1
        torch.manual_seed(seed)
        try:
            params = tr._get_params(7, torch.device("cpu"), (20, 24))
        except TypeError:
            params = tr._get_params(7, torch.device("cpu"))
        out[f"params|{key}|seed"] = np.int64(seed)
        for i, p in enumerate(params):
            out[f"params|{key}|{i}"] = np_(p)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of an unmodified triton-augment v0.3.0 checkout")
    args = ap.parse_args()
    ta = load_reference(args.reference)

    cases = fused_cases(ta)
    flat = {"names": np.array([c["name"] for c in cases])}
    for c in cases:
        for k, v in c.items():
            if k != "name":
                flat[f"{c['name']}|{k}"] = np.asarray(v)
    np.savez_compressed(os.path.join(HERE, "fused_cases.npz"), **flat)
    np.savez_compressed(os.path.join(HERE, "functional_cases.npz"), **functional_cases(ta))
    np.savez_compressed(os.path.join(HERE, "class_cases.npz"), **class_cases(ta))
    for f in ("fused_cases.npz", "functional_cases.npz", "class_cases.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)) // 1024, "KiB")


if __name__ == "__main__":
    main()
