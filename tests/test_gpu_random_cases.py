"""Randomised parity: shapes, crop windows, affine parameters, colour flags, dtypes and sampling
modes drawn from a seeded generator, each case checked against the CPU oracle (float32 <= 1e-5,
float16 <= 1e-2; uint8 input against the oracle on image / 255).  Ranges go well beyond the
benchmark's: rotations up to +-180 degrees, scales 0.3 .. 3, windows partly off the image,
non-zero fill, widths that cannot be staged."""
import numpy as np
import pytest
import torch

from conftest import MEAN, STD
from oracle import fused_oracle as O

pytestmark = pytest.mark.gpu


def run_cases(seed, count, big=False, channels=(3,)):
    import triton_augment_b200 as ta
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(seed)
    worst = {}
    for case in range(count):
        kind = ["f32", "f16", "u8", "u8h"][int(rng.integers(0, 4))]
        interp = ["none", "nearest", "bilinear"][int(rng.integers(0, 3))]
        n = int(rng.integers(1, 3 if big else 5))
        ch = int(rng.choice(channels))
        h, w = (int(rng.integers(300, 1300)), int(rng.integers(300, 1300))) if big else \
               (int(rng.integers(20, 300)), int(rng.integers(20, 400)))
        if rng.random() < 0.6:
            w = (w + 15) // 16 * 16                          # rows that can be staged, for every dtype
        oh, ow = int(rng.integers(1, h + 1)), int(rng.integers(1, w + 1))
        wild = rng.random() < 0.3
        top = rng.integers(-10 if wild else 0, (h - oh + 1) + (10 if wild else 0), n).astype(np.float32)
        left = rng.integers(-10 if wild else 0, (w - ow + 1) + (10 if wild else 0), n).astype(np.float32)
        flip = rng.random(n) < 0.5
        amax = 180.0 if wild else 20.0
        angle = rng.uniform(-amax, amax, n).astype(np.float32)
        translate = np.stack([rng.uniform(-0.3 * w, 0.3 * w, n), rng.uniform(-0.3 * h, 0.3 * h, n)], 1).astype(np.float32)
        scale = rng.uniform(0.3 if wild else 0.8, 3.0 if wild else 1.25, n).astype(np.float32)
        shear = rng.uniform(-20 if wild else -5, 20 if wild else 5, (n, 2)).astype(np.float32)
        fill = float(rng.choice([0.0, 0.0, 0.5, -1.0]))
        bits = int(rng.integers(0, 32)) & (31 if ch == 3 else 19)       # one channel: no saturation, no grayscale
        bytes_in = kind in ("u8", "u8h")
        half = kind in ("f16", "u8h")
        fdt = np.float16 if half else np.float32
        if bytes_in:
            raw = rng.integers(0, 256, (n, ch, h, w), dtype=np.uint8)
            scaled = raw.astype(np.float32) * np.float32(1.0 / 255.0)
            ref_img = scaled.astype(np.float16) if half else scaled
            img = raw
        else:
            img = rng.random((n, ch, h, w), dtype=np.float32).astype(fdt)
            ref_img = img
        b = rng.uniform(0.6, 1.4, n).astype(np.float32) if bits & 1 else np.ones(n, np.float32)
        c = rng.uniform(0.6, 1.4, n).astype(np.float32) if bits & 2 else np.ones(n, np.float32)
        s = rng.uniform(0.0, 2.0, n).astype(np.float32) if bits & 4 else np.ones(n, np.float32)
        g = (rng.random(n) < 0.5) if bits & 8 else np.zeros(n, bool)
        norm = bool(bits & 16)
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
        akw, matrix = {}, None
        if interp != "none":
            akw = dict(angle=t(angle), translate=t(translate), scale=t(scale), shear=t(shear), interpolation=interp, fill=fill)
            matrix = ta.functional._prepare_affine_matrix_only(n, dev, h, w, t(angle), t(translate), t(scale), t(shear),
                                                               None).cpu().numpy()
        got = ta.fused_augment(t(img), t(top), t(left), oh, ow, t(flip), brightness_factor=t(b), contrast_factor=t(c),
                               saturation_factor=t(s), grayscale=t(g), mean=MEAN if norm else None,
                               std=STD if norm else None, out_dtype=torch.float16 if kind == "u8h" else None, **akw)
        assert got.dtype == (torch.float16 if half else torch.float32)
        got = got.float().cpu().numpy()
        want = O.fused_augment(ref_img, top, left, oh, ow, flip, matrix=matrix,
                               interpolation=interp if interp != "none" else "nearest", fill=fill if matrix is not None else 0.0,
                               brightness=b.astype(fdt), contrast=c.astype(fdt), saturation=s.astype(fdt), grayscale=g,
                               mean=MEAN if norm else None, std=STD if norm else None).astype(np.float32)
        tol = 1e-2 if half else 1e-5
        diff = np.abs(got - want)
        if interp == "bilinear" and bytes_in:
            # bytes are blended raw and scaled once; the oracle blends scaled (for float16: rounded)
            # taps - the same value up to the rounding of the taps
            tol = 2e-2 if half else 2e-5
        err = float(diff.max()) if diff.size else 0.0
        # a source coordinate within float32 rounding of a texel boundary may pick the neighbour:
        # allowed for a handful of pixels per case, never as a pattern
        bad = int((diff > tol).sum())
        allowed = 0 if interp != "nearest" else max(2, diff.size // 20000)
        key = (kind, interp)
        worst[key] = max(worst.get(key, 0.0), err if bad == 0 else 0.0)
        assert bad <= allowed, (case, kind, interp, (n, ch, h, w, oh, ow), bits, wild, err, bad)
    return worst


def test_random_cases():
    run_cases(2024, 120)


def test_random_cases_large_images_and_single_channel():
    run_cases(2025, 24, big=True)
    run_cases(2026, 40, channels=(1,))


def test_random_transforms_agree_across_entry_points():
    """TritonFusedAugment on random image and video batches: the host-buffer call and the sharded
    wrapper (three shards on one GPU) give the bits of the plain forward for the same seed."""
    import triton_augment_b200 as ta
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(5)
    for case in range(60):
        dtype = [torch.float32, torch.float16, torch.uint8][int(rng.integers(0, 3))]
        video = rng.random() < 0.4
        n, t = int(rng.integers(1, 12)), int(rng.integers(1, 5))
        h, w = int(rng.integers(24, 200)), int(rng.integers(24, 260))
        if rng.random() < 0.5:
            w = (w + 15) // 16 * 16
        oh, ow = int(rng.integers(8, h + 1)), int(rng.integers(8, w + 1))
        kw = {}
        if rng.random() < 0.7:
            kw = dict(degrees=float(rng.choice([5, 15, 90])), translate=(0.1, 0.1), scale=(0.8, 1.2),
                      shear=float(rng.uniform(0, 10)), interpolation=str(rng.choice(["nearest", "bilinear"])),
                      fill=float(rng.choice([0.0, 0.3])))
        colour = dict(brightness=0.2, contrast=0.2, saturation=0.2, grayscale_p=0.3, mean=MEAN, std=STD) \
            if rng.random() < 0.7 else {}
        exact = bool(colour) and rng.random() < 0.3 and not (dtype == torch.uint8 and w % 16)
        aug = ta.TritonFusedAugment(crop_size=(oh, ow), horizontal_flip_p=0.5,
                                    contrast_mode="torchvision" if exact else "fast", fast_rng=bool(rng.random() < 0.5),
                                    same_on_batch=bool(rng.random() < 0.2), same_on_frame=bool(rng.random() < 0.6),
                                    **kw, **colour)
        shape = (n, t, 3, h, w) if video else (n, 3, h, w)
        g = torch.Generator().manual_seed(case)
        x = (torch.randint(0, 256, shape, generator=g, dtype=torch.uint8) if dtype == torch.uint8
             else torch.rand(shape, generator=g).to(dtype))
        torch.manual_seed(case); want = aug(x.to(dev))
        torch.manual_seed(case); host = aug.forward_host(x.pin_memory(), device=dev)
        assert host.equal(want.cpu()), (case, dtype, shape, (oh, ow), kw)
        if not aug.fast_rng:
            torch.manual_seed(case); got = ta.ShardedAugment(aug, [0, 0, 0])(x.to(dev), gather_to=dev)
            assert got.equal(want), (case, dtype, shape, (oh, ow), kw)
