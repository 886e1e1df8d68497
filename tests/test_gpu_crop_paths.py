"""Calls without a matrix (crop / flip / colour) can run through the crop kernels or through the
staged kernel; large fp32 batches pick the latter.  Both must give the same bits, and plain
crop + flip must equal tensor indexing exactly.  Also: the CUDA-graph wrapper."""
import numpy as np
import pytest
import torch

from conftest import MEAN, STD

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda:0")


@pytest.fixture
def crop_path():
    from triton_augment_b200 import _lib
    yield _lib.crop_path
    _lib.crop_path(0)


def _launch(img, top, left, flip, oh, ow, flags=0, colour=None, checked=False):
    from triton_augment_b200 import _lib
    dev = img.device
    n, c = img.shape[:2]
    out = torch.empty(n, c, oh, ow, dtype=img.dtype, device=dev)
    b, cf, s, g = colour if colour is not None else (None, None, None, None)
    norm = bool(flags & 16)
    p = _lib.make_params(img, out, top, left, flip, None, 0.0, False, flags, b, cf, s, g,
                         MEAN if norm else None, STD if norm else None)
    _lib.launch_fused(p, dev, checked=checked)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("channels", [1, 3])
def test_staged_crop_flip_equals_indexing(crop_path, channels):
    """Pure data movement: every output element is one input element (or 0 outside the image)."""
    from triton_augment_b200 import _lib
    dev = _dev()
    g = torch.Generator(device="cpu").manual_seed(5)
    for (n, h, w, oh, ow) in [(3, 200, 256, 150, 192), (2, 97, 132, 97, 132), (4, 64, 64, 33, 61), (2, 300, 512, 260, 330)]:
        img = torch.rand(n, channels, h, w, generator=g).to(dev)
        top = torch.randint(0, h - oh + 1, (n,), generator=g).float()
        left = torch.randint(0, w - ow + 1, (n,), generator=g).float()
        flip = torch.rand(n, generator=g) < 0.5
        want = torch.stack([
            (img[i, :, int(top[i]):int(top[i]) + oh, int(left[i]):int(left[i]) + ow].flip(-1) if flip[i]
             else img[i, :, int(top[i]):int(top[i]) + oh, int(left[i]):int(left[i]) + ow]) for i in range(n)])
        _lib.debug_counters(reset=True)
        crop_path(2)
        got = _launch(img, top.to(dev), left.to(dev), flip.to(dev).to(torch.uint8), oh, ow, checked=True)
        staged, direct, violations, timeouts = _lib.debug_counters()
        assert torch.equal(got, want), (n, h, w, oh, ow)
        assert violations == 0 and timeouts == 0 and staged > 0 and direct == 0


def test_staged_crop_window_outside_the_image_reads_zero(crop_path):
    dev = _dev()
    img = torch.rand(2, 3, 96, 128, device=dev) + 1.0
    top = torch.tensor([-7.0, 40.0], device=dev)
    left = torch.tensor([-12.0, 60.0], device=dev)
    flip = torch.tensor([0, 1], device=dev, dtype=torch.uint8)
    outs = []
    for path in (1, 2):
        crop_path(path)
        outs.append(_launch(img, top, left, flip, 80, 100))
    assert torch.equal(outs[0], outs[1])
    assert float(outs[1][0, :, :7].abs().max()) == 0.0 and float(outs[1][0, :, :, :12].abs().max()) == 0.0
    assert float(outs[1][1, :, 56:].abs().max()) == 0.0


def test_every_flag_combination_same_bits_on_both_paths(crop_path):
    dev = _dev()
    g = torch.Generator(device="cpu").manual_seed(11)
    n, h, w, oh, ow = 4, 160, 224, 130, 200
    img = torch.rand(n, 3, h, w, generator=g).to(dev)
    top = torch.randint(0, h - oh + 1, (n,), generator=g).float().to(dev)
    left = torch.randint(0, w - ow + 1, (n,), generator=g).float().to(dev)
    flip = (torch.rand(n, generator=g) < 0.5).to(torch.uint8).to(dev)
    colour = tuple((torch.rand(n, generator=g) * 0.8 + 0.6).to(dev) for _ in range(3)) + (
        (torch.rand(n, generator=g) < 0.5).to(torch.uint8).to(dev),)
    for flags in range(32):
        outs = []
        for path in (1, 2):
            crop_path(path)
            outs.append(_launch(img, top, left, flip, oh, ow, flags=flags, colour=colour))
        assert torch.equal(outs[0], outs[1]), flags


def test_large_fp32_batches_choose_the_staged_kernel(crop_path):
    from triton_augment_b200 import _lib
    dev = _dev()
    crop_path(0)
    img = torch.rand(16, 3, 768, 768, device=dev)
    top = torch.full((16,), 17.0, device=dev)
    left = torch.full((16,), 33.0, device=dev)
    flip = torch.zeros(16, dtype=torch.uint8, device=dev)
    _lib.debug_counters(reset=True)
    got = _launch(img, top, left, flip, 704, 704)          # 95 MB of output, 704 columns
    staged = _lib.debug_counters()[0]
    assert staged == 16 * -(-704 // 64) * -(-704 // 32)       # (matrix-free float calls use the 64 x 32 tile shape)
    assert torch.equal(got, img[:, :, 17:17 + 704, 33:33 + 704])
    _lib.debug_counters(reset=True)
    _launch(img[:1], top[:1], left[:1], flip[:1], 704, 704)  # small: the crop kernels
    assert _lib.debug_counters()[0] == 0


def test_graphed_transform_replays_the_eager_sequence():
    """One captured call replayed three times draws the same parameters as three eager calls
    from the same seed, and gives a new result on every replay."""
    import triton_augment_b200 as ta
    dev = _dev()
    aug = ta.TritonFusedAugment(crop_size=96, horizontal_flip_p=0.5, degrees=15, translate=(0.1, 0.1), scale=(0.9, 1.1),
                                shear=5, interpolation="bilinear", brightness=0.2, contrast=0.2, saturation=0.2,
                                grayscale_p=0.2, mean=MEAN, std=STD)
    img = torch.rand(8, 3, 128, 128, device=dev)
    graphed = ta.GraphedTransform(aug, img, warmup=2)
    torch.manual_seed(99)
    eager = [aug(img).clone() for _ in range(3)]
    torch.manual_seed(99)
    replayed = []
    for _ in range(3):
        out = graphed()
        torch.cuda.synchronize()
        replayed.append(out.clone())
    assert not torch.equal(replayed[0], replayed[1])
    for a, b in zip(eager, replayed):
        assert torch.equal(a, b)
    other = torch.rand(8, 3, 128, 128, device=dev)
    torch.manual_seed(3)
    want = aug(other).clone()
    torch.manual_seed(3)
    assert torch.equal(graphed(other), want)
    with pytest.raises(ValueError):
        graphed(torch.rand(4, 3, 128, 128, device=dev))
