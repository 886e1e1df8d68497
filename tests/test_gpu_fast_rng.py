"""fast_rng=True: every parameter of a TritonFusedAugment call from ONE sampler launch (the
library's own Philox stream) instead of ~18 torch draws.  Same distributions, same kernel;
checked here: ranges and frequencies of the draws, the matrix against the torch formula on the
same draws, frame / batch sharing for videos, repeatability under torch.manual_seed, and that
the image result is the fused kernel on exactly those parameters."""
import pytest
import torch

from conftest import MEAN, STD

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _aug(ta, **kw):
    base = dict(crop_size=(40, 48), horizontal_flip_p=0.3, degrees=15, translate=(0.1, 0.2), scale=(0.9, 1.1),
                shear=(-5, 5, -2, 2), interpolation="bilinear", brightness=0.2, contrast=(0.7, 1.4), saturation=0.3,
                grayscale_p=0.25, mean=MEAN, std=STD, fast_rng=True)
    base.update(kw)
    return ta.TritonFusedAugment(**base)


def test_draws_have_the_reference_distributions():
    import triton_augment_b200 as ta
    aug = _aug(ta)
    n, h, w = 20000, 64, 80
    lay = aug._layout(torch.empty(n, 3, h, w, device=DEV))
    torch.manual_seed(1)
    p = aug._sample_fast(lay, torch.float32, want_draws=True)
    torch.cuda.synchronize()
    inside = lambda t, lo, hi: float(t.min()) >= lo and float(t.max()) <= hi
    assert inside(p["angle"], -15, 15) and abs(float(p["angle"].mean())) < 0.3 and float(p["angle"].std()) > 8
    assert inside(p["translate"][:, 0], -8, 8) and inside(p["translate"][:, 1], -12.8, 12.8)
    assert float(p["translate"][:, 1].abs().max()) > 12 and float(p["translate"][:, 0].abs().max()) > 7.5
    assert inside(p["scale"], 0.9, 1.1) and inside(p["shear"][:, 0], -5, 5) and inside(p["shear"][:, 1], -2, 2)
    assert inside(p["brightness"], 0.8, 1.2) and inside(p["contrast"], 0.7, 1.4) and inside(p["saturation"], 0.7, 1.3)
    assert abs(float(p["contrast"].mean()) - 1.05) < 0.01
    for name, span in (("top", h - 40), ("left", w - 48)):
        t = p[name]
        assert torch.equal(t, t.round()) and inside(t, 0, span)
        counts = torch.bincount(t.long(), minlength=span + 1).float()
        assert float(counts.min()) > 0.8 * n / (span + 1) and float(counts.max()) < 1.2 * n / (span + 1)
    assert abs(float(p["flip"].float().mean()) - 0.3) < 0.015 and abs(float(p["gray"].float().mean()) - 0.25) < 0.015
    # independent draws: no correlation between any two of them
    cols = torch.stack([p["angle"], p["translate"][:, 0], p["translate"][:, 1], p["scale"], p["shear"][:, 0], p["top"],
                        p["left"], p["flip"].float(), p["brightness"], p["contrast"], p["saturation"], p["gray"].float()])
    corr = torch.corrcoef(cols) - torch.eye(cols.shape[0], device=DEV)
    assert float(corr.abs().max()) < 0.03
    # the matrix is the reference formula on these draws, bit for bit
    want = ta.functional._prepare_affine_matrix_only(n, DEV, h, w, p["angle"], p["translate"], p["scale"], p["shear"], None)
    assert torch.equal(p["matrix"], want)


def test_sharing_over_frames_and_batch():
    import triton_augment_b200 as ta
    video = torch.empty(5, 7, 3, 64, 80, device=DEV)
    for sob, sof, distinct in ((False, True, 5), (True, False, 7), (False, False, 35), (True, True, 1)):
        aug = _aug(ta, same_on_batch=sob, same_on_frame=sof)
        lay = aug._layout(video)
        p = aug._sample_fast(lay, torch.float32, want_draws=True)
        a = p["angle"].view(5, 7)
        assert len(torch.unique(p["angle"])) == distinct
        if sof:
            assert torch.equal(a, a[:, :1].expand(5, 7))
        if sob:
            assert torch.equal(a, a[:1].expand(5, 7))
        assert p["matrix"][:, 2].unique().numel() <= distinct and p["top"].unique().numel() <= distinct


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.uint8])
def test_result_is_the_fused_kernel_on_the_sampled_parameters(dtype):
    import triton_augment_b200 as ta
    aug = _aug(ta)
    g = torch.Generator().manual_seed(3)
    img = (torch.randint(0, 256, (6, 3, 64, 80), generator=g, dtype=torch.uint8) if dtype == torch.uint8
           else torch.rand(6, 3, 64, 80, generator=g).to(dtype)).to(DEV)
    torch.manual_seed(11)
    out = aug(img)
    torch.manual_seed(11)
    again = aug(img)
    torch.manual_seed(12)
    other = aug(img)
    assert torch.equal(out, again) and not torch.equal(out, other)
    work = torch.float32 if dtype == torch.uint8 else dtype
    assert out.dtype == work and out.shape == (6, 3, 40, 48)
    torch.manual_seed(11)
    p = aug._sample_fast(aug._layout(img), work, want_draws=True)
    want = ta.fused_augment(img, p["top"], p["left"], 40, 48, p["flip"].bool(), angle=p["angle"], translate=p["translate"],
                            scale=p["scale"], shear=p["shear"], interpolation="bilinear", brightness_factor=p["brightness"],
                            contrast_factor=p["contrast"], saturation_factor=p["saturation"], grayscale=p["gray"].bool(),
                            mean=MEAN, std=STD)
    assert torch.equal(out, want)


def test_no_affine_no_crop_video_and_graph_capture():
    import triton_augment_b200 as ta
    aug = ta.TritonFusedAugment(horizontal_flip_p=0.5, brightness=0.2, saturation=0.2, mean=MEAN, std=STD, fast_rng=True)
    video = torch.rand(2, 3, 3, 32, 48, device=DEV)
    out = aug(video)
    assert out.shape == video.shape
    assert torch.equal(out[:, 0] - out[:, 0], torch.zeros_like(out[:, 0]))     # finite
    graphed = ta.GraphedTransform(aug, video)
    torch.manual_seed(5)
    a = graphed().clone()
    b = graphed().clone()
    torch.manual_seed(5)
    c = aug(video)
    assert torch.equal(a, c) and not torch.equal(a, b)
    with pytest.raises(ValueError):
        ta.TritonFusedAugment(crop_size=64, fast_rng=True)(torch.rand(1, 3, 32, 48, device=DEV))
    # the host-buffer entry samples the same way
    full = _aug(ta)
    host = torch.rand(5, 3, 64, 80).pin_memory()
    torch.manual_seed(21)
    want = full(host.to(DEV))
    torch.manual_seed(21)
    got = full.forward_host(host, device=DEV)
    assert torch.equal(got, want.cpu())
