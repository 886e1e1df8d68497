"""All parameters of a forward from ONE launch that reproduces PyTorch's CUDA generator.

The reference draws each parameter with its own `uniform_` / `randint` / `rand` call.  The
sampler kernel's torch_compat mode computes the very same values (Philox4x32-10, counter =
(offset / 4 + draw number, element index), PyTorch's word -> value transformations) and the
generator is advanced by what those calls would have consumed, so seeds keep their meaning.
Checked here: the start-up self-check accepts this PyTorch build; parameters are bit-identical
to `_get_params` for every parameter-set count the task names; whole forwards (4-D, 5-D, every
same_on_* setting, partial configurations) are identical with the feature on and off, leave the
generator at the same offset, and stay identical over several calls and through graph replays."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
MEAN, STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)

CONFIGS = [
    dict(crop_size=96, horizontal_flip_p=0.5, degrees=15, translate=(0.1, 0.2), scale=(0.9, 1.1), shear=5,
         interpolation="bilinear", brightness=0.2, contrast=0.2, saturation=0.2, grayscale_p=0.3, mean=MEAN, std=STD),
    dict(crop_size=(80, 100), horizontal_flip_p=0.5, brightness=0.2, grayscale_p=0.1),            # no affine
    dict(degrees=20, shear=(-5, 5, -3, 3), contrast=0.4, mean=MEAN, std=STD),                     # no crop, no flip, shear y drawn
    dict(crop_size=64, degrees=(-10, 30), scale=(0.7, 0.8), interpolation="nearest", saturation=(0.5, 1.5)),
    dict(translate=(0.3, 0.0), horizontal_flip_p=1.0),                                            # degrees 0 but affine on
]


def _gen():
    return torch.cuda.default_generators[0]


def test_self_check_accepts_this_pytorch_build():
    from triton_augment_b200 import _torch_rng
    flags = _torch_rng.flags_for(DEV)
    assert flags & 1, "the sampler kernel could not reproduce this PyTorch build's CUDA draws"
    assert _torch_rng.max_values_per_draw(DEV) >= 4096


@pytest.mark.parametrize("count", [1, 64, 128, 4096])
@pytest.mark.parametrize("cfg", range(len(CONFIGS)))
def test_parameters_equal_the_separate_draws(cfg, count):
    import triton_augment_b200 as ta
    from triton_augment_b200 import _torch_rng
    from triton_augment_b200.transforms import _Layout
    aug = ta.TritonFusedAugment(**CONFIGS[cfg])
    img = torch.empty(count, 3, 128, 144, device=DEV)
    lay = _Layout(img, False, True)
    flags = _torch_rng.flags_for(DEV)
    torch.manual_seed(1000 + cfg)
    torch.rand(5, device=DEV)                                     # a generator that is not at offset 0
    start = _gen().get_offset()
    want = aug._spread_all(lay, aug._get_params(count, DEV, (128, 144)))
    end = _gen().get_offset()
    torch.manual_seed(1000 + cfg)
    torch.rand(5, device=DEV)
    got = aug._sample_fast(lay, torch.float32, want_draws=True, torch_flags=flags)
    assert _gen().get_offset() == end and end - start == 4 * aug._draw_plan()[1]
    angle, translate, scale, shear, top, left, flip, b, c, s, g = want
    if aug.has_affine:
        assert torch.equal(got["angle"], angle) and torch.equal(got["translate"], translate)
        assert torch.equal(got["scale"], scale) and torch.equal(got["shear"], shear)
        m = ta.functional._prepare_affine_matrix_only(count, DEV, 128, 144, angle, translate, scale, shear, None)
        assert torch.equal(got["matrix"].view(torch.int32), m.contiguous().view(torch.int32))
    assert torch.equal(got["top"], top) and torch.equal(got["left"], left)
    assert torch.equal(got["flip"].bool(), flip) and torch.equal(got["gray"].bool(), g)
    assert torch.equal(got["brightness"], b) and torch.equal(got["contrast"], c) and torch.equal(got["saturation"], s)


@pytest.mark.parametrize("cfg", range(len(CONFIGS)))
@pytest.mark.parametrize("layout", ["4d", "5d", "5d_per_frame", "same_on_batch", "5d_batch_not_frame", "3d", "f16"])
def test_forward_is_identical_with_the_feature_on_and_off(cfg, layout):
    import triton_augment_b200 as ta
    kw = dict(CONFIGS[cfg])
    if layout == "5d_per_frame":
        kw.update(same_on_frame=False)
    if layout == "same_on_batch":
        kw.update(same_on_batch=True)
    if layout == "5d_batch_not_frame":
        kw.update(same_on_batch=True, same_on_frame=False)
    shape = {"4d": (6, 3, 128, 144), "3d": (3, 128, 144), "f16": (5, 3, 128, 144), "same_on_batch": (6, 3, 128, 144)}.get(layout, (3, 4, 3, 128, 144))
    x = torch.rand(shape, device=DEV, generator=torch.Generator(device=DEV).manual_seed(3))
    if layout == "f16":
        x = x.half()
    aug = ta.TritonFusedAugment(**kw)
    outs, offsets = {}, {}
    for on in (True, False):
        aug.one_launch_draws = on
        torch.manual_seed(77)
        outs[on] = [aug(x) for _ in range(3)]                         # three calls: the stream position carries over
        offsets[on] = _gen().get_offset()
    assert offsets[True] == offsets[False]
    for a, b in zip(outs[True], outs[False]):
        assert torch.equal(a, b)


def test_graph_replays_follow_the_eager_sequence():
    import triton_augment_b200 as ta
    aug = ta.TritonFusedAugment(**CONFIGS[0])
    x = torch.rand(8, 3, 128, 144, device=DEV)
    g = ta.GraphedTransform(aug, x)
    assert g._draws == 13 and len(g._samplers) == 1                    # the capture used the library's sampler
    torch.manual_seed(5)
    replayed = [g().clone() for _ in range(4)]
    end_graph = _gen().get_offset()
    torch.manual_seed(5)
    eager = [aug(x) for _ in range(4)]
    assert _gen().get_offset() == end_graph
    for a, b in zip(replayed, eager):
        assert torch.equal(a, b)
    aug.one_launch_draws = False                                       # ... and PyTorch's own draws give the same again
    torch.manual_seed(5)
    for a in replayed:
        assert torch.equal(a, aug(x))


@pytest.mark.parametrize("name,kw", [
    ("TritonColorJitter", dict(brightness=0.3, saturation=(0.5, 1.5))),
    ("TritonColorJitterNormalize", dict(brightness=0.2, contrast=0.2, saturation=0.2, grayscale_p=0.4, mean=MEAN, std=STD)),
    ("TritonColorJitterNormalize", dict(contrast=0.5, contrast_mode="torchvision")),
    ("TritonRandomCropFlip", dict(size=(90, 70), horizontal_flip_p=0.5)),
    ("TritonRandomCropFlip", dict(size=64, horizontal_flip_p=0.0)),          # the flip draw happens even for p = 0
    ("TritonRandomCrop", dict(size=(100, 77))),
    ("TritonRandomHorizontalFlip", dict(p=0.5)),
    ("TritonRandomAffine", dict(degrees=25, translate=(0.1, 0.2), scale=(0.8, 1.2), shear=(-5, 5, -3, 3), interpolation="bilinear", fill=0.25)),
    ("TritonRandomAffine", dict(degrees=(-10, 40), interpolation="nearest")),
    ("TritonRandomRotation", dict(degrees=30, interpolation="bilinear")),
])
@pytest.mark.parametrize("ndim", [4, 5])
def test_other_classes_through_the_one_launch_sampler(name, kw, ndim):
    """The classes whose draws are a subset of TritonFusedAugment's borrow its sampler; their own
    draw order (no grayscale draw; flip always drawn) must survive, as must graph replays."""
    import triton_augment_b200 as ta
    x = torch.rand((5, 3, 128, 144) if ndim == 4 else (2, 3, 3, 128, 144), device=DEV)
    aug = getattr(ta, name)(**kw)
    outs, offsets = {}, {}
    for on in (True, False):
        aug.one_launch_draws = on
        torch.manual_seed(21)
        outs[on] = [aug(x) for _ in range(3)]
        offsets[on] = _gen().get_offset()
    assert offsets[True] == offsets[False] and offsets[True] > 0
    for a, b in zip(outs[True], outs[False]):
        assert torch.equal(a, b)
    aug.one_launch_draws = True
    g = ta.GraphedTransform(aug, x)
    assert g._draws > 0
    torch.manual_seed(21)
    for want in outs[False]:
        assert torch.equal(g(), want)
    assert _gen().get_offset() == offsets[False]


def test_a_rank_draws_only_its_own_slice():
    """Per-rank sharding: every rank seeds alike, samples just its slice (the sampler computes
    value i of a draw from the seed, the offset and i) and leaves its generator where the
    whole-batch call leaves it; the slices tile the single-GPU result."""
    import triton_augment_b200 as ta
    aug = ta.TritonFusedAugment(**CONFIGS[0])
    for shape, world in (((10, 3, 128, 144), 3), ((4, 3, 3, 128, 144), 2)):
        x = torch.rand(shape, device=DEV)
        torch.manual_seed(31)
        want = aug(x)
        end = _gen().get_offset()
        flat_want = want.reshape(-1, *want.shape[-3:])
        group = shape[1] if len(shape) == 5 else 1
        flat = x.reshape(-1, *x.shape[-3:])
        for rank, (a, b) in enumerate(ta.shard_bounds(flat.shape[0], world, group)):
            torch.manual_seed(31)
            got = ta.ShardedAugment.for_rank(aug, rank, world, device=DEV)((flat[a:b], shape))
            assert _gen().get_offset() == end
            assert torch.equal(got, flat_want[a:b]), (shape, rank)


def test_a_capture_by_someone_else_keeps_pytorch_draws():
    """Only GraphedTransform refreshes the sampler's generator state before a replay; a graph that
    the user captures directly must therefore fall back to PyTorch's own (graph-safe) draws, so
    that its replays keep producing fresh parameters."""
    import triton_augment_b200 as ta
    aug = ta.TritonFusedAugment(**CONFIGS[1])
    x = torch.rand(6, 3, 128, 144, device=DEV)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            aug(x)
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = aug(x)
    g.replay(); a = out.clone()
    g.replay(); b = out.clone()
    assert not torch.equal(a, b)                                  # fresh parameters on every replay
