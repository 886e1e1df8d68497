"""Host-side logic that needs no GPU: random-draw order against parameters captured from the
reference's classes, shape / broadcast rules, argument validation, sharding arithmetic, and
that the C-ABI library exports everything its header declares."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import triton_augment_b200 as ta
from triton_augment_b200 import _lib, transforms as T
from triton_augment_b200.multi_gpu import shard_bounds, slice_params

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SPEC_PATH = os.path.join(ROOT, "tests", "golden", "make_golden.py")


def _class_specs():
    """CLASS_SPECS of the generator script, read without importing it (it needs the reference)."""
    src = open(SPEC_PATH).read()
    start = src.index("CLASS_SPECS = {")
    end = src.index("\n}\n", start) + 3
    ns = {"MEAN": (0.485, 0.456, 0.406), "STD": (0.229, 0.224, 0.225)}
    exec(src[start:end], ns)
    return ns["CLASS_SPECS"]


SPECS = _class_specs()


@pytest.mark.parametrize("key", sorted(SPECS))
def test_random_draw_order_matches_reference(class_golden, key):
    """Same seed on the CPU generator -> bit-identical sampled parameters (count 7, 20x24 image)."""
    cls_name, kwargs = SPECS[key]
    tr = getattr(ta, cls_name)(**kwargs)
    if not hasattr(tr, "_get_params") or f"params|{key}|seed" not in class_golden.files:
        pytest.skip("class draws inside forward only")
    torch.manual_seed(int(class_golden[f"params|{key}|seed"]))
    try:
        params = tr._get_params(7, torch.device("cpu"), (20, 24))
    except TypeError:
        params = tr._get_params(7, torch.device("cpu"))
    for i, p in enumerate(params):
        want = class_golden[f"params|{key}|{i}"]
        assert np.array_equal(np.asarray(p), want), (key, i)


def test_param_count_and_broadcast_rules():
    cnt = T._compute_param_count
    assert cnt(None, None, False, True) == 1
    assert (cnt(4, None, False, True), cnt(4, None, True, True)) == (4, 1)
    assert [cnt(2, 3, sb, sf) for sb, sf in ((True, True), (True, False), (False, True), (False, False))] == [1, 3, 2, 6]
    p = torch.tensor([10.0, 20.0])
    out = T._broadcast_params_to_all_samples(p, 2, 3, 6, False, True)       # per video, video-major
    assert out.tolist() == [10, 10, 10, 20, 20, 20]
    q = torch.tensor([1.0, 2.0, 3.0])
    out = T._broadcast_params_to_all_samples(q, 2, 3, 6, True, False)       # per frame index
    assert out.tolist() == [1, 2, 3, 1, 2, 3]
    assert T._broadcast_params_to_all_samples(torch.tensor([7.0]), 2, 3, 6, True, True).tolist() == [7.0] * 6
    full = torch.arange(6.0)
    assert T._broadcast_params_to_all_samples(full, 2, 3, 6, False, False) is full
    with pytest.raises(ValueError):
        T._broadcast_params_to_all_samples(torch.zeros(4), 2, 3, 6, False, True)
    two = T._broadcast_2d_params(torch.tensor([[1.0, 2.0], [3.0, 4.0]]), 2, 2, 4, False, True)
    assert two.tolist() == [[1, 2], [1, 2], [3, 4], [3, 4]]
    with pytest.raises(ValueError):
        T._normalize_video_shape(torch.zeros(2, 2))


def test_constructor_validation_matches_reference():
    with pytest.raises(ValueError):
        ta.TritonColorJitter(brightness=-0.1)
    with pytest.raises(TypeError):
        ta.TritonColorJitter(contrast="x")
    with pytest.raises(ValueError):
        ta.TritonColorJitterNormalize(grayscale_p=1.5)
    with pytest.raises(ValueError):
        ta.TritonColorJitterNormalize(mean=(0.5, 0.5, 0.5))
    with pytest.raises(ValueError):
        ta.TritonRandomAffine(degrees=-1)
    with pytest.raises(ValueError):
        ta.TritonRandomAffine(degrees=10, translate=(0.5, 1.5))
    with pytest.raises(ValueError):
        ta.TritonRandomAffine(degrees=10, scale=(1.2, 0.8))
    with pytest.raises(ValueError):
        ta.TritonRandomAffine(degrees=10, shear=(1, 2, 3))
    assert ta.TritonRandomRotation(10, expand=True).expand          # built here; the reference raises NotImplementedError
    with pytest.raises(ValueError):
        ta.TritonRandomRotation(10, expand=True, center=(3, 4))
    with pytest.raises(ValueError):
        ta.TritonRandomCrop(8, padding=(1, 2, 3))
    with pytest.raises(ValueError):
        ta.TritonRandomHorizontalFlip(p=2)
    with pytest.raises(ValueError):
        ta.TritonGrayscale(num_output_channels=2)
    with pytest.raises(ValueError):
        ta.TritonFusedAugment(contrast_mode="nope")
    assert ta.TritonColorJitter(brightness=0).brightness is None            # (1, 1) cannot change anything
    assert ta.TritonColorJitter(brightness=0.2).brightness == (0.8, 1.2)
    assert ta.TritonRandomAffine(5, shear=3).shear == (-3.0, 3.0, 0.0, 0.0)
    assert "TritonFusedAugment(" in repr(ta.TritonFusedAugment(crop_size=8, brightness=0.1))   # reference's repr raises


def test_functional_argument_errors_without_a_gpu():
    img = torch.rand(1, 3, 4, 4)
    with pytest.raises(TypeError):
        ta.fused_augment([1, 2], 0, 0, 4, 4)
    with pytest.raises(ValueError, match="CUDA"):
        ta.fused_augment(img, 0, 0, 4, 4)                 # no CPU fallback, same error as the reference
    with pytest.raises(ValueError):
        ta.adjust_brightness(img, 1.2)
    with pytest.raises(ValueError):
        ta.TritonGrayscale()(img)
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):
            ta.TritonFusedAugment(crop_size=2)(img)       # class API uploads host tensors; needs CUDA


def test_uint8_is_accepted_by_the_fused_entry_points_only():
    """Bytes are an extension of fused_augment / TritonFusedAugment (result float32); the
    stand-alone functionals keep the reference's float-only check (tested on the GPU, where
    the dtype check is reached).  Host-side checks only."""
    from triton_augment_b200 import functional as F
    u8 = torch.zeros(2, 3, 8, 8, dtype=torch.uint8)
    assert F._work_dtype(u8) == torch.float32 and F._work_dtype(u8.half()) == torch.float16
    with pytest.raises(ValueError, match="CUDA"):
        ta.fused_augment(u8, 0, 0, 4, 4)                  # the device check comes first, as in the reference
    assert _lib.U8 == 2 and _lib.F32 == 0 and _lib.F16 == 1
    header = open(os.path.join(ROOT, "include", "ta_b200.h")).read()
    assert "TA_B200_F32 = 0, TA_B200_F16 = 1, TA_B200_U8 = 2" in header


def test_inverse_matrix_matches_torchvision_and_golden(functional_golden):
    z = functional_golden
    t = lambda k: torch.from_numpy(z[k])
    got = ta.functional._get_inverse_affine_matrix(t("mat_center"), t("mat_angle"), t("mat_translate"),
                                                   t("mat_scale"), t("mat_shear"))
    assert np.array_equal(got.numpy(), z["mat_out"])     # same torch ops, same order, same device -> same bits
    from torchvision.transforms.functional import _get_inverse_affine_matrix as tv_inv
    for i in range(4):
        want = tv_inv(z["mat_center"][i].tolist(), float(z["mat_angle"][i]), z["mat_translate"][i].tolist(),
                      float(z["mat_scale"][i]), z["mat_shear"][i].tolist())
        np.testing.assert_allclose(got[i].numpy(), np.array(want, np.float32), rtol=1e-4, atol=1e-4)


def test_shard_bounds():
    assert shard_bounds(10, 4) == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert shard_bounds(4096, 8) == [(i * 512, (i + 1) * 512) for i in range(8)]
    assert shard_bounds(2, 4) == [(0, 1), (1, 2), (2, 2), (2, 2)]
    assert shard_bounds(8 * 16, 3, group=16) == [(0, 48), (48, 96), (96, 128)]      # whole videos per GPU
    with pytest.raises(ValueError):
        shard_bounds(10, 2, group=4)
    p = slice_params((torch.arange(6.0), 1.0, torch.arange(12.0).reshape(6, 2)), 2, 5)
    assert p[0].tolist() == [2, 3, 4] and p[1] == 1.0 and p[2].shape == (3, 2)


def test_missing_library_fails_loudly():
    """No fallback: with the shared library gone, the first use raises instead of computing on
    the CPU.  Run in a child process so that this process keeps its loaded library."""
    import subprocess
    import sys
    code = ("import sys; sys.path.insert(0, %r)\n"
            "from triton_augment_b200 import _lib\n"
            "try:\n    _lib.load()\nexcept Exception as e:\n    print('RAISED', type(e).__name__)\n"
            "else:\n    print('LOADED')\n") % ROOT
    env = dict(os.environ, TA_B200_LIB=os.path.join(ROOT, "no_such_dir", "libta_b200.so"))
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300).stdout
    assert "RAISED" in out and "LOADED" not in out, out


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "ta_b200.h")).read()
    declared = set(re.findall(r"\b(ta_b200_[a-z_0-9]+)\s*\(", header))
    assert declared == set(_lib.SYMBOLS), declared ^ set(_lib.SYMBOLS)
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name
    assert _lib.load().ta_b200_abi_version() == _lib.ABI_VERSION
    assert ctypes.sizeof(_lib.FusedParams) == 184       # sizeof(ta_b200_fused_params) on LP64 (168 before fill_rgb)
    assert _lib.FusedParams.fill_rgb.offset == 168      # the older layout ends here and is still accepted
    assert ctypes.sizeof(_lib.SampleSpec) == 272 and _lib.SampleSpec.torch_compat.offset == 216     # the older layout ends at 216        # sizeof(ta_b200_sample_spec) on LP64


def test_diagnostic_switches_refuse_values_they_do_not_know():
    """The process-wide switches touch no device, so their argument checks run on any host."""
    for call, bad in ((_lib.tile_height, 48), (_lib.crop_path, 3), (_lib.host_upload, 5)):
        with pytest.raises(_lib.LibraryError):
            call(bad)
        call(0 if call is not _lib.host_upload else 1)          # back to the default


def test_a_failing_shard_does_not_stop_the_others():
    """ShardedAugment runs every shard even when one raises and reports the failure per shard
    (host logic only: the 'devices' are the CPU and the transform's kernel call is a stand-in)."""
    import triton_augment_b200 as ta

    class Stub(ta.TritonFusedAugment):
        def _apply(self, image4d, spread_params, matrix=None, first_image=0):
            if first_image == 4:                                     # the second of three shards
                raise RuntimeError("device lost")
            top = spread_params[4]
            assert top.shape[0] == image4d.shape[0]
            return image4d[:, :, :8, :8] + first_image

    aug = Stub(crop_size=8, horizontal_flip_p=0.5, brightness=0.2, grayscale_p=0.1)
    cpu = torch.device("cpu")
    x = torch.zeros(10, 3, 16, 16)
    sharder = ta.ShardedAugment(aug, [cpu, cpu, cpu])
    with pytest.raises(ta.ShardError) as info:
        sharder(x)
    err = info.value
    assert list(err.errors) == [1] and "device lost" in str(err) and "shard 1 (samples 4..7)" in str(err)
    assert err.bounds == [(0, 4), (4, 7), (7, 10)]
    assert err.outputs[1] is None
    assert err.outputs[0].shape[0] == 4 and float(err.outputs[2].max()) == 7.0       # both others completed

    class Fine(Stub):
        def _apply(self, image4d, spread_params, matrix=None, first_image=0):
            return image4d[:, :, :8, :8] + first_image

    parts = ta.ShardedAugment(Fine(crop_size=8), [cpu, cpu])(x)
    assert [p.shape[0] for p in parts] == [5, 5]
