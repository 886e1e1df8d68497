"""The grayscale-mean pre-pass (torchvision-exact contrast) has two kernels: the staged one
(fp32, rows the tensor copies can read, scratch as large as ta_b200_gray_mean_scratch_bytes
reports) and the gather one (everything else, or a smaller scratch).  Both must be
deterministic and agree with each other and with a torch evaluation of the same mean."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _params(_lib, ta, n, h, w, oh, ow, mode, seed, bright=True):
    g = torch.Generator().manual_seed(seed)
    img = torch.rand(n, 3, h, w, generator=g).to(DEV)
    top = torch.randint(0, h - oh + 1, (n,), generator=g).float().to(DEV)
    left = torch.randint(0, w - ow + 1, (n,), generator=g).float().to(DEV)
    flip = (torch.rand(n, generator=g) < 0.5).to(torch.uint8).to(DEV)
    bf = (torch.rand(n, generator=g) * 0.6 + 0.7).to(DEV)
    matrix = None
    if mode != "none":
        angle = (torch.rand(n, generator=g) * 30 - 15).to(DEV)
        matrix = ta.functional._prepare_affine_matrix_only(n, DEV, h, w, angle, [2.5, -3.0], 1.07, [4.0, 0.0], None).contiguous()
    out = torch.empty(n, 3, oh, ow, device=DEV)
    p = _lib.make_params(img, out, top, left, flip, matrix, 0.0, mode == "bilinear",
                         _lib.APPLY_BRIGHTNESS if bright else 0, bf, None, None, None, None, None)
    return p, (img, top, left, flip, bf, matrix, out)


def _run(lib, p, scratch_bytes):
    means = torch.full((p.n,), -1.0, device=DEV)
    scratch = torch.empty(scratch_bytes, dtype=torch.uint8, device=DEV)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.ta_b200_gray_mean(C.byref(p), C.c_void_p(means.data_ptr()), C.c_void_p(scratch.data_ptr()), scratch_bytes, stream)
    assert rc == 0, lib.ta_b200_last_error().decode()
    torch.cuda.synchronize()
    return means


@pytest.mark.parametrize("mode", ["none", "nearest", "bilinear"])
def test_staged_and_gather_prepass_agree_and_are_deterministic(mode):
    import triton_augment_b200 as ta
    from triton_augment_b200 import _lib
    lib = _lib.load()
    for (n, h, w, oh, ow) in ((5, 160, 192, 130, 150), (3, 96, 128, 96, 128)):
        p, keep = _params(_lib, ta, n, h, w, oh, ow, mode, seed=4)
        full = int(lib.ta_b200_gray_mean_scratch_bytes(C.byref(p)))
        small = (4 * n + 255) // 256 * 256 + 4 * n * min(128, (oh * ow + 4095) // 4096)      # the gather kernel's need
        assert full > small
        staged, staged2 = _run(lib, p, full), _run(lib, p, full)
        gather, gather2 = _run(lib, p, small), _run(lib, p, small)
        assert torch.equal(staged, staged2) and torch.equal(gather, gather2)
        assert float((staged - gather).abs().max()) <= 2e-6
        # the same mean from the fused kernel's own output: geometry + brightness only, then gray
        img, top, left, flip, bf, matrix, out = keep
        q = _lib.make_params(img, out, top, left, flip, matrix, 0.0, mode == "bilinear", _lib.APPLY_BRIGHTNESS, bf,
                             None, None, None, None, None)
        _lib.launch_fused(q, DEV)
        gray = 0.2989 * out[:, 0] + 0.587 * out[:, 1] + 0.114 * out[:, 2]
        want = gray.double().mean(dim=(1, 2)).float()
        assert float((staged - want).abs().max()) <= 2e-6


def test_prepass_for_half_images_uses_the_gather_kernel_and_small_scratch():
    import triton_augment_b200 as ta
    from triton_augment_b200 import _lib
    lib = _lib.load()
    p, keep = _params(_lib, ta, 4, 64, 80, 48, 64, "bilinear", seed=9)
    img16 = keep[0].half()
    bf16 = keep[4].half()
    out16 = torch.empty(4, 3, 48, 64, device=DEV, dtype=torch.float16)
    q = _lib.make_params(img16, out16, keep[1], keep[2], keep[3], keep[5], 0.0, True, _lib.APPLY_BRIGHTNESS, bf16,
                         None, None, None, None, None)
    need = int(lib.ta_b200_gray_mean_scratch_bytes(C.byref(q)))
    assert need == (4 * 4 + 255) // 256 * 256 + 4 * 4 * 1
    m16 = _run(lib, q, need)
    m32 = _run(lib, p, int(lib.ta_b200_gray_mean_scratch_bytes(C.byref(p))))
    assert float((m16 - m32).abs().max()) <= 2e-3
