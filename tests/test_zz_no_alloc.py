"""The allocation-free variant of the grayscale-mean pre-pass.

ta_b200_gray_mean_static() is for callers that are not allowed to allocate device memory
(a plugin whose host application owns the allocator, a service with a frozen memory budget):
its scratch is a fixed array inside the library instead of a buffer the caller passes.  The
test calls it through the C ABI and requires the same means as the ordinary entry point
(ta_b200_gray_mean with caller-provided scratch) gives - on two calls in a row with different
batch sizes, because the array is shared and keeps the previous call's contents.  It also
checks that a batch too large for the fixed array is refused with a clear error, and the
property the entry point exists for: once warm, a call leaves the amount of free device memory
and torch's allocator counters exactly where they were.

This file sorts last on purpose: if it fails, a run that stops at the first failure has
already run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _means(lib, _lib, image, top, left, flip, matrix, bilinear, brightness, static):
    n, c, h, w = image.shape
    oh, ow = 48, 56
    out = torch.empty(n, c, oh, ow, dtype=image.dtype, device=image.device)      # not written by the pre-pass
    p = _lib.make_params(image, out, top, left, flip, matrix, 0.0, bilinear, _lib.APPLY_BRIGHTNESS, brightness,
                         None, None, None, None, None)
    means = torch.full((n,), -1.0, dtype=torch.float32, device=image.device)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    if static:
        rc = lib.ta_b200_gray_mean_static(C.byref(p), C.c_void_p(means.data_ptr()), stream)
    else:
        need = int(lib.ta_b200_gray_mean_scratch_bytes(C.byref(p)))
        scratch = torch.empty(need, dtype=torch.uint8, device=image.device)
        rc = lib.ta_b200_gray_mean(C.byref(p), C.c_void_p(means.data_ptr()), C.c_void_p(scratch.data_ptr()), need, stream)
    assert rc == 0, lib.ta_b200_last_error().decode()
    torch.cuda.synchronize()
    return means.cpu().numpy()


def test_static_scratch_entry_point_matches_the_allocating_one():
    from triton_augment_b200 import _lib, functional as F
    lib = _lib.load()
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(17)
    for n, dtype, bilinear in ((9, torch.float32, True), (4, torch.float16, False), (9, torch.float32, False)):
        image = torch.rand(n, 3, 64, 72, generator=g).to(dtype).to(dev)
        top = torch.randint(0, 17, (n,), generator=g).float().to(dev)
        left = torch.randint(0, 17, (n,), generator=g).float().to(dev)
        flip = (torch.rand(n, generator=g) < 0.5).to(dev)
        angle = torch.empty(n).uniform_(-15, 15, generator=g).to(dev)
        matrix = F._prepare_affine_matrix_only(n, dev, 64, 72, angle, [1.5, -2.0], 1.05, [3.0, 0.0], None).contiguous()
        brightness = torch.empty(n).uniform_(0.8, 1.2, generator=g).to(dtype).to(dev)
        want = _means(lib, _lib, image, top, left, flip, matrix, bilinear, brightness, static=False)
        got = _means(lib, _lib, image, top, left, flip, matrix, bilinear, brightness, static=True)
        again = _means(lib, _lib, image, top, left, flip, matrix, bilinear, brightness, static=True)
        tol = 1e-2 if dtype == torch.float16 else 1e-5
        assert np.all(want > 0.2) and np.all(want < 0.8)
        assert np.abs(got - want).max() <= tol and np.abs(again - want).max() <= tol


def test_static_scratch_refuses_what_does_not_fit():
    from triton_augment_b200 import _lib
    lib = _lib.load()
    p = _lib.FusedParams()
    p.struct_size = C.sizeof(_lib.FusedParams)
    p.dtype, p.n, p.c, p.h, p.w, p.oh, p.ow = 0, 4000, 3, 1024, 1024, 1024, 1024     # needs ~2 MiB of partial sums
    p.inp = p.out = 256                                # never dereferenced: the size check comes first
    rc = lib.ta_b200_gray_mean_static(C.byref(p), C.c_void_p(256), None)
    assert rc == -8
    assert b"built-in buffer" in lib.ta_b200_last_error()


def test_static_scratch_call_allocates_no_device_memory():
    """Free device memory (cudaMemGetInfo) and torch's allocator statistics are identical before
    and after warm calls; p->out is NULL, which this entry accepts because it writes no image."""
    from triton_augment_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda:0")
    n = 6
    image = torch.rand(n, 3, 96, 112, device=dev)
    dummy = torch.empty(n, 3, 80, 96, device=dev)
    top = torch.full((n,), 3.0, device=dev)
    left = torch.full((n,), 5.0, device=dev)
    bright = torch.full((n,), 1.1, device=dev)
    means = torch.zeros(n, device=dev)
    p = _lib.make_params(image, dummy, top, left, None, None, 0.0, False, _lib.APPLY_BRIGHTNESS, bright, None, None,
                         None, None, None)
    p.out = None
    del dummy
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    call = lambda: lib.ta_b200_gray_mean_static(C.byref(p), C.c_void_p(means.data_ptr()), stream)
    assert call() == 0, lib.ta_b200_last_error().decode()      # warm: symbol lookup, kernel code loaded
    torch.cuda.synchronize()
    first = means.clone()
    torch.cuda.synchronize()
    before = (torch.cuda.mem_get_info(dev)[0], torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev))
    for _ in range(3):
        assert call() == 0
    torch.cuda.synchronize()
    after = (torch.cuda.mem_get_info(dev)[0], torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev))
    assert after == before
    assert means.equal(first) and bool((first > 0.3).all())
