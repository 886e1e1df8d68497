"""A barrier wait that runs out inside the staged kernel must reach the caller.

The staged kernel's consumer warps wait (with a time limit) for the tile their producer warp
is fetching.  Here the limit is set to a few milliseconds and the producer of ONE tile is told
to leave without signalling, so the consumers of that tile give up: the thread block takes its
abort path, the launch completes, every other tile is written, and the condition is reported
through ta_b200_status() and by the next call.  Nothing faults, traps or waits without bound.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _case():
    from triton_augment_b200 import _lib, functional as F
    g = torch.Generator().manual_seed(5)
    n, h, w, oh, ow = 2, 256, 256, 192, 192
    img = torch.rand(n, 3, h, w, generator=g).to(DEV)
    angle = torch.tensor([7.0, -11.0], device=DEV)
    matrix = F._prepare_affine_matrix_only(n, DEV, h, w, angle, [3.0, -2.0], 1.05, [2.0, 0.0], None).contiguous()
    top = torch.tensor([20.0, 31.0], device=DEV)
    left = torch.tensor([11.0, 40.0], device=DEV)
    flip = torch.tensor([True, False], device=DEV)
    bf = torch.tensor([1.1, 0.9], device=DEV)

    def launch(out):
        p = _lib.make_params(img, out, top, left, flip, matrix, 0.0, True, _lib.APPLY_BRIGHTNESS, bf, None, None, None,
                             None, None)
        _lib.launch_fused(p, DEV)
    return launch, (n, 3, oh, ow)


def test_a_wait_that_runs_out_is_reported_and_only_that_tile_is_lost():
    from triton_augment_b200 import _lib
    launch, shape = _case()
    good = torch.empty(shape, device=DEV)
    launch(good)
    torch.cuda.synchronize()
    _lib.debug_counters(reset=True)
    assert not _lib.status(DEV, acknowledge=True)

    tile_w, tile_h = _lib.tile_shape()[:2]
    tiles_x = (shape[3] + tile_w - 1) // tile_w
    lost = 3                                                   # tile number: image 0, tile row / column below
    ty, tx = divmod(lost, tiles_x)
    out = torch.full(shape, -7.0, device=DEV)
    _lib.debug_wait(limit_ns=5_000_000, skip_arrive_tile=lost)
    try:
        launch(out)                                            # returns OK: the launch itself is asynchronous
        torch.cuda.synchronize()                               # ... and the kernel ends by itself
    finally:
        _lib.debug_wait(0, -1)
    assert _lib.debug_counters()[3] == 1                       # one thread block gave up
    assert _lib.status(DEV)                                    # raised, and stays raised
    assert _lib.status(DEV)
    with pytest.raises(_lib.LibraryError, match="-9"):
        launch(torch.empty(shape, device=DEV))                 # the next call reports it and enqueues nothing
    # the tile whose producer never signalled keeps the sentinel, everything else is complete
    region = (slice(0, 1), slice(None), slice(ty * tile_h, (ty + 1) * tile_h), slice(tx * tile_w, (tx + 1) * tile_w))
    assert bool((out[region] == -7.0).all())
    patched = out.clone()
    patched[region] = good[region]
    assert patched.equal(good)

    with pytest.raises(_lib.LibraryError):
        _lib.check_status(DEV)                                 # raises once and acknowledges
    assert not _lib.status(DEV)
    again = torch.empty(shape, device=DEV)
    launch(again)
    torch.cuda.synchronize()
    assert again.equal(good) and not _lib.status(DEV)
    _lib.debug_counters(reset=True)


def test_the_host_buffer_call_reports_a_timeout_at_its_final_synchronisation():
    import triton_augment_b200 as ta
    from triton_augment_b200 import _lib
    aug = ta.TritonFusedAugment(crop_size=192, degrees=10, interpolation="bilinear", brightness=0.2)
    x = torch.rand(4, 3, 256, 256).pin_memory()
    torch.manual_seed(3)
    want = aug.forward_host(x, device=DEV).clone()
    _lib.debug_wait(limit_ns=5_000_000, skip_arrive_tile=0)
    try:
        torch.manual_seed(3)
        with pytest.raises(_lib.LibraryError, match="-9"):
            aug.forward_host(x, device=DEV)
    finally:
        _lib.debug_wait(0, -1)
    assert _lib.status(DEV, acknowledge=True)
    _lib.debug_counters(reset=True)
    torch.manual_seed(3)
    assert aug.forward_host(x, device=DEV).equal(want)         # the pipeline is usable again
    ta.utils.release_host_buffers(DEV)
    torch.manual_seed(3)
    assert aug.forward_host(x, device=DEV).equal(want)         # ... also after its buffers were released
