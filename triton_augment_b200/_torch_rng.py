"""Reproducing PyTorch's CUDA random stream inside the library's sampler kernel.

The reference draws every per-sample parameter with its own `uniform_` / `randint` / `rand`
call (triton_augment/transforms.py:1431-1481, 1712-1751, 637-668): about a dozen small
launches per forward.  PyTorch's CUDA generator is a counter-based Philox4x32-10: value i of
such a draw is a pure function of (seed, offset, i), and each draw moves the offset on by 4.
`ta_b200_sample_params` in its `torch_compat` mode computes those same values for all
parameters in ONE launch, after which the generator's offset is advanced by what the separate
draws would have consumed - so a seed keeps giving the reference's parameters, bit for bit.

Two float roundings (whether a multiply-add pair is fused) are properties of the PyTorch
build, not of the algorithm.  `flags_for()` therefore checks the kernel against real draws
from a private generator the first time a device is used, picks the variant that matches and
returns 0 - "do not use" - if none does; callers then keep drawing with PyTorch itself.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

_FLAGS = {}            # device index -> torch_compat value (0: unavailable)
# Sampler launches recorded while a CUDA graph is being captured: (state tensor, draws), in launch
# order.  GraphedTransform empties it before a capture and keeps what the capture added.
CAPTURED = []
# True only while GraphedTransform captures: it is the one that refreshes the captured launches'
# generator state before every replay.  A capture started by anyone else keeps PyTorch's own
# draws (whose graph-safe generator advances by itself on replay).
REPLAY_MANAGED = False
DRAW_SLOTS = ("angle", "tx", "ty", "scale", "shear_x", "shear_y", "top", "left", "flip", "brightness", "contrast",
              "saturation", "gray")


def max_values_per_draw(device) -> int:
    """Largest draw whose value i comes from the first word of thread i (beyond it PyTorch's
    threads produce several values each and the mapping used here no longer holds)."""
    p = torch.cuda.get_device_properties(device)
    return p.multi_processor_count * (p.max_threads_per_multi_processor // 256) * 256


def _probe(device, flags: int, count: int) -> bool:
    """One kernel call against three real PyTorch draws (uniform_, randint, rand < p) from a
    private generator with a known seed; offset 0."""
    seed, lo, hi, span, prob = 0x5EED0000 + count, -15.25, 37.5, 193, 0.37
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    want_u = torch.empty(count, device=device).uniform_(lo, hi, generator=g)
    want_i = torch.randint(0, span, (count,), device=device, dtype=torch.float32, generator=g)
    want_b = torch.rand(count, device=device, generator=g) < prob
    if g.get_offset() != 12:
        return False
    angle = torch.empty(count, device=device)
    top = torch.empty(count, device=device)
    flip = torch.empty(count, dtype=torch.uint8, device=device)
    sp = _lib.SampleSpec()
    sp.struct_size = C.sizeof(_lib.SampleSpec)
    sp.total, sp.frames, sp.same_on_batch, sp.same_on_frame = count, 1, 0, 1
    sp.img_h = sp.img_w = span + 63
    sp.crop_h = sp.crop_w = 64
    sp.factor_dtype = _lib.F32
    sp.degrees[:] = (lo, hi)
    sp.scale[:] = (1.0, 1.0)
    sp.flip_p = prob
    sp.torch_compat = flags
    sp.draw[:] = [0, -1, -1, -1, -1, -1, 1, -1, 2, -1, -1, -1, -1]
    sp.torch_seed, sp.torch_offset = seed, 0
    sp.angle_out, sp.top, sp.flip = angle.data_ptr(), top.data_ptr(), flip.data_ptr()
    _lib.launch_sample_params(sp, device)
    return bool(torch.equal(angle, want_u) and torch.equal(top, want_i) and torch.equal(flip.bool(), want_b))


def flags_for(device) -> int:
    """The `torch_compat` value to use on `device`, or 0 when the kernel cannot reproduce this
    PyTorch build's draws (checked once per device)."""
    device = torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    hit = _FLAGS.get(idx)
    if hit is None:
        hit = 0
        try:
            for flags in (7, 3, 5, 1):           # bit 0 on; bits 1, 2: which multiply-adds are fused
                if all(_probe(device, flags, n) for n in (1, 257, 4096)):
                    hit = flags
                    break
        except Exception:                        # an unexpected generator API: keep PyTorch's own draws
            hit = 0
        _FLAGS[idx] = hit
    return hit


def generator_of(device):
    device = torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    return torch.cuda.default_generators[idx]
