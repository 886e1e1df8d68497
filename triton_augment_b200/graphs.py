"""Replay one transform call as a CUDA graph (extra; the reference has no counterpart).

A `TritonFusedAugment.forward` on a device-resident batch is ~19 small launches (one per random
draw, as in the reference, so that a seed gives the reference's parameters) followed by the
fused kernel.  For large batches the GPU work hides the launches; once the fused kernel runs
in a quarter of a millisecond the host cannot issue them fast enough.  `GraphedTransform`
captures the whole call once and replays it with a single launch.  Every replay draws fresh
parameters: PyTorch's CUDA generator advances its Philox offset per replay exactly as the
eager calls would, so graphed and eager runs started from the same seed produce the same
outputs (tests/test_gpu_crop_paths.py checks this).

The price is the usual one of CUDA graphs: input and output live at fixed addresses, and the
captured call must not read device values on the host.  The transform classes never do (they
know from their constructor arguments which operations are on); the functional entry points
called with tensor-valued factors decide that from the values with one device-to-host read and
therefore cannot be captured.

    aug = ta.TritonFusedAugment(...)
    g = ta.GraphedTransform(aug, batch)      # `batch` is the staging tensor the loader refills
    for _ in loader_steps:
        batch.copy_(next_batch, non_blocking=True)   # or fill it in place some other way
        out = g()                            # same tensor every time; consume before the next call
"""
from __future__ import annotations

from typing import Optional

import torch

__all__ = ["GraphedTransform"]


class GraphedTransform:
    """``transform(example)`` captured as a CUDA graph.

    ``example`` becomes the static input: later calls either pass nothing (the caller has
    refilled ``example`` in place), the same tensor, or another tensor of the same shape and
    dtype, which is copied into it first.  The returned tensor is the graph's static output
    and is overwritten by the next call.  ``warmup`` eager calls run before the capture (lazy
    initialisation must not happen inside it); they consume random draws like any other call.
    """

    def __init__(self, transform, example: torch.Tensor, warmup: int = 3):
        if not isinstance(example, torch.Tensor) or not example.is_cuda:
            raise ValueError("GraphedTransform needs a CUDA tensor as the static input")
        self.transform = transform
        self.static_input = example
        device = example.device
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            for _ in range(max(int(warmup), 1)):
                transform(example)
        torch.cuda.current_stream(device).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        from . import _torch_rng
        del _torch_rng.CAPTURED[:]
        _torch_rng.REPLAY_MANAGED = True
        try:
            with torch.cuda.device(device), torch.cuda.graph(self.graph):
                self.static_output = transform(example)
        finally:
            _torch_rng.REPLAY_MANAGED = False
        # A transform that draws its parameters inside the library in PyTorch-compatible mode has
        # captured a launch that reads the generator's (seed, offset) from device memory: every
        # replay is preceded by a refresh of those two words (per captured sampler launch, each
        # starting where the one before stops) and followed by the same advance of PyTorch's
        # generator that eager calls make.
        self._samplers = list(_torch_rng.CAPTURED)
        del _torch_rng.CAPTURED[:]
        self._draws = sum(d for _, d in self._samplers)
        self._device = device

    def __call__(self, image: Optional[torch.Tensor] = None) -> torch.Tensor:
        if image is not None and image is not self.static_input:
            if image.shape != self.static_input.shape or image.dtype != self.static_input.dtype:
                raise ValueError(f"expected {tuple(self.static_input.shape)} {self.static_input.dtype}, "
                                 f"got {tuple(image.shape)} {image.dtype}")
            if not image.is_cuda or image.data_ptr() != self.static_input.data_ptr():
                self.static_input.copy_(image, non_blocking=True)
        if self._samplers:
            from . import _lib, _torch_rng
            gen = _torch_rng.generator_of(self._device)
            seed, offset = gen.initial_seed(), gen.get_offset()
            for state, draws in self._samplers:
                _lib.store_words(state, seed, offset)
                offset += 4 * draws
            gen.set_offset(offset)
        self.graph.replay()
        return self.static_output

    forward = __call__
