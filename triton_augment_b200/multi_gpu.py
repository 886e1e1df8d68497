"""Batch sharding over the GPUs of one box.  No collective, no peer access, no NCCL.

Images are independent, so a batch is cut into contiguous slices, one per GPU, and each
GPU runs the same kernel on its slice.  The only thing that must be coordinated is the
random parameters: they are drawn ONCE for the whole batch, with the transform's own
draw order, and then sliced - so the sharded result is bit-identical to running the
whole batch on one GPU under the same seed.

Two ways to use it:

* one process driving several devices: ``ShardedAugment(transform, devices)(batch)``;
* one process per GPU (``torchrun``): every rank seeds the same generator state, calls
  ``ShardedAugment.for_rank(transform, rank, world)`` and passes only its own slice.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

import contextlib

__all__ = ["shard_bounds", "slice_params", "ShardedAugment", "ShardError"]


class ShardError(RuntimeError):
    """One or more shards of a ``ShardedAugment`` call failed; the others ran to the end.

    ``errors`` maps shard index -> the exception that shard raised, ``bounds`` holds every
    shard's ``[start, stop)`` and ``outputs`` the per-shard results (None for failed shards),
    so a caller can keep what succeeded and retry only the failed slices."""

    def __init__(self, errors, bounds, outputs):
        self.errors, self.bounds, self.outputs = dict(errors), list(bounds), list(outputs)
        what = "; ".join(f"shard {i} (samples {bounds[i][0]}..{bounds[i][1]}): {type(e).__name__}: {e}"
                         for i, e in sorted(self.errors.items()))
        super().__init__(f"{len(self.errors)} of {len(bounds)} shards failed: {what}")


def _on(device):
    """Make ``device`` current for the block (nothing to do for a host 'device', which the
    CPU tests of the sharding logic use)."""
    return torch.cuda.device(device) if device.type == "cuda" else contextlib.nullcontext()


def shard_bounds(total: int, parts: int, group: int = 1) -> List[Tuple[int, int]]:
    """``parts`` contiguous ``[start, stop)`` slices of ``total`` samples.

    Slices are whole multiples of ``group`` (frames per video, so a video never straddles
    two GPUs); the first ``(total/group) % parts`` slices get one group more.  Slices can be
    empty when there are fewer groups than parts.
    """
    if parts < 1 or group < 1 or total < 0 or total % group:
        raise ValueError(f"cannot split {total} samples in groups of {group} over {parts} parts")
    groups = total // group
    base, extra = divmod(groups, parts)
    bounds, start = [], 0
    for i in range(parts):
        stop = start + (base + (1 if i < extra else 0)) * group
        bounds.append((start, stop))
        start = stop
    return bounds


def slice_params(spread_params: Sequence, start: int, stop: int, device=None):
    """Cut per-sample parameter tensors to ``[start, stop)`` (Python scalars / lists pass through)."""
    out = []
    for p in spread_params:
        if isinstance(p, torch.Tensor):
            p = p[start:stop]
            if device is not None:
                p = p.to(device, non_blocking=True)
        out.append(p)
    return tuple(out)


class ShardedAugment:
    """Run a ``TritonFusedAugment`` over a batch split across GPUs."""

    def __init__(self, transform, devices: Optional[Sequence] = None):
        for attr in ("_get_params", "_spread_all", "_apply"):
            if not hasattr(transform, attr):
                raise TypeError("ShardedAugment needs a TritonFusedAugment-like transform")
        if devices is None:
            devices = list(range(torch.cuda.device_count()))
        self.transform = transform
        self.devices = [torch.device("cuda", d) if isinstance(d, int) else torch.device(d) for d in devices]
        if not self.devices:
            raise RuntimeError("ShardedAugment needs at least one CUDA device")
        self._rank = None
        self._world = None

    @classmethod
    def for_rank(cls, transform, rank: int, world_size: int, device=None):
        """One-process-per-GPU flavour: this object handles slice ``rank`` of ``world_size``."""
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self = cls(transform, [device])
        self._rank, self._world = rank, world_size
        return self

    # ------------------------------------------------------------------ parameter plan (pure host logic)
    def plan(self, batch_shape: Sequence[int], param_device):
        """Draw and spread the parameters of a whole batch of ``batch_shape``; returns
        ``(layout, spread_params, bounds)``.  ``bounds`` has one entry per device (or per
        rank in the per-rank flavour)."""
        from .transforms import _Layout

        meta = torch.empty(batch_shape, device="meta")
        lay = _Layout.__new__(_Layout)
        flat_shape, lay.batch, lay.frames, lay.shape, lay.was_3d = _meta_layout(meta)
        lay.sob, lay.sof = self.transform.same_on_batch, self.transform.same_on_frame
        lay.total = flat_shape[0]
        from .transforms import _compute_param_count
        lay.count = _compute_param_count(lay.batch, lay.frames, lay.sob, lay.sof)
        lay.image = None
        params = self.transform._get_params(lay.count, param_device, (flat_shape[2], flat_shape[3]))
        spread = self.transform._spread_all(lay, params)
        parts = self._world if self._world is not None else len(self.devices)
        bounds = shard_bounds(lay.total, parts, lay.frames or 1)
        return lay, spread, bounds

    def _one_launch_slice(self, flat, full_shape):
        """Per-rank flavour, fast path: where the transform can draw its parameters with the
        library's sampler in PyTorch-compatible mode, the rank draws ONLY its own slice - the
        sampler computes value i of a draw from (seed, offset, i), so no rank needs the rest -
        and advances its generator as the whole-batch draw would.  Same bits as plan() + _apply().
        None when that path is not available."""
        t = self.transform
        if not (hasattr(t, "_torch_flags") and hasattr(t, "_forward_fast")) or getattr(t, "fast_rng", False):
            return None
        dev = self.devices[0]
        if dev.type != "cuda":
            return None
        lay = self._meta_layout(full_shape, dev)
        flags = t._torch_flags(lay, dev)
        if not flags:
            return None
        start, stop = shard_bounds(lay.total, self._world, lay.frames or 1)[self._rank]
        if flat.shape[0] != stop - start:
            raise ValueError(f"rank {self._rank} owns samples [{start}, {stop}) but got {flat.shape[0]}")
        with _on(dev):
            return t._forward_fast(lay, flags, part=(start, stop), image=flat.to(dev))

    def _meta_layout(self, batch_shape, param_device):
        """Shape bookkeeping of a batch of ``batch_shape`` without any data."""
        from .transforms import _Layout, _compute_param_count
        meta = torch.empty(batch_shape, device="meta")
        lay = _Layout.__new__(_Layout)
        flat_shape, lay.batch, lay.frames, lay.shape, lay.was_3d = _meta_layout(meta)
        lay.sob, lay.sof = self.transform.same_on_batch, self.transform.same_on_frame
        lay.total = flat_shape[0]
        lay.count = _compute_param_count(lay.batch, lay.frames, lay.sob, lay.sof)
        lay.image = torch.empty(flat_shape, device="meta")
        lay.param_device = torch.device(param_device)
        return lay

    # ------------------------------------------------------------------ execution
    def __call__(self, batch, gather_to=None):
        """``batch``: one tensor holding the whole batch (host or any GPU; slices are copied to
        their GPU), or - per-rank flavour - ``(local_slice, full_batch_shape)``.  Returns the
        list of per-device outputs, or one tensor on ``gather_to`` if given."""
        if self._world is not None:
            local, full_shape = batch
            flat = local.reshape(-1, *local.shape[-3:]) if local.ndim != 4 else local
            fast = self._one_launch_slice(flat, full_shape)
            if fast is not None:
                return fast
            lay, spread, bounds = self.plan(full_shape, self.devices[0])
            start, stop = bounds[self._rank]
            if flat.shape[0] != stop - start:
                raise ValueError(f"rank {self._rank} owns samples [{start}, {stop}) but got {flat.shape[0]}")
            with _on(self.devices[0]):
                return self.transform._apply(flat.to(self.devices[0]), slice_params(spread, start, stop), first_image=start)
        lay, spread, bounds = self.plan(tuple(batch.shape), self.devices[0])
        flat = batch.reshape(-1, *batch.shape[-3:]) if batch.ndim != 4 else batch
        # Shards are independent: one that fails (a device out of memory, a bad device) is
        # recorded and the loop goes on, so the other GPUs still deliver their slices.
        outs, errors = [], {}
        for i, (dev, (start, stop)) in enumerate(zip(self.devices, bounds)):
            try:
                with _on(dev):
                    part = flat[start:stop].to(dev, non_blocking=True)
                    outs.append(self.transform._apply(part, slice_params(spread, start, stop, dev), first_image=start))
            except Exception as e:          # noqa: BLE001 - reported per shard below
                outs.append(None)
                errors[i] = e
        if errors:
            raise ShardError(errors, bounds, outs)
        if gather_to is None:
            return outs
        whole = torch.cat([o.to(gather_to) for o in outs], dim=0)
        return lay.restore(whole)


def _meta_layout(meta: torch.Tensor):
    """Shape bookkeeping of transforms._normalize_video_shape without touching data."""
    from .transforms import _normalize_video_shape
    flat, batch, frames, shape, was_3d = _normalize_video_shape(meta)
    return tuple(flat.shape), batch, frames, shape, was_3d
