"""TritonFusedAugment: every augmentation in one kernel launch (re-exported by transforms.py)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import functional as F
from . import transforms as T
from ._transforms_color import TritonColorJitterNormalize
from ._transforms_geometric import TritonRandomAffine
from .functional import InterpolationMode

__all__ = ["TritonFusedAugment"]


class TritonFusedAugment(T._BatchAware):
    """RandomAffine -> RandomCrop -> RandomHorizontalFlip -> ColorJitter -> RandomGrayscale ->
    Normalize as ONE pass over the image.

    Constructor arguments, defaults and the order of random draws are the reference's
    (transforms.py:1252-1580).  Draw order per call, each a separate draw of ``param_count``
    values from the device's default generator: the affine draws (only if any affine
    argument was given), crop top and left as fp32 ``randint`` (only with ``crop_size``),
    the flip mask (only if ``horizontal_flip_p > 0``), brightness, contrast, saturation
    (only those that are set), and the grayscale mask (always).

    ``contrast_mode="torchvision"`` (extra) uses torchvision's mean-based contrast instead
    of the reference's fast formula, at the cost of one more read of the source footprint.

    ``fast_rng=True`` (extra, opt-in) replaces those ~18 separate draws and small elementwise
    operations by one launch that samples every parameter, spreads it over video frames and
    builds the affine matrices.  Same distributions; a different random stream (a Philox
    generator of the library, seeded per call by one draw from torch's generator, so
    ``torch.manual_seed`` still makes runs repeatable), hence not the reference's parameters
    for a given seed.

    ``out_dtype=torch.float16`` (extra) makes a uint8 batch come out as float16 instead of
    float32 (see ``functional.fused_augment``); float batches are not affected.
    """

    def __init__(self, crop_size=None, horizontal_flip_p: float = 0.0, degrees=0, translate=None, scale=None,
                 shear=None, interpolation=InterpolationMode.NEAREST, fill: float = 0.0, brightness=0, contrast=0,
                 saturation=0, grayscale_p: float = 0.0, mean=None, std=None, same_on_batch: bool = False,
                 same_on_frame: bool = True, contrast_mode: str = "fast", fast_rng: bool = False,
                 out_dtype=None):
        super().__init__(same_on_batch, same_on_frame)
        self.fast_rng = bool(fast_rng)
        if out_dtype not in (None, torch.float32, torch.float16):
            raise TypeError(f"out_dtype must be torch.float32 or torch.float16, got {out_dtype}")
        self.out_dtype = out_dtype             # result dtype for uint8 images (None: float32)
        if crop_size is None:
            self.crop_height = self.crop_width = None
        elif isinstance(crop_size, int):
            self.crop_height = self.crop_width = crop_size
        else:
            self.crop_height, self.crop_width = crop_size
        self.horizontal_flip_p = horizontal_flip_p
        self.has_affine = any([degrees != 0, translate is not None, scale is not None, shear is not None])
        if self.has_affine:
            self.affine_helper = TritonRandomAffine(degrees=degrees, translate=translate, scale=scale, shear=shear,
                                                    interpolation=interpolation, fill=fill,
                                                    same_on_batch=same_on_batch, same_on_frame=same_on_frame)
            self.interpolation = interpolation
            self.fill = fill
        self.color_helper = TritonColorJitterNormalize(brightness=brightness, contrast=contrast, saturation=saturation,
                                                       grayscale_p=grayscale_p, mean=mean, std=std,
                                                       same_on_batch=same_on_batch, same_on_frame=same_on_frame,
                                                       contrast_mode=contrast_mode)
        self.contrast_mode = contrast_mode

    def _check_input(self, value, name, center=1.0, bound=(0, float("inf")), clip_first_on_zero=True):
        return T._check_range(value, name, center, bound, clip_first_on_zero)

    def _get_params(self, param_count: int, device, img_size: Tuple[int, int]):
        """All parameters of one call: (angle, translate, scale, shear, top, left, flip,
        brightness, contrast, saturation, grayscale mask).  Reference: transforms.py:1431-1481."""
        img_height, img_width = img_size
        angle, translate, scale, shear = 0.0, [0.0, 0.0], 1.0, [0.0, 0.0]
        if self.has_affine:
            angle, translate, scale, shear = self.affine_helper._get_params(param_count, device, (img_height, img_width))
        if self.crop_height is None:
            top = torch.zeros(param_count, device=device, dtype=torch.float32)
            left = torch.zeros(param_count, device=device, dtype=torch.float32)
        else:
            top = torch.randint(0, img_height - self.crop_height + 1, (param_count,), device=device, dtype=torch.float32)
            left = torch.randint(0, img_width - self.crop_width + 1, (param_count,), device=device, dtype=torch.float32)
        if self.horizontal_flip_p > 0:
            flip = F._sample_bernoulli_tensor(param_count, self.horizontal_flip_p, device)
        else:
            flip = torch.zeros(param_count, device=device, dtype=torch.bool)
        b, c, s, g = self.color_helper._get_params(param_count, device)
        return angle, translate, scale, shear, top, left, flip, b, c, s, g

    def _spread_all(self, lay, params):
        """Sampled parameter sets -> one value per flattened sample."""
        angle, translate, scale, shear, top, left, flip, b, c, s, g = params
        if self.has_affine:
            angle, scale = lay.spread(angle), lay.spread(scale)
            translate, shear = lay.spread2(translate), lay.spread2(shear)
        return (angle, translate, scale, shear, lay.spread(top), lay.spread(left), lay.spread(flip),
                lay.spread(b), lay.spread(c), lay.spread(s), lay.spread(g))

    def _matrix_for(self, spread_params, total, device, h, w):
        """Inverse affine matrices ``[total, 6]`` of already spread parameters (None without affine)."""
        if not self.has_affine:
            return None
        angle, translate, scale, shear = spread_params[:4]
        return F._prepare_affine_matrix_only(total, device, h, w, angle, translate, scale, shear, None).contiguous()

    def _apply(self, image4d, spread_params, matrix=None, first_image=0):
        """Run the kernel on a (slice of a) flattened batch with per-sample parameters;
        ``first_image`` is the slice's position in the batch."""
        angle, translate, scale, shear, top, left, flip, b, c, s, g = spread_params
        h, w = image4d.shape[2:]
        return F.fused_augment(
            image4d, top=top, left=left, _matrix=matrix,
            height=self.crop_height if self.crop_height is not None else h,
            width=self.crop_width if self.crop_width is not None else w,
            flip_horizontal=flip, angle=angle, translate=translate, scale=scale, shear=shear,
            interpolation=self.interpolation if self.has_affine else "nearest",
            fill=self.fill if self.has_affine else 0.0,
            brightness_factor=b, contrast_factor=c, saturation_factor=s, grayscale=g,
            mean=self.color_helper.mean, std=self.color_helper.std, contrast_mode=self.contrast_mode,
            out_dtype=self.out_dtype if image4d.dtype == torch.uint8 else None, _first_image=first_image,
            _flags=self.color_helper._colour_flags(affine=self.has_affine))

    # True: when PyTorch's CUDA generator can be reproduced inside the sampler kernel (checked per
    # device, see _torch_rng), forward() draws all parameters with ONE launch and advances the
    # generator as the reference's separate draws would - same parameters for a seed, a dozen
    # launches fewer.  False: always draw with PyTorch itself.
    one_launch_draws = True
    # The reference's TritonFusedAugment draws the flip mask only for horizontal_flip_p > 0 and the
    # grayscale mask always; classes that borrow this sampler (TritonRandomCropFlip: flip always;
    # TritonColorJitter, TritonRandomCropFlip: no grayscale draw) say so here.
    _draw_flip_always = False
    _draw_gray = True

    def _draw_plan(self):
        """Which draw of a call (0, 1, ... in the reference's order, transforms.py:1431-1481) each
        parameter comes from; -1 = not drawn.  Returns (13 indices, number of draws)."""
        ch, k, plan = self.color_helper, 0, {}
        def take(name, drawn):
            nonlocal k
            plan[name] = k if drawn else -1
            k += 1 if drawn else 0
        ah = self.affine_helper if self.has_affine else None
        take("angle", ah is not None)
        take("tx", ah is not None and ah.translate is not None)
        take("ty", ah is not None and ah.translate is not None)
        take("scale", ah is not None and ah.scale is not None)
        take("shear_x", ah is not None and ah.shear is not None)
        take("shear_y", ah is not None and ah.shear is not None)
        take("top", self.crop_height is not None)
        take("left", self.crop_height is not None)
        take("flip", self.horizontal_flip_p > 0 or self._draw_flip_always)
        take("brightness", ch.brightness is not None)
        take("contrast", ch.contrast is not None)
        take("saturation", ch.saturation is not None)
        take("gray", self._draw_gray)
        from ._torch_rng import DRAW_SLOTS
        return [plan[s] for s in DRAW_SLOTS], k

    def _torch_flags(self, lay, dev) -> int:
        """Non-zero: this call's parameters can come from the sampler kernel in PyTorch-compatible mode."""
        from . import _torch_rng
        if not self.one_launch_draws or self._param_device is not None or dev.type != "cuda":
            return 0
        if lay.count > _torch_rng.max_values_per_draw(dev):
            return 0
        if torch.cuda.is_current_stream_capturing():
            # only under GraphedTransform, which refreshes the state before each replay, and only if the
            # state words exist already (nothing may be allocated and zeroed inside the capture)
            if not _torch_rng.REPLAY_MANAGED or getattr(self, "_torch_state", None) is None:
                return 0
        elif _torch_rng.generator_of(dev).get_offset() % 4:
            return 0                      # PyTorch itself only ever leaves multiples of 4
        return _torch_rng.flags_for(dev)

    def _static_spec(self, work_dtype, h, w, frames, torch_flags):
        """The part of a sampler call that depends on the configuration and the image size only,
        as a filled ta_b200_sample_spec (cached; the per-call fields are set by _sample_fast)."""
        from . import _lib
        ch = self.color_helper
        ah = self.affine_helper if self.has_affine else None
        key = (work_dtype, h, w, frames, torch_flags, self.same_on_batch, self.same_on_frame, self.crop_height,
               self.crop_width, self.horizontal_flip_p, ch.grayscale_p, ch.brightness, ch.contrast, ch.saturation,
               (ah.degrees, ah.translate, ah.scale, ah.shear) if ah else None, self._draw_flip_always, self._draw_gray)
        cache = self.__dict__.setdefault("_spec_cache", {})
        hit = cache.get(key)
        if hit is not None:
            return hit
        sp = _lib.SampleSpec()
        sp.struct_size = _lib.C.sizeof(_lib.SampleSpec)
        sp.frames = frames
        sp.same_on_batch, sp.same_on_frame = int(self.same_on_batch), int(self.same_on_frame)
        sp.img_h, sp.img_w = h, w
        sp.crop_h, sp.crop_w = (self.crop_height or 0), (self.crop_width or 0)
        sp.factor_dtype = _lib.F16 if work_dtype == torch.float16 else _lib.F32
        sp.degrees[:] = ah.degrees if ah else (0.0, 0.0)
        sp.translate[:] = ah.translate if ah and ah.translate is not None else (0.0, 0.0)
        sp.scale[:] = ah.scale if ah and ah.scale is not None else (1.0, 1.0)
        sp.shear[:] = ah.shear if ah and ah.shear is not None else (0.0, 0.0, 0.0, 0.0)
        sp.flip_p, sp.grayscale_p = float(self.horizontal_flip_p), float(ch.grayscale_p)
        sp.brightness[:] = ch.brightness or (1.0, 1.0)
        sp.contrast[:] = ch.contrast or (1.0, 1.0)
        sp.saturation[:] = ch.saturation or (1.0, 1.0)
        draws = 0
        if torch_flags:
            plan, draws = self._draw_plan()
            sp.torch_compat = torch_flags
            sp.draw[:] = plan
            if ah and ah.translate is not None:           # pixels, multiplied in double like the reference
                sp.translate[:] = (float(ah.translate[0] * w), float(ah.translate[1] * h))
        if len(cache) > 32:
            cache.clear()
        cache[key] = (sp, draws)
        return sp, draws

    def _sample_fast(self, lay, work_dtype, want_draws: bool = False, device=None, torch_flags: int = 0, part=None,
                     views: bool = True):
        """Every per-sample parameter of one call from the library's sampler kernel: dict of
        device tensors ``top, left, flip, gray, matrix, brightness, contrast, saturation``
        (``matrix`` None without affine arguments; with ``want_draws`` also ``angle, translate,
        scale, shear``, the draws behind the matrix).  ``torch_flags`` != 0: the values PyTorch's
        generator would give the reference's separate draws (and the generator is advanced
        accordingly); 0: the library's own random stream, seeded by one PyTorch draw.  ``part =
        (start, stop)``: only the samples of that slice of the batch ``lay`` describes (a shard);
        the values are those the whole-batch call gives these samples.  ``views=False``: the
        entries are bare device addresses into one buffer (kept alive under ``"buffer"``) instead of
        tensor views - all the fused launch needs, and a dozen tensor objects fewer per call."""
        from . import _lib
        dev = lay.image.device if device is None else torch.device(device)     # host batches: where to sample
        h, w = lay.image.shape[2:]
        first, total = (0, lay.total) if part is None else (part[0], part[1] - part[0])
        sp, draws = self._static_spec(work_dtype, h, w, lay.frames or 1, torch_flags)
        sp.total, sp.first_sample = total, first
        seed = None
        if torch_flags:
            from . import _torch_rng
            gen = _torch_rng.generator_of(dev)
            if getattr(self, "_torch_state", None) is None or self._torch_state.device != dev:
                self._torch_state = torch.zeros(2, dtype=torch.int64, device=dev)      # (seed, offset) for graph replays
            if torch.cuda.is_current_stream_capturing():
                sp.torch_state = self._torch_state.data_ptr()      # refreshed before every replay (GraphedTransform)
                _torch_rng.CAPTURED.append((self._torch_state, draws))
            else:
                offset = gen.get_offset()
                sp.torch_state = None
                sp.torch_seed, sp.torch_offset = gen.initial_seed(), offset
                gen.set_offset(offset + 4 * draws)                 # what the separate draws would have consumed
        else:
            seed = torch.randint(-2 ** 63, 2 ** 63 - 1, (1,), dtype=torch.int64, device=dev)    # one draw from torch's generator
            sp.seed = seed.data_ptr()
        words = 8 + 3 + (6 if want_draws else 0)                 # fp32 slots per sample: top, left, matrix(6), 3 factors, draws
        buf = torch.empty(total * words * 4 + total * 2, dtype=torch.uint8, device=dev)
        base = buf.data_ptr()
        at = lambda slot: base + 4 * total * slot                # address of fp32 slot `slot`
        sp.top, sp.left, sp.matrix = at(0), at(1), (at(2) if self.has_affine else None)
        sp.brightness_out, sp.contrast_out, sp.saturation_out = at(8), at(9), at(10)
        sp.flip, sp.gray = at(words), at(words) + total
        if want_draws:
            sp.angle_out, sp.translate_out, sp.scale_out, sp.shear_out = at(11), at(12), at(14), at(15)
        else:
            sp.angle_out = sp.translate_out = sp.scale_out = sp.shear_out = None
        _lib.launch_sample_params(sp, dev)
        if not views:
            R = _lib.RawPointer
            return dict(top=R(at(0)), left=R(at(1)), flip=R(at(words)), gray=R(at(words) + total),
                        matrix=R(at(2)) if self.has_affine else None, brightness=R(at(8)), contrast=R(at(9)),
                        saturation=R(at(10)), buffer=buf, seed=seed)
        f32 = buf[: total * words * 4].view(torch.float32)
        u8 = buf[total * words * 4:]
        factors = [f32[(8 + i) * total: (9 + i) * total] for i in range(3)]
        if work_dtype == torch.float16:
            factors = [f.view(torch.float16)[:total] for f in factors]
        out = dict(top=f32[:total], left=f32[total: 2 * total], flip=u8[:total], gray=u8[total:],
                   matrix=f32[2 * total: 8 * total].view(total, 6) if self.has_affine else None,
                   brightness=factors[0], contrast=factors[1], saturation=factors[2])
        if want_draws:
            d = f32[11 * total:]
            out.update(angle=d[:total], translate=d[total: 3 * total].view(total, 2), scale=d[3 * total: 4 * total],
                       shear=d[4 * total: 6 * total].view(total, 2))
        return out

    def _forward_fast(self, lay, torch_flags: int = 0, part=None, image=None):
        """Sampler launch + fused kernel.  ``part`` / ``image``: run only the slice ``part`` of the
        batch that ``lay`` describes, ``image`` holding that slice's samples."""
        from . import _lib
        img = lay.image if image is None else image
        h, w = img.shape[2:]
        if self.crop_height is not None and (self.crop_height > h or self.crop_width > w):
            raise ValueError(f"Crop size ({self.crop_height}, {self.crop_width}) is larger than the image ({h}, {w})")
        out_dtype = self.out_dtype if img.dtype == torch.uint8 else None
        work = F._work_dtype(img, out_dtype)
        p = self._sample_fast(lay, work, torch_flags=torch_flags, part=part, device=img.device, views=False)
        flags = self.color_helper._colour_flags(affine=self.has_affine)
        mean, std = self.color_helper.mean, self.color_helper.std
        bits = ((_lib.APPLY_BRIGHTNESS if flags["brightness"] else 0) | (_lib.APPLY_CONTRAST if flags["contrast"] else 0)
                | (_lib.APPLY_SATURATION if flags["saturation"] else 0) | (_lib.APPLY_GRAYSCALE if flags["grayscale"] else 0)
                | (_lib.APPLY_NORMALIZE if mean is not None else 0))
        return F._run_fused(img, self.crop_height if self.crop_height is not None else h,
                            self.crop_width if self.crop_width is not None else w, p["top"], p["left"], p["flip"], p["matrix"],
                            self.has_affine and F._is_bilinear(self.interpolation), self.fill if self.has_affine else 0.0,
                            p["brightness"], p["contrast"], p["saturation"], p["gray"],
                            F._rounded_triple(mean, work) if mean is not None else None,
                            F._rounded_triple(std, work) if std is not None else None, bits,
                            F._contrast_mode(self.contrast_mode), out_dtype, first_image=part[0] if part else 0)

    def forward(self, image: torch.Tensor) -> torch.Tensor:
        lay = self._layout(image)
        if self.fast_rng:
            return lay.restore(self._forward_fast(lay))
        torch_flags = self._torch_flags(lay, lay.param_device)
        if torch_flags:
            return lay.restore(self._forward_fast(lay, torch_flags))
        h, w = lay.image.shape[2:]
        # (Drawing the parameters on a side stream so that they overlap the previous call's
        # kernel was tried and measured slower: 0.66 ms instead of 0.41 ms per 64-image call.)
        spread = self._spread_all(lay, self._get_params(lay.count, lay.param_device, (h, w)))
        return lay.restore(self._apply(lay.image, spread))

    def forward_host(self, image: torch.Tensor, out: Optional[torch.Tensor] = None, device=None) -> torch.Tensor:
        """Host tensor in, host tensor out (extra; the reference's ``forward`` uploads a host
        batch and leaves the result on the GPU).  Parameters are drawn on ``device`` exactly
        as in ``forward``; the images then flow host -> GPU -> host in slices through the
        library's pipelined entry point, so the copies in both directions overlap the kernel.
        Use pinned memory for ``image`` and ``out`` to get full PCIe speed."""
        from . import _lib
        if image.is_cuda:
            raise ValueError("forward_host takes a host tensor; use forward() for CUDA tensors")
        if not torch.cuda.is_available():
            raise RuntimeError("Triton-Augment requires CUDA, but CUDA is not available.")
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        lay = T._Layout(image, self.same_on_batch, self.same_on_frame, upload=False)
        flat = lay.image.contiguous()
        F_ = F
        if flat.ndim != 4 or flat.shape[1] not in (1, 3) or flat.dtype not in (torch.float32, torch.float16, torch.uint8):
            raise ValueError(f"expected float32/float16/uint8 images with 1 or 3 channels, got {tuple(image.shape)} {image.dtype}")
        work = F._work_dtype(flat, self.out_dtype if flat.dtype == torch.uint8 else None)    # bytes: float32 unless out_dtype
        n, c, h, w = flat.shape
        oh = self.crop_height if self.crop_height is not None else h
        ow = self.crop_width if self.crop_width is not None else w
        matrix = None
        if self.fast_rng:
            fp = self._sample_fast(lay, work, device=dev)
            top, left, flip, b, cf, s, g = (fp[k] for k in ("top", "left", "flip", "brightness", "contrast", "saturation", "gray"))
            if self.has_affine:
                matrix = fp["matrix"].cpu().contiguous()
        else:
            params = self._spread_all(lay, self._get_params(lay.count, dev, (h, w)))
            angle, translate, scale, shear, top, left, flip, b, cf, s, g = params
            if self.has_affine:
                matrix = F_._prepare_affine_matrix_only(n, dev, h, w, angle, translate, scale, shear, None).cpu().contiguous()
        flags = self.color_helper._colour_flags(affine=self.has_affine)
        mean, std = self.color_helper.mean, self.color_helper.std
        bits = ((_lib.APPLY_BRIGHTNESS if flags["brightness"] else 0) | (_lib.APPLY_CONTRAST if flags["contrast"] else 0)
                | (_lib.APPLY_SATURATION if flags["saturation"] else 0) | (_lib.APPLY_GRAYSCALE if flags["grayscale"] else 0)
                | (_lib.APPLY_NORMALIZE if mean is not None else 0))
        if out is None:
            out = torch.empty((n, c, oh, ow), dtype=work, pin_memory=True)
        elif out.is_cuda or not out.is_contiguous() or out.numel() != n * c * oh * ow or out.dtype != work:
            raise ValueError("out must be a contiguous host tensor with the output's size and dtype")
        host = lambda t, dt: t.to(dtype=dt).cpu().contiguous()
        keep = [host(top, torch.float32), host(left, torch.float32), host(flip, torch.uint8), matrix,
                host(b, work), host(cf, work), host(s, work), host(g, torch.uint8)]
        p = _lib.make_params(flat, out.view(n, c, oh, ow), keep[0], keep[1], keep[2], keep[3],
                             self.fill if self.has_affine else 0.0,
                             self.has_affine and F_._is_bilinear(self.interpolation), bits, keep[4], keep[5], keep[6],
                             keep[7], F_._rounded_triple(mean, work) if mean is not None else None,
                             F_._rounded_triple(std, work) if std is not None else None,
                             F_._contrast_mode(self.contrast_mode))
        _lib.launch_fused_host(p, dev)
        return lay.restore(out.view(n, c, oh, ow))

    def __repr__(self):
        ch = self.color_helper
        parts = [f"crop_size=({self.crop_height}, {self.crop_width})" if self.crop_height is not None
                 else "crop_size=None", f"horizontal_flip_p={self.horizontal_flip_p}"]
        if self.has_affine:
            ah = self.affine_helper
            parts.append(f"degrees={ah.degrees}, translate={ah.translate}, scale={ah.scale}, shear={ah.shear}")
        for name in ("brightness", "contrast", "saturation"):
            if getattr(ch, name):
                parts.append(f"{name}={getattr(ch, name)}")
        if ch.grayscale_p > 0:
            parts.append(f"grayscale_p={ch.grayscale_p}")
        if ch.mean is not None:
            parts.append(f"mean={ch.mean}, std={ch.std}")
        return f"{self.__class__.__name__}(" + ", ".join(parts) + ")"
