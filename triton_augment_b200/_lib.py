"""ctypes binding of libta_b200.so (C ABI in include/ta_b200.h).

There is no fallback: if the library is missing or the device is not a B200-class
GPU the call raises.  Pointers handed to the library are raw ``data_ptr()`` values
and the stream is torch's current stream on the tensor's device.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("TA_B200_LIB") or os.path.join(_HERE, "lib", "libta_b200.so")

ABI_VERSION = 1
F32, F16, U8, U8_F16 = 0, 1, 2, 3       # U8 / U8_F16: bytes in (read as value / 255), float32 / float16 out
NEAREST, BILINEAR = 0, 1
CONTRAST_FAST, CONTRAST_MEAN = 0, 1
ERR_TIMEOUT = -9
APPLY_BRIGHTNESS, APPLY_CONTRAST, APPLY_SATURATION, APPLY_GRAYSCALE, APPLY_NORMALIZE = 1, 2, 4, 8, 16

# Every symbol include/ta_b200.h declares.
SYMBOLS = (
    "ta_b200_abi_version", "ta_b200_last_error", "ta_b200_fused_augment", "ta_b200_fused_augment_at", "ta_b200_gray_mean",
    "ta_b200_gray_mean_scratch_bytes", "ta_b200_gray_mean_static", "ta_b200_fused_augment_host", "ta_b200_inverse_affine_matrix",
    "ta_b200_debug_counters", "ta_b200_debug_fused_checked", "ta_b200_debug_tile_footprint",
    "ta_b200_debug_crop_path", "ta_b200_debug_host_upload", "ta_b200_sample_params",
    "ta_b200_debug_tile_shape", "ta_b200_status", "ta_b200_host_release", "ta_b200_debug_wait",
    "ta_b200_fused_augment_mean", "ta_b200_fused_augment_mean_scratch_bytes", "ta_b200_mean_path",
    "ta_b200_store_words", "ta_b200_debug_tile_height",
)


class FusedParams(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("dtype", C.c_int32),
        ("n", C.c_int32), ("c", C.c_int32), ("h", C.c_int32), ("w", C.c_int32),
        ("oh", C.c_int32), ("ow", C.c_int32),
        ("inp", C.c_void_p), ("out", C.c_void_p),
        ("top", C.c_void_p), ("left", C.c_void_p), ("flip", C.c_void_p), ("matrix", C.c_void_p),
        ("fill", C.c_float), ("interp", C.c_int32), ("apply", C.c_uint32),
        ("brightness", C.c_void_p), ("contrast", C.c_void_p), ("saturation", C.c_void_p), ("gray", C.c_void_p),
        ("mean", C.c_float * 3), ("std", C.c_float * 3),
        ("contrast_mode", C.c_int32), ("gray_mean", C.c_void_p),
        ("fill_rgb", C.c_float * 3), ("fill_per_channel", C.c_uint32),
    ]


class SampleSpec(C.Structure):
    """ta_b200_sample_spec of include/ta_b200.h."""
    _fields_ = [
        ("struct_size", C.c_uint32), ("total", C.c_int32), ("frames", C.c_int32),
        ("same_on_batch", C.c_int32), ("same_on_frame", C.c_int32),
        ("img_h", C.c_int32), ("img_w", C.c_int32), ("crop_h", C.c_int32), ("crop_w", C.c_int32),
        ("factor_dtype", C.c_int32),
        ("degrees", C.c_float * 2), ("translate", C.c_float * 2), ("scale", C.c_float * 2), ("shear", C.c_float * 4),
        ("flip_p", C.c_float), ("grayscale_p", C.c_float),
        ("brightness", C.c_float * 2), ("contrast", C.c_float * 2), ("saturation", C.c_float * 2),
        ("seed", C.c_void_p), ("top", C.c_void_p), ("left", C.c_void_p), ("flip", C.c_void_p), ("gray", C.c_void_p),
        ("matrix", C.c_void_p), ("brightness_out", C.c_void_p), ("contrast_out", C.c_void_p),
        ("saturation_out", C.c_void_p), ("angle_out", C.c_void_p), ("translate_out", C.c_void_p),
        ("scale_out", C.c_void_p), ("shear_out", C.c_void_p),
        ("torch_compat", C.c_int32), ("draw", C.c_int8 * 13), ("pad_", C.c_int8 * 3),
        ("torch_seed", C.c_uint64), ("torch_offset", C.c_uint64), ("torch_state", C.c_void_p),
        ("first_sample", C.c_int32), ("pad2_", C.c_int32),
    ]


class LibraryError(RuntimeError):
    """A call into libta_b200.so returned a negative status."""


_lib = None


def load():
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m triton_augment_b200.build` "
            "(needs nvcc; the library targets sm_100a and has no CPU or other-GPU fallback)")
    lib = C.CDLL(LIB_PATH)
    lib.ta_b200_abi_version.restype = C.c_int
    lib.ta_b200_last_error.restype = C.c_char_p
    lib.ta_b200_fused_augment.argtypes = [C.POINTER(FusedParams), C.c_void_p]
    lib.ta_b200_fused_augment.restype = C.c_int
    lib.ta_b200_debug_fused_checked.argtypes = [C.POINTER(FusedParams), C.c_void_p]
    lib.ta_b200_debug_fused_checked.restype = C.c_int
    lib.ta_b200_fused_augment_at.argtypes = [C.POINTER(FusedParams), C.c_uint32, C.c_void_p]
    lib.ta_b200_fused_augment_at.restype = C.c_int
    lib.ta_b200_gray_mean.argtypes = [C.POINTER(FusedParams), C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    lib.ta_b200_gray_mean.restype = C.c_int
    lib.ta_b200_gray_mean_scratch_bytes.argtypes = [C.POINTER(FusedParams)]
    lib.ta_b200_gray_mean_scratch_bytes.restype = C.c_size_t
    lib.ta_b200_gray_mean_static.argtypes = [C.POINTER(FusedParams), C.c_void_p, C.c_void_p]
    lib.ta_b200_gray_mean_static.restype = C.c_int
    lib.ta_b200_fused_augment_host.argtypes = [C.POINTER(FusedParams)]
    lib.ta_b200_fused_augment_host.restype = C.c_int
    lib.ta_b200_inverse_affine_matrix.argtypes = [C.c_int32] + [C.c_void_p] * 7
    lib.ta_b200_inverse_affine_matrix.restype = C.c_int
    lib.ta_b200_sample_params.argtypes = [C.POINTER(SampleSpec), C.c_void_p]
    lib.ta_b200_sample_params.restype = C.c_int
    lib.ta_b200_debug_crop_path.argtypes = [C.c_int32]
    lib.ta_b200_debug_crop_path.restype = C.c_int
    lib.ta_b200_debug_tile_height.argtypes = [C.c_int32]
    lib.ta_b200_debug_tile_height.restype = C.c_int
    lib.ta_b200_debug_host_upload.argtypes = [C.c_int32]
    lib.ta_b200_debug_host_upload.restype = C.c_int
    lib.ta_b200_debug_counters.argtypes = [C.POINTER(C.c_uint64), C.c_int]
    lib.ta_b200_debug_counters.restype = C.c_int
    lib.ta_b200_debug_tile_footprint.argtypes = (
        [C.c_int32] * 6 + [C.c_float, C.c_float, C.c_int32, C.POINTER(C.c_float), C.c_int32, C.c_int32,
                           C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.c_int32])
    lib.ta_b200_debug_tile_footprint.restype = C.c_int
    lib.ta_b200_debug_tile_shape.argtypes = [C.POINTER(C.c_int32)]
    lib.ta_b200_debug_tile_shape.restype = None
    lib.ta_b200_fused_augment_mean.argtypes = [C.POINTER(FusedParams), C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    lib.ta_b200_fused_augment_mean.restype = C.c_int
    lib.ta_b200_fused_augment_mean_scratch_bytes.argtypes = [C.POINTER(FusedParams)]
    lib.ta_b200_fused_augment_mean_scratch_bytes.restype = C.c_size_t
    lib.ta_b200_mean_path.argtypes = [C.c_int32]
    lib.ta_b200_mean_path.restype = C.c_int
    lib.ta_b200_store_words.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_void_p]
    lib.ta_b200_store_words.restype = C.c_int
    lib.ta_b200_status.argtypes = [C.c_int]
    lib.ta_b200_status.restype = C.c_int
    lib.ta_b200_host_release.argtypes = []
    lib.ta_b200_host_release.restype = C.c_int
    lib.ta_b200_debug_wait.argtypes = [C.c_uint64, C.c_int32]
    lib.ta_b200_debug_wait.restype = C.c_int
    if lib.ta_b200_abi_version() != ABI_VERSION:
        raise RuntimeError(f"libta_b200.so has ABI {lib.ta_b200_abi_version()}, this package expects {ABI_VERSION}")
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().ta_b200_last_error().decode("utf-8", "replace")
        raise LibraryError(f"{what} failed with status {rc}: {msg}")


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


class RawPointer:
    """A device address that quacks like a tensor for make_params() (`data_ptr()`): lets a caller
    carve one allocation into many vectors without creating a tensor view per vector."""
    __slots__ = ("address",)

    def __init__(self, address: int):
        self.address = address

    def data_ptr(self) -> int:
        return self.address


def _index_of(device):
    """Device index of a torch.device / "cuda:1" / 1 / None (None: whichever device is current)."""
    if device is None or isinstance(device, int):
        return device
    if not isinstance(device, torch.device):
        device = torch.device(device)
    return device.index


class _OnDevice:
    """`with torch.cuda.device(d)` only when d is not current already (the switch costs microseconds)."""
    __slots__ = ("guard",)

    def __init__(self, device):
        idx = _index_of(device)
        self.guard = None if idx is None or idx == torch.cuda.current_device() else torch.cuda.device(idx)

    def __enter__(self):
        if self.guard is not None:
            self.guard.__enter__()

    def __exit__(self, *a):
        if self.guard is not None:
            self.guard.__exit__(*a)


try:
    _raw_stream = torch._C._cuda_getCurrentRawStream          # the current stream's handle without a Stream object
except AttributeError:                                        # pragma: no cover - older or newer torch
    _raw_stream = None


def _stream(device) -> "C.c_void_p":
    """torch's current stream on `device` as a cudaStream_t."""
    idx = _index_of(device)
    if idx is None:
        idx = torch.cuda.current_device()
    if _raw_stream is not None:
        return C.c_void_p(_raw_stream(idx))
    return C.c_void_p(torch.cuda.current_stream(idx).cuda_stream)


def make_params(image, out, top, left, flip, matrix, fill, bilinear, apply_bits, brightness, contrast,
                saturation, gray, mean, std, contrast_mode=CONTRAST_FAST, gray_mean=None) -> FusedParams:
    """Fill a FusedParams from tensors (device or host; the caller picks the entry point)."""
    p = FusedParams()
    p.struct_size = C.sizeof(FusedParams)
    if image.dtype == torch.uint8:
        p.dtype = U8_F16 if out.dtype == torch.float16 else U8
    else:
        p.dtype = F16 if image.dtype == torch.float16 else F32
    p.n, p.c, p.h, p.w = image.shape
    p.oh, p.ow = out.shape[2], out.shape[3]
    p.inp, p.out = _ptr(image), _ptr(out)
    p.top, p.left, p.flip, p.matrix = _ptr(top), _ptr(left), _ptr(flip), _ptr(matrix)
    if isinstance(fill, (list, tuple)):               # per channel (1 value: all channels)
        vals = [float(v) for v in fill]
        if len(vals) not in (1, 3):
            raise ValueError(f"fill must be a number or a sequence of 1 or 3 numbers, got {len(vals)} values")
        vals = vals * 3 if len(vals) == 1 else vals
        p.fill = vals[0]
        p.fill_per_channel = 1
        for i in range(3):
            p.fill_rgb[i] = vals[i]
    else:
        p.fill = float(fill)
    p.interp = BILINEAR if bilinear else NEAREST
    p.apply = int(apply_bits)
    p.brightness, p.contrast, p.saturation, p.gray = _ptr(brightness), _ptr(contrast), _ptr(saturation), _ptr(gray)
    m = mean if mean is not None else (0.0, 0.0, 0.0)
    s = std if std is not None else (1.0, 1.0, 1.0)
    for i in range(3):
        p.mean[i] = float(m[i])
        p.std[i] = float(s[i])
    p.contrast_mode = int(contrast_mode)
    p.gray_mean = _ptr(gray_mean)
    return p


def launch_fused(params: FusedParams, device: torch.device, checked: bool = False, first_image: int = 0) -> None:
    """``first_image``: index of the first image within the batch this call is a piece of (see
    ta_b200_fused_augment_at in the header)."""
    lib = load()
    with _OnDevice(device):
        stream = _stream(device)
        if checked:
            check(lib.ta_b200_debug_fused_checked(C.byref(params), stream), "ta_b200_fused_augment")
        elif first_image:
            check(lib.ta_b200_fused_augment_at(C.byref(params), int(first_image), stream), "ta_b200_fused_augment_at")
        else:
            check(lib.ta_b200_fused_augment(C.byref(params), stream), "ta_b200_fused_augment")


def launch_fused_host(params: FusedParams, device: torch.device) -> None:
    """Host-buffer entry point: every pointer in ``params`` is a host pointer; uploads, runs
    and downloads slice by slice on ``device`` and returns when the output is complete."""
    with torch.cuda.device(device):
        check(load().ta_b200_fused_augment_host(C.byref(params)), "ta_b200_fused_augment_host")


def launch_gray_mean(params: FusedParams, device: torch.device) -> torch.Tensor:
    """Run the grayscale-mean pre-pass; returns the fp32 ``[n]`` means on ``device``."""
    lib = load()
    with torch.cuda.device(device):
        need = int(lib.ta_b200_gray_mean_scratch_bytes(C.byref(params)))
        scratch = torch.empty(need, dtype=torch.uint8, device=device)
        means = torch.empty(params.n, dtype=torch.float32, device=device)
        stream = C.c_void_p(torch.cuda.current_stream(device).cuda_stream)
        check(lib.ta_b200_gray_mean(C.byref(params), _ptr(means), _ptr(scratch), need, stream), "ta_b200_gray_mean")
    return means


def launch_fused_mean(params: FusedParams, device: torch.device) -> torch.Tensor:
    """Mean-mode contrast in one library call (one cooperative launch where the images allow it):
    reduction + fused pass; returns the fp32 ``[n]`` means it computed on the way."""
    lib = load()
    with torch.cuda.device(device):
        need = int(lib.ta_b200_fused_augment_mean_scratch_bytes(C.byref(params)))
        scratch = torch.empty(need, dtype=torch.uint8, device=device)
        means = torch.empty(params.n, dtype=torch.float32, device=device)
        stream = C.c_void_p(torch.cuda.current_stream(device).cuda_stream)
        check(lib.ta_b200_fused_augment_mean(C.byref(params), _ptr(means), _ptr(scratch), need, stream),
              "ta_b200_fused_augment_mean")
    return means


def mean_path(one_launch) -> None:
    """ta_b200_fused_augment_mean: 0 two launches (default), 1 / 2 one cooperative launch, the fused pass one / two images behind."""
    check(load().ta_b200_mean_path(int(one_launch)), "ta_b200_mean_path")


def inverse_affine_matrix(center, angle, translate, scale, shear) -> torch.Tensor:
    """``[n, 6]`` inverse affine matrices from device fp32 parameter tensors in one launch."""
    dev = angle.device
    n = angle.shape[0]
    args = [t.contiguous() for t in (center, angle, translate, scale, shear)]
    out = torch.empty(n, 6, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        check(load().ta_b200_inverse_affine_matrix(n, *[_ptr(t) for t in args], _ptr(out), stream),
              "ta_b200_inverse_affine_matrix")
    return out


def launch_sample_params(spec: SampleSpec, device: torch.device) -> None:
    """Enqueue the fused parameter sampler on torch's current stream of ``device``."""
    with _OnDevice(device):
        check(load().ta_b200_sample_params(C.byref(spec), _stream(device)), "ta_b200_sample_params")


def store_words(dst: torch.Tensor, a: int, b: int) -> None:
    """dst[0], dst[1] = a, b (a 2-element int64 device tensor) on torch's current stream."""
    with torch.cuda.device(dst.device):
        stream = C.c_void_p(torch.cuda.current_stream(dst.device).cuda_stream)
        check(load().ta_b200_store_words(_ptr(dst), int(a) & (2 ** 64 - 1), int(b) & (2 ** 64 - 1), stream), "ta_b200_store_words")


def crop_path(path: int) -> None:
    """0: pick the kernel for matrix-free calls by size, 1: crop kernels only, 2: staged kernel (tests)."""
    check(load().ta_b200_debug_crop_path(int(path)), "ta_b200_debug_crop_path")


def tile_height(rows: int) -> None:
    """Tile height of the staged kernel for float32 / float16 images: 0 = by output height, 32 or 64 = forced (tests)."""
    check(load().ta_b200_debug_tile_height(int(rows)), "ta_b200_debug_tile_height")


def host_upload(mode: int) -> None:
    """Host-buffer path: 1 = upload the box of each large image that is read where that is cheaper
    (default), 0 = whole images, 2 = boxes for every call on large images (tests)."""
    check(load().ta_b200_debug_host_upload(int(mode)), "ta_b200_debug_host_upload")


def status(device=None, acknowledge: bool = False) -> bool:
    """True if a kernel of the library gave up a bounded wait on ``device`` (default: the current
    one) since the last acknowledged check, i.e. some launch left its output incomplete.  Does not
    synchronise: call it after your own synchronisation point."""
    with torch.cuda.device(device):
        rc = load().ta_b200_status(int(acknowledge))
    if rc not in (0, ERR_TIMEOUT):
        check(rc, "ta_b200_status")
    return rc == ERR_TIMEOUT


def check_status(device=None) -> None:
    """Raise ``LibraryError`` (and acknowledge) if ``status(device)`` is raised."""
    if status(device, acknowledge=True):
        raise LibraryError("a kernel of libta_b200 gave up a bounded barrier wait on this device: "
                           "outputs produced since the last check may be incomplete")


def host_release(device=None) -> None:
    """Free the staging buffers and streams the host-buffer entry point keeps on ``device``."""
    with torch.cuda.device(device):
        check(load().ta_b200_host_release(), "ta_b200_host_release")


def debug_wait(limit_ns: int = 0, skip_arrive_tile: int = -1) -> None:
    """Barrier wait limit of the staged kernels and the tile whose barrier is never signalled (tests)."""
    check(load().ta_b200_debug_wait(int(limit_ns), int(skip_arrive_tile)), "ta_b200_debug_wait")


def debug_counters(reset: bool = False):
    """(staged tiles, direct tiles, staging violations, barrier time-outs) on the current device."""
    buf = (C.c_uint64 * 4)()
    check(load().ta_b200_debug_counters(buf, int(reset)), "ta_b200_debug_counters")
    return tuple(int(x) for x in buf)


def tile_shape():
    """(tile width, tile height and source-row capacity for float pixels, staged row pitch for 4-, 2-,
    1-byte elements, tile height and source-row capacity for half pixels)."""
    buf = (C.c_int32 * 8)()
    load().ta_b200_debug_tile_shape(buf)
    return tuple(int(x) for x in buf)


def tile_footprint(bilinear, elem_bytes, h, w, oh, ow, top, left, flip, matrix, tile_x, tile_y):
    """Host-side evaluation of the staged kernel's footprint for one tile (tests)."""
    cap = max(tile_shape()[2], tile_shape()[7])
    row0 = C.c_int32(0)
    xs = (C.c_int32 * cap)()
    xe = (C.c_int32 * cap)()
    m = (C.c_float * 6)(*[float(v) for v in matrix])
    rows = load().ta_b200_debug_tile_footprint(int(bool(bilinear)), elem_bytes, h, w, oh, ow, float(top), float(left),
                                               int(bool(flip)), m, tile_x, tile_y, C.byref(row0), xs, xe, cap)
    return rows, int(row0.value), [int(v) for v in xs[:rows]], [int(v) for v in xe[:rows]]
