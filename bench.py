"""Benchmark of the fused augmentation hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--interp bilinear|nearest] [--impl reference]

Headline workload (`value`, `roofline`, `e2e`): the "ultimate fusion with affine" configuration -
64 x 3 x 1280 x 1280 fp32 images, random affine (15 deg, translate 0.1, scale 0.9-1.1, shear 5) +
crop 1024 + flip 0.5 + colour jitter 0.2 + grayscale 0.1 + ImageNet normalize - on synthetic
uniform[0,1) pixels.  One step = one direct call of ``TritonFusedAugment.forward`` on the batch
(parameter sampling included); `graph_replay` is the same call captured once and replayed.  With N > 1 (torchrun, one process per GPU) every rank runs the
same workload on its own GPU: images are independent, there is no collective on the data path,
scaling is weak.

Every number is the median over >= 10 timed blocks of K steps each (CUDA events around a block,
barrier + synchronize on both sides of every block); `timing` gives min / median / max.

Also in the line: `configs` (the other benchmark configurations: colour only, crop + flip +
colour, fp16 affine, video, the 4096-image batch - kernel alone, class forward called directly
and replayed as a CUDA graph, rotating over buffer sets where a configuration fits the L2),
`c5b_sharded` (the 4096-image batch cut into one slice per rank, strong scaling, with a SHA-256
check of every rank's output against a single-GPU run of the same slice), `triton_reference`
(the unmodified reference package timed on the same tensors on the same GPU, N = 1 only) and
`e2e_copy_control` (plain pinned copies of the end-to-end path's bytes).

Prints ONE JSON line (rank 0).  ``--impl reference`` times the CPU restatement of the
reference's kernel (oracle/) on the host cores instead, on a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MEAN, STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)
N_IMG, SRC, CROP = 64, 1280, 1024
METRIC, UNIT = "fused-augment throughput, 1280x1280 -> 1024x1024 affine config", "images/s"
L2_BYTES = 126e6
MIN_TIMED_MS = 150.0          # every measurement times at least this much GPU work ...
MIN_BLOCKS = 10               # ... in at least this many blocks of `steps` steps
# dram__bytes_read.sum + dram__bytes_write.sum of one full 64-image affine-kernel launch (single-pass
# ncu capture with `--profile-case 64`, summarised in profiles/affine_kernel_c3_fp32.md), divided by 64.
NCU_TRAFFIC_PER_IMAGE = {"bilinear": (830525696 + 759459840) / 64, "nearest": (829769984 + 756168704) / 64}


def workload_name(interp):
    """`config.workload` of both arms (this one and ``--impl reference``)."""
    return (f"C3 affine({interp})+crop{CROP}+flip+colour+gray+normalize, N={N_IMG} per GPU, 3x{SRC}x{SRC} fp32")


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def make_transform(interp, fast_rng=False, contrast_mode="fast", out_dtype=None, module=None):
    """The headline transform; `module` = the reference package builds the reference's class with
    the same arguments (it has no fast_rng / contrast_mode / out_dtype)."""
    kw = dict(crop_size=CROP, horizontal_flip_p=0.5, degrees=15, translate=(0.1, 0.1), scale=(0.9, 1.1), shear=5,
              interpolation=interp, brightness=0.2, contrast=0.2, saturation=0.2, grayscale_p=0.1, mean=MEAN, std=STD)
    if module is not None:
        return module.TritonFusedAugment(**kw)
    import triton_augment_b200 as ta
    return ta.TritonFusedAugment(fast_rng=fast_rng, contrast_mode=contrast_mode, out_dtype=out_dtype, **kw)


# ----------------------------------------------------------------------------- host placement
def bind_to_gpu_numa_node(index):
    """Pin this process to the CPUs of the NUMA node the GPU hangs off, BEFORE any host buffer is
    allocated or pinned, so that pinned pages are first touched on that node and the copies do
    not cross the socket interconnect.  Returns what was done (goes into the JSON line)."""
    try:
        out = subprocess.run(["nvidia-smi", "--query-gpu=pci.bus_id", "--format=csv,noheader", "-i", str(index)],
                             stdout=subprocess.PIPE, text=True, timeout=20).stdout.strip()
        bdf = out.lower()
        if bdf.count(":") == 2 and len(bdf.split(":")[0]) == 8:       # nvidia-smi prints an 8-digit domain
            bdf = bdf[4:]
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return {"bound": False, "why": f"GPU {index} ({bdf}) reports no NUMA node"}
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0) & cpus
        if not allowed:
            return {"bound": False, "why": f"no allowed CPU on node {node}", "node": node}
        os.sched_setaffinity(0, allowed)
        return {"bound": True, "node": node, "cpus": len(allowed), "pci": bdf}
    except Exception as e:                                            # containers often hide sysfs: report, go on
        return {"bound": False, "why": f"{type(e).__name__}: {e}"[:120]}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,clocks.mem,power.draw,utilization.gpu")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=lambda: self.rows.extend(self.proc.stdout), daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, busy_sm, mem, power, mx, reasons = [], [], [], [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            f = [x.strip() for x in r.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])); mx = max(mx, float(f[1]))
            except ValueError:
                continue
            reasons.update(n for n, v in zip(names, f[2:6]) if v.lower().startswith("active"))
            try:
                mem.append(float(f[6])); power.append(float(f[7]))
                if float(f[8]) >= 50:
                    busy_sm.append(sm[-1])
            except (ValueError, IndexError):
                pass
        under_load = busy_sm or sm                  # samples taken while the GPU was busy, if any
        return {"sm_mhz": statistics.median(under_load) if under_load else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm), "samples_under_load": len(busy_sm),
                "sm_mhz_min_under_load": min(under_load) if under_load else None,
                "mem_mhz_min": min(mem) if mem else None, "power_w_max": max(power) if power else None,
                "power_w_median": statistics.median(power) if power else None}


# ----------------------------------------------------------------------------- timing
class Timer:
    """W warm-up calls, then blocks of K calls between CUDA events on the current stream.  The
    number of blocks is chosen so that at least MIN_TIMED_MS of device time is measured, never
    fewer than MIN_BLOCKS; every block has a barrier and a synchronize on both sides.  Ranks
    agree on the block count (rank 0 decides), so the barriers line up."""

    def __init__(self, steps, warmup, barrier=None, agree=None):
        self.steps, self.warmup, self.barrier, self.agree = steps, warmup, barrier, agree
        self.fixed_blocks = 0
        self.total_ms = 0.0
        self.launch_blocks = 0

    def __call__(self, fn):
        for _ in range(self.warmup):
            fn()
        torch.cuda.synchronize()
        blocks, times = (self.fixed_blocks or MIN_BLOCKS), []
        i = 0
        while i < blocks:
            if self.barrier:
                self.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(self.steps):
                fn()
            b.record()
            torch.cuda.synchronize()
            if self.barrier:
                self.barrier()
            times.append(a.elapsed_time(b))
            if i == 0 and not self.fixed_blocks:          # size the run from the first block
                want = int(min(200, max(MIN_BLOCKS, math.ceil(MIN_TIMED_MS / max(times[0], 1e-3)))))
                blocks = self.agree(want) if self.agree else want
            i += 1
        self.total_ms += sum(times)
        self.launch_blocks += len(times)
        per = sorted(t / self.steps for t in times)
        return {"ms": statistics.median(per), "min_ms": per[0], "max_ms": per[-1], "blocks": len(per),
                "timed_ms": round(sum(times), 2)}


def wall_timed(fn, steps, warmup, barrier=None):
    """Host-synchronous calls (the end-to-end path returns when the host buffer is complete):
    wall clock per call, median over `steps` calls."""
    for _ in range(warmup):
        fn()
    if barrier:
        barrier()
    per = []
    for _ in range(steps):
        t0 = time.perf_counter()
        fn()
        per.append(1e3 * (time.perf_counter() - t0))
    if barrier:
        barrier()
    per.sort()
    return {"ms": statistics.median(per), "min_ms": per[0], "max_ms": per[-1], "calls": len(per)}


# ----------------------------------------------------------------------------- CPU arms
def cpu_oracle_rate(interp, sample, threads=0):
    """images/s of the CPU restatement of the reference kernel on `sample` images of the workload."""
    import numpy as np
    from oracle import fused_oracle as O
    rng = np.random.default_rng(0)
    img = rng.random((sample, 3, SRC, SRC), dtype=np.float32)
    ang = np.deg2rad(rng.uniform(-15, 15, sample)); s = rng.uniform(0.9, 1.1, sample)
    tx, ty = rng.uniform(-128, 128, sample), rng.uniform(-128, 128, sample)
    m = np.stack([np.cos(ang) / s, np.sin(ang) / s, -tx, -np.sin(ang) / s, np.cos(ang) / s, -ty], 1).astype(np.float32)
    top = rng.integers(0, SRC - CROP + 1, sample); left = rng.integers(0, SRC - CROP + 1, sample)
    vec = dict(flip=rng.random(sample) < 0.5, matrix=m, brightness=rng.uniform(.8, 1.2, sample),
               contrast=rng.uniform(.8, 1.2, sample), saturation=rng.uniform(.8, 1.2, sample),
               grayscale=rng.random(sample) < 0.1)
    fixed = dict(interpolation=interp, mean=MEAN, std=STD, threads=threads)
    O.fused_augment(img[:1], top[:1], left[:1], CROP, CROP, **{k: v[:1] for k, v in vec.items()}, **fixed)   # warm
    done, dt = 0, 0.0
    while dt < 2.0 and done < 16 * sample:          # repeat the sample until ~2 s of work has been timed
        t0 = time.perf_counter()
        O.fused_augment(img, top, left, CROP, CROP, **vec, **fixed)
        dt += time.perf_counter() - t0
        done += sample
    return done / dt, (threads or O.max_threads())


def torchvision_cpu_rate(interp, sample):
    """images/s of the torchvision.transforms.v2 functional composition of the same operations
    on the host cores (per-image loop: the parameters differ per image)."""
    import torchvision.transforms.v2.functional as tvF
    from torchvision.transforms import InterpolationMode as IM
    g = torch.Generator().manual_seed(0)
    imgs = torch.rand(sample, 3, SRC, SRC, generator=g)
    mode = IM.BILINEAR if interp == "bilinear" else IM.NEAREST

    def one(i):
        u = lambda lo, hi: float(torch.empty(1).uniform_(lo, hi, generator=g))
        x = tvF.affine(imgs[i], angle=u(-15, 15), translate=[u(-128, 128), u(-128, 128)], scale=u(0.9, 1.1),
                       shear=[u(-5, 5), 0.0], interpolation=mode, fill=0.0)
        t, l = int(u(0, SRC - CROP)), int(u(0, SRC - CROP))
        x = tvF.crop(x, t, l, CROP, CROP)
        if u(0, 1) < 0.5:
            x = tvF.horizontal_flip(x)
        x = tvF.adjust_brightness(x, u(0.8, 1.2))
        x = tvF.adjust_contrast(x, u(0.8, 1.2))
        x = tvF.adjust_saturation(x, u(0.8, 1.2))
        if u(0, 1) < 0.1:
            x = tvF.rgb_to_grayscale(x, 3)
        return tvF.normalize(x, MEAN, STD)

    one(0)
    t0 = time.perf_counter()
    for i in range(sample):
        one(i)
    return sample / (time.perf_counter() - t0), torch.get_num_threads()


def run_reference_arm(args, rank):
    """The reference's own path has no CPU implementation; its restatement in oracle/ is timed
    on the host cores with all threads.  Rank 0 only."""
    if rank != 0:
        return
    sample = 4
    rates = []
    for _ in range(max(1, min(args.steps, 3))):
        r, cores = cpu_oracle_rate(args.interp, sample)
        rates.append(r)
    value = statistics.median(rates)
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * N_IMG / value, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(args.interp)},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                             "sample": f"{sample} of {N_IMG} images per step, CPU restatement of the reference kernel, all host threads"},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- kernel alone
def fixed_params(aug, img, exact_contrast=False):
    """Parameters drawn once -> a filled ta_b200_fused_params for `img` (plus the tensors it points to)."""
    from triton_augment_b200 import _lib, functional as F
    from triton_augment_b200.transforms import _Layout
    dev = img.device
    lay = _Layout(img, getattr(aug, "same_on_batch", False), getattr(aug, "same_on_frame", True))
    flat = lay.image
    n, c, src_h, src_w = flat.shape
    if hasattr(aug, "_spread_all"):
        angle, translate, scale, shear, top, left, flip, b, cf, s, g = aug._spread_all(
            lay, aug._get_params(lay.count, dev, (src_h, src_w)))
        has_affine, interp = aug.has_affine, getattr(aug, "interpolation", "nearest")
        oh = aug.crop_height if aug.crop_height is not None else src_h
        ow = aug.crop_width if aug.crop_width is not None else src_w
        helper = aug.color_helper
    else:                                                   # TritonColorJitterNormalize: colour only
        b, cf, s, g = (lay.spread(p) for p in aug._get_params(lay.count, dev))
        top = left = torch.zeros(n, device=dev)
        flip = torch.zeros(n, dtype=torch.bool, device=dev)
        has_affine, interp, oh, ow, helper = False, "nearest", src_h, src_w, aug
    matrix = None
    if has_affine:
        matrix = F._prepare_affine_matrix_only(n, dev, src_h, src_w, angle, translate, scale, shear, None).contiguous()
    work = F._work_dtype(flat, getattr(aug, "out_dtype", None) if flat.dtype == torch.uint8 else None)
    out = torch.empty(n, c, oh, ow, device=dev, dtype=work)
    tensors = [flat, out, top.float(), left.float(), flip, matrix, b.to(work), cf.to(work), s.to(work), g]
    p = _lib.make_params(flat, out, tensors[2], tensors[3], flip, matrix, 0.0, has_affine and F._is_bilinear(interp), 31,
                         tensors[6], tensors[7], tensors[8], g, F._rounded_triple(helper.mean, work),
                         F._rounded_triple(helper.std, work))
    if exact_contrast:
        p.contrast_mode = _lib.CONTRAST_MEAN
    return p, tensors


def kernel_only(aug, imgs, timer, exact_contrast=False):
    """The fused kernel alone (parameters drawn once, then fixed), round-robin over `imgs` (one
    parameter block and one output per input, so a rotation never re-reads or re-writes lines
    that are still in L2).  ``exact_contrast``: mean reduction + fused kernel in mean mode."""
    from triton_augment_b200 import _lib
    sets = [fixed_params(aug, img, exact_contrast) for img in imgs]
    dev = imgs[0].device
    state = {"i": 0}

    def one():
        p, keep = sets[state["i"] % len(sets)]
        state["i"] += 1
        if exact_contrast:
            _lib.launch_fused_mean(p, dev)                  # reduction + fused pass (one cooperative launch)
        else:
            _lib.launch_fused(p, dev)
    return timer(one)


# The benchmark configurations besides the headline one: images (or videos x frames), source size,
# crop, dtype, affine, interpolation.
CONFIGS = {
    "c1": dict(shape=(32, 3, 224, 224), crop=None, dtype=torch.float32, affine=False,
               what="colour jitter + grayscale + normalize, N=32, 3x224x224 fp32"),
    "c2": dict(shape=(256, 3, 224, 224), crop=112, dtype=torch.float32, affine=False,
               what="crop 112 + flip + colour + grayscale + normalize, N=256, 3x224x224 fp32"),
    "c4": dict(shape=(512, 3, 512, 512), crop=448, dtype=torch.float16, affine=True, interp="nearest",
               what="fp16 affine(nearest) + crop 448 + flip + colour + grayscale + normalize, N=512, 3x512x512"),
    "c5a": dict(shape=(8, 16, 3, 224, 224), crop=112, dtype=torch.float32, affine=False,
                what="video [8,16,3,224,224] fp32, same_on_frame, crop 112 + flip + colour + normalize"),
    "c5b": dict(shape=(4096, 3, 224, 224), crop=112, dtype=torch.float32, affine=False,
                what="crop 112 + flip + colour + grayscale + normalize, N=4096, 3x224x224 fp32"),
}
# for profiler captures only (--profile-config)
PROFILE_ONLY = {
    "c3": dict(shape=(N_IMG, 3, SRC, SRC), crop=CROP, dtype=torch.float32, affine=True),
    "c3exact": dict(shape=(N_IMG, 3, SRC, SRC), crop=CROP, dtype=torch.float32, affine=True),   # + mean pre-pass
    "c3u8": dict(shape=(N_IMG, 3, SRC, SRC), crop=CROP, dtype=torch.uint8, affine=True),       # bytes in, float32 out
    "c3u8h": dict(shape=(N_IMG, 3, SRC, SRC), crop=CROP, dtype=torch.uint8, affine=True),      # bytes in, float16 out
}


def config_transform(name, cfg, interp=None):
    import triton_augment_b200 as ta
    colour = dict(brightness=0.2, contrast=0.2, saturation=0.2, grayscale_p=0.1, mean=MEAN, std=STD)
    if name == "c1":
        return ta.TritonColorJitterNormalize(**colour)
    kw = {}
    if cfg["affine"]:
        kw = dict(degrees=15, translate=(0.1, 0.1), scale=(0.9, 1.1), shear=5, interpolation=interp or cfg.get("interp", "bilinear"))
    return ta.TritonFusedAugment(crop_size=cfg["crop"], horizontal_flip_p=0.5, same_on_frame=True,
                                 out_dtype=torch.float16 if name == "c3u8h" else None, **colour, **kw)


def config_images(cfg, dev, sets, seed=0):
    g = torch.Generator(device=dev).manual_seed(seed)
    if cfg["dtype"] == torch.uint8:
        return [torch.randint(0, 256, cfg["shape"], device=dev, dtype=torch.uint8, generator=g) for _ in range(sets)]
    return [torch.rand(cfg["shape"], device=dev, generator=g).to(cfg["dtype"]) for _ in range(sets)]


def measure_config(name, cfg, dev, timer, peak):
    """One entry of `configs`: kernel alone, forward called directly, forward replayed as a graph."""
    import triton_augment_b200 as ta
    shape = cfg["shape"]
    samples = shape[0] * (shape[1] if len(shape) == 5 else 1)
    c, h, w = shape[-3:]
    oh = ow = cfg["crop"] or h
    es = torch.empty((), dtype=cfg["dtype"]).element_size()
    in_bytes, out_bytes = samples * c * h * w * es, samples * c * oh * ow * es
    alg = 2 * out_bytes                                     # one source texel read per output texel written
    # A working set that fits the L2 is rotated over enough buffer sets that a launch never finds
    # its input (or the lines it is about to overwrite) in the cache: > 2.5 x the L2 in total.
    sets = 1 if in_bytes + out_bytes > 2.5 * L2_BYTES else int(math.ceil(2.5 * L2_BYTES / (in_bytes + out_bytes)))
    imgs = config_images(cfg, dev, sets)
    aug = config_transform(name, cfg)
    k = kernel_only(aug, imgs, timer)
    ring = [None] * sets
    state = {"i": 0}

    def eager():
        i = state["i"] % sets
        state["i"] += 1
        ring[i] = aug(imgs[i])                              # keeping the last `sets` results alive rotates the outputs too
    e = timer(eager)
    del ring
    graphs = [ta.GraphedTransform(aug, img) for img in imgs]

    def replay():
        graphs[state["i"] % sets]()
        state["i"] += 1
    g = timer(replay)
    ach = alg / (k["ms"] * 1e-3) / 1e9
    return {"what": cfg["what"], "images_per_step": samples, "dtype": str(cfg["dtype"]).replace("torch.", ""),
            "algorithmic_bytes": alg, "ms_per_launch": round(k["ms"], 5),
            "roofline": {"bound": "hbm", "achieved": round(ach, 1), "peak": peak, "unit": "GB/s", "frac": round(ach / peak, 4)},
            "ms_per_step": round(g["ms"], 5), "ms_per_step_eager": round(e["ms"], 5),
            "value": samples / (g["ms"] * 1e-3), "value_eager": samples / (e["ms"] * 1e-3), "unit": UNIT,
            "l2": (f"working set {(in_bytes + out_bytes) / 1e6:.0f} MB fits the L2: every measurement rotates over {sets} "
                   f"input/output sets ({sets * (in_bytes + out_bytes) / 1e6:.0f} MB)") if sets > 1 else
                  f"working set {(in_bytes + out_bytes) / 1e6:.0f} MB, larger than the L2 (no rotation)"}


def measure_c5b_sharded(dev, rank, world, timer, dist):
    """The 4096-image batch cut into one contiguous slice per rank (strong scaling).  Parameters are
    drawn once for the whole batch from the same seed on every rank and sliced, as ShardedAugment
    does.  Rank 0 then re-runs every other rank's slice on its own GPU and compares SHA-256 digests:
    the sharded result equals the single-GPU result bit for bit."""
    import triton_augment_b200 as ta
    cfg = CONFIGS["c5b"]
    full = cfg["shape"]
    bounds = ta.shard_bounds(full[0], world)
    aug = config_transform("c5b", cfg)

    def slice_input(r):
        a, b = bounds[r]
        g = torch.Generator(device=dev).manual_seed(5000 + r)
        return torch.rand((b - a,) + tuple(full[1:]), device=dev, generator=g)

    def run_slice(r, local):
        torch.manual_seed(4242)
        return ta.ShardedAugment.for_rank(aug, r, world, device=dev)((local, full))

    mine = slice_input(rank)
    digest = hashlib.sha256(run_slice(rank, mine).cpu().numpy()).hexdigest()
    sharder = ta.ShardedAugment.for_rank(aug, rank, world, device=dev)
    t = timer(lambda: sharder((mine, full)))
    result = {"ms_local": t["ms"]}
    if world > 1:
        digests = [None] * world
        dist.all_gather_object(digests, digest)
    else:
        digests = [digest]
    if rank == 0:
        ok = True
        for r in range(1, world):
            ok = ok and hashlib.sha256(run_slice(r, slice_input(r)).cpu().numpy()).hexdigest() == digests[r]
        result["sha256_equal_to_single_gpu"] = bool(ok) if world > 1 else None
        result["slices"] = [b - a for a, b in bounds]
    return result


def measure_triton_reference(img, timer):
    """The unmodified reference package (baseline/_ref) on the same tensor on this GPU: its
    TritonFusedAugment built with the headline arguments, forward() timed like ours; plus its
    functional entry point with fixed parameter tensors (closest to its kernel alone: one Triton
    launch and the host code around it)."""
    path = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(path, "triton_augment")):
        return {"unavailable": "the reference is not installed under baseline/_ref"}
    try:
        os.environ["TRITON_AUGMENT_SUPPRESS_FIRST_RUN_MESSAGE"] = "1"
        sys.path.insert(0, path)
        import triton_augment as ref
        out = {"package": f"triton_augment {ref.__version__} (unmodified), Triton {__import__('triton').__version__}"}
        n = img.shape[0]
        for interp in ("nearest", "bilinear"):
            aug = make_transform(interp, module=ref)
            fwd = timer(lambda: aug(img))
            torch.manual_seed(99)
            angle, translate, scale, shear, top, left, flip, b, c, s, g = aug._get_params(n, img.device, (SRC, SRC))
            fn = timer(lambda: ref.functional.fused_augment(
                img, top, left, CROP, CROP, flip, angle=angle, translate=translate, scale=scale, shear=shear,
                interpolation=interp, brightness_factor=b, contrast_factor=c, saturation_factor=s, grayscale=g,
                mean=MEAN, std=STD))
            out[interp] = {"ms_per_step": round(fwd["ms"], 4), "min_ms": round(fwd["min_ms"], 4), "max_ms": round(fwd["max_ms"], 4),
                           "value": n / (fwd["ms"] * 1e-3), "unit": UNIT, "functional_ms": round(fn["ms"], 4),
                           "algorithmic_gbs": round(2 * n * 3 * CROP * CROP * 4 / (fn["ms"] * 1e-3) / 1e9, 1)}
        out["what"] = ("reference TritonFusedAugment.forward on the same 64x3x1280x1280 tensor (ms_per_step) and "
                       "reference functional.fused_augment with fixed parameter tensors (functional_ms); same timer as ours")
        return out
    except Exception as e:                                   # noqa: BLE001 - report, do not fail the bench
        return {"unavailable": f"{type(e).__name__}: {e}"[:200]}


class _PlainTimer(Timer):
    """One warm-up call and one block (profiler captures must stay short)."""

    def __call__(self, fn):
        for _ in range(self.warmup):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(self.steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return {"ms": a.elapsed_time(b) / self.steps}


def profile_case(config, images, interp):
    """For profilers: the configuration's tensors for `images` images, three launches of the fused
    kernel through the C ABI, nothing else.  Prints no benchmark line."""
    cfg = dict(CONFIGS.get(config) or PROFILE_ONLY[config])
    if images:
        cfg["shape"] = (images,) + tuple(cfg["shape"][1:])
    torch.cuda.set_device(0)
    torch.manual_seed(1234)
    dev = torch.device("cuda:0")
    imgs = config_images(cfg, dev, 1, seed=1234)
    aug = config_transform(config, cfg, interp)
    exact = config == "c3exact"
    ms = kernel_only(aug, imgs, _PlainTimer(2, 1), exact_contrast=exact)["ms"]
    shape = cfg["shape"]
    n = shape[0] * (shape[1] if len(shape) == 5 else 1)
    crop = cfg["crop"] or shape[-1]
    in_es = imgs[0].element_size()
    out_es = 2 if config == "c3u8h" else 4 if cfg["dtype"] == torch.uint8 else in_es
    gbs = n * 3 * crop * crop * (in_es * (2 if exact else 1) + out_es) / (ms * 1e-3) / 1e9
    print(f"profile case {config}: {n} images, {interp if cfg['affine'] else 'no affine'}, {ms:.4f} ms per launch, "
          f"{gbs:.0f} GB/s algorithmic")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--interp", default="bilinear", choices=["bilinear", "nearest"])
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--profile-case", type=int, default=None, metavar="IMAGES",
                    help="only launch the fused kernel 3 times on IMAGES images (0 = the configuration's own batch); for ncu")
    ap.add_argument("--profile-config", default="c3", choices=sorted(set(CONFIGS) | set(PROFILE_ONLY)),
                    help="which configuration --profile-case builds")
    ap.add_argument("--skip", default="", help="comma-separated parts to leave out: configs,sharded,triton,e2e,cpu")
    ap.add_argument("--blocks", type=int, default=0,
                    help="time exactly this many blocks per measurement and skip the burn-in (0 = at least 10 blocks and "
                         "150 ms of device time); 1 keeps a profiler's launch list short")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    skip = set(filter(None, args.skip.split(",")))
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if args.profile_case is not None:
        profile_case(args.profile_config, args.profile_case, args.interp)
        return

    numa = bind_to_gpu_numa_node(local)                                # before anything allocates or pins host memory
    import torch.distributed as dist
    barrier = agree = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("gloo", rank=rank, world_size=world)   # control plane only: barriers, max of times
        barrier = dist.barrier

        def agree(v):
            t = torch.tensor([v], dtype=torch.int64)
            dist.broadcast(t, src=0)
            return int(t[0])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    import triton_augment_b200 as ta  # noqa: F401  (fails loudly if the CUDA library is missing)

    timer = Timer(args.steps, args.warmup, barrier, agree)
    if args.blocks > 0:
        timer.fixed_blocks = args.blocks
    torch.manual_seed(1234)
    img = torch.rand(N_IMG, 3, SRC, SRC, device=dev)            # 1.26 GB: far larger than the 126 MB L2
    if args.blocks == 0:
        # Burn-in: the fused kernel back to back for ~0.3 s, untimed.  Under sustained load the 1 kW
        # power cap pulls the SM clock down (1965 -> ~1550 MHz measured here); without this the first
        # measurements of the run would be taken on a cool GPU and the later ones on a capped one.
        warm_p, warm_keep = fixed_params(make_transform(args.interp), img)
        from triton_augment_b200 import _lib as _warm_lib
        t_end = time.perf_counter() + 0.3
        while time.perf_counter() < t_end:
            for _ in range(50):
                _warm_lib.launch_fused(warm_p, dev)
            torch.cuda.synchronize()
        del warm_p, warm_keep
    peak, peak_kind = measured_peak_gbs()
    alg_bytes = 2 * N_IMG * 3 * CROP * CROP * 4                 # one read + one write per output element
    result, extra = {}, {}
    with ClockSampler(local) as clocks:
        headline_blocks = 0
        for interp in (args.interp, "nearest" if args.interp == "bilinear" else "bilinear"):
            aug = make_transform(interp)
            eager = timer(lambda: aug(img))
            kern = kernel_only(aug, [img], timer)
            # the same call (parameter draws + matrix + fused kernel) captured once and replayed
            graphed = ta.GraphedTransform(aug, img)
            graph = timer(lambda: graphed())
            if interp == args.interp:
                headline_blocks = eager["blocks"]
            del graphed
            result[interp] = (eager, kern, graph)
        # what a plain device copy of the same bytes (805 MB read, 805 MB written) reaches under this very
        # timing protocol: the measured peak is a burst figure, long runs settle lower under the power cap
        src, dst = torch.empty(N_IMG * 3 * CROP * CROP, device=dev), torch.empty(N_IMG * 3 * CROP * CROP, device=dev)
        extra["copy"] = timer(lambda: dst.copy_(src))
        del src, dst
        # opt-in sampler: all parameters of a step from one launch of the library (its own random stream)
        fast = make_transform(args.interp, fast_rng=True)
        extra["fast"] = timer(lambda: fast(img))
        graphed = ta.GraphedTransform(fast, img)
        extra["fast_graph"] = timer(lambda: graphed())
        del graphed
        # torchvision-exact contrast: one more read of the footprint (mean pre-pass), 1.5 x the bytes
        exact = make_transform(args.interp, fast_rng=True, contrast_mode="torchvision")
        extra["exact"] = timer(lambda: exact(img))

        configs = {}
        if "configs" not in skip:
            for name, cfg in CONFIGS.items():
                configs[name] = measure_config(name, cfg, dev, timer, peak)
                torch.cuda.empty_cache()
        sharded = None if "sharded" in skip else measure_c5b_sharded(dev, rank, world, timer, dist)
        triton_ref = None
        if world == 1 and "triton" not in skip:
            triton_ref = measure_triton_reference(img, timer)

        e2e = {}
        if "e2e" not in skip:
            # end to end: pinned host batch in, pinned host result out, copies inside the timed region
            host_in = torch.empty(N_IMG, 3, SRC, SRC, pin_memory=True).copy_(img)
            host_out = torch.empty(N_IMG, 3, CROP, CROP, pin_memory=True)
            aug = make_transform(args.interp)
            e2e_steps = max(5, min(args.steps, 10))
            e2e["f32"] = wall_timed(lambda: aug.forward_host(host_in, out=host_out, device=dev), e2e_steps, 2, barrier)
            # control: nothing but the copies of the same bytes, both directions at once, same pinned buffers
            d_in, d_out = torch.empty_like(img), torch.empty(N_IMG, 3, CROP, CROP, device=dev)
            s_up, s_down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

            def copies():
                with torch.cuda.stream(s_up):
                    d_in.copy_(host_in, non_blocking=True)
                with torch.cuda.stream(s_down):
                    host_out.copy_(d_out, non_blocking=True)
                s_up.synchronize(); s_down.synchronize()
            e2e["control"] = wall_timed(copies, e2e_steps, 2, barrier)
            del d_in, d_out
            # the same end-to-end call fed with bytes (extension: the kernel reads value / 255 itself)
            host_u8 = torch.randint(0, 256, (N_IMG, 3, SRC, SRC), dtype=torch.uint8).pin_memory()
            e2e["u8"] = wall_timed(lambda: aug.forward_host(host_u8, out=host_out, device=dev), e2e_steps, 2, barrier)
            # ... and with a float16 result (half the download)
            aug_h = make_transform(args.interp, out_dtype=torch.float16)
            host_out_h = torch.empty(N_IMG, 3, CROP, CROP, dtype=torch.float16).pin_memory()
            e2e["u8h"] = wall_timed(lambda: aug_h.forward_host(host_u8, out=host_out_h, device=dev), e2e_steps, 2, barrier)
    clk = clocks.summary()
    ta.utils.check_status(dev)                                   # no kernel gave up a wait anywhere above

    def over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    def ms_of(t):
        return over_ranks(t["ms"])

    eager, kern, graph = result[args.interp]
    ms_eager, ms_kernel, ms_step = ms_of(eager), ms_of(kern), ms_of(graph)
    other = "nearest" if args.interp == "bilinear" else "bilinear"
    ms_eager_o, ms_kernel_o, ms_step_o = (ms_of(v) for v in result[other])
    ms_fast, ms_fast_graph, ms_exact = ms_of(extra["fast"]), ms_of(extra["fast_graph"]), ms_of(extra["exact"])
    ms_copy = ms_of(extra["copy"])
    copy_ctl = {"gbs": round(alg_bytes / (ms_copy * 1e-3) / 1e9, 1), "ms": round(ms_copy, 4),
                "best_block_gbs": round(alg_bytes / (extra["copy"]["min_ms"] * 1e-3) / 1e9, 1),
                "what": "torch copy_ of the launch's algorithmic bytes (805 MB -> 805 MB), same timer, same run"}
    ms_e2e = {k: over_ranks(v["ms"]) for k, v in e2e.items()}
    for name, c in configs.items():            # per-rank numbers; rank 0's line reports the slowest rank
        for key in ("ms_per_launch", "ms_per_step", "ms_per_step_eager"):
            c[key] = round(over_ranks(c[key]), 5)
        ach = c["algorithmic_bytes"] / (c["ms_per_launch"] * 1e-3) / 1e9
        c["roofline"].update(achieved=round(ach, 1), frac=round(ach / peak, 4))
        c["value"] = world * c["images_per_step"] / (c["ms_per_step"] * 1e-3)
        c["value_eager"] = world * c["images_per_step"] / (c["ms_per_step_eager"] * 1e-3)
    if sharded is not None:
        sharded["ms_per_step"] = over_ranks(sharded.pop("ms_local"))
    if rank != 0:
        return

    def roof(ms, interp, t):
        ach = alg_bytes / (ms * 1e-3) / 1e9
        best = alg_bytes / (t["min_ms"] * 1e-3) / 1e9
        per_img = NCU_TRAFFIC_PER_IMAGE.get(interp)
        return {"bound": "hbm", "achieved": round(ach, 1), "peak": peak, "unit": "GB/s", "frac": round(ach / peak, 4),
                "traffic": None if per_img is None else per_img * N_IMG, "peak_source": f"{peak_kind} copy bandwidth",
                "kernel": f"affine_kernel<float,3,{interp}>", "ms_per_launch": round(ms, 4),
                "best_block": {"ms_per_launch": round(t["min_ms"], 4), "achieved": round(best, 1), "frac": round(best / peak, 4),
                               "what": "fastest of rank 0's blocks (the burst figure; `frac` is the median block, i.e. "
                                       "sustained under the power cap)"},
                "copy_same_protocol": copy_ctl}

    line = {"metric": METRIC, "value": world * N_IMG / (ms_eager * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_eager, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(args.interp),
                       "step": "one TritonFusedAugment.forward per step, called directly (fresh random parameters from "
                               "PyTorch's generator stream and the matrices by one sampler launch, then the fused kernel); "
                               "measured after a 0.3 s burn-in, i.e. at power-capped clocks",
                       "l2": "input 1.26 GB per step, larger than L2 (no flush needed)",
                       "parallelism": f"dp{world} (batch sharded, no collective)"},
            "timing": {"blocks": eager["blocks"], "steps_per_block": args.steps, "timed_region_ms": eager["timed_ms"],
                       "ms_per_step_min": round(eager["min_ms"], 5), "ms_per_step_median": round(eager["ms"], 5),
                       "ms_per_step_max": round(eager["max_ms"], 5),
                       "what": "rank 0's blocks of the headline measurement; every other number in this line is a "
                               "median over blocks sized the same way (>= 10 blocks, >= 150 ms of device time)"},
            "roofline": roof(ms_kernel, args.interp, kern),
            "kernel_only_images_per_s": world * N_IMG / (ms_kernel * 1e-3),
            "graph_replay": {"value": world * N_IMG / (ms_step * 1e-3), "ms_per_step": ms_step,
                             "what": "the same forward captured once through GraphedTransform and replayed (a store of the "
                                     "generator state, then the graph: sampler + fused kernel); measured after the other "
                                     "two, i.e. on the hottest GPU of the three"},
            "fast_rng": {"value": world * N_IMG / (ms_fast_graph * 1e-3), "ms_per_step": ms_fast_graph,
                         "eager_ms_per_step": ms_fast,
                         "what": "fast_rng=True (not the reference's random stream): every parameter of the step from "
                                 "one sampler launch of the library, then the fused kernel"},
            "exact_contrast": {"value": world * N_IMG / (ms_exact * 1e-3), "ms_per_step": ms_exact,
                               "achieved_gbs": round(1.5 * alg_bytes / (ms_exact * 1e-3) / 1e9, 1),
                               "frac": round(1.5 * alg_bytes / (ms_exact * 1e-3) / 1e9 / peak, 4),
                               "what": "contrast_mode='torchvision' (mean pre-pass + fused kernel, fast_rng forward): "
                                       "algorithmic bytes are 1.5 x those of the roofline entry"},
            other: {"value": world * N_IMG / (ms_eager_o * 1e-3), "ms_per_step": ms_eager_o,
                    "graph_replay_ms_per_step": ms_step_o, "roofline": roof(ms_kernel_o, other, result[other][1])},
            # per step: sample_params_kernel (all parameters + matrices) and affine_kernel
            "gpu_launches": 2 * args.steps * headline_blocks,
            "numa": numa,
            "clocks": clk}
    if e2e:
        up, down = N_IMG * 3 * SRC * SRC * 4, N_IMG * 3 * CROP * CROP * 4
        line["e2e"] = {"value": world * N_IMG / (ms_e2e["f32"] * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e["f32"],
                       "h2d_bytes_per_step": up, "d2h_bytes_per_step": down,
                       "api": "TritonFusedAugment.forward_host (pinned host in/out, pipelined slices)"}
        line["e2e_copy_control"] = {"value": world * N_IMG / (ms_e2e["control"] * 1e-3), "unit": UNIT,
                                    "ms_per_step": ms_e2e["control"], "h2d_bytes_per_step": up, "d2h_bytes_per_step": down,
                                    "what": "no kernel: cudaMemcpyAsync of the same bytes from / to the same pinned buffers, both "
                                            "directions at once on two streams - the ceiling the host side sets for e2e at this N"}
        line["e2e_uint8_input"] = {"value": world * N_IMG / (ms_e2e["u8"] * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e["u8"],
                                   "h2d_bytes_per_step": up // 4, "d2h_bytes_per_step": down,
                                   "what": "not the reference's configuration: the same call with a uint8 host batch, "
                                           "scaled by 1/255 inside the kernel"}
        line["e2e_uint8_to_float16"] = {"value": world * N_IMG / (ms_e2e["u8h"] * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e["u8h"],
                                        "h2d_bytes_per_step": up // 4, "d2h_bytes_per_step": down // 2,
                                        "what": "not the reference's configuration: uint8 host batch in, float16 result out "
                                                "(out_dtype=torch.float16)"}
    if configs:
        line["configs"] = configs
    if sharded is not None:
        n_all = CONFIGS["c5b"]["shape"][0]
        sharded.update(value=n_all / (sharded["ms_per_step"] * 1e-3), unit=UNIT, scaling="strong", images=n_all,
                       what="the 4096 x 3 x 224 x 224 batch cut into one contiguous slice per rank (ShardedAugment.for_rank): "
                            "parameters drawn for the whole batch from one seed and sliced, each rank's forward on its "
                            "resident slice timed, max over ranks; digests of every rank's output compared with a "
                            "single-GPU run of the same slice on rank 0")
        line["c5b_sharded"] = sharded
    if triton_ref is not None:
        line["triton_reference"] = triton_ref
    if world == 1 and "cpu" not in skip:
        sample = 4
        v, cores = cpu_oracle_rate(args.interp, sample)
        line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": f"{sample} of {N_IMG} images, CPU restatement of the reference kernel (oracle/), all host threads"}
        try:
            tv, tcores = torchvision_cpu_rate(args.interp, 2)
            line["torchvision_cpu"] = {"value": tv, "unit": UNIT, "cores": tcores,
                                       "sample": "2 images, torchvision.transforms.v2.functional composition, per-image loop"}
        except Exception as e:       # torchvision missing or too old: report, do not fail the bench
            line["torchvision_cpu"] = {"unavailable": str(e)[:100]}
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
