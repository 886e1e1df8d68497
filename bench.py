"""Benchmark of the fused augmentation hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--interp bilinear|nearest] [--impl reference]

Workload: the "ultimate fusion with affine" configuration - 64 x 3 x 1280 x 1280 fp32 images,
random affine (15 deg, translate 0.1, scale 0.9-1.1, shear 5) + crop 1024 + flip 0.5 + colour
jitter 0.2 + grayscale 0.1 + ImageNet normalize - on synthetic uniform[0,1) pixels.  One step =
one call of ``TritonFusedAugment.forward`` on the batch (parameter sampling included).  With
N > 1 (torchrun, one process per GPU) every rank runs the same workload on its own GPU: images
are independent, there is no collective on the data path, scaling is weak.

Prints ONE JSON line (rank 0).  ``--impl reference`` times the CPU restatement of the
reference's kernel (oracle/) on the host cores instead, on a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import json
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
# dram__bytes_read.sum + dram__bytes_write.sum of one full 64-image affine-kernel launch (single-pass
# ncu capture with `--profile-case 64`, summarised under profiles/), divided by 64.
NCU_TRAFFIC_PER_IMAGE = {"bilinear": (832564992 + 761615616) / 64, "nearest": (832006400 + 759964928) / 64}


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def make_transform(interp, fast_rng=False, contrast_mode="fast", out_dtype=None):
    import triton_augment_b200 as ta
    return ta.TritonFusedAugment(crop_size=CROP, horizontal_flip_p=0.5, degrees=15, translate=(0.1, 0.1),
                                 scale=(0.9, 1.1), shear=5, interpolation=interp, brightness=0.2, contrast=0.2,
                                 saturation=0.2, grayscale_p=0.1, mean=MEAN, std=STD, fast_rng=fast_rng,
                                 contrast_mode=contrast_mode, out_dtype=out_dtype)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

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
        sm, mx, reasons = [], 0.0, set()
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
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def timed(fn, steps, warmup, barrier=None):
    """W warm-up calls, then K calls between CUDA events on the current stream; ms per call."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return a.elapsed_time(b) / steps


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
    for _ in range(args.warmup):
        pass                                       # nothing to warm on the CPU beyond the call inside cpu_oracle_rate
    rates = []
    for _ in range(max(1, min(args.steps, 3))):
        r, cores = cpu_oracle_rate(args.interp, sample)
        rates.append(r)
    value = statistics.median(rates)
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * N_IMG / value, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"C3 affine({args.interp})+crop{CROP}+flip+colour+normalize, N={N_IMG}, 3x{SRC}x{SRC} fp32"},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                             "sample": f"{sample} of {N_IMG} images per step, CPU restatement of the reference kernel, all host threads"},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def kernel_only(aug, img, steps, warmup, barrier, exact_contrast=False):
    """The fused kernel alone (parameters drawn once, then fixed): ms per launch, CUDA events.
    ``exact_contrast``: the grayscale-mean pre-pass + the fused kernel in mean-contrast mode."""
    from triton_augment_b200 import _lib, functional as F
    from triton_augment_b200.transforms import _Layout
    dev = img.device
    n, _, src_h, src_w = img.shape
    crop = aug.crop_height
    lay = _Layout(img, False, True)
    angle, translate, scale, shear, top, left, flip, b, c, s, g = aug._spread_all(
        lay, aug._get_params(lay.count, dev, (src_h, src_w)))
    matrix = None
    if aug.has_affine:
        matrix = F._prepare_affine_matrix_only(n, dev, src_h, src_w, angle, translate, scale, shear, None).contiguous()
    work = F._work_dtype(img, aug.out_dtype if img.dtype == torch.uint8 else None)
    out = torch.empty(n, 3, crop, crop, device=dev, dtype=work)
    p = _lib.make_params(img, out, top, left, flip, matrix, 0.0, aug.has_affine and F._is_bilinear(aug.interpolation), 31,
                         b.to(work), c.to(work), s.to(work), g,
                         F._rounded_triple(MEAN, work), F._rounded_triple(STD, work))
    if not exact_contrast:
        return timed(lambda: _lib.launch_fused(p, dev), steps, warmup, barrier)
    p.contrast_mode = _lib.CONTRAST_MEAN

    def both():
        means = _lib.launch_gray_mean(p, dev)
        p.gray_mean = means.data_ptr()
        _lib.launch_fused(p, dev)
    return timed(both, steps, warmup, barrier)


# Other configurations of the reference's benchmark list, for profiler captures (--profile-config):
# images, source size, crop, dtype, affine
PROFILE_CONFIGS = {
    "c1": (32, 224, 224, torch.float32, False),          # colour + grayscale + normalize only
    "c2": (256, 224, 112, torch.float32, False),         # crop 112 + flip + colour + normalize
    "c3": (N_IMG, SRC, CROP, torch.float32, True),
    "c3exact": (N_IMG, SRC, CROP, torch.float32, True),  # C3 with torchvision-exact contrast: mean pre-pass + fused kernel
    "c3u8": (N_IMG, SRC, CROP, torch.uint8, True),       # C3 fed with bytes (scaled by 1/255 in the kernel), float32 out
    "c3u8h": (N_IMG, SRC, CROP, torch.uint8, True),      # ... float16 out
    "c4": (512, 512, 448, torch.float16, True),          # fp16 affine + crop 448 + flip + colour + normalize
    "c5b": (4096, 224, 112, torch.float32, False),       # crop 112 + flip + colour + normalize, image batch
}


def profile_case(config, images, interp):
    """For profilers: the configuration's tensors for `images` images, three launches of the fused
    kernel through the C ABI, nothing else.  Prints no benchmark line."""
    import triton_augment_b200 as ta
    n, src, crop, dtype, affine = PROFILE_CONFIGS[config]
    n = images or n
    torch.cuda.set_device(0)
    torch.manual_seed(1234)
    img = (torch.randint(0, 256, (n, 3, src, src), device="cuda:0", dtype=torch.uint8) if dtype == torch.uint8
           else torch.rand(n, 3, src, src, device="cuda:0").to(dtype))
    kw = dict(degrees=15, translate=(0.1, 0.1), scale=(0.9, 1.1), shear=5, interpolation=interp) if affine else {}
    aug = ta.TritonFusedAugment(crop_size=crop, horizontal_flip_p=0.5, brightness=0.2, contrast=0.2, saturation=0.2,
                                grayscale_p=0.1, mean=MEAN, std=STD,
                                out_dtype=torch.float16 if config == "c3u8h" else None, **kw)
    exact = config == "c3exact"
    ms = kernel_only(aug, img, 2, 1, None, exact_contrast=exact)
    out_bytes = 2 if config == "c3u8h" else 4 if dtype == torch.uint8 else img.element_size()
    gbs = n * 3 * crop * crop * (img.element_size() * (2 if exact else 1) + out_bytes) / (ms * 1e-3) / 1e9
    print(f"profile case {config}: {n} images, {interp if affine else 'no affine'}, {ms:.4f} ms per launch, "
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
    ap.add_argument("--profile-config", default="c3", choices=sorted(PROFILE_CONFIGS),
                    help="which configuration --profile-case builds")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if args.profile_case is not None:
        profile_case(args.profile_config, args.profile_case, args.interp)
        return

    import torch.distributed as dist
    barrier = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("gloo", rank=rank, world_size=world)   # control plane only: barriers, max of times
        barrier = dist.barrier
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    import triton_augment_b200 as ta  # noqa: F401  (fails loudly if the CUDA library is missing)

    torch.manual_seed(1234)
    img = torch.rand(N_IMG, 3, SRC, SRC, device=dev)            # 1.26 GB: far larger than the 126 MB L2
    peak, peak_kind = measured_peak_gbs()
    alg_bytes = 2 * N_IMG * 3 * CROP * CROP * 4                 # one read + one write per output element
    result = {}
    with ClockSampler(local) as clocks:
        for interp in (args.interp, "nearest" if args.interp == "bilinear" else "bilinear"):
            aug = make_transform(interp)
            ms_step = timed(lambda: aug(img), args.steps, args.warmup, barrier)
            ms_kernel = kernel_only(aug, img, args.steps, args.warmup, barrier)
            # the same call (parameter draws + matrix + fused kernel) captured once and replayed
            import triton_augment_b200 as ta
            graphed = ta.GraphedTransform(aug, img)
            ms_graph = timed(lambda: graphed(), args.steps, args.warmup, barrier)
            del graphed
            result[interp] = (ms_step, ms_kernel, ms_graph)
        # opt-in sampler: all parameters of a step from one launch of the library (its own random stream)
        fast = make_transform(args.interp, fast_rng=True)
        ms_fast = timed(lambda: fast(img), args.steps, args.warmup, barrier)
        graphed = ta.GraphedTransform(fast, img)
        ms_fast_graph = timed(lambda: graphed(), args.steps, args.warmup, barrier)
        del graphed
        # torchvision-exact contrast: one more read of the footprint (mean pre-pass), 1.5 x the bytes
        exact = make_transform(args.interp, fast_rng=True, contrast_mode="torchvision")
        ms_exact = timed(lambda: exact(img), args.steps, args.warmup, barrier)
        # end to end: pinned host batch in, pinned host result out, copies inside the timed region
        host_in = torch.empty(N_IMG, 3, SRC, SRC, pin_memory=True).copy_(img)
        host_out = torch.empty(N_IMG, 3, CROP, CROP, pin_memory=True)
        aug = make_transform(args.interp)
        e2e_steps = max(3, min(args.steps, 10))
        for _ in range(2):
            aug.forward_host(host_in, out=host_out, device=dev)
        if barrier:
            barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            aug.forward_host(host_in, out=host_out, device=dev)   # returns when host_out is complete
        ms_e2e = 1e3 * (time.perf_counter() - t0) / e2e_steps
        # the same end-to-end call fed with bytes (extension: the kernel reads value / 255 itself)
        host_u8 = torch.randint(0, 256, (N_IMG, 3, SRC, SRC), dtype=torch.uint8).pin_memory()
        for _ in range(2):
            aug.forward_host(host_u8, out=host_out, device=dev)
        if barrier:
            barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            aug.forward_host(host_u8, out=host_out, device=dev)
        ms_e2e_u8 = 1e3 * (time.perf_counter() - t0) / e2e_steps
        # ... and with a float16 result (half the download)
        aug_h = make_transform(args.interp, out_dtype=torch.float16)
        host_out_h = torch.empty(N_IMG, 3, CROP, CROP, dtype=torch.float16).pin_memory()
        for _ in range(2):
            aug_h.forward_host(host_u8, out=host_out_h, device=dev)
        if barrier:
            barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            aug_h.forward_host(host_u8, out=host_out_h, device=dev)
        ms_e2e_u8h = 1e3 * (time.perf_counter() - t0) / e2e_steps
    clk = clocks.summary()

    def over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    ms_eager, ms_kernel, ms_step = (over_ranks(v) for v in result[args.interp])
    other = "nearest" if args.interp == "bilinear" else "bilinear"
    ms_eager_o, ms_kernel_o, ms_step_o = (over_ranks(v) for v in result[other])
    ms_e2e = over_ranks(ms_e2e)
    ms_e2e_u8 = over_ranks(ms_e2e_u8)
    ms_e2e_u8h = over_ranks(ms_e2e_u8h)
    ms_fast, ms_fast_graph = over_ranks(ms_fast), over_ranks(ms_fast_graph)
    ms_exact = over_ranks(ms_exact)
    if rank != 0:
        return

    def roof(ms, interp):
        ach = alg_bytes / (ms * 1e-3) / 1e9
        per_img = NCU_TRAFFIC_PER_IMAGE.get(interp)
        return {"bound": "hbm", "achieved": round(ach, 1), "peak": peak, "unit": "GB/s", "frac": round(ach / peak, 4),
                "traffic": None if per_img is None else per_img * N_IMG, "peak_source": f"{peak_kind} copy bandwidth",
                "kernel": f"affine_kernel<float,3,{interp}>", "ms_per_launch": round(ms, 4)}

    line = {"metric": METRIC, "value": world * N_IMG / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"C3 affine({args.interp})+crop{CROP}+flip+colour+gray+normalize, N={N_IMG} per GPU, "
                                   f"3x{SRC}x{SRC} fp32, one TritonFusedAugment.forward (fresh random parameters, matrix, "
                                   f"fused kernel) per step, replayed as a CUDA graph through GraphedTransform",
                       "l2": "input 1.26 GB per step, larger than L2 (no flush needed)", "parallelism": f"dp{world} (batch sharded, no collective)"},
            "roofline": roof(ms_kernel, args.interp),
            "kernel_only_images_per_s": world * N_IMG / (ms_kernel * 1e-3),
            "eager": {"value": world * N_IMG / (ms_eager * 1e-3), "ms_per_step": ms_eager,
                      "what": "the same forward called directly (about 19 small launches per step issued from Python)"},
            "fast_rng": {"value": world * N_IMG / (ms_fast_graph * 1e-3), "ms_per_step": ms_fast_graph,
                         "eager_ms_per_step": ms_fast,
                         "what": "fast_rng=True (not the reference's random stream): every parameter of the step from "
                                 "one sampler launch of the library, then the fused kernel"},
            "exact_contrast": {"value": world * N_IMG / (ms_exact * 1e-3), "ms_per_step": ms_exact,
                               "achieved_gbs": round(1.5 * alg_bytes / (ms_exact * 1e-3) / 1e9, 1),
                               "frac": round(1.5 * alg_bytes / (ms_exact * 1e-3) / 1e9 / peak, 4),
                               "what": "contrast_mode='torchvision' (mean pre-pass + fused kernel, fast_rng forward): "
                                       "algorithmic bytes are 1.5 x those of the roofline entry"},
            other: {"value": world * N_IMG / (ms_step_o * 1e-3), "ms_per_step": ms_step_o,
                    "eager_ms_per_step": ms_eager_o, "roofline": roof(ms_kernel_o, other)},
            "e2e": {"value": world * N_IMG / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": N_IMG * 3 * SRC * SRC * 4, "d2h_bytes_per_step": N_IMG * 3 * CROP * CROP * 4,
                    "api": "TritonFusedAugment.forward_host (pinned host in/out, pipelined slices)"},
            "e2e_uint8_input": {"value": world * N_IMG / (ms_e2e_u8 * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e_u8,
                                "h2d_bytes_per_step": N_IMG * 3 * SRC * SRC, "d2h_bytes_per_step": N_IMG * 3 * CROP * CROP * 4,
                                "what": "not the reference's configuration: the same call with a uint8 host batch, "
                                        "scaled by 1/255 inside the kernel"},
            "e2e_uint8_to_float16": {"value": world * N_IMG / (ms_e2e_u8h * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e_u8h,
                                     "h2d_bytes_per_step": N_IMG * 3 * SRC * SRC, "d2h_bytes_per_step": N_IMG * 3 * CROP * CROP * 2,
                                     "what": "not the reference's configuration: uint8 host batch in, float16 result out "
                                             "(out_dtype=torch.float16)"},
            "gpu_launches": 2 * args.steps,       # per step: inverse_matrix_kernel + affine_kernel (inside the graph)
            "clocks": clk}
    if world == 1:
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
