"""Builds libta_b200.so (sm_100a only) from csrc/ with nvcc, in-tree.

    python -m triton_augment_b200.build [--force] [--jobs N]

Each translation unit is compiled to an object file in parallel and the objects are
linked into lib/libta_b200.so next to this file.  No libtorch, no Python headers: the
library has a plain C ABI (include/ta_b200.h) and is loaded with ctypes.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "lib", "obj")
LIB = os.path.join(HERE, "lib", "libta_b200.so")

UNITS = (["ta_api.cu", "ta_inst_f32_crop_staged.cu", "ta_inst_f32_bilinear_mix.cu", "ta_inst_f32_mean.cu",
          "ta_inst_f32_two_phase.cu"]
         + [f"ta_inst_f32_short_{k}.cu" for k in ("crop_staged", "nearest", "bilinear", "bilinear_mix")]
         + [f"ta_inst_f16_short_{k}.cu" for k in ("nearest", "bilinear")]
         + [f"ta_inst_u8_{k}.cu" for k in ("crop_staged", "nearest", "bilinear", "bilinear_mix")]
         + [f"ta_inst_u8h_{k}.cu" for k in ("crop_staged", "nearest", "bilinear")]
         + [f"ta_inst_{t}_{k}.cu" for t in ("f32", "f16") for k in ("direct", "nearest", "bilinear")])

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _newest_source() -> float:
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    paths.append(os.path.join(os.path.dirname(HERE), "include", "ta_b200.h"))
    return max(os.path.getmtime(p) for p in paths)


def up_to_date() -> bool:
    return os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_source()


def _compile(unit: str, verbose: bool) -> str:
    out = os.path.join(OBJ, unit.replace(".cu", ".o"))
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", os.path.join(CSRC, unit), "-o", out]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {unit}:\n{r.stdout}")
    if verbose:
        print(r.stdout)
    return out


def build(force: bool = False, jobs: int | None = None, verbose: bool = False) -> str:
    if not force and up_to_date():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    jobs = jobs or min(len(UNITS), os.cpu_count() or 1)
    with cf.ThreadPoolExecutor(max_workers=jobs) as ex:
        objs = list(ex.map(lambda u: _compile(u, verbose), UNITS))
    cmd = [_nvcc(), "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--jobs", type=int, default=None)
    ap.add_argument("--verbose", action="store_true", help="print ptxas resource usage")
    a = ap.parse_args()
    print(build(a.force, a.jobs, a.verbose))
    sys.exit(0)
