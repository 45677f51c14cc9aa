"""Builds the sm_100a kernel library in-tree with nvcc.

Every `csrc/*.cu` is compiled with `-gencode arch=compute_100a,code=sm_100a` and
linked into `libdmb200.so` beside this file.  No torch headers are involved:
the library exports a flat C ABI (pointers + stream) that `cuda_ops.py` calls
through ctypes, so a full rebuild is a few tens of seconds.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libdmb200.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-O3"]
# Fast math (approximate exp / division / sqrt, flush-to-zero) is a choice for the bf16 activation kernels,
# whose results are rounded to 8 mantissa bits anyway.  The optimizer updates fp32 master weights and
# moments and is compiled with IEEE division and square root.
PRECISE = {"fused_optim.cu"}


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found")
    return exe


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(SRC, f) for f in os.listdir(SRC) if f.endswith((".cuh", ".h"))]
    sources = sorted(f for f in os.listdir(SRC) if f.endswith(".cu"))
    nvcc = _nvcc()
    jobs = []
    for s in sources:
        src, obj = os.path.join(SRC, s), os.path.join(OBJ, s[:-3] + ".o")
        if force or _stale(obj, [src] + headers):
            fast = [] if s in PRECISE else ["--use_fast_math"]
            jobs.append([nvcc] + NVCC_FLAGS + fast + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj])

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stderr

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        logs = list(ex.map(run, jobs))
    if verbose:
        print("\n".join(logs))
    objs = [os.path.join(OBJ, s[:-3] + ".o") for s in sources]
    if force or jobs or _stale(LIB, objs):
        run([nvcc, "-shared", "-o", LIB] + objs + ["-lcudart"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
