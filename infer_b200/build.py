"""Builds libfth_b200.so (hand-written CUDA for sm_100a behind the C ABI of include/fth_b200.h) in-tree.

nvcc cross-compiles without a GPU.  Objects are cached under infer_b200/csrc/_obj and rebuilt when a
source or header is newer.  Run as `python -m infer_b200.build`.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(HERE, "libfth_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "-Xptxas", "-v"]


def _newest_header() -> float:
    headers = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    return max(os.path.getmtime(h) for h in headers)


def _compile(src: str, verbose: bool) -> str:
    obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
    stamp = max(os.path.getmtime(src), _newest_header())
    if os.path.exists(obj) and os.path.getmtime(obj) >= stamp:
        return obj
    proc = subprocess.run([NVCC, *FLAGS, "-c", src, "-o", obj], capture_output=True, text=True)
    log = proc.stdout + proc.stderr
    with open(obj[:-2] + ".ptxas.log", "w") as f:
        f.write(log)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{log}")
    if verbose:
        spills = [l for l in log.splitlines() if "spill" in l and "0 bytes spill stores, 0 bytes spill loads" not in l]
        print(f"[build] {os.path.basename(src)} ok" + (f" ({len(spills)} kernels spill)" if spills else ""))
    return obj


def build(verbose: bool = True) -> str:
    os.makedirs(OBJ, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    with cf.ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), sources))
    if not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        subprocess.check_call([NVCC, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a"])
        if verbose:
            print(f"[build] linked {LIB}")
    return LIB


if __name__ == "__main__":
    build(verbose="-q" not in sys.argv)
