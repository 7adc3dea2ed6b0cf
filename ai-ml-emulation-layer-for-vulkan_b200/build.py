"""Builds ``libmlel_b200.so`` (the C-ABI library of include/mlel_b200.h) in-tree with nvcc for sm_100a.

    python ai-ml-emulation-layer-for-vulkan_b200/build.py [--force] [--verbose]

Every source is compiled to an object under ``csrc/_obj`` (only when older than its inputs) and
linked into ``ai-ml-emulation-layer-for-vulkan_b200/libmlel_b200.so``.
"""
from __future__ import annotations

import concurrent.futures
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(HERE, "libmlel_b200.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CFLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-Wall", "--expt-relaxed-constexpr",
          "-I", os.path.join(HERE, "..", "include")]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cpp")) + glob.glob(os.path.join(CSRC, "*.cu")) +
                  glob.glob(os.path.join(CSRC, "kernels", "*.cu")))


def headers():
    return (glob.glob(os.path.join(CSRC, "*.hpp")) + glob.glob(os.path.join(CSRC, "kernels", "*.hpp")) +
            glob.glob(os.path.join(CSRC, "kernels", "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h")))


def _compile(src: str, obj: str, verbose: bool) -> None:
    cmd = [NVCC, *ARCH, *CFLAGS, "-x", "cu", "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}")


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    newest_header = max(os.path.getmtime(h) for h in headers())
    jobs, objs = [], []
    for src in sources():
        obj = os.path.join(OBJ, os.path.relpath(src, CSRC).replace(os.sep, "_") + ".o")
        objs.append(obj)
        stale = (not os.path.exists(obj)) or os.path.getmtime(obj) < max(os.path.getmtime(src), newest_header)
        if force or stale:
            jobs.append((src, obj))
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        for f in [pool.submit(_compile, s, o, verbose) for s, o in jobs]:
            f.result()
    if jobs or not os.path.exists(LIB):
        cmd = [NVCC, *ARCH, "-shared", "-o", LIB, *objs]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
