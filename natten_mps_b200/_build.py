"""Build the CUDA library in-tree: ``natten_mps_b200/libnatten_b200.so``.

nvcc cross-compiles for sm_100a without a GPU.  Each ``.cu`` file is compiled to
an object in ``csrc/build/`` (in parallel, skipped when the object is newer than
every source and header) and the objects are linked into one shared library.
"""
from __future__ import annotations

import concurrent.futures
import glob
import os
import subprocess

_PKG = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_PKG, "csrc")
LIB_PATH = os.path.join(_PKG, "libnatten_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def build(force: bool = False, verbose: bool = False) -> str:
    sources = sorted(glob.glob(os.path.join(_CSRC, "*.cu")))
    headers = glob.glob(os.path.join(_CSRC, "*.cuh")) + glob.glob(
        os.path.join(os.path.dirname(_PKG), "include", "*.h"))
    newest_header = max((os.path.getmtime(h) for h in headers), default=0.0)
    objdir = os.path.join(_CSRC, "build")
    os.makedirs(objdir, exist_ok=True)
    flags = list(NVCC_FLAGS)
    if verbose:
        flags = flags + ["-Xptxas", "-v"]

    def compile_one(src: str) -> str:
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(
            os.path.getmtime(src), newest_header)
        if stale:
            subprocess.check_call([_nvcc(), *flags, "-c", src, "-o", obj])
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, min(8, len(sources)))) as pool:
        objects = list(pool.map(compile_one, sources))
    if force or not os.path.exists(LIB_PATH) or any(
            os.path.getmtime(o) > os.path.getmtime(LIB_PATH) for o in objects):
        subprocess.check_call([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared",
                               "-o", LIB_PATH, *objects, "-lcuda"])
    return LIB_PATH


if __name__ == "__main__":
    import sys
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
