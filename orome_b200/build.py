"""Compile the CUDA library in-tree for sm_100a.

    python -m orome_b200.build [--force] [--verbose]

Produces orome_b200/liborome_cuda.so with nvcc (cross-compiles without a GPU): every
csrc/*.cu becomes an object file (compiled side by side), then one link step.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "liborome_cuda.so")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build liborome_cuda.so")
    return exe


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _deps() -> list[str]:
    return glob.glob(os.path.join(CSRC, "*")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))


def stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(d) > t for d in _deps() if os.path.exists(d))


def build(force: bool = False, verbose: bool = False, defines: tuple[str, ...] = ()) -> str:
    if not force and not stale():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    # every translation unit includes the shared headers, so a change to any of them recompiles all
    newest_header = max(os.path.getmtime(d) for d in _deps() if not d.endswith(".cu") and os.path.exists(d))
    extra = [f"-D{d}" for d in defines] + (["-Xptxas", "-v"] if verbose else [])

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), newest_header):
            subprocess.check_call([nvcc(), *NVCC_FLAGS, *extra, "-c", "-o", obj, src])
        return obj

    with ThreadPoolExecutor(max_workers=max(1, min(len(sources()), os.cpu_count() or 1))) as pool:
        objs = list(pool.map(compile_one, sources()))
    subprocess.check_call([nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv,
                defines=tuple(a[2:] for a in sys.argv[1:] if a.startswith("-D"))))
