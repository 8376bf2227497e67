"""Build recipe for libplx_sm100.so (hand-written CUDA for sm_100a + the C ABI).

    python -m parallax_b200.build [--force]

The library is built in-tree (``parallax_b200/lib/libplx_sm100.so``) with nvcc;
nvcc cross-compiles for sm_100a, so no GPU is needed to build.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

from ._paths import CSRC, INCLUDE, LIB_DIR, LIB_PATH

SOURCES = ["plx_abi.cu", "plx_decode.cu", "plx_train_mma.cu", "plx_fwd_sm100.cu", "plx_bwd_sm100.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; cannot build libplx_sm100.so")
    return exe


def _inputs():
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    files.append(os.path.join(INCLUDE, "plx_abi.h"))
    return files


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(f) > built for f in _inputs())


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources; returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [_nvcc(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", LIB_PATH,
           *[os.path.join(CSRC, s) for s in SOURCES]]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
