"""Compile the CUDA sources of this package into ``libb200proj.so`` (in-tree, sm_100a only).

The library has no torch dependency: it is built with ``nvcc`` alone from
``../csrc/b200proj.cu`` (which includes the kernel headers next to it) and the public
header ``include/b200proj.h`` at the repository root.

Usage:  python -m torch_projectors_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC_DIR = PKG_DIR.parent / "csrc"
INCLUDE_DIR = PKG_DIR.parent.parent / "include"
LIB_PATH = PKG_DIR / "libb200proj.so"

SOURCES = [CSRC_DIR / "b200proj.cu"]
HEADERS = [CSRC_DIR / "fourier_slice_device.cuh", CSRC_DIR / "fourier_slice_kernels.cuh",
           INCLUDE_DIR / "b200proj.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def find_nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def needs_build() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    return any(p.exists() and p.stat().st_mtime > t for p in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Build the library if it is missing or older than its sources; return its path."""
    if not force and not needs_build():
        return LIB_PATH
    cmd = [find_nvcc(), *NVCC_FLAGS, f"-I{INCLUDE_DIR}", f"-I{CSRC_DIR}"]
    if ptxas_info:
        cmd += ["-Xptxas", "-v"]
    cmd += [str(s) for s in SOURCES] + ["-o", str(LIB_PATH)]
    if verbose:
        print("[torch_projectors_b200.build]", " ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas-info" in sys.argv)
    print(LIB_PATH)
