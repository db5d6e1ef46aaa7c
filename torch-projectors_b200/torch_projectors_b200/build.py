"""Compile the native pieces of this package in-tree (sm_100a only).

* ``libb200proj.so`` -- the CUDA kernels behind the C ABI of ``include/b200proj.h``; built with
  ``nvcc`` alone from ``../csrc/b200proj.cu`` (which includes the kernel headers next to it); no
  torch dependency.
* ``_C.so`` -- the C++ operator layer (``../csrc/torch_binding.cpp``): ``TORCH_LIBRARY``
  definitions of the eight raw operators, their CUDA implementations and autograd, linked against
  the installed libtorch and ``libb200proj.so``; built with ``g++``.

A library is rebuilt when the hash of its sources differs from the stamp recorded beside it at
build time (file times do not survive a copy of the tree).  Builds write to a temporary file and
rename it into place under a file lock, so several ranks starting at once build once and nobody
loads a half-written file.

Usage:  python -m torch_projectors_b200.build [--force] [--verbose] [--ptxas-info]
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
from contextlib import contextmanager
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC_DIR = PKG_DIR.parent / "csrc"
INCLUDE_DIR = PKG_DIR.parent.parent / "include"
LIB_PATH = PKG_DIR / "libb200proj.so"
BINDING_PATH = PKG_DIR / "_C.so"

SOURCES = [CSRC_DIR / "b200proj.cu"]
HEADERS = [CSRC_DIR / "fourier_slice_device.cuh", CSRC_DIR / "fourier_slice_kernels.cuh",
           INCLUDE_DIR / "b200proj.h"]
BINDING_SOURCES = [CSRC_DIR / "torch_binding.cpp"]

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


def _stamp_of(files) -> str:
    h = hashlib.sha256()
    for f in files:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()[:16]


def source_stamp() -> str:
    """Hash of the CUDA library's sources; the library reports the one it was built from
    (``b200proj_source_stamp``)."""
    return _stamp_of(SOURCES + HEADERS)


def binding_stamp() -> str:
    import torch
    return _stamp_of(BINDING_SOURCES + [INCLUDE_DIR / "b200proj.h"]) + "-torch" + torch.__version__


def _recorded(path: Path) -> str:
    side = Path(str(path) + ".stamp")
    return side.read_text().strip() if side.exists() else ""


def needs_build() -> bool:
    return not LIB_PATH.exists() or _recorded(LIB_PATH) != source_stamp()


def binding_needs_build() -> bool:
    return not BINDING_PATH.exists() or _recorded(BINDING_PATH) != binding_stamp()


@contextmanager
def _build_lock():
    with open(PKG_DIR / ".build.lock", "w") as fh:
        fcntl.flock(fh, fcntl.LOCK_EX)
        try:
            yield
        finally:
            fcntl.flock(fh, fcntl.LOCK_UN)


def _run_into_place(cmd, out: Path, stamp: str, verbose: bool) -> None:
    tmp = out.with_name(f".{out.name}.{os.getpid()}.tmp")
    full = cmd + ["-o", str(tmp)]
    if verbose:
        print("[torch_projectors_b200.build]", " ".join(full), flush=True)
    try:
        subprocess.run(full, check=True)
        os.replace(tmp, out)
        Path(str(out) + ".stamp").write_text(stamp + "\n")
    finally:
        if tmp.exists():
            tmp.unlink()


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Build the CUDA library if it is missing or was built from other sources; return its path."""
    if not force and not needs_build():
        return LIB_PATH
    with _build_lock():
        if not force and not needs_build():          # another process built it while we waited
            return LIB_PATH
        stamp = source_stamp()
        cmd = [find_nvcc(), *NVCC_FLAGS, f"-I{INCLUDE_DIR}", f"-I{CSRC_DIR}", f'-DB200PROJ_SOURCE_STAMP="{stamp}"']
        if ptxas_info:
            cmd += ["-Xptxas", "-v"]
        cmd += [str(s) for s in SOURCES]
        _run_into_place(cmd, LIB_PATH, stamp, verbose)
    return LIB_PATH


def build_binding(force: bool = False, verbose: bool = False) -> Path:
    """Build the C++ operator layer (needs the CUDA library, which it links) if it is missing or
    stale; return its path."""
    build(verbose=verbose)
    if not force and not binding_needs_build():
        return BINDING_PATH
    import torch
    from torch.utils import cpp_extension
    with _build_lock():
        if not force and not binding_needs_build():
            return BINDING_PATH
        stamp = binding_stamp()
        torch_lib = Path(torch.__file__).resolve().parent / "lib"
        cuda_home = Path(os.environ.get("CUDA_HOME") or "/usr/local/cuda")
        cmd = [os.environ.get("CXX") or shutil.which("g++") or "g++", "-O2", "-std=c++17", "-fPIC", "-shared",
               "-D_GLIBCXX_USE_CXX11_ABI=" + str(int(torch._C._GLIBCXX_USE_CXX11_ABI)),
               f"-I{INCLUDE_DIR}", f"-I{cuda_home / 'include'}"]
        cmd += [f"-I{p}" for p in cpp_extension.include_paths()]
        cmd += [str(s) for s in BINDING_SOURCES]
        cmd += [f"-L{PKG_DIR}", "-lb200proj", f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
                "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
        _run_into_place(cmd, BINDING_PATH, stamp, verbose)
    return BINDING_PATH


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas-info" in sys.argv)
    print(LIB_PATH)
    if BINDING_SOURCES[0].exists():
        print(build_binding(force="--force" in sys.argv, verbose=True))
