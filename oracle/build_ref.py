#!/usr/bin/env python
"""Build the reference's own CPU operators into ``oracle/_ref/`` (test infrastructure).

The reference (warpem/torch-projectors) keeps its CPU backend in a handful of C++
translation units: ``csrc/torch_projectors.cpp`` (op schemas + CPU registration) and
``csrc/cpu/{2d,3d}/*.cpp``.  This script compiles exactly those files, where they lie
in the reference checkout, with ``g++`` directly (it does not run the reference's
``setup.py``) and links them against the installed libtorch into one shared object:

    oracle/_ref/torch_projectors_ref.so

Loading that file with ``torch.ops.load_library`` registers the reference's eight raw
operators under ``torch.ops.torch_projectors.*`` (CPU dispatch key only).  They are used
as (i) the checker that pins ``oracle/fourier_slice_oracle.c`` and generates the golden
vectors under ``tests/golden/``, and (ii) the timed CPU baseline of ``bench.py``.

Nothing from the reference is copied into this repository: sources are read in place and
only the built object is written, into a git-ignored folder.

Flags follow the reference's own build (``setup.py``: ``-O3 -std=c++20 -fopenmp``); no
``-march`` flag is given, so the compiler cannot contract ``a*b+c`` into FMA and the fp32
coordinate arithmetic keeps one rounding per operation.

Usage:  python oracle/build_ref.py [--reference /path/to/torch-projectors] [--force]
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
OUT_SO = OUT_DIR / "torch_projectors_ref.so"

OUT_SO_CUDA = OUT_DIR / "torch_projectors_ref_cuda.so"

# The reference's CUDA backend (generic SIMT kernels, no sm_100-specific code), compiled with the
# flags of its own build (setup.py: -O3 --use_fast_math -DUSE_CUDA) for sm_100: the kernels a user
# of the reference would run on a B200.  Used only as a speed comparator by bench.py.
CUDA_SOURCES = [
    "csrc/cuda/2d/projection_2d_kernels.cu",
    "csrc/cuda/2d/backprojection_2d_kernels.cu",
    "csrc/cuda/3d/projection_3d_to_2d_kernels.cu",
    "csrc/cuda/3d/backprojection_2d_to_3d_kernels.cu",
]

SOURCES = [
    "csrc/torch_projectors.cpp",
    "csrc/cpu/2d/projection_2d_kernels.cpp",
    "csrc/cpu/2d/backprojection_2d_kernels.cpp",
    "csrc/cpu/3d/projection_3d_to_2d_kernels.cpp",
    "csrc/cpu/3d/backprojection_2d_to_3d_kernels.cpp",
]


def default_reference() -> Path:
    """The reference checkout: $TORCH_PROJECTORS_REFERENCE, else a folder named ``reference``
    beside this repository (absent on machines that only use the prebuilt object)."""
    env = os.environ.get("TORCH_PROJECTORS_REFERENCE")
    return Path(env) if env else HERE.parent.parent / "reference"


def build(reference: Path | None = None, force: bool = False, verbose: bool = True) -> Path | None:
    """Compile the reference CPU backend; returns the .so path, or None if the
    reference checkout is not present (then a previously built .so is kept as is)."""
    reference = Path(reference) if reference else default_reference()
    if not (reference / SOURCES[0]).exists():
        if verbose:
            print(f"[build_ref] no reference checkout at {reference}; "
                  f"{'using prebuilt ' + str(OUT_SO) if OUT_SO.exists() else 'nothing built'}")
        return OUT_SO if OUT_SO.exists() else None

    srcs = [reference / s for s in SOURCES]
    if OUT_SO.exists() and not force:
        newest = max(p.stat().st_mtime for p in srcs)
        if OUT_SO.stat().st_mtime >= newest:
            return OUT_SO

    import torch  # noqa: F401  (only for its include/lib dirs)
    from torch.utils import cpp_extension as ce

    OUT_DIR.mkdir(parents=True, exist_ok=True)
    obj_dir = OUT_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}"]
    cxx11 = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    common = ["g++", "-O3", "-std=c++20", "-fopenmp", "-fPIC", "-w",
              f"-D_GLIBCXX_USE_CXX11_ABI={cxx11}",
              "-DTORCH_EXTENSION_NAME=torch_projectors_ref",
              "-DTORCH_API_INCLUDE_EXTENSION_H"] + inc

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        cmd = common + ["-c", str(src), "-o", str(obj)]
        if verbose:
            print("[build_ref]", " ".join(cmd[:6]), "...", src.name, flush=True)
        subprocess.run(cmd, check=True)
        return obj

    with ThreadPoolExecutor(max_workers=min(5, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, srcs))

    libdirs = ce.library_paths()
    link = (["g++", "-shared", "-fopenmp", "-o", str(OUT_SO)] + [str(o) for o in objs]
            + [f"-L{d}" for d in libdirs] + [f"-Wl,-rpath,{d}" for d in libdirs]
            + ["-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python"])
    subprocess.run(link, check=True)
    if verbose:
        print(f"[build_ref] wrote {OUT_SO}")
    return OUT_SO


def build_cuda(reference: Path | None = None, force: bool = False, verbose: bool = True) -> Path | None:
    """Compile the reference's CPU + CUDA backends into one library (registers the CUDA
    dispatch key too).  Takes several minutes (nvcc on torch headers); returns the .so path,
    or a previously built one / None when the reference checkout is absent."""
    reference = Path(reference) if reference else default_reference()
    if not (reference / CUDA_SOURCES[0]).exists():
        return OUT_SO_CUDA if OUT_SO_CUDA.exists() else None
    if OUT_SO_CUDA.exists() and not force:
        return OUT_SO_CUDA
    import torch  # noqa: F401
    from torch.utils import cpp_extension as ce

    OUT_DIR.mkdir(parents=True, exist_ok=True)
    obj_dir = OUT_DIR / "obj_cuda"
    obj_dir.mkdir(exist_ok=True)
    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}", "-I/usr/local/cuda/include"]
    cxx11 = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    defs = [f"-D_GLIBCXX_USE_CXX11_ABI={cxx11}", "-DTORCH_EXTENSION_NAME=torch_projectors_ref_cuda",
            "-DTORCH_API_INCLUDE_EXTENSION_H", "-DUSE_CUDA"]
    host = ["g++", "-O3", "-std=c++20", "-fopenmp", "-fPIC", "-w"] + defs + inc
    dev = ["nvcc", "-O3", "--use_fast_math", "-std=c++17", "-gencode", "arch=compute_100,code=sm_100",
           "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-w",
           "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__",
           "-D__CUDA_NO_BFLOAT16_CONVERSIONS__"] + defs + inc

    def compile_one(rel: str) -> Path:
        src = reference / rel
        obj = obj_dir / (src.stem + ("_cu.o" if src.suffix == ".cu" else ".o"))
        cmd = (dev if src.suffix == ".cu" else host) + ["-c", str(src), "-o", str(obj)]
        if verbose:
            print("[build_ref cuda]", cmd[0], "...", src.name, flush=True)
        subprocess.run(cmd, check=True)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, SOURCES + CUDA_SOURCES))
    libdirs = ce.library_paths() + ["/usr/local/cuda/lib64"]
    link = (["g++", "-shared", "-fopenmp", "-o", str(OUT_SO_CUDA)] + [str(o) for o in objs]
            + [f"-L{d}" for d in libdirs] + [f"-Wl,-rpath,{d}" for d in libdirs]
            + ["-lc10", "-lc10_cuda", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-ltorch_python", "-lcudart"])
    subprocess.run(link, check=True)
    if verbose:
        print(f"[build_ref cuda] wrote {OUT_SO_CUDA}")
    return OUT_SO_CUDA


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--cuda", action="store_true", help="also build the reference's CUDA backend (minutes)")
    a = ap.parse_args()
    ok = build(a.reference, a.force)
    if a.cuda:
        ok = build_cuda(a.reference, a.force) and ok
    sys.exit(0 if ok else 1)
