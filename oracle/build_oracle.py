#!/usr/bin/env python
"""Compile ``oracle/fourier_slice_oracle.c`` (test infrastructure) with gcc.

The one C file is compiled twice -- ``-DREAL=float -DSUFFIX=f32`` and
``-DREAL=double -DSUFFIX=f64`` -- and linked into
``oracle/_build/libfourier_slice_oracle.so``.  ``-ffp-contract=off`` keeps every
multiply and add separately rounded, which is what the reference's x86-64 build does
and what the fp32 coordinate parity depends on.

Usage:  python oracle/build_oracle.py [--force]
"""
from __future__ import annotations

import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "fourier_slice_oracle.c"
OUT_DIR = HERE / "_build"
OUT_SO = OUT_DIR / "libfourier_slice_oracle.so"

CFLAGS = ["-O2", "-std=c99", "-fPIC", "-ffp-contract=off", "-fno-fast-math", "-Wall", "-Wextra"]


def build(force: bool = False, verbose: bool = False) -> Path:
    if OUT_SO.exists() and not force and OUT_SO.stat().st_mtime >= SRC.stat().st_mtime:
        return OUT_SO
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    objs = []
    for real, suffix in (("float", "f32"), ("double", "f64")):
        obj = OUT_DIR / f"oracle_{suffix}.o"
        cmd = ["gcc", *CFLAGS, f"-DREAL={real}", f"-DSUFFIX={suffix}", "-c", str(SRC), "-o", str(obj)]
        if verbose:
            print("[build_oracle]", " ".join(cmd))
        subprocess.run(cmd, check=True)
        objs.append(str(obj))
    subprocess.run(["gcc", "-shared", "-o", str(OUT_SO), *objs, "-lm"], check=True)
    if verbose:
        print(f"[build_oracle] wrote {OUT_SO}")
    return OUT_SO


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
