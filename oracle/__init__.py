"""CPU oracles for the Fourier-slice operators -- TEST INFRASTRUCTURE, not product code.

Two checkers live here:

* ``oracle.port``  -- ctypes wrapper around ``fourier_slice_oracle.c``, a plain-C
  restatement of the reference's CPU algorithm (fp32 and fp64 variants).
* ``oracle.reference_ops()`` -- the reference's own CPU operators, compiled in place from
  its sources by ``oracle/build_ref.py`` into ``oracle/_ref/`` (present only where that
  build has been run; the built object travels, the sources do not).

Only ``tests/``, the smoke check and the CPU-baseline / reference legs of ``bench.py`` may
import this package, and only as the checker or the timed CPU baseline.  The product
package never imports it.
"""
from __future__ import annotations

from pathlib import Path

from . import port  # noqa: F401

_REF_SO = Path(__file__).resolve().parent / "_ref" / "torch_projectors_ref.so"
_ref_loaded = False


def reference_available() -> bool:
    return _REF_SO.exists()


def reference_ops():
    """Return ``torch.ops.torch_projectors`` backed by the reference's CPU kernels, or
    raise FileNotFoundError when ``oracle/_ref`` has not been built."""
    global _ref_loaded
    import torch

    if not _ref_loaded:
        if not _REF_SO.exists():
            raise FileNotFoundError(
                f"{_REF_SO} not built; run `python oracle/build_ref.py` where the reference checkout exists")
        torch.ops.load_library(str(_REF_SO))
        _ref_loaded = True
    return torch.ops.torch_projectors


_REF_CUDA_SO = Path(__file__).resolve().parent / "_ref" / "torch_projectors_ref_cuda.so"


def reference_cuda_available() -> bool:
    return _REF_CUDA_SO.exists()


def reference_cuda_ops():
    """``torch.ops.torch_projectors`` backed by the reference's CPU AND CUDA kernels (its CUDA
    sources recompiled for sm_100 by ``oracle/build_ref.py --cuda``).  Speed comparator only.
    The CPU-only library and this one define the same op namespace, so a process can load just
    one of them."""
    global _ref_loaded
    import torch

    if _ref_loaded == "cuda":
        return torch.ops.torch_projectors
    if _ref_loaded:
        raise RuntimeError("the CPU-only reference library is already loaded in this process")
    if not _REF_CUDA_SO.exists():
        raise FileNotFoundError(f"{_REF_CUDA_SO} not built; run `python oracle/build_ref.py --cuda`")
    torch.ops.load_library(str(_REF_CUDA_SO))
    _ref_loaded = "cuda"
    return torch.ops.torch_projectors
