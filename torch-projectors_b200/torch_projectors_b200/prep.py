"""The steps either side of the Fourier-slice operators, as the reference's README and test
utilities perform them (``README.md:96-160`` and ``tests/test_utils.py:174-293`` there):

* ``pad_and_fftshift``  real-space image / volume -> zero-padded (oversampled), fftshifted,
  rfft'd reconstruction in the layout the projection operators read;
* ``ifftshift_and_crop``  the inverse, for a back-projected reconstruction;
* ``normalize_by_weights``  the usual consumer of the (data, weight) pair of a weighted
  back-projection: data / max(weight, eps)  (``paper/main.tex:72`` there).

These are thin compositions of torch's FFT (cuFFT on a GPU) and elementwise operators; they
run wherever their input lives and are differentiable through torch's own autograd.
"""
from __future__ import annotations

import torch


def pad_and_fftshift(real: torch.Tensor, oversampling: float = 1.0, dims: int = 3) -> torch.Tensor:
    """Zero-pad the last `dims` (2 or 3) axes of a real tensor symmetrically to
    ``round(n * oversampling)`` (made even), move the centre to index 0 and take the real FFT
    with ``norm='forward'``: [..., n, n(, n)] -> [..., m, m(, m/2+1)] complex."""
    if dims not in (2, 3):
        raise ValueError("dims must be 2 or 3")
    n = real.shape[-1]
    if any(s != n for s in real.shape[-dims:]):
        raise ValueError(f"the last {dims} axes must have equal length, got {tuple(real.shape[-dims:])}")
    m = int(round(n * oversampling))
    m += m % 2
    if m < n:
        raise ValueError("oversampling must be >= 1")
    lo = (m - n) // 2
    hi = m - n - lo
    padded = torch.nn.functional.pad(real, (lo, hi) * dims) if m > n else real
    axes = tuple(range(-dims, 0))
    shifted = torch.fft.fftshift(padded, dim=axes)
    return torch.fft.rfftn(shifted, dim=axes, norm="forward")


def ifftshift_and_crop(rec: torch.Tensor, oversampling: float = 1.0, dims: int = 3) -> torch.Tensor:
    """Inverse of ``pad_and_fftshift``: inverse real FFT (``norm='forward'``), centre back to
    the middle, crop the last `dims` axes to ``int(m / oversampling)``."""
    if dims not in (2, 3):
        raise ValueError("dims must be 2 or 3")
    axes = tuple(range(-dims, 0))
    m = rec.shape[-2]
    real = torch.fft.irfftn(rec, s=(m,) * dims, dim=axes, norm="forward")
    real = torch.fft.ifftshift(real, dim=axes)
    n = int(m / oversampling)
    lo = (m - n) // 2
    index = (Ellipsis,) + (slice(lo, lo + n),) * dims
    return real[index]


def normalize_by_weights(data_rec: torch.Tensor, weight_rec: torch.Tensor, eps: float = 1e-3) -> torch.Tensor:
    """Weighted-average reconstruction from the two outputs of a weighted back-projection:
    ``data / max(weight, eps)`` (voxels that received almost no weight stay near zero)."""
    if data_rec.shape != weight_rec.shape:
        raise ValueError("data and weight reconstructions must have the same shape")
    return data_rec / torch.clamp(weight_rec, min=eps)
