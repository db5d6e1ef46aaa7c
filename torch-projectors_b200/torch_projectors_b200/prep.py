"""The steps either side of the Fourier-slice operators, as the reference's README and test
utilities perform them (``README.md:96-160`` and ``tests/test_utils.py:174-293`` there):

* ``pad_and_fftshift``  real-space image / volume -> zero-padded (oversampled), fftshifted,
  rfft'd reconstruction in the layout the projection operators read;
* ``ifftshift_and_crop``  the inverse, for a back-projected reconstruction;
* ``normalize_by_weights``  the usual consumer of the (data, weight) pair of a weighted
  back-projection: data / max(weight, eps)  (``paper/main.tex:72`` there).

The FFTs are torch's (cuFFT on a GPU).  On a CUDA device the zero-padding and the shift that
moves the real-space centre to index 0 run as ONE pass of this package's library
(``b200proj_pad_fftshift`` / ``b200proj_ifftshift_crop``, each the adjoint of the other, which
is what their autograd needs) instead of a pad followed by a roll; CPU tensors take the plain
torch composition (host-side convenience and the reference for the tests).
"""
from __future__ import annotations

import torch


def _launch_in_batches(fn, src: torch.Tensor, dst: torch.Tensor, dims: int, a: int, b: int) -> None:
    """Call fn(src_chunk, batch, dims, a, b, dst_chunk) over the flattened leading axes, in chunks
    that fit one launch (grid z = batch * outer axis of the output <= 65535)."""
    src2 = src.reshape((-1,) + tuple(src.shape[-dims:]))
    dst2 = dst.reshape((-1,) + tuple(dst.shape[-dims:]))
    per_launch = max(1, 65535 // (dst.shape[-1] if dims == 3 else 1))
    for lo in range(0, src2.shape[0], per_launch):
        hi = min(src2.shape[0], lo + per_launch)
        fn(src2[lo:hi], hi - lo, dims, a, b, dst2[lo:hi])


class _PadShift(torch.autograd.Function):
    """[..., n(, n), n] real -> [..., m(, m), m]: zero-pad by (m-n)//2 in front of every axis and
    roll by m/2 (fftshift of the padded array), in one pass."""

    @staticmethod
    def forward(ctx, real, dims, m):
        from . import _abi
        real = real.contiguous()
        n = real.shape[-1]
        out = torch.empty(real.shape[:-dims] + (m,) * dims, dtype=real.dtype, device=real.device)
        if out.numel():
            _launch_in_batches(_abi.pad_fftshift, real, out, dims, n, m)
        ctx.dims, ctx.n = dims, n
        return out

    @staticmethod
    def backward(ctx, grad):
        return _CropUnshift.apply(grad, ctx.dims, ctx.n), None, None


class _CropUnshift(torch.autograd.Function):
    """[..., m(, m), m] real -> [..., n(, n), n]: roll back by m/2 (ifftshift) and keep the centred
    box n, in one pass; the adjoint of _PadShift."""

    @staticmethod
    def forward(ctx, full, dims, n):
        from . import _abi
        full = full.contiguous()
        m = full.shape[-1]
        out = torch.empty(full.shape[:-dims] + (n,) * dims, dtype=full.dtype, device=full.device)
        if out.numel():
            _launch_in_batches(_abi.ifftshift_crop, full, out, dims, m, n)
        ctx.dims, ctx.m = dims, m
        return out

    @staticmethod
    def backward(ctx, grad):
        return _PadShift.apply(grad, ctx.dims, ctx.m), None, None


def _fused(t: torch.Tensor, m: int) -> bool:
    return t.is_cuda and t.dtype in (torch.float32, torch.float64) and m % 2 == 0


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
    axes = tuple(range(-dims, 0))
    if _fused(real, m):
        shifted = _PadShift.apply(real, dims, m)
    else:
        lo = (m - n) // 2
        hi = m - n - lo
        padded = torch.nn.functional.pad(real, (lo, hi) * dims) if m > n else real
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
    n = int(m / oversampling)
    if _fused(real, m) and 1 <= n <= m:
        return _CropUnshift.apply(real, dims, n)
    real = torch.fft.ifftshift(real, dim=axes)
    lo = (m - n) // 2
    index = (Ellipsis,) + (slice(lo, lo + n),) * dims
    return real[index]


def normalize_by_weights(data_rec: torch.Tensor, weight_rec: torch.Tensor, eps: float = 1e-3) -> torch.Tensor:
    """Weighted-average reconstruction from the two outputs of a weighted back-projection:
    ``data / max(weight, eps)`` (voxels that received almost no weight stay near zero)."""
    if data_rec.shape != weight_rec.shape:
        raise ValueError("data and weight reconstructions must have the same shape")
    return data_rec / torch.clamp(weight_rec, min=eps)
