"""Host-to-host streaming wrappers: the operators of this package with HOST tensors on both
sides, pipelined so that PCIe copies overlap the kernels.

The reference API takes and returns device tensors, so a caller whose slices live in host
memory pays three serial phases: copy in, compute, copy out.  At B200 kernel speeds the
copies dominate (10,000 box-128 projections are 666 MB; the kernel that makes them runs
4 ms), so these helpers split the poses into chunks and use a second CUDA stream: while
chunk k is computed on the current stream, chunk k-1 is copied by the copy stream.  Pinned
host memory is required for the copies to be asynchronous; unpinned tensors still work, just
without overlap.  No autograd: these are inference / reconstruction paths.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import ops
from .sharding import PartialVolumes
from ._abi import rec_boxsize


def _device(device) -> torch.device:
    dev = torch.device(device if device is not None else "cuda")
    if dev.type != "cuda":
        raise RuntimeError("torch_projectors_b200 runs on CUDA devices only (there is no CPU path)")
    return dev if dev.index is not None else torch.device("cuda", torch.cuda.current_device())


def project_3d_to_2d_to_host(reconstruction: torch.Tensor, rotations: torch.Tensor,
                             shifts: Optional[torch.Tensor] = None, *,
                             out: Optional[torch.Tensor] = None, chunk: int = 1024, device=None,
                             output_shape: Optional[Tuple[int, int]] = None,
                             interpolation: str = "linear", oversampling: float = 1.0,
                             fourier_radius_cutoff: Optional[float] = None, packed: bool = False):
    """``project_3d_to_2d_forw`` from host (or device) inputs to a HOST result.

    ``packed=True``: only the pixels inside the cutoff are produced and copied (at the default
    cutoff 78 % of the bytes): returns (out [B,P,n_inside] pinned host tensor, index [N*Nh] int32
    host tensor); ``ops.unpack_projections(out, index, N)`` gives the dense slices.

    reconstruction [B,D,H,W/2+1], rotations [B_rot,P,3,3], shifts [B_s,P,2] may live on the
    host (ideally pinned) or on the device.  Projections are produced `chunk` poses at a time
    and copied into ``out`` (a pinned host tensor [B,P,N,Nh], allocated if not given) while
    the next chunk is computed.  On return all work has been ENQUEUED; the current stream is
    ordered after the last copy, so ``torch.cuda.current_stream().synchronize()`` (or any
    later work on it) makes ``out`` safe to read.
    """
    dev = _device(device if device is not None else (reconstruction.device if reconstruction.is_cuda else None))
    if rotations.dim() == 3:
        rotations = rotations.unsqueeze(0)
    if shifts is not None and shifts.dim() == 2:
        shifts = shifts.unsqueeze(0)
    with torch.cuda.device(dev):
        main = torch.cuda.current_stream(dev)
        copy = _copy_stream(dev)
        rec = reconstruction.to(dev, non_blocking=True)
        rot = rotations.to(dev, non_blocking=True)
        sh = shifts.to(dev, non_blocking=True) if shifts is not None else None
        B, P = rec.shape[0], rot.shape[1]
        N = int(output_shape[0]) if output_shape is not None else rec.shape[2]
        index = None
        shape = (B, P, N, N // 2 + 1)
        if packed:
            from . import _abi
            index, count = _abi.cutoff_pack_index(N, fourier_radius_cutoff if fourier_radius_cutoff is not None else N / 2.0, dev)
            shape = (B, P, count)
        if out is None:
            out = torch.empty(shape, dtype=torch.complex64, pin_memory=True)
        elif tuple(out.shape) != shape or out.dtype != torch.complex64 or out.is_cuda:
            raise ValueError(f"out must be a host complex64 tensor of shape {shape}")
        kw = dict(output_shape=(N, N), interpolation=interpolation, oversampling=oversampling,
                  fourier_radius_cutoff=fourier_radius_cutoff)
        for lo in range(0, P, max(1, chunk)):
            hi = min(P, lo + chunk)
            if packed:
                part, _ = ops.project_3d_to_2d_forw_packed(rec, rot[:, lo:hi], sh[:, lo:hi] if sh is not None else None, **kw)
            else:
                with torch.no_grad():
                    part = ops.project_3d_to_2d_forw(rec, rot[:, lo:hi], sh[:, lo:hi] if sh is not None else None, **kw)
            copy.wait_stream(main)
            with torch.cuda.stream(copy):
                out[:, lo:hi].copy_(part, non_blocking=True)
            part.record_stream(copy)          # keep the chunk alive until its copy has run
        main.wait_stream(copy)
    if packed:
        return out, index.cpu()
    return out


def backproject_2d_to_3d_from_host(projections: torch.Tensor, rotations: torch.Tensor,
                                   weights: Optional[torch.Tensor] = None,
                                   shifts: Optional[torch.Tensor] = None, *, chunk: int = 4096,
                                   device=None, interpolation: str = "linear",
                                   oversampling: float = 1.0,
                                   fourier_radius_cutoff: Optional[float] = None,
                                   into: Optional[PartialVolumes] = None) -> PartialVolumes:
    """``backproject_2d_to_3d_forw`` of HOST slices [B,P,N,Nh] (ideally pinned) into device
    volumes: chunk k+1 is copied to the device by the copy stream while chunk k is scattered.
    Returns the (data, weights) volumes as a ``PartialVolumes`` (pass ``into=`` to keep adding
    to existing ones)."""
    dev = _device(device)
    if rotations.dim() == 3:
        rotations = rotations.unsqueeze(0)
    if shifts is not None and shifts.dim() == 2:
        shifts = shifts.unsqueeze(0)
    B, P, N, _ = projections.shape
    with torch.cuda.device(dev):
        main = torch.cuda.current_stream(dev)
        copy = _copy_stream(dev)
        rot = rotations.to(dev, non_blocking=True)
        sh = shifts.to(dev, non_blocking=True) if shifts is not None else None
        vols = into if into is not None else PartialVolumes(B, rec_boxsize(N, oversampling), dev,
                                                            with_weights=weights is not None)
        copy.wait_stream(main)
        staged = None
        spans = [(lo, min(P, lo + chunk)) for lo in range(0, P, max(1, chunk))]

        def stage(span):
            lo, hi = span
            with torch.cuda.stream(copy):
                p = projections[:, lo:hi].to(dev, non_blocking=True)
                w = weights[:, lo:hi].to(dev, non_blocking=True) if weights is not None else None
                ev = torch.cuda.Event()
                ev.record(copy)
            return p, w, ev

        if spans:
            staged = stage(spans[0])
        for k, (lo, hi) in enumerate(spans):
            p, w, ev = staged
            if k + 1 < len(spans):
                staged = stage(spans[k + 1])
            main.wait_event(ev)
            vols.add_(p, rot[:, lo:hi], w, sh[:, lo:hi] if sh is not None else None,
                      interpolation=interpolation, oversampling=oversampling,
                      fourier_radius_cutoff=fourier_radius_cutoff)
            p.record_stream(main)
            if w is not None:
                w.record_stream(main)
        vols.flush()
    return vols


_copy_streams = {}


def _copy_stream(dev: torch.device) -> torch.cuda.Stream:
    s = _copy_streams.get(dev.index)
    if s is None:
        s = torch.cuda.Stream(device=dev)
        _copy_streams[dev.index] = s
    return s
