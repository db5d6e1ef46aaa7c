"""Public API and autograd glue over the C++ operator layer.

The seven public functions and the eight raw operators keep the names, argument lists,
defaults and error behaviour of warpem/torch-projectors (``torch_projectors/ops.py`` and
``csrc/torch_projectors.cpp:23-36`` in the reference) so that user code switches by
changing the import.  The raw operators are defined and implemented in C++
(``csrc/torch_binding.cpp``, built into ``_C.so``: ``TORCH_LIBRARY`` with the reference's schema
strings, ``TORCH_LIBRARY_IMPL`` for the CUDA key, shape-only Meta implementations) under the op
namespace ``torch_projectors_b200``; each calls one entry point of the C ABI
(``include/b200proj.h``).  Calling them with CPU (or MPS) tensors raises from the dispatcher --
there is no CPU fallback.  complex128 / float64 inputs, which the reference's CUDA wrappers
silently route through its CPU kernels (``csrc/cuda/3d/projection_3d_to_2d_kernels.cu:902-918``),
run on the GPU here (the same kernels instantiated for double); mixed precisions raise
``RuntimeError``.

As in the reference, autograd lives in Python (four ``autograd.Function``s).  Calls that cannot
need a gradient (no input requires one, or gradients are switched off) go straight to the raw
operator, which keeps small problems from paying for the autograd machinery.
"""
from __future__ import annotations

from typing import Optional, Union

import torch

from . import _abi
from . import build as _build

NAMESPACE = "torch_projectors_b200"


def _load_operator_library():
    """Load ``_C.so`` (building it first when absent or stale); ImportError when impossible."""
    path = _build.BINDING_PATH
    if _build.binding_needs_build():
        try:
            _build.build_binding()
        except Exception as e:  # noqa: BLE001
            raise ImportError(f"torch_projectors_b200: {path} is missing or stale and building it failed ({e}); "
                              "run `python -m torch_projectors_b200.build` on a machine with g++ and nvcc") from e
    try:
        torch.ops.load_library(str(path))
    except OSError as e:
        raise ImportError(f"torch_projectors_b200: cannot load {path}: {e}") from e


_load_operator_library()
_ops = getattr(torch.ops, NAMESPACE)


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _interp_code(interpolation: str) -> int:
    _check(interpolation in ("linear", "cubic"), "Supported interpolation methods: 'linear', 'cubic'")
    return _abi.CUBIC if interpolation == "cubic" else _abi.LINEAR


_REAL_OF = {torch.complex64: torch.float32, torch.complex128: torch.float64}


def _check_fp32(name: str, t: torch.Tensor, complex_: bool, like: Optional[torch.Tensor] = None) -> None:
    """Precision check: complex64 with float32 (the fast path) or complex128 with float64 (same
    kernels instantiated for double); every tensor of a call must be of the same precision as
    `like` (the call's main complex tensor).  Nothing else is accepted and nothing is converted."""
    allowed = (torch.complex64, torch.complex128) if complex_ else (torch.float32, torch.float64)
    if t.dtype not in allowed:
        raise RuntimeError(
            f"{name} has dtype {t.dtype}; the B200 kernels compute in complex64/float32 or "
            f"complex128/float64 only and there is no CPU fallback for other precisions")
    if like is not None:
        want = like.dtype if complex_ else _REAL_OF[like.dtype]
        if t.dtype != want:
            raise RuntimeError(f"{name} has dtype {t.dtype} but {want} is needed to match the {like.dtype} data "
                               f"(mixed precisions are not supported)")


def _check_pose_inputs(dim: int, what: str, B: int, rotations, shifts, like: torch.Tensor):
    """Shape / device / dtype checks shared by all operators; returns (P, rot, shifts)
    as contiguous tensors (expanded or sliced pose tensors are legal inputs)."""
    _check(rotations.is_cuda, "Input rotations must be on CUDA device")
    _check(rotations.dim() == 4 and rotations.size(2) == dim and rotations.size(3) == dim,
           f"Rotations must be (B_rot, P, {dim}, {dim})")
    _check(rotations.device == like.device, "rotations must be on the same device as the data")
    _check_fp32("rotations", rotations, False, like)
    B_rot, P = rotations.size(0), rotations.size(1)
    _check(B_rot == B or B_rot == 1, f"Batch size of rotations must be 1 or same as {what}")
    if shifts is not None:
        _check(shifts.is_cuda, "Shifts must be on CUDA device")
        _check(shifts.dim() == 3, "Shifts must be (B_shift, P, 2)")
        _check(shifts.size(2) == 2, "Shifts must have 2 components (x, y)")
        _check(shifts.size(0) == B or shifts.size(0) == 1, f"Batch size of shifts must be 1 or same as {what}")
        _check(shifts.size(1) == P, "Number of poses in shifts must match rotations")
        _check(shifts.dtype == rotations.dtype, "Shifts and rotations must have the same dtype")
        _check(shifts.device == like.device, "shifts must be on the same device as the data")
        shifts = shifts.contiguous()
    return P, rotations.contiguous(), shifts


def _backproject_workspace(dim, B, R, P, N, interp, weights, device):
    """Scratch for the interleaved accumulation path of the back-projection kernels (from
    torch's caching allocator, so nothing is freed behind the stream); None when the
    library says a workspace would not help."""
    if weights is not None and weights.dtype != torch.float32:
        return None                      # the interleaved accumulation path is fp32 only
    n = _abi.backproject_workspace_bytes(dim, B, R, P, N, interp, weights is not None)
    return torch.empty(n, dtype=torch.uint8, device=device) if n else None


# Volumes (one batch item) at least this large get a locality-preserving processing order of
# their slices when the caller gives none; below it the whole volume stays in the 126 MB L2 and
# the order changes nothing.  Change them with set_pose_order_thresholds (the C++ layer holds a copy).
POSE_ORDER_MIN_BYTES = 96 << 20
POSE_ORDER_MIN_POSES = 64


def set_pose_order_thresholds(min_volume_bytes: int = 96 << 20, min_poses: int = 64) -> None:
    """When the 3D operators that read a volume derive a processing order of the slices by
    themselves: volumes of at least `min_volume_bytes` per batch item and at least `min_poses` poses."""
    global POSE_ORDER_MIN_BYTES, POSE_ORDER_MIN_POSES
    POSE_ORDER_MIN_BYTES, POSE_ORDER_MIN_POSES = int(min_volume_bytes), int(min_poses)
    _ops._set_pose_order_thresholds(POSE_ORDER_MIN_BYTES, POSE_ORDER_MIN_POSES)


# Saved derivatives: when the rotations of a cubic 3D projection need gradients, the forward pass can
# also write every pixel's derivatives with respect to its sample position (three more tensors of
# the projections' size), and the backward pass then forms the pose gradients from them instead of
# gathering the volume a second time -- and skips the scatter into the volume's gradient altogether
# when the volume needs none.  Measured on B200, box 512, 4,096 poses of 256 x 256, cubic: forward
# 6.5 -> 8.9 ms, backward 20.3 -> 15.1 ms (1.9 ms with a fixed volume).
# When the reconstruction needs a gradient too, the backward pass still scatters, and onto a small
# reconstruction that scatter is bound by contention, not by the gather beside it (one 128 x 65
# reference, 65,536 poses, cubic: 9.8 ms either way, while the forward pass pays 1.4 ms for the
# derivatives): below SAVE_DERIVATIVES_MIN_VOLUME_BYTES per batch item the plain pair stays.
SAVE_DERIVATIVES = True
SAVE_DERIVATIVES_MAX_BYTES = 16 << 30
SAVE_DERIVATIVES_MIN_VOLUME_BYTES = 2 << 20


def set_save_derivatives(enabled: bool = True, max_bytes: int = 16 << 30, min_volume_bytes: int = 2 << 20) -> None:
    """Whether ``project_2d_forw`` / ``project_3d_to_2d_forw`` keep their pixels' derivatives for the
    backward pass when the rotations require gradients (complex64; when the reconstruction needs a
    gradient as well: cubic interpolation and at least `min_volume_bytes` per batch item), and up to
    which size of that extra tensor (2 or 3 x the projections)."""
    global SAVE_DERIVATIVES, SAVE_DERIVATIVES_MAX_BYTES, SAVE_DERIVATIVES_MIN_VOLUME_BYTES
    SAVE_DERIVATIVES, SAVE_DERIVATIVES_MAX_BYTES = bool(enabled), int(max_bytes)
    SAVE_DERIVATIVES_MIN_VOLUME_BYTES = int(min_volume_bytes)


def plane_locality_order(rotations: torch.Tensor, batch: int = 1) -> torch.Tensor:
    """int32 [batch * P] processing order of the slices of a 3D operator that reads a volume:
    slices whose planes lie close together come one after the other, so that a volume larger than
    L2 is read from DRAM far less often.  Results of the operators do not depend on it.  Compute it
    once per set of rotations and pass it as ``pose_order=`` to ``project_3d_to_2d_forw`` (its
    backward reuses it) for as many iterations as the rotations stay (roughly) the same.
    rotations: [B_rot, P, 3, 3] (or [P, 3, 3]) on the device."""
    if rotations.dim() == 3:
        rotations = rotations.unsqueeze(0)
    return _ops.plane_locality_order(rotations.detach(), int(batch))


_NATURAL = {}


def _natural_order(device) -> torch.Tensor:
    """The empty int32 tensor that tells the operators to keep the given order of the slices."""
    t = _NATURAL.get(device)
    if t is None:
        t = _NATURAL[device] = torch.empty(0, dtype=torch.int32, device=device)
    return t


def _resolve_order(pose_order, vol: torch.Tensor, rotations: torch.Tensor) -> torch.Tensor:
    """pose_order argument of the public 3D functions -> the tensor handed to the operators (and
    kept for the backward pass): a given order as it is, ``False`` = natural order, ``None`` = made
    here when the volume is large enough for it to matter."""
    if isinstance(pose_order, torch.Tensor):
        return pose_order
    if pose_order is None and rotations.size(1) >= POSE_ORDER_MIN_POSES and \
            vol[0].numel() * vol.element_size() >= POSE_ORDER_MIN_BYTES and vol.is_cuda:
        return _ops.plane_locality_order(rotations.detach(), vol.size(0))
    return _natural_order(vol.device)


def _cutoff(fourier_radius_cutoff: Optional[float], N: int) -> float:
    # default: Nyquist radius of the projection (reference: projection_3d_to_2d_kernels.cu:892)
    return float(fourier_radius_cutoff) if fourier_radius_cutoff is not None else N / 2.0


# ---------------------------------------------------------------------------------------
# public functions (reference: torch_projectors/ops.py:6-296)
# ---------------------------------------------------------------------------------------
def _validate_rec_box(boxsize: int, boxsize_half: int) -> None:
    if boxsize % 2 != 0:
        raise ValueError(f"Boxsize ({boxsize}) must be even. Only even dimensions are supported.")
    if boxsize != (boxsize_half - 1) * 2:
        raise ValueError(f"Reconstruction shape mismatch: expected boxsize {boxsize} to match 2*(boxsize_half-1) = {(boxsize_half - 1) * 2}")


def _validate_output_shape(output_shape, boxsize: int):
    if output_shape is None:
        return (boxsize, boxsize)
    if len(output_shape) != 2 or output_shape[0] != output_shape[1]:
        raise ValueError(f"Output shape {output_shape} must be square (height == width)")
    if output_shape[0] % 2 != 0:
        raise ValueError(f"Output boxsize {output_shape[0]} must be even")
    return output_shape


def _validate_projections(projections, weights) -> None:
    if projections.dim() != 4:
        raise ValueError("Projections must be a 4D tensor (B, P, height, width/2+1)")
    _, _, proj_boxsize, proj_boxsize_half = projections.shape
    if proj_boxsize % 2 != 0:
        raise ValueError(f"Projection boxsize ({proj_boxsize}) must be even. Only even dimensions are supported.")
    if proj_boxsize != (proj_boxsize_half - 1) * 2:
        raise ValueError(f"Projection shape mismatch: expected boxsize {proj_boxsize} to match 2*(boxsize_half-1) = {(proj_boxsize_half - 1) * 2}")
    if weights is not None:
        if weights.shape != projections.shape:
            raise ValueError(f"Weights shape {weights.shape} must match projections shape {projections.shape}")
        if not weights.is_floating_point():
            raise ValueError("Weights must be real-valued (floating point)")


def _wants_grad(*tensors) -> bool:
    return torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors)


def project_2d_forw(reconstruction: torch.Tensor, rotations: torch.Tensor,
                    shifts: Optional[torch.Tensor] = None,
                    output_shape: Optional[tuple[int, ...]] = None,
                    interpolation: str = "linear", oversampling: float = 1.0,
                    fourier_radius_cutoff: Optional[float] = None) -> torch.Tensor:
    """Sample P rotated 2D rfft images from 2D rfft reconstructions [B, H, W/2+1]
    -> [B, P, H_out, W_out/2+1].  (reference: torch_projectors/ops.py:6-38)"""
    if reconstruction.dim() < 2:
        raise ValueError("Reconstruction must have at least 2 dimensions")
    _validate_rec_box(reconstruction.shape[-2], reconstruction.shape[-1])
    output_shape = _validate_output_shape(output_shape, reconstruction.shape[-2])
    if not _wants_grad(reconstruction, rotations, shifts):
        reconstruction, rotations, shifts = _canon_project(2, reconstruction, rotations, shifts)
        return _ops.project_2d_forw(reconstruction, rotations, shifts, output_shape, interpolation,
                                    oversampling, fourier_radius_cutoff)
    return _Project2D.apply(reconstruction, rotations, shifts, output_shape, interpolation,
                            oversampling, fourier_radius_cutoff)


def project_2d_back(projections: torch.Tensor, reconstruction: torch.Tensor,
                    rotations: torch.Tensor, shifts: Optional[torch.Tensor] = None,
                    interpolation: str = "linear", oversampling: float = 1.0) -> torch.Tensor:
    """Gradient of ``project_2d_forw`` w.r.t. the reconstruction only.
    (reference: torch_projectors/ops.py:40-59)"""
    grad_reconstruction, _, _ = _ops.project_2d_back(
        projections, reconstruction, rotations, shifts, interpolation, oversampling, None)
    return grad_reconstruction


def backproject_2d_forw(projections: torch.Tensor, rotations: torch.Tensor,
                        weights: Optional[torch.Tensor] = None,
                        shifts: Optional[torch.Tensor] = None, interpolation: str = "linear",
                        oversampling: float = 1.0,
                        fourier_radius_cutoff: Optional[float] = None
                        ) -> tuple[torch.Tensor, torch.Tensor]:
    """Adjoint of ``project_2d_forw``: accumulate projections [B, P, H, W/2+1] (and optional
    real weights) into 2D rfft reconstructions.  Returns (data, weights); the second is an
    empty ``(0,)`` tensor without weights.  (reference: torch_projectors/ops.py:61-117)"""
    _validate_projections(projections, weights)
    if not _wants_grad(projections, weights, rotations, shifts):
        projections, weights, rotations, shifts = _canon_backproject(projections, weights, rotations, shifts)
        return _ops.backproject_2d_forw(projections, weights, rotations, shifts, interpolation,
                                        oversampling, fourier_radius_cutoff)
    return _Backproject2D.apply(projections, weights, rotations, shifts, interpolation,
                                oversampling, fourier_radius_cutoff)


def project_3d_to_2d_forw(reconstruction: torch.Tensor, rotations: torch.Tensor,
                          shifts: Optional[torch.Tensor] = None,
                          output_shape: Optional[tuple[int, ...]] = None,
                          interpolation: str = "linear", oversampling: float = 1.0,
                          fourier_radius_cutoff: Optional[float] = None,
                          pose_order: Union[torch.Tensor, bool, None] = None) -> torch.Tensor:
    """Sample P rotated central slices from 3D rfft volumes [B, D, H, W/2+1]
    -> [B, P, H_out, W_out/2+1].  (reference: torch_projectors/ops.py:119-174)

    ``pose_order`` (not in the reference API) is the processing order of the slices
    (``plane_locality_order``): None = derived here when the volume is larger than L2 and there are
    enough poses, once per call and reused by the backward pass; a tensor = reused as given (compute
    it once for a training loop over the same rotations); False = the order given.  Results do not
    depend on it."""
    if reconstruction.dim() != 4:
        raise ValueError("Reconstruction must be a 4D tensor (B, D, H, W/2+1)")
    _validate_rec_box(reconstruction.shape[2], reconstruction.shape[3])
    output_shape = _validate_output_shape(output_shape, reconstruction.shape[2])
    if not _wants_grad(reconstruction, rotations, shifts):
        reconstruction, rotations, shifts = _canon_project(3, reconstruction, rotations, shifts)
        if pose_order is None:        # the operator derives the order by the same thresholds
            return _ops.project_3d_to_2d_forw(reconstruction, rotations, shifts, output_shape, interpolation,
                                              oversampling, fourier_radius_cutoff)
        return _ops.project_3d_to_2d_forw_ordered(reconstruction, rotations, shifts, output_shape, interpolation,
                                                  oversampling, fourier_radius_cutoff,
                                                  _resolve_order(pose_order, reconstruction, rotations))
    return _Project3DTo2D.apply(reconstruction, rotations, shifts, output_shape, interpolation,
                                oversampling, fourier_radius_cutoff, pose_order)


def project_3d_to_2d_back(projections: torch.Tensor, reconstruction: torch.Tensor,
                          rotations: torch.Tensor, shifts: Optional[torch.Tensor] = None,
                          interpolation: str = "linear", oversampling: float = 1.0) -> torch.Tensor:
    """Gradient of ``project_3d_to_2d_forw`` w.r.t. the volume only.
    (reference: torch_projectors/ops.py:176-206)"""
    grad_reconstruction, _, _ = _ops.project_3d_to_2d_back(
        projections, reconstruction, rotations, shifts, interpolation, oversampling, None)
    return grad_reconstruction


def backproject_2d_to_3d_forw(projections: torch.Tensor, rotations: torch.Tensor,
                              weights: Optional[torch.Tensor] = None,
                              shifts: Optional[torch.Tensor] = None,
                              interpolation: str = "linear", oversampling: float = 1.0,
                              fourier_radius_cutoff: Optional[float] = None
                              ) -> tuple[torch.Tensor, torch.Tensor]:
    """Adjoint of ``project_3d_to_2d_forw``: accumulate 2D slices (and optional real weights)
    into cubic 3D rfft volumes of box ceil(N*oversampling) rounded up to even.
    (reference: torch_projectors/ops.py:208-264)"""
    _validate_projections(projections, weights)
    if not _wants_grad(projections, weights, rotations, shifts):
        projections, weights, rotations, shifts = _canon_backproject(projections, weights, rotations, shifts)
        return _ops.backproject_2d_to_3d_forw(projections, weights, rotations, shifts, interpolation,
                                              oversampling, fourier_radius_cutoff)
    return _Backproject2DTo3D.apply(projections, weights, rotations, shifts, interpolation,
                                    oversampling, fourier_radius_cutoff)


def backproject_2d_to_3d_back(reconstruction: torch.Tensor, projections: torch.Tensor,
                              rotations: torch.Tensor, shifts: Optional[torch.Tensor] = None,
                              interpolation: str = "linear", oversampling: float = 1.0) -> torch.Tensor:
    """Gradient of ``backproject_2d_to_3d_forw`` w.r.t. the projections only, given the
    gradient of the data volume.  (reference: torch_projectors/ops.py:266-296; the reference
    wrapper passes 7 arguments to a 9-argument operator and cannot run -- this one passes
    ``None`` for the weight-related arguments, which is what its docstring describes.)"""
    grad_projections, _, _, _ = _ops.backproject_2d_to_3d_back(
        reconstruction, None, projections, None, rotations, shifts, interpolation, oversampling, None)
    return grad_projections


def backproject_2d_to_3d_accumulate_(data_rec: torch.Tensor, weight_rec: Optional[torch.Tensor],
                                     projections: torch.Tensor, rotations: torch.Tensor,
                                     weights: Optional[torch.Tensor] = None,
                                     shifts: Optional[torch.Tensor] = None,
                                     interpolation: str = "linear", oversampling: float = 1.0,
                                     fourier_radius_cutoff: Optional[float] = None) -> None:
    """In-place streaming variant of ``backproject_2d_to_3d_forw`` (no autograd): adds the
    given chunk of projections into existing volumes instead of returning fresh ones, so
    that many chunks accumulate without a per-chunk volume-sized sum.  Not in the reference
    API; its callers sum per-call outputs
    (tests/3d/back/test_performance_back_2d_to_3d.py:357-369 there)."""
    _validate_projections(projections, weights)
    if projections.dim() == 4 and rotations.dim() == 3:
        rotations = rotations.unsqueeze(0)
    if shifts is not None and shifts.dim() == 2:
        shifts = shifts.unsqueeze(0)
    _check(projections.is_cuda, "Input projections must be on CUDA device")
    _check_fp32("projections", projections, True)
    B, P_p, N, _ = projections.shape
    interp = _interp_code(interpolation)
    if weights is not None:
        _check(weight_rec is not None, "weights given but weight_rec is None")
        _check(weights.is_cuda, "Weights must be on CUDA device")
        _check_fp32("weights", weights, False, projections)
        weights = weights.contiguous()
    P, rot, sh = _check_pose_inputs(3, "projections", B, rotations, shifts, projections)
    _check(P == P_p, "Number of poses in rotations must match projections")
    R = _abi.rec_boxsize(N, oversampling)
    want = (B, R, R, R // 2 + 1)
    _check(tuple(data_rec.shape) == want and data_rec.dtype == projections.dtype and data_rec.is_contiguous()
           and data_rec.device == projections.device, f"data_rec must be a contiguous {projections.dtype} tensor of shape {want}")
    if weights is not None:
        _check(tuple(weight_rec.shape) == want and weight_rec.dtype == _REAL_OF[projections.dtype] and weight_rec.is_contiguous()
               and weight_rec.device == projections.device, f"weight_rec must be a contiguous {_REAL_OF[projections.dtype]} tensor of shape {want}")
    if P == 0:
        return
    _abi.backproject_forw(3, projections.contiguous(), weights, rot, sh, interp, oversampling,
                          _cutoff(fourier_radius_cutoff, N), data_rec,
                          weight_rec if weights is not None else None, True,
                          _backproject_workspace(3, B, R, P, N, interp, weights, projections.device))


def new_backprojection_accumulator(batch: int, box: int, device) -> torch.Tensor:
    """Zero-filled persistent accumulator for ``backproject_2d_to_3d_accumulate_interleaved_``:
    float32 [batch, box, box, box//2+1, 4], one 16-byte (re, im, weight, 0) slot per voxel."""
    _check(box >= 2 and box % 2 == 0, f"reconstruction boxsize {box} must be even")
    assert _abi.accumulator_bytes(batch, box) == batch * box * box * (box // 2 + 1) * 16
    return torch.zeros((batch, box, box, box // 2 + 1, 4), dtype=torch.float32, device=device)


def prepare_accumulate_interleaved(accumulator: torch.Tensor, projections: torch.Tensor,
                                   rotations: torch.Tensor, weights: torch.Tensor,
                                   shifts: Optional[torch.Tensor] = None,
                                   interpolation: str = "linear", oversampling: float = 1.0,
                                   fourier_radius_cutoff: Optional[float] = None):
    """Validate one chunk for the interleaved accumulator and return the positional arguments of
    ``_abi.backproject_accumulate`` / ``_abi.backproject_accumulate_slabs`` (contiguous tensors
    included, so holding the tuple keeps them alive), or None for an empty chunk."""
    _validate_projections(projections, weights)
    _check(weights is not None, "the interleaved accumulator needs weights")
    if projections.dim() == 4 and rotations.dim() == 3:
        rotations = rotations.unsqueeze(0)
    if shifts is not None and shifts.dim() == 2:
        shifts = shifts.unsqueeze(0)
    _check(projections.is_cuda and weights.is_cuda, "projections and weights must be on a CUDA device")
    _check(projections.dtype == torch.complex64 and weights.dtype == torch.float32,
           "the interleaved accumulator holds float32 sums: projections must be complex64 and weights float32")
    B, P_p, N, _ = projections.shape
    interp = _interp_code(interpolation)
    P, rot, sh = _check_pose_inputs(3, "projections", B, rotations, shifts, projections)
    _check(P == P_p, "Number of poses in rotations must match projections")
    R = _abi.rec_boxsize(N, oversampling)
    want = (B, R, R, R // 2 + 1, 4)
    _check(tuple(accumulator.shape) == want and accumulator.dtype == torch.float32 and accumulator.is_contiguous()
           and accumulator.device == projections.device, f"accumulator must be a contiguous float32 tensor of shape {want}")
    if P == 0:
        return None
    return (projections.contiguous(), weights.contiguous(), rot, sh, interp, oversampling,
            _cutoff(fourier_radius_cutoff, N), R, accumulator)


def backproject_2d_to_3d_accumulate_interleaved_(accumulator: torch.Tensor, projections: torch.Tensor,
                                                 rotations: torch.Tensor, weights: torch.Tensor,
                                                 shifts: Optional[torch.Tensor] = None,
                                                 interpolation: str = "linear", oversampling: float = 1.0,
                                                 fourier_radius_cutoff: Optional[float] = None) -> None:
    """Streaming weighted back-projection (no autograd) that adds a chunk of slices into a
    persistent interleaved accumulator (``new_backprojection_accumulator``): data and weight of
    a tap leave as ONE vector reduction, nothing is zero-filled or folded per chunk, and
    volumes beyond L2 take the slab-ordered kernel.  ``fold_backprojection_accumulator``
    turns the sums into the usual data / weight volumes.  complex64 / float32 only.  Not in the
    reference API."""
    call = prepare_accumulate_interleaved(accumulator, projections, rotations, weights, shifts,
                                          interpolation, oversampling, fourier_radius_cutoff)
    if call is not None:
        _abi.backproject_accumulate(*call)


def fold_backprojection_accumulator(accumulator: torch.Tensor, data_rec: Optional[torch.Tensor] = None,
                                    weight_rec: Optional[torch.Tensor] = None, accumulate: bool = False,
                                    voxel_range: Optional[tuple] = None):
    """(data_rec, weight_rec) = the sums held by the accumulator, written into (or, with
    ``accumulate=True``, added to) the given volumes; fresh ones are made when none are given.
    ``voxel_range=(first, stop)`` folds only that range of the flattened volumes (the rest of the
    outputs is left as it is).  The accumulator itself is left unchanged."""
    _check(accumulator.is_cuda and accumulator.dtype == torch.float32 and accumulator.dim() == 5
           and accumulator.size(-1) == 4 and accumulator.is_contiguous(), "accumulator must come from new_backprojection_accumulator")
    shape = tuple(accumulator.shape[:-1])
    B, R = shape[0], shape[1]
    if data_rec is None:
        _check(not accumulate, "accumulate=True needs existing volumes")
        data_rec = torch.empty(shape, dtype=torch.complex64, device=accumulator.device)
    if weight_rec is None:
        _check(not accumulate, "accumulate=True needs existing volumes")
        weight_rec = torch.empty(shape, dtype=torch.float32, device=accumulator.device)
    for t, dt, what in ((data_rec, torch.complex64, "data_rec"), (weight_rec, torch.float32, "weight_rec")):
        _check(tuple(t.shape) == shape and t.dtype == dt and t.is_contiguous() and t.device == accumulator.device,
               f"{what} must be a contiguous {dt} tensor of shape {shape}")
    if voxel_range is not None:
        first, stop = int(voxel_range[0]), int(voxel_range[1])
        _check(0 <= first <= stop <= data_rec.numel(), f"voxel_range {voxel_range} outside the volume of {data_rec.numel()} voxels")
        voxel_range = (first, stop)
    _abi.accumulator_fold(accumulator, B, R, data_rec, weight_rec, accumulate, voxel_range)
    return data_rec, weight_rec


def fold_backprojection_accumulator_normalized(accumulator: torch.Tensor, eps: float = 1e-3,
                                               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The weighted-average reconstruction ``data / max(weight, eps)`` straight from the
    accumulator (fold and division in one pass; the same values as
    ``prep.normalize_by_weights(*fold_backprojection_accumulator(acc), eps)``).  For reconstructions
    made on one GPU; partial volumes of several ranks have to be reduced before they are divided."""
    _check(accumulator.is_cuda and accumulator.dtype == torch.float32 and accumulator.dim() == 5
           and accumulator.size(-1) == 4 and accumulator.is_contiguous(), "accumulator must come from new_backprojection_accumulator")
    _check(eps > 0, "eps must be positive")
    shape = tuple(accumulator.shape[:-1])
    if out is None:
        out = torch.empty(shape, dtype=torch.complex64, device=accumulator.device)
    _check(tuple(out.shape) == shape and out.dtype == torch.complex64 and out.is_contiguous() and out.device == accumulator.device,
           f"out must be a contiguous complex64 tensor of shape {shape}")
    if out.numel():
        _abi.accumulator_fold_normalized(accumulator, eps, out)
    return out


def project_3d_to_2d_forw_packed(reconstruction: torch.Tensor, rotations: torch.Tensor,
                                 shifts: Optional[torch.Tensor] = None, output_shape: Optional[tuple] = None,
                                 interpolation: str = "linear", oversampling: float = 1.0,
                                 fourier_radius_cutoff: Optional[float] = None,
                                 pose_order: Union[torch.Tensor, bool, None] = None):
    """``project_3d_to_2d_forw`` (no autograd, complex64) that produces only the pixels inside the
    cutoff: returns (packed [B, P, n_inside] complex64, index [N * Nh] int32 with the position of
    every pixel among the packed ones, -1 outside).  ``unpack_projections`` restores the dense
    slices.  For results that leave the device: the zeros outside the cutoff are never moved."""
    if reconstruction.dim() != 4:
        raise ValueError("Reconstruction must be a 4D tensor (B, D, H, W/2+1)")
    _validate_rec_box(reconstruction.shape[2], reconstruction.shape[3])
    output_shape = _validate_output_shape(output_shape, reconstruction.shape[2])
    reconstruction, rotations, shifts = _canon_project(3, reconstruction, rotations, shifts)
    _check(reconstruction.is_cuda and reconstruction.dtype == torch.complex64, "the packed projection takes complex64 CUDA volumes")
    interp = _interp_code(interpolation)
    B, N = reconstruction.size(0), int(output_shape[0])
    P, rot, sh = _check_pose_inputs(3, "reconstruction", B, rotations, shifts, reconstruction)
    cutoff = _cutoff(fourier_radius_cutoff, N)
    index, count = _abi.cutoff_pack_index(N, cutoff, reconstruction.device)
    packed = torch.empty((B, P, count), dtype=torch.complex64, device=reconstruction.device)
    if packed.numel():
        rec = reconstruction.contiguous()
        order = _resolve_order(pose_order, rec, rot)
        _abi.project_3d_to_2d_forw_packed(rec, rot, sh, P, N, interp, oversampling, cutoff, packed, index, count,
                                          order if order.numel() else None)
    return packed, index


def unpack_projections(packed: torch.Tensor, index: torch.Tensor, boxsize: int) -> torch.Tensor:
    """Dense [B, P, N, N/2+1] slices (zeros outside the cutoff) from the output of
    ``project_3d_to_2d_forw_packed``; works on host or device tensors."""
    Nh = boxsize // 2 + 1
    index = index.to(packed.device).long()
    inside = index >= 0
    dense = torch.zeros(packed.shape[:-1] + (boxsize * Nh,), dtype=packed.dtype, device=packed.device)
    dense[..., inside] = packed[..., index[inside]]
    return dense.view(packed.shape[:-1] + (boxsize, Nh))


# ---------------------------------------------------------------------------------------
# autograd glue (reference: torch_projectors/ops.py:300-514)
# ---------------------------------------------------------------------------------------
def _canon_poses(rotations, shifts):
    if rotations.dim() == 2:
        rotations = rotations.unsqueeze(0)
    if rotations.dim() == 3:
        rotations = rotations.unsqueeze(0)
    if shifts is not None:
        if shifts.dim() == 1:
            shifts = shifts.unsqueeze(0)
        if shifts.dim() == 2:
            shifts = shifts.unsqueeze(0)
    return rotations, shifts


def _canon_project(rec_rank: int, reconstruction, rotations, shifts):
    """Ranks of the raw operators: [B, (R,) R, Rh], [B_rot, P, d, d], [B_s, P, 2]."""
    if reconstruction.dim() == rec_rank:
        reconstruction = reconstruction.unsqueeze(0)
    rotations, shifts = _canon_poses(rotations, shifts)
    if rotations.size(0) != reconstruction.size(0) and rotations.size(0) != 1:
        raise ValueError("Batch size of rotations must be 1 or match reconstruction")
    return reconstruction, rotations, shifts


_PLAIN, _KEEP_DERIVATIVES, _KEEP_OUTPUT = 0, 1, 2


def _save_derivatives(dim, reconstruction, rotations, output_shape, interpolation, need_rec, need_rot, need_shift=False) -> int:
    """What a projection's forward pass keeps for the backward pass: nothing but its inputs (the
    backward pass gathers the reconstruction again), its pixels' derivatives and its output
    (rotation gradients wanted), or its output alone (shift gradients wanted but no rotation
    gradients: they are Im(grad * conj(output)) times the frequency)."""
    if not (SAVE_DERIVATIVES and reconstruction.is_cuda and reconstruction.dtype == torch.complex64
            and rotations.dtype == torch.float32):
        return _PLAIN
    if not need_rot:
        return _KEEP_OUTPUT if need_shift else _PLAIN      # costs the forward pass nothing and spares the backward pass its gather
    if need_rec and not (interpolation == "cubic" and reconstruction[0].numel() * 8 >= SAVE_DERIVATIVES_MIN_VOLUME_BYTES):
        return _PLAIN
    N = int(output_shape[0])
    fits = 8 * dim * reconstruction.size(0) * rotations.size(1) * N * (N // 2 + 1) <= SAVE_DERIVATIVES_MAX_BYTES
    return _KEEP_DERIVATIVES if fits else _PLAIN


class _Project2D(torch.autograd.Function):
    @staticmethod
    def forward(ctx, reconstruction, rotations, shifts, output_shape, interpolation, oversampling,
                fourier_radius_cutoff):
        reconstruction, rotations, shifts = _canon_project(2, reconstruction, rotations, shifts)
        need_rec = ctx.needs_input_grad[0]
        ctx.saving = _save_derivatives(2, reconstruction, rotations, output_shape, interpolation, need_rec, ctx.needs_input_grad[1],
                                       shifts is not None and ctx.needs_input_grad[2])
        ctx.need_rec = need_rec
        if ctx.saving == _KEEP_DERIVATIVES:
            projection, derivatives = _ops.project_2d_forw_saving(reconstruction, rotations, shifts, output_shape, interpolation,
                                                                  oversampling, fourier_radius_cutoff)
            ctx.save_for_backward(reconstruction, rotations, shifts, projection, derivatives)
        elif ctx.saving == _KEEP_OUTPUT:
            projection = _ops.project_2d_forw(reconstruction, rotations, shifts, output_shape, interpolation,
                                              oversampling, fourier_radius_cutoff)
            ctx.save_for_backward(reconstruction, rotations, shifts, projection, projection.new_empty(0))
        else:
            projection = _ops.project_2d_forw(reconstruction, rotations, shifts, output_shape, interpolation,
                                              oversampling, fourier_radius_cutoff)
            ctx.save_for_backward(reconstruction, rotations, shifts)
        ctx.interpolation = interpolation
        ctx.oversampling = oversampling
        ctx.fourier_radius_cutoff = fourier_radius_cutoff
        return projection

    @staticmethod
    def backward(ctx, grad_output):
        if ctx.saving:
            reconstruction, rotations, shifts, projection, derivatives = ctx.saved_tensors
            grad_reconstruction, grad_rotations, grad_shifts = _ops.project_2d_back_saved(
                grad_output.contiguous(), projection, derivatives, reconstruction, rotations, shifts, ctx.interpolation,
                ctx.oversampling, ctx.fourier_radius_cutoff, ctx.need_rec)
            if not ctx.need_rec:
                grad_reconstruction = None
        else:
            reconstruction, rotations, shifts = ctx.saved_tensors
            grad_reconstruction, grad_rotations, grad_shifts = _ops.project_2d_back(
                grad_output.contiguous(), reconstruction, rotations, shifts, ctx.interpolation,
                ctx.oversampling, ctx.fourier_radius_cutoff)
        if shifts is None:
            grad_shifts = None
        return grad_reconstruction, grad_rotations, grad_shifts, None, None, None, None


class _Project3DTo2D(torch.autograd.Function):
    @staticmethod
    def forward(ctx, reconstruction, rotations, shifts, output_shape, interpolation, oversampling,
                fourier_radius_cutoff, pose_order):
        reconstruction, rotations, shifts = _canon_project(3, reconstruction, rotations, shifts)
        # the processing order of the slices is settled once here and kept for the backward pass
        order = _resolve_order(pose_order, reconstruction, rotations)
        need_rec = ctx.needs_input_grad[0]
        saving = _save_derivatives(3, reconstruction, rotations, output_shape, interpolation, need_rec, ctx.needs_input_grad[1],
                                   shifts is not None and ctx.needs_input_grad[2])
        ctx.saving = saving
        ctx.need_rec = need_rec
        if saving == _KEEP_DERIVATIVES:
            projection, derivatives = _ops.project_3d_to_2d_forw_saving(reconstruction, rotations, shifts, output_shape, interpolation,
                                                                        oversampling, fourier_radius_cutoff, order)
            ctx.save_for_backward(reconstruction, rotations, shifts, projection, derivatives)
        elif saving == _KEEP_OUTPUT:
            projection = _ops.project_3d_to_2d_forw_ordered(reconstruction, rotations, shifts, output_shape, interpolation,
                                                            oversampling, fourier_radius_cutoff, order)
            ctx.save_for_backward(reconstruction, rotations, shifts, projection, projection.new_empty(0))
        else:
            projection = _ops.project_3d_to_2d_forw_ordered(reconstruction, rotations, shifts, output_shape, interpolation,
                                                            oversampling, fourier_radius_cutoff, order)
            ctx.save_for_backward(reconstruction, rotations, shifts)
        ctx.pose_order = order
        ctx.interpolation = interpolation
        ctx.oversampling = oversampling
        ctx.fourier_radius_cutoff = fourier_radius_cutoff
        return projection

    @staticmethod
    def backward(ctx, grad_output):
        if ctx.saving:
            reconstruction, rotations, shifts, projection, derivatives = ctx.saved_tensors
            grad_reconstruction, grad_rotations, grad_shifts = _ops.project_3d_to_2d_back_saved(
                grad_output.contiguous(), projection, derivatives, reconstruction, rotations, shifts, ctx.interpolation,
                ctx.oversampling, ctx.fourier_radius_cutoff, ctx.pose_order, ctx.need_rec)
            if not ctx.need_rec:
                grad_reconstruction = None
        else:
            reconstruction, rotations, shifts = ctx.saved_tensors
            grad_reconstruction, grad_rotations, grad_shifts = _ops.project_3d_to_2d_back_ordered(
                grad_output.contiguous(), reconstruction, rotations, shifts, ctx.interpolation,
                ctx.oversampling, ctx.fourier_radius_cutoff, ctx.pose_order)
        if shifts is None:
            grad_shifts = None
        return grad_reconstruction, grad_rotations, grad_shifts, None, None, None, None, None


def _canon_backproject(projections, weights, rotations, shifts):
    if projections.dim() == 3:
        projections = projections.unsqueeze(0)
    rotations, shifts = _canon_poses(rotations, shifts)
    if weights is not None and weights.dim() == 3:
        weights = weights.unsqueeze(0)
    if rotations.size(0) != projections.size(0) and rotations.size(0) != 1:
        raise ValueError("Batch size of rotations must be 1 or match projections")
    return projections, weights, rotations, shifts


class _BackprojectBase(torch.autograd.Function):
    _forw = None
    _back = None
    _ordered = False

    @classmethod
    def _run_forward(cls, ctx, projections, weights, rotations, shifts, interpolation,
                     oversampling, fourier_radius_cutoff):
        projections, weights, rotations, shifts = _canon_backproject(projections, weights, rotations, shifts)
        data_reconstruction, weight_reconstruction = getattr(_ops, cls._forw)(
            projections, weights, rotations, shifts, interpolation, oversampling, fourier_radius_cutoff)
        ctx.save_for_backward(projections, weights, rotations, shifts)
        ctx.interpolation = interpolation
        ctx.oversampling = oversampling
        ctx.fourier_radius_cutoff = fourier_radius_cutoff
        return data_reconstruction, weight_reconstruction

    @classmethod
    def _run_backward(cls, ctx, grad_data_rec, grad_weight_rec):
        projections, weights, rotations, shifts = ctx.saved_tensors
        if grad_weight_rec is not None and grad_weight_rec.numel() == 0:
            grad_weight_rec = None
        grad_projections, grad_weights, grad_rotations, grad_shifts = getattr(_ops, cls._back)(
            grad_data_rec.contiguous(),
            grad_weight_rec.contiguous() if grad_weight_rec is not None else None,
            projections, weights, rotations, shifts, ctx.interpolation, ctx.oversampling,
            ctx.fourier_radius_cutoff)
        if weights is None:
            grad_weights = None
        if shifts is None:
            grad_shifts = None
        return grad_projections, grad_weights, grad_rotations, grad_shifts, None, None, None


class _Backproject2D(_BackprojectBase):
    _forw, _back = "backproject_2d_forw", "backproject_2d_back"

    @staticmethod
    def forward(ctx, *args):
        return _Backproject2D._run_forward(ctx, *args)

    @staticmethod
    def backward(ctx, grad_data_rec, grad_weight_rec):
        return _Backproject2D._run_backward(ctx, grad_data_rec, grad_weight_rec)


class _Backproject2DTo3D(_BackprojectBase):
    _forw, _back = "backproject_2d_to_3d_forw", "backproject_2d_to_3d_back"

    @staticmethod
    def forward(ctx, *args):
        return _Backproject2DTo3D._run_forward(ctx, *args)

    @staticmethod
    def backward(ctx, grad_data_rec, grad_weight_rec):
        return _Backproject2DTo3D._run_backward(ctx, grad_data_rec, grad_weight_rec)
