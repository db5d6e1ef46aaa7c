"""ctypes binding of ``libb200proj.so`` (the C ABI declared in ``include/b200proj.h``).

This is the only place that hands raw device pointers to the CUDA library.  Tensors given
to the functions below must already be validated, contiguous CUDA tensors of
complex64 / float32; the stream is torch's current stream of the tensors' device.

There is no fallback of any kind: if the library is missing and cannot be built, importing
the package fails; if a call returns an error code, ``RuntimeError`` is raised with the
library's message.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import build as _build

LINEAR, CUBIC = 0, 1

_i64, _dbl, _int, _ptr = C.c_int64, C.c_double, C.c_int, C.c_void_p

# name -> argument ctypes, mirroring include/b200proj.h
_COMMON = [_i64, _i64, _ptr, _i64, _ptr, _i64, _i64, _i64, _int, _dbl, _dbl]  # B,R,rot,B_rot,shifts,B_shift,P,N,interp,os,cutoff
SIGNATURES = {
    "b200proj_project_2d_forw": [_ptr] + _COMMON + [_ptr, _ptr],
    "b200proj_project_3d_to_2d_forw": [_ptr] + _COMMON + [_ptr, _ptr, _ptr],
    "b200proj_project_2d_back": [_ptr, _ptr] + _COMMON + [_ptr, _ptr, _ptr, _ptr],
    "b200proj_project_3d_to_2d_back": [_ptr, _ptr] + _COMMON + [_ptr, _ptr, _ptr, _ptr, _ptr],
    "b200proj_backproject_2d_forw": [_ptr, _ptr] + _COMMON + [_ptr, _ptr, _int, _ptr, C.c_size_t, _ptr],
    "b200proj_backproject_2d_to_3d_forw": [_ptr, _ptr] + _COMMON + [_ptr, _ptr, _int, _ptr, C.c_size_t, _ptr],
    "b200proj_backproject_2d_to_3d_forw_noalloc": [_ptr, _ptr] + _COMMON + [_ptr, _ptr, _int, _ptr],
    "b200proj_backproject_2d_back": [_ptr, _ptr, _ptr] + _COMMON + [_ptr, _ptr, _ptr, _ptr, _ptr],
    "b200proj_backproject_2d_to_3d_back": [_ptr, _ptr, _ptr] + _COMMON + [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr],
    "b200proj_pose_order_3d": [_ptr, _i64, _i64, _i64, _ptr, _ptr],
    "b200proj_pad_fftshift": [_ptr, _i64, _int, _i64, _i64, _ptr, _ptr],
    "b200proj_ifftshift_crop": [_ptr, _i64, _int, _i64, _i64, _ptr, _ptr],
}
# complex128 / float64 variants: same argument lists (pointers are void* here)
SIGNATURES.update({name + "_f64": sig for name, sig in list(SIGNATURES.items()) if not name.endswith("_noalloc")})
# fp32-only entry points of the persistent interleaved accumulator
SIGNATURES["b200proj_backproject_2d_to_3d_accumulate"] = [_ptr, _ptr] + _COMMON + [_ptr, _ptr]
SIGNATURES["b200proj_accumulator_fold"] = [_ptr, _i64, _i64, _ptr, _ptr, _int, _ptr]
SIGNATURES["b200proj_accumulator_fold_range"] = [_ptr, _i64, _i64, _ptr, _ptr, _int, _ptr]
SIGNATURES["b200proj_accumulator_fold_normalized"] = [_ptr, _i64, _i64, _dbl, _ptr, _ptr]
SIGNATURES["b200proj_project_2d_forw_saving"] = [_ptr] + _COMMON + [_ptr, _ptr, _ptr]
SIGNATURES["b200proj_project_2d_back_saved"] = [_ptr, _ptr, _ptr] + _COMMON + [_ptr, _ptr, _ptr, _ptr]
SIGNATURES["b200proj_project_3d_to_2d_forw_saving"] = [_ptr] + _COMMON + [_ptr, _ptr, _ptr, _ptr]
SIGNATURES["b200proj_project_3d_to_2d_back_saved"] = [_ptr, _ptr, _ptr] + _COMMON + [_ptr, _ptr, _ptr, _ptr, _ptr]
SIGNATURES["b200proj_project_3d_to_2d_forw_packed"] = [_ptr] + _COMMON + [_ptr, _ptr, _i64, _ptr, _ptr]
SIGNATURES["b200proj_reduction_rate_probe"] = [_int, _ptr, C.c_size_t, _int, _int, _ptr]
SIGNATURES["b200proj_reduction_rate_probe_streaming"] = [_ptr, C.c_size_t, C.c_size_t, _ptr, C.c_size_t, _int, _int, _int, _ptr]
SIGNATURES["b200proj_backproject_2d_to_3d_accumulate_slabs"] = [_ptr, _ptr] + _COMMON + [_ptr, _int, _int, _ptr]
EXPORTS = list(SIGNATURES) + ["b200proj_version", "b200proj_last_error", "b200proj_rec_boxsize",
                                "b200proj_backproject_workspace_bytes", "b200proj_accumulator_bytes",
                                "b200proj_source_stamp", "b200proj_accumulator_slab_plan",
                                "b200proj_accumulator_slab_voxels", "b200proj_debug_index", "b200proj_cutoff_pack_index"]

_lib: Optional[C.CDLL] = None


def library_path():
    return _build.LIB_PATH


def load() -> C.CDLL:
    """Load the CUDA library, building it first when it is absent or was built from other sources
    than the ones beside it; raises ImportError when it cannot be built or when the file that
    loads reports other sources than it should.  Never substitutes another implementation."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB_PATH
    if _build.needs_build():
        try:
            _build.build()
        except Exception as e:  # noqa: BLE001
            raise ImportError(
                f"torch_projectors_b200: {path} is missing or stale and building it failed ({e}); "
                "run `python -m torch_projectors_b200.build` on a machine with nvcc") from e
    try:
        lib = C.CDLL(str(path))
    except OSError as e:
        raise ImportError(f"torch_projectors_b200: cannot load {path}: {e}") from e
    lib.b200proj_source_stamp.restype = C.c_char_p
    lib.b200proj_source_stamp.argtypes = []
    built_from = (lib.b200proj_source_stamp() or b"").decode()
    if built_from != _build.source_stamp():
        raise ImportError(f"torch_projectors_b200: {path} was built from other sources (stamp {built_from!r}, "
                          f"expected {_build.source_stamp()!r}); run `python -m torch_projectors_b200.build --force`")
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = _int
    lib.b200proj_version.restype = _int
    lib.b200proj_version.argtypes = []
    lib.b200proj_last_error.restype = C.c_char_p
    lib.b200proj_last_error.argtypes = []
    lib.b200proj_rec_boxsize.restype = _i64
    lib.b200proj_rec_boxsize.argtypes = [_i64, _dbl]
    lib.b200proj_backproject_workspace_bytes.restype = C.c_size_t
    lib.b200proj_backproject_workspace_bytes.argtypes = [_int, _i64, _i64, _i64, _i64, _int, _int]
    lib.b200proj_accumulator_bytes.restype = C.c_size_t
    lib.b200proj_accumulator_bytes.argtypes = [_i64, _i64]
    lib.b200proj_cutoff_pack_index.restype = _i64
    lib.b200proj_cutoff_pack_index.argtypes = [_i64, _dbl, _ptr]
    lib.b200proj_accumulator_slab_plan.restype = _int
    lib.b200proj_accumulator_slab_plan.argtypes = [_i64, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    lib.b200proj_accumulator_slab_voxels.restype = _int
    lib.b200proj_accumulator_slab_voxels.argtypes = [_i64, _int, _int, C.POINTER(_i64), C.POINTER(_i64)]
    _lib = lib
    return lib


def version() -> int:
    return int(load().b200proj_version())


def rec_boxsize(N: int, oversampling: float) -> int:
    return int(load().b200proj_rec_boxsize(int(N), float(oversampling)))


def backproject_workspace_bytes(dim: int, B: int, R: int, P: int, N: int, interp: int, has_weights: bool) -> int:
    return int(load().b200proj_backproject_workspace_bytes(dim, B, R, P, N, interp, int(has_weights)))


def _p(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _call(name: str, anchor: torch.Tensor, *args) -> None:
    """Invoke an entry point (its _f64 variant for double precision tensors) on the current
    stream of anchor's device.  This is the per-call hot path of small problems, so it avoids
    Python-level context managers and stream objects where it can."""
    if anchor.dtype in (torch.complex128, torch.float64):
        name += "_f64"
    if not anchor.is_cuda:
        raise RuntimeError(f"{name}: tensors must be on a CUDA device (there is no CPU path)")
    lib = _lib if _lib is not None else load()
    fn = getattr(lib, name)
    index = anchor.device.index
    if torch.cuda.current_device() == index:
        stream = _raw_stream(index) if _raw_stream is not None else torch.cuda.current_stream(index).cuda_stream
        rc = fn(*args, stream)
    else:
        with torch.cuda.device(index):
            rc = fn(*args, torch.cuda.current_stream(index).cuda_stream)
    if rc != 0:
        msg = lib.b200proj_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{name}: {msg} (code {rc})")


def _geom(B, R, rot, shifts, P, N, interp, oversampling, cutoff):
    return (int(B), int(R), _p(rot), int(rot.shape[0]), _p(shifts),
            int(shifts.shape[0]) if shifts is not None else 0, int(P), int(N), int(interp),
            float(oversampling), float(cutoff))


def pose_order_3d(rot, B, P, order):
    """Fill order (int32 [B*P], CUDA) with a processing order of the slices that keeps slices
    with nearby planes together (b200proj_pose_order_3d)."""
    _call("b200proj_pose_order_3d", rot, _p(rot), int(B), int(rot.shape[0]), int(P), _p(order))


def _order_arg(dim, order):
    """Trailing pose_order argument: the 3D entry points take it, the 2D ones do not."""
    return (_p(order),) if dim == 3 else ()


def project_forw(dim, rec, rot, shifts, P, N, interp, oversampling, cutoff, out, order=None):
    name = "b200proj_project_2d_forw" if dim == 2 else "b200proj_project_3d_to_2d_forw"
    B, R = rec.shape[0], rec.shape[-2]
    _call(name, rec, _p(rec), *_geom(B, R, rot, shifts, P, N, interp, oversampling, cutoff), _p(out),
          *_order_arg(dim, order))


def project_back(dim, grad_proj, rec, rot, shifts, P, N, interp, oversampling, cutoff,
                 grad_rec, grad_rot, grad_shifts, order=None):
    name = "b200proj_project_2d_back" if dim == 2 else "b200proj_project_3d_to_2d_back"
    B, R = rec.shape[0], rec.shape[-2]
    _call(name, rec, _p(grad_proj), _p(rec), *_geom(B, R, rot, shifts, P, N, interp, oversampling, cutoff),
          _p(grad_rec), _p(grad_rot), _p(grad_shifts), *_order_arg(dim, order))


def project_3d_to_2d_forw_saving(rec, rot, shifts, P, N, interp, oversampling, cutoff, out, derivatives, order=None):
    """Forward projection that also writes the pixels' derivatives [3, B, P, N, Nh] (complex64)."""
    B, R = rec.shape[0], rec.shape[-2]
    _call("b200proj_project_3d_to_2d_forw_saving", rec, _p(rec), *_geom(B, R, rot, shifts, P, N, interp, oversampling, cutoff),
          _p(out), _p(derivatives), _p(order))


def project_3d_to_2d_back_saved(grad_proj, out, derivatives, B, R, rot, shifts, P, N, interp, oversampling, cutoff,
                                grad_rec, grad_rot, grad_shifts, order=None):
    """Backward pass from the saved projections and derivatives (any of the three outputs may be None)."""
    _call("b200proj_project_3d_to_2d_back_saved", grad_proj, _p(grad_proj), _p(out), _p(derivatives),
          *_geom(B, R, rot, shifts, P, N, interp, oversampling, cutoff), _p(grad_rec), _p(grad_rot), _p(grad_shifts), _p(order))


def backproject_forw(dim, proj, weights, rot, shifts, interp, oversampling, cutoff,
                     data_rec, weight_rec, accumulate, workspace=None):
    """workspace: optional uint8 CUDA tensor (see backproject_workspace_bytes)."""
    name = "b200proj_backproject_2d_forw" if dim == 2 else "b200proj_backproject_2d_to_3d_forw"
    B, P, N = proj.shape[0], proj.shape[1], proj.shape[2]
    R = data_rec.shape[-2]
    _call(name, proj, _p(proj), _p(weights), *_geom(B, R, rot, shifts, P, N, interp, oversampling, cutoff),
          _p(data_rec), _p(weight_rec), int(bool(accumulate)), _p(workspace),
          0 if workspace is None else workspace.numel() * workspace.element_size())


NOALLOC_MAX_VOXELS = 64 * 64 * 33


def backproject_2d_to_3d_forw_noalloc(proj, weights, rot, shifts, interp, oversampling, cutoff,
                                      data_rec, weight_rec, accumulate):
    """Weighted 2D->3D back-projection through the library's built-in scratch: for callers that
    may not allocate device memory (no workspace tensor is involved).  Volumes are limited to
    NOALLOC_MAX_VOXELS voxels; calls that overlap on the GPU race on the shared scratch."""
    B, P, N = proj.shape[0], proj.shape[1], proj.shape[2]
    R = data_rec.shape[-2]
    _call("b200proj_backproject_2d_to_3d_forw_noalloc", proj, _p(proj), _p(weights),
          *_geom(B, R, rot, shifts, P, N, interp, oversampling, cutoff),
          _p(data_rec), _p(weight_rec), int(bool(accumulate)))


def pad_fftshift(real, batch, dims, n, m, out):
    _call("b200proj_pad_fftshift", real, _p(real), int(batch), int(dims), int(n), int(m), _p(out))


def ifftshift_crop(full, batch, dims, m, n, out):
    _call("b200proj_ifftshift_crop", full, _p(full), int(batch), int(dims), int(m), int(n), _p(out))


def accumulator_bytes(B: int, R: int) -> int:
    return int(load().b200proj_accumulator_bytes(int(B), int(R)))


def backproject_accumulate(proj, weights, rot, shifts, interp, oversampling, cutoff, R, accumulator):
    """Add the slices into the persistent interleaved accumulator (a zero-initialised CUDA tensor
    of accumulator_bytes(B, R) bytes); see b200proj_backproject_2d_to_3d_accumulate."""
    B, P, N = proj.shape[0], proj.shape[1], proj.shape[2]
    _call("b200proj_backproject_2d_to_3d_accumulate", proj, _p(proj), _p(weights),
          *_geom(B, R, rot, shifts, P, N, interp, oversampling, cutoff), _p(accumulator))


def backproject_accumulate_slabs(proj, weights, rot, shifts, interp, oversampling, cutoff, R, accumulator,
                                 slab_first, slab_count):
    """The same for slabs [slab_first, slab_first + slab_count) of the accumulator's slab plan only."""
    B, P, N = proj.shape[0], proj.shape[1], proj.shape[2]
    _call("b200proj_backproject_2d_to_3d_accumulate_slabs", proj, _p(proj), _p(weights),
          *_geom(B, R, rot, shifts, P, N, interp, oversampling, cutoff), _p(accumulator), int(slab_first), int(slab_count))


def _host_call(fn, *args) -> None:
    rc = fn(*args)
    if rc != 0:
        raise RuntimeError(f"{fn.__name__}: {load().b200proj_last_error().decode('utf-8', 'replace')} (code {rc})")


def accumulator_slab_plan(R: int):
    """(slabs, planes per slab) of the slab-ordered passes that fill an accumulator of box R;
    slabs == 1 when it is small enough for one pass."""
    slabs, planes = C.c_int32(0), C.c_int32(0)
    _host_call(load().b200proj_accumulator_slab_plan, int(R), C.byref(slabs), C.byref(planes))
    return slabs.value, planes.value


def accumulator_slab_voxels(R: int, slab_first: int, slab_count: int):
    """[(first, stop), ...] voxel ranges (relative to a batch item's first voxel) that slabs
    [slab_first, slab_first + slab_count) own: at most two, in ascending order."""
    first, count = (_i64 * 2)(), (_i64 * 2)()
    _host_call(load().b200proj_accumulator_slab_voxels, int(R), int(slab_first), int(slab_count), first, count)
    return sorted((int(f), int(f + n)) for f, n in zip(first, count) if n > 0)


def accumulator_fold(accumulator, B, R, data_rec, weight_rec, accumulate, voxel_range=None):
    if voxel_range is None:
        _call("b200proj_accumulator_fold", data_rec, _p(accumulator), int(B), int(R), _p(data_rec), _p(weight_rec),
              int(bool(accumulate)))
    else:
        _call("b200proj_accumulator_fold_range", data_rec, _p(accumulator), int(voxel_range[0]),
              int(voxel_range[1] - voxel_range[0]), _p(data_rec), _p(weight_rec), int(bool(accumulate)))


def backproject_back(dim, grad_data_rec, grad_weight_rec, proj, rot, shifts, interp, oversampling,
                     cutoff, grad_proj, grad_weights, grad_rot, grad_shifts, order=None):
    name = "b200proj_backproject_2d_back" if dim == 2 else "b200proj_backproject_2d_to_3d_back"
    B, P, N = proj.shape[0], proj.shape[1], proj.shape[2]
    R = grad_data_rec.shape[-2]
    _call(name, proj, _p(grad_data_rec), _p(grad_weight_rec), _p(proj),
          *_geom(B, R, rot, shifts, P, N, interp, oversampling, cutoff),
          _p(grad_proj), _p(grad_weights), _p(grad_rot), _p(grad_shifts), *_order_arg(dim, order))


def accumulator_fold_normalized(accumulator, eps, normalized, voxel_range=None):
    """normalized[k] = accumulator data[k] / max(accumulator weight[k], eps), for the whole
    volume or for the flattened voxel range (first, stop)."""
    first, stop = voxel_range if voxel_range is not None else (0, normalized.numel())
    _call("b200proj_accumulator_fold_normalized", normalized, _p(accumulator), int(first), int(stop - first), float(eps), _p(normalized))


_pack_tables = {}


def cutoff_pack_index(N: int, cutoff: float, device):
    """(index, count): int32 [N * Nh] device table with the position of every pixel among the
    `count` pixels inside the cutoff (-1 outside), made by the library's own cutoff test; cached."""
    key = (int(N), float(cutoff), str(device))
    hit = _pack_tables.get(key)
    if hit is None:
        host = torch.empty(N * (N // 2 + 1), dtype=torch.int32)
        count = int(load().b200proj_cutoff_pack_index(int(N), float(cutoff), host.data_ptr()))
        if count < 0:
            raise RuntimeError("b200proj_cutoff_pack_index: " + load().b200proj_last_error().decode("utf-8", "replace"))
        hit = _pack_tables[key] = (host.to(device), count)
    return hit


def project_3d_to_2d_forw_packed(rec, rot, shifts, P, N, interp, oversampling, cutoff, out_packed, pack_index, pack_count, order=None):
    B, R = rec.shape[0], rec.shape[-2]
    _call("b200proj_project_3d_to_2d_forw_packed", rec, _p(rec), *_geom(B, R, rot, shifts, P, N, interp, oversampling, cutoff),
          _p(out_packed), _p(pack_index), int(pack_count), _p(order))


def reduction_rate_probe(pattern: int, buffer, blocks: int, iterations: int):
    _call("b200proj_reduction_rate_probe", buffer, int(pattern), _p(buffer), buffer.numel() * buffer.element_size(), int(blocks), int(iterations))


def reduction_rate_probe_streaming(target, window_bytes: int, source, blocks: int, iterations: int, evict_last: bool = False):
    """Pattern 1 of the probe inside a window that moves through `target`, with 8 bytes per four
    reductions streamed from `source` (both float32 CUDA tensors); evict_last: with the L2 hint
    of the slab-ordered kernel."""
    _call("b200proj_reduction_rate_probe_streaming", target, _p(target), target.numel() * target.element_size(), int(window_bytes),
          _p(source), source.numel() * source.element_size(), int(blocks), int(iterations), int(bool(evict_last)))
