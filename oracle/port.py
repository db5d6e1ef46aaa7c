"""ctypes wrapper around ``fourier_slice_oracle.c`` (TEST INFRASTRUCTURE, CPU only).

The functions take and return CPU torch tensors in the canonical ranks of the reference's
raw operators (csrc/torch_projectors.cpp:23-36 in the reference):

    rec [B,(R,)R,Rh] complex   proj [B,P,N,Nh] complex   rot [B_rot,P,d,d]   shifts [B_s,P,2]

and follow the same return conventions (results that were not requested are empty ``(0,)``
tensors).  complex64/float32 inputs use the ``_f32`` build, complex128/float64 the
``_f64`` build.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch

from . import build_oracle

_lib = None


def _load():
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(build_oracle.build()))
        for suf in ("f32", "f64"):
            for name in ("oracle_project_forw", "oracle_project_back",
                         "oracle_backproject_forw", "oracle_backproject_back"):
                getattr(_lib, f"{name}_{suf}").restype = None
            getattr(_lib, f"oracle_rec_boxsize_{suf}").restype = C.c_int64
            getattr(_lib, f"oracle_rec_boxsize_{suf}").argtypes = [C.c_int64, C.c_double]
    return _lib


def _suffix(t: torch.Tensor) -> str:
    if t.dtype in (torch.complex64, torch.float32):
        return "f32"
    if t.dtype in (torch.complex128, torch.float64):
        return "f64"
    raise TypeError(f"unsupported dtype {t.dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _real_dtype(t: torch.Tensor):
    return torch.float32 if _suffix(t) == "f32" else torch.float64


def _prep(t: Optional[torch.Tensor], dtype=None):
    if t is None:
        return None
    t = t.detach().cpu()
    if dtype is not None:
        t = t.to(dtype)
    return t.contiguous()


def _interp(s: str) -> int:
    if s == "linear":
        return 0
    if s == "cubic":
        return 1
    raise ValueError("Supported interpolation methods: 'linear', 'cubic'")


def rec_boxsize(N: int, oversampling: float) -> int:
    return int(_load().oracle_rec_boxsize_f32(N, float(oversampling)))


def _project_forw(dim, rec, rot, shifts, output_shape, interpolation, oversampling, cutoff):
    lib = _load()
    suf = _suffix(rec)
    rd = _real_dtype(rec)
    rec_c, rot_c, sh_c = _prep(rec), _prep(rot, rd), _prep(shifts, rd)
    B, R = rec_c.shape[0], rec_c.shape[-2]
    B_rot, P = rot_c.shape[0], rot_c.shape[1]
    N = int(output_shape[0])
    cut = float(cutoff) if cutoff is not None else N / 2.0
    out = torch.empty((B, P, N, N // 2 + 1), dtype=rec_c.dtype)
    getattr(lib, f"oracle_project_forw_{suf}")(
        C.c_int(dim), C.c_int(_interp(interpolation)), _ptr(rec_c), C.c_int64(B), C.c_int64(R),
        _ptr(rot_c), C.c_int64(B_rot), _ptr(sh_c), C.c_int64(0 if sh_c is None else sh_c.shape[0]),
        C.c_int64(P), C.c_int64(N), C.c_double(oversampling), C.c_double(cut), _ptr(out))
    return out


def _project_back(dim, grad_proj, rec, rot, shifts, interpolation, oversampling, cutoff,
                  need_rot_grad, need_shift_grad):
    lib = _load()
    suf = _suffix(rec)
    rd = _real_dtype(rec)
    if need_rot_grad is None:
        need_rot_grad = rot.requires_grad
    if need_shift_grad is None:
        need_shift_grad = shifts is not None and shifts.requires_grad
    gp_c, rec_c, rot_c, sh_c = _prep(grad_proj), _prep(rec), _prep(rot, rd), _prep(shifts, rd)
    B, P, N = gp_c.shape[0], gp_c.shape[1], gp_c.shape[2]
    R = rec_c.shape[-2]
    cut = float(cutoff) if cutoff is not None else N / 2.0
    grad_rec = torch.empty_like(rec_c)
    grad_rot = torch.empty_like(rot_c) if need_rot_grad else None
    grad_sh = torch.empty_like(sh_c) if (need_shift_grad and sh_c is not None) else None
    getattr(lib, f"oracle_project_back_{suf}")(
        C.c_int(dim), C.c_int(_interp(interpolation)), _ptr(gp_c), _ptr(rec_c), C.c_int64(B),
        C.c_int64(R), _ptr(rot_c), C.c_int64(rot_c.shape[0]), _ptr(sh_c),
        C.c_int64(0 if sh_c is None else sh_c.shape[0]), C.c_int64(P), C.c_int64(N),
        C.c_double(oversampling), C.c_double(cut), _ptr(grad_rec), _ptr(grad_rot), _ptr(grad_sh))
    empty = torch.empty((0,), dtype=rd)
    return grad_rec, (grad_rot if grad_rot is not None else empty), (grad_sh if grad_sh is not None else empty)


def _backproject_forw(dim, proj, weights, rot, shifts, interpolation, oversampling, cutoff,
                      out=None):
    lib = _load()
    suf = _suffix(proj)
    rd = _real_dtype(proj)
    pr_c, w_c, rot_c, sh_c = _prep(proj), _prep(weights, rd), _prep(rot, rd), _prep(shifts, rd)
    B, P, N = pr_c.shape[0], pr_c.shape[1], pr_c.shape[2]
    raw = math.ceil(N * oversampling)
    R = raw + raw % 2
    Rh = R // 2 + 1
    cut = float(cutoff) if cutoff is not None else N / 2.0
    shape = (B, R, R, Rh) if dim == 3 else (B, R, Rh)
    accumulate = out is not None
    if accumulate:
        data, wrec = out
    else:
        data = torch.empty(shape, dtype=pr_c.dtype)
        wrec = torch.empty(shape, dtype=rd) if w_c is not None else None
    getattr(lib, f"oracle_backproject_forw_{suf}")(
        C.c_int(dim), C.c_int(_interp(interpolation)), _ptr(pr_c), _ptr(w_c), C.c_int64(B),
        C.c_int64(R), _ptr(rot_c), C.c_int64(rot_c.shape[0]), _ptr(sh_c),
        C.c_int64(0 if sh_c is None else sh_c.shape[0]), C.c_int64(P), C.c_int64(N),
        C.c_double(oversampling), C.c_double(cut), _ptr(data), _ptr(wrec), C.c_int(int(accumulate)))
    return data, (wrec if wrec is not None else torch.empty((0,), dtype=rd))


def _backproject_back(dim, grad_data_rec, grad_weight_rec, proj, weights, rot, shifts,
                      interpolation, oversampling, cutoff, need_rot_grad, need_shift_grad):
    lib = _load()
    suf = _suffix(proj)
    rd = _real_dtype(proj)
    if need_rot_grad is None:
        need_rot_grad = rot.requires_grad
    if need_shift_grad is None:
        need_shift_grad = shifts is not None and shifts.requires_grad
    gd_c, gw_c = _prep(grad_data_rec), _prep(grad_weight_rec, rd)
    pr_c, rot_c, sh_c = _prep(proj), _prep(rot, rd), _prep(shifts, rd)
    B, P, N = pr_c.shape[0], pr_c.shape[1], pr_c.shape[2]
    R = gd_c.shape[-2]
    cut = float(cutoff) if cutoff is not None else N / 2.0
    grad_proj = torch.empty_like(pr_c)
    # the reference allocates zeros_like(weights) whenever weights exist and fills it
    # only when grad_weight_rec exists too
    grad_w = torch.zeros(pr_c.shape, dtype=rd) if weights is not None else None
    grad_rot = torch.empty_like(rot_c) if need_rot_grad else None
    grad_sh = torch.empty_like(sh_c) if (need_shift_grad and sh_c is not None) else None
    getattr(lib, f"oracle_backproject_back_{suf}")(
        C.c_int(dim), C.c_int(_interp(interpolation)), _ptr(gd_c), _ptr(gw_c), _ptr(pr_c),
        C.c_int64(B), C.c_int64(R), _ptr(rot_c), C.c_int64(rot_c.shape[0]), _ptr(sh_c),
        C.c_int64(0 if sh_c is None else sh_c.shape[0]), C.c_int64(P), C.c_int64(N),
        C.c_double(oversampling), C.c_double(cut), _ptr(grad_proj),
        _ptr(grad_w if gw_c is not None else None), _ptr(grad_rot), _ptr(grad_sh))
    empty = torch.empty((0,), dtype=rd)
    return (grad_proj, (grad_w if grad_w is not None else empty),
            (grad_rot if grad_rot is not None else empty), (grad_sh if grad_sh is not None else empty))


# ---- the eight raw operators, named as in the reference --------------------------------
def project_2d_forw(rec, rot, shifts, output_shape, interpolation, oversampling, cutoff=None):
    return _project_forw(2, rec, rot, shifts, output_shape, interpolation, oversampling, cutoff)


def project_3d_to_2d_forw(rec, rot, shifts, output_shape, interpolation, oversampling, cutoff=None):
    return _project_forw(3, rec, rot, shifts, output_shape, interpolation, oversampling, cutoff)


def project_2d_back(grad_proj, rec, rot, shifts, interpolation, oversampling, cutoff=None,
                    need_rot_grad=None, need_shift_grad=None):
    return _project_back(2, grad_proj, rec, rot, shifts, interpolation, oversampling, cutoff,
                         need_rot_grad, need_shift_grad)


def project_3d_to_2d_back(grad_proj, rec, rot, shifts, interpolation, oversampling, cutoff=None,
                          need_rot_grad=None, need_shift_grad=None):
    return _project_back(3, grad_proj, rec, rot, shifts, interpolation, oversampling, cutoff,
                         need_rot_grad, need_shift_grad)


def backproject_2d_forw(proj, weights, rot, shifts, interpolation, oversampling, cutoff=None, out=None):
    return _backproject_forw(2, proj, weights, rot, shifts, interpolation, oversampling, cutoff, out)


def backproject_2d_to_3d_forw(proj, weights, rot, shifts, interpolation, oversampling, cutoff=None, out=None):
    return _backproject_forw(3, proj, weights, rot, shifts, interpolation, oversampling, cutoff, out)


def backproject_2d_back(grad_data_rec, grad_weight_rec, proj, weights, rot, shifts, interpolation,
                        oversampling, cutoff=None, need_rot_grad=None, need_shift_grad=None):
    return _backproject_back(2, grad_data_rec, grad_weight_rec, proj, weights, rot, shifts,
                             interpolation, oversampling, cutoff, need_rot_grad, need_shift_grad)


def backproject_2d_to_3d_back(grad_data_rec, grad_weight_rec, proj, weights, rot, shifts,
                              interpolation, oversampling, cutoff=None, need_rot_grad=None,
                              need_shift_grad=None):
    return _backproject_back(3, grad_data_rec, grad_weight_rec, proj, weights, rot, shifts,
                             interpolation, oversampling, cutoff, need_rot_grad, need_shift_grad)
