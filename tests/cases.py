"""Seeded synthetic inputs and error metrics shared by the tests, the golden-vector
generator and the benchmark.  No dataset is involved: the reference itself benchmarks and
tests on ``torch.randn`` data (paper/results/benchmarks/benchmark_base.py:146-174 there)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field, asdict
from typing import Optional

import torch


@dataclass(frozen=True)
class Case:
    name: str
    dim: int                 # 2 or 3
    interp: str              # 'linear' | 'cubic'
    B: int
    P: int
    N: int                   # projection box
    R: int                   # reconstruction box for the projection ops
    os: float                # oversampling
    cutoff: Optional[float] = None
    B_rot: int = 1
    B_shift: int = 1         # 0 = no shifts
    weights: bool = True
    shift_range: float = 4.0
    seed: int = 0
    special_poses: bool = True   # pose 0 identity, pose 1 a 90-degree turn (exact lattice hits)

    def as_dict(self):
        return asdict(self)


def random_rotations_3d(P: int, gen: torch.Generator, dtype=torch.float32) -> torch.Tensor:
    """Uniform SO(3) from normalised N(0,1) quaternions."""
    q = torch.randn(P, 4, generator=gen, dtype=torch.float64)
    q = q / q.norm(dim=1, keepdim=True)
    w, x, y, z = q.unbind(1)
    m = torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w),
                     2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w),
                     2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)], 1)
    return m.reshape(P, 3, 3).to(dtype)


def random_rotations_2d(P: int, gen: torch.Generator, dtype=torch.float32) -> torch.Tensor:
    a = torch.rand(P, generator=gen, dtype=torch.float64) * (2 * math.pi)
    return torch.stack([a.cos(), -a.sin(), a.sin(), a.cos()], 1).reshape(P, 2, 2).to(dtype)


def make_rotations(dim: int, B_rot: int, P: int, gen: torch.Generator, special: bool = True,
                   dtype=torch.float32) -> torch.Tensor:
    f = random_rotations_3d if dim == 3 else random_rotations_2d
    rot = f(B_rot * P, gen, dtype).reshape(B_rot, P, dim, dim).clone()
    if special and P >= 1:
        rot[0, 0] = torch.eye(dim, dtype=dtype)
    if special and P >= 2:
        turn = torch.zeros(dim, dim, dtype=dtype)
        turn[0, 1], turn[1, 0] = -1.0, 1.0          # (c, r) -> (-r, c): half the samples mirror
        if dim == 3:
            turn[2, 2] = 1.0
        rot[0, 1] = turn
    return rot


def axis_aligned_rotations(gen: torch.Generator, perturbed: int = 8) -> torch.Tensor:
    """The 24 proper rotations that map the axes onto each other (every sample of a slice hits
    the lattice exactly, whole rows and columns land on one plane) followed by `perturbed` of them
    turned by 1e-6 .. 1e-3 rad about all three axes (samples a hair off the lattice)."""
    import itertools
    out = []
    for perm in itertools.permutations(range(3)):
        for signs in itertools.product((1.0, -1.0), repeat=3):
            m = torch.zeros(3, 3, dtype=torch.float64)
            for r, c in enumerate(perm):
                m[r, c] = signs[r]
            if abs(torch.det(m).item() - 1.0) < 1e-9:
                out.append(m)
    for k in range(perturbed):
        ax, ay, az = ((torch.rand(3, generator=gen, dtype=torch.float64) - 0.5) * 2e-6 * 10 ** (k % 4)).tolist()
        rx = torch.tensor([[1, 0, 0], [0, math.cos(ax), -math.sin(ax)], [0, math.sin(ax), math.cos(ax)]], dtype=torch.float64)
        ry = torch.tensor([[math.cos(ay), 0, math.sin(ay)], [0, 1, 0], [-math.sin(ay), 0, math.cos(ay)]], dtype=torch.float64)
        rz = torch.tensor([[math.cos(az), -math.sin(az), 0], [math.sin(az), math.cos(az), 0], [0, 0, 1]], dtype=torch.float64)
        out.append(rz @ ry @ rx @ out[(k * 5) % 24])
    return torch.stack(out).float()


def hermitian_dc_column_(proj: torch.Tensor) -> torch.Tensor:
    """Make the j = 0 column of rfft-format slices [..., N, Nh] consistent with a real image:
    p[N-i, 0] = conj(p[i, 0]); imaginary part 0 at i = 0 and i = N/2."""
    N = proj.shape[-2]
    col = proj[..., :, 0]
    col[..., 0] = col[..., 0].real.to(col.dtype)
    col[..., N // 2] = col[..., N // 2].real.to(col.dtype)
    idx = torch.arange(1, N // 2)
    col[..., N - idx] = col[..., idx].conj()
    return proj


def make_inputs(case: Case, device="cpu", cdtype=torch.complex64):
    """All tensors any of the eight operators of `case` needs (on `device`)."""
    rdtype = torch.float32 if cdtype == torch.complex64 else torch.float64
    gen = torch.Generator().manual_seed(1234 + case.seed)
    Rh, Nh = case.R // 2 + 1, case.N // 2 + 1
    rec_shape = (case.B, case.R, case.R, Rh) if case.dim == 3 else (case.B, case.R, Rh)
    rec = torch.randn(rec_shape, generator=gen, dtype=torch.float64) + 1j * torch.randn(rec_shape, generator=gen, dtype=torch.float64)
    rot = make_rotations(case.dim, case.B_rot, case.P, gen, case.special_poses, rdtype)
    shifts = None
    if case.B_shift:
        shifts = ((torch.rand(case.B_shift, case.P, 2, generator=gen, dtype=torch.float64) * 2 - 1) * case.shift_range).to(rdtype)
    pshape = (case.B, case.P, case.N, Nh)
    proj = torch.randn(pshape, generator=gen, dtype=torch.float64) + 1j * torch.randn(pshape, generator=gen, dtype=torch.float64)
    weights = torch.rand(pshape, generator=gen, dtype=torch.float64).to(rdtype) if case.weights else None
    # gradient volumes for the backward of back-projection (box from the size rule)
    raw = math.ceil(case.N * case.os)
    Rb = raw + raw % 2
    bshape = (case.B, Rb, Rb, Rb // 2 + 1) if case.dim == 3 else (case.B, Rb, Rb // 2 + 1)
    grad_data = torch.randn(bshape, generator=gen, dtype=torch.float64) + 1j * torch.randn(bshape, generator=gen, dtype=torch.float64)
    grad_weight = torch.randn(bshape, generator=gen, dtype=torch.float64).to(rdtype)
    out = dict(rec=rec.to(cdtype), rot=rot, shifts=shifts, proj=proj.to(cdtype), weights=weights,
               grad_data=grad_data.to(cdtype), grad_weight=grad_weight)
    return {k: (v.to(device) if v is not None else None) for k, v in out.items()}


def rel_err(a: torch.Tensor, ref: torch.Tensor) -> float:
    """max|a - ref| / max|ref| over the whole tensor (point-wise relative error is
    meaningless at the zeros outside the cutoff)."""
    if a.shape != ref.shape:
        raise AssertionError(f"shape mismatch {tuple(a.shape)} vs {tuple(ref.shape)}")
    if ref.numel() == 0:
        return 0.0
    a = a.detach().cpu()
    ref = ref.detach().cpu()
    if a.is_complex():
        a, ref = a.to(torch.complex128), ref.to(torch.complex128)
    else:
        a, ref = a.to(torch.float64), ref.to(torch.float64)
    denom = ref.abs().max().item()
    num = (a - ref).abs().max().item()
    return num / denom if denom > 0 else num


def rel_err_on_device(a: torch.Tensor, ref: torch.Tensor) -> float:
    """rel_err for volumes of gigabytes: the same metric evaluated on a's device in the tensors'
    own precision (the difference of two nearby floats is exact to an ulp of the difference),
    which avoids several double-precision host copies of a 3 GB volume."""
    if a.shape != ref.shape:
        raise AssertionError(f"shape mismatch {tuple(a.shape)} vs {tuple(ref.shape)}")
    ref = ref.to(a.device)
    denom = ref.abs().max().item()
    num = (a.detach() - ref).abs().max().item()
    return num / denom if denom > 0 else num


# Tolerances of the parity contract: global-normalised max error against the reference's
# fp32 CPU result.
TOL_FORWARD = 1e-5        # forward projection (gather)
TOL_ATOMIC = 1e-4         # atomically accumulated back-projection and all gradients


SMALL_CASES = [
    Case("3d_lin_os2", 3, "linear", 1, 6, 16, 32, 2.0, None, 1, 1),
    Case("3d_cub_os2", 3, "cubic", 1, 6, 16, 32, 2.0, None, 1, 1, seed=1),
    Case("3d_lin_batch_bcast", 3, "linear", 2, 5, 12, 12, 1.0, None, 1, 2, seed=2),
    Case("3d_cub_batch_full", 3, "cubic", 2, 4, 12, 18, 1.5, 5.0, 2, 2, seed=3),
    Case("3d_lin_noshift", 3, "linear", 1, 4, 16, 16, 1.0, None, 1, 0, seed=4),
    Case("3d_cub_overreach", 3, "cubic", 1, 4, 16, 16, 1.5, None, 1, 0, seed=5),   # samples leave the volume: clamp / drop
    Case("3d_lin_overreach", 3, "linear", 2, 3, 8, 10, 1.5, 3.0, 1, 2, seed=6),
    Case("3d_lin_tiny", 3, "linear", 1, 3, 6, 6, 1.0, None, 1, 1, seed=7),
    Case("3d_cub_tiny_noweights", 3, "cubic", 1, 3, 6, 10, 1.5, None, 1, 1, weights=False, seed=8),
    Case("2d_lin_os2", 2, "linear", 1, 8, 16, 32, 2.0, None, 1, 1, seed=9),
    Case("2d_cub_os2", 2, "cubic", 1, 8, 16, 32, 2.0, None, 1, 1, seed=10),
    Case("2d_lin_batch", 2, "linear", 3, 4, 12, 12, 1.0, 4.5, 3, 1, seed=11),
    Case("2d_cub_batch", 2, "cubic", 2, 5, 10, 16, 1.5, None, 1, 2, seed=12),
    Case("2d_lin_overreach", 2, "linear", 1, 4, 16, 16, 1.5, None, 1, 0, seed=13),
    Case("2d_cub_noweights", 2, "cubic", 1, 4, 8, 8, 1.0, None, 1, 1, weights=False, seed=14),
]

MEDIUM_CASES = [
    Case("3d_cub_cfg2_like", 3, "cubic", 1, 24, 64, 128, 2.0, 32.0, 1, 1, shift_range=8.0, seed=20, special_poses=False),
    Case("3d_lin_cfg3_like", 3, "linear", 1, 32, 64, 128, 2.0, None, 1, 1, shift_range=8.0, seed=21, special_poses=False),
    Case("2d_lin_cfg1_like", 2, "linear", 1, 64, 64, 128, 2.0, None, 1, 1, seed=22, special_poses=False),
    Case("3d_cub_odd_tiles", 3, "cubic", 2, 5, 34, 70, 2.0, None, 2, 2, seed=23),
    # many poses on a small 2D reconstruction: every voxel receives reductions from many slices
    Case("2d_cub_many_poses", 2, "cubic", 2, 70, 16, 32, 2.0, None, 2, 2, seed=24),
    Case("2d_lin_many_poses_noweights", 2, "linear", 1, 80, 12, 24, 2.0, 4.5, 1, 0, weights=False, seed=25),
    Case("2d_lin_many_poses_overreach", 2, "linear", 1, 66, 16, 16, 1.5, None, 1, 1, seed=26),
]


def random_case(k: int) -> Case:
    """Seeded random small configuration: every combination of the optional arguments, odd
    oversampling factors, cutoffs from tight to beyond the corners, boxes that leave the volume."""
    import random
    rnd = random.Random(1000 + k)
    dim = rnd.choice([2, 3])
    interp = rnd.choice(["linear", "cubic"])
    B = rnd.choice([1, 1, 2, 3])
    P = rnd.choice([1, 2, 5, 9])
    N = rnd.choice([2, 4, 6, 10, 14, 18])
    os_ = rnd.choice([1.0, 1.25, 1.3, 1.5, 2.0, 2.5, 3.0])
    R = math.ceil(N * os_)
    R += R % 2                                   # the box back-projection produces (projection accepts any even box)
    cutoff = rnd.choice([None, None, 1.0, N / 4, N / 2 - 0.5, float(N)])
    B_rot = rnd.choice([1, B])
    B_shift = rnd.choice([0, 1, B])
    return Case(f"random{k}", dim, interp, B, P, N, R, os_, cutoff, B_rot, B_shift, weights=rnd.random() < 0.7,
                shift_range=rnd.choice([0.5, 3.0]), seed=2000 + k, special_poses=rnd.random() < 0.5)
