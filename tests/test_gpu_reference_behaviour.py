"""Behaviour of the public API on the themes of the reference's own suite
(tests/{2d,3d}/{forw,back}/test_basic_*.py, test_batching_*.py, test_oversampling_*.py,
test_gradients_*.py there), with expectations derived by hand: where a peak must land, what a
shift does to every pixel, which calls must agree with which.  Inputs are seeded."""
import math

import pytest
import torch

from cases import TOL_ATOMIC, random_rotations_2d, random_rotations_3d, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def tp(cuda_device):
    import torch_projectors_b200
    return torch_projectors_b200


def _crandn(*shape, gen):
    return torch.complex(torch.randn(*shape, generator=gen), torch.randn(*shape, generator=gen)).to(DEV)


def _freqs(N):
    kr = torch.arange(N, device=DEV)
    kr = torch.where(kr <= N // 2, kr, kr - N).float().view(N, 1)
    kc = torch.arange(N // 2 + 1, device=DEV).float().view(1, -1)
    return kr, kc


def _inside(N, cutoff=None):
    kr, kc = _freqs(N)
    c = N / 2.0 if cutoff is None else cutoff
    return (kr * kr + kc * kc) <= c * c


def _eye(dim, P=1):
    return torch.eye(dim, device=DEV).view(1, 1, dim, dim).repeat(1, P, 1, 1)


def _rot3(ax, ay, az):
    cx, sx, cy, sy, cz, sz = math.cos(ax), math.sin(ax), math.cos(ay), math.sin(ay), math.cos(az), math.sin(az)
    rx = torch.tensor([[1, 0, 0], [0, cx, -sx], [0, sx, cx]])
    ry = torch.tensor([[cy, 0, sy], [0, 1, 0], [-sy, 0, cy]])
    rz = torch.tensor([[cz, -sz, 0], [sz, cz, 0], [0, 0, 1]])
    return (rz @ ry @ rx).float()


# ---- forward projection: known answers -----------------------------------------------------
@pytest.mark.parametrize("interp", ["linear", "cubic"])
def test_2d_peak_follows_quarter_turns(tp, interp):
    """(themes: tests/2d/forw/test_basic_projection.py:56)  Output pixel k reads the image at R k,
    so a peak stored at (row 0, column 5) shows up where R k = (5, 0) in (column, row) order."""
    N = 32
    rec = torch.zeros(1, N, N // 2 + 1, dtype=torch.complex64, device=DEV)
    rec[0, 0, 5] = 1 + 1j
    rot = torch.stack([torch.eye(2), torch.tensor([[0., 1.], [-1., 0.]]), torch.tensor([[0., -1.], [1., 0.]])]).view(1, 3, 2, 2).to(DEV)
    out = tp.project_2d_forw(rec, rot, output_shape=(N, N), interpolation=interp)
    for p, (i, j) in enumerate([(0, 5), (5, 0), (N - 5, 0)]):
        mag = out[0, p].abs()
        assert mag[i, j] == mag.max() and mag[i, j] > 0.9, (p, mag[i, j].item())
        # the turned peak keeps its value, or its conjugate when it is read through the Friedel mirror
        assert torch.allclose(out[0, p, i, j].real, torch.tensor(1.0, device=DEV), atol=1e-6)


@pytest.mark.parametrize("dim", [2, 3])
@pytest.mark.parametrize("interp", ["linear", "cubic"])
def test_identity_pose_returns_the_central_section_inside_the_cutoff(tp, dim, interp):
    """(themes: tests/3d/forw/test_basic_projection_3d_to_2d.py:48 and :227)"""
    N = 16
    gen = torch.Generator().manual_seed(42)
    rec = _crandn(1, *([N] * (dim - 1)), N // 2 + 1, gen=gen)
    fn = tp.project_2d_forw if dim == 2 else tp.project_3d_to_2d_forw
    out = fn(rec, _eye(dim), output_shape=(N, N), interpolation=interp)
    assert out.shape == (1, 1, N, N // 2 + 1)
    section = rec[0] if dim == 2 else rec[0, 0]
    want = torch.where(_inside(N), section, torch.zeros_like(section))
    assert torch.allclose(out[0, 0], want, atol=1e-5)
    # a tighter cutoff removes exactly the pixels beyond it
    tight = fn(rec, _eye(dim), output_shape=(N, N), interpolation=interp, fourier_radius_cutoff=5.0)
    assert torch.allclose(tight[0, 0], torch.where(_inside(N, 5.0), section, torch.zeros_like(section)), atol=1e-5)


@pytest.mark.parametrize("interp", ["linear", "cubic"])
def test_3d_different_orientations_give_different_slices(tp, interp):
    """(themes: tests/3d/forw/test_basic_projection_3d_to_2d.py:98)"""
    N = 64
    gen = torch.Generator().manual_seed(1)
    rec = _crandn(1, N, N, N // 2 + 1, gen=gen)
    rot = torch.stack([_rot3(0, 0, 0), _rot3(math.pi / 4, math.pi / 6, math.pi / 3), _rot3(math.pi / 2, math.pi / 3, math.pi / 4)]).view(1, 3, 3, 3).to(DEV)
    out = tp.project_3d_to_2d_forw(rec, rot, interpolation=interp)
    assert out.shape == (1, 3, N, N // 2 + 1)
    for a in range(3):
        for b in range(a + 1, 3):
            assert (out[0, a] - out[0, b]).abs().pow(2).sum().sqrt() > 1e-3


@pytest.mark.parametrize("dim", [2, 3])
@pytest.mark.parametrize("interp", ["linear", "cubic"])
def test_a_shift_multiplies_every_pixel_by_its_phase_ramp(tp, dim, interp):
    """(themes: tests/2d/forw/test_basic_projection.py:101, tests/3d/forw/test_basic_projection_3d_to_2d.py:173)
    shifts[..., 0] pairs with rows, shifts[..., 1] with columns; a zero shift changes nothing."""
    N = 32
    gen = torch.Generator().manual_seed(7)
    rec = _crandn(1, *([N] * (dim - 1)), N // 2 + 1, gen=gen)
    rot = (random_rotations_2d(2, gen) if dim == 2 else random_rotations_3d(2, gen)).view(1, 2, dim, dim).to(DEV)
    shifts = torch.tensor([[[0.0, 0.0], [2.5, -1.8]]], device=DEV)
    fn = tp.project_2d_forw if dim == 2 else tp.project_3d_to_2d_forw
    plain = fn(rec, rot, output_shape=(N, N), interpolation=interp)
    moved = fn(rec, rot, shifts=shifts, output_shape=(N, N), interpolation=interp)
    assert torch.equal(moved[0, 0], plain[0, 0])
    kr, kc = _freqs(N)
    ramp = torch.polar(torch.ones(N, N // 2 + 1, device=DEV), -2 * math.pi * (kr * 2.5 + kc * -1.8) / N)
    assert rel_err(moved[0, 1], plain[0, 1] * ramp) < 1e-5
    assert (moved[0, 1] - plain[0, 1]).abs().max() > 1e-3


def test_2d_integer_shift_rolls_a_real_space_dot(tp):
    """(themes: tests/2d/forw/test_basic_projection.py:101)"""
    N = 32
    dot = torch.zeros(N, N, device=DEV)
    dot[N // 2, N // 2] = 1.0
    rec = torch.fft.rfft2(dot).unsqueeze(0)
    out = tp.project_2d_forw(rec, _eye(2), shifts=torch.tensor([[[2.0, 3.0]]], device=DEV), output_shape=(N, N))
    got = torch.fft.irfft2(out[0, 0], s=(N, N))
    want_f = torch.fft.rfft2(torch.roll(dot, shifts=(2, 3), dims=(0, 1)))
    want = torch.fft.irfft2(torch.where(_inside(N), want_f, torch.zeros_like(want_f)), s=(N, N))
    assert torch.allclose(got, want, atol=1e-4)
    assert got.argmax().item() == (N // 2 + 2) * N + (N // 2 + 3)


# ---- validation ------------------------------------------------------------------------------
def test_shape_rules_are_enforced_with_the_reference_messages(tp):
    """(themes: tests/2d/forw/test_basic_projection.py:144, tests/3d/back/test_basic_backprojection_2d_to_3d.py:218)"""
    rot2, rot3 = _eye(2), _eye(3)
    with pytest.raises(ValueError, match="expected boxsize .* to match"):
        tp.project_2d_forw(torch.zeros(1, 30, 17, dtype=torch.complex64, device=DEV), rot2)
    with pytest.raises(ValueError, match="Boxsize .* must be even"):
        tp.project_2d_forw(torch.zeros(1, 29, 15, dtype=torch.complex64, device=DEV), rot2)
    with pytest.raises(ValueError, match="must be square"):
        tp.project_2d_forw(torch.zeros(1, 32, 17, dtype=torch.complex64, device=DEV), rot2, output_shape=(16, 32))
    with pytest.raises(ValueError, match="must be even"):
        tp.project_3d_to_2d_forw(torch.zeros(1, 32, 32, 17, dtype=torch.complex64, device=DEV), rot3, output_shape=(15, 15))
    with pytest.raises(ValueError, match="4D tensor"):
        tp.backproject_2d_to_3d_forw(torch.zeros(1, 32, 17, dtype=torch.complex64, device=DEV), rot3)
    with pytest.raises(ValueError, match="Projection boxsize .* must be even"):
        tp.backproject_2d_forw(torch.zeros(1, 1, 29, 15, dtype=torch.complex64, device=DEV), rot2)
    with pytest.raises(ValueError, match="Weights shape"):
        tp.backproject_2d_forw(torch.zeros(1, 1, 32, 17, dtype=torch.complex64, device=DEV), rot2, weights=torch.zeros(1, 1, 32, 16, device=DEV))
    with pytest.raises(ValueError, match="real-valued"):
        tp.backproject_2d_forw(torch.zeros(1, 1, 32, 17, dtype=torch.complex64, device=DEV), rot2,
                               weights=torch.zeros(1, 1, 32, 17, dtype=torch.complex64, device=DEV))
    # and the valid shapes pass, forward and backward
    rec = torch.zeros(1, 32, 17, dtype=torch.complex64, device=DEV)
    assert tp.project_2d_forw(rec, rot2).shape == (1, 1, 32, 17)
    assert tp.project_2d_back(torch.zeros(1, 1, 32, 17, dtype=torch.complex64, device=DEV), rec, rot2).shape == rec.shape


# ---- batching --------------------------------------------------------------------------------
@pytest.mark.parametrize("dim", [2, 3])
def test_forward_batching_equals_single_calls(tp, dim):
    """(themes: tests/2d/forw/test_batching.py:16-100, tests/3d/forw/test_batching_3d_to_2d.py:16-108)
    B reconstructions x 1 pose, 1 reconstruction x P poses, B x P with shared and with per-item
    poses: every slice equals the single-slice call, bit for bit."""
    N, B, P = 16, 3, 4
    gen = torch.Generator().manual_seed(21)
    recs = _crandn(B, *([N] * (dim - 1)), N // 2 + 1, gen=gen)
    make = random_rotations_2d if dim == 2 else random_rotations_3d
    shared = make(P, gen).view(1, P, dim, dim).to(DEV)
    own = make(B * P, gen).view(B, P, dim, dim).to(DEV)
    shifts = ((torch.rand(B, P, 2, generator=gen) * 2 - 1) * 3).to(DEV)
    fn = tp.project_2d_forw if dim == 2 else tp.project_3d_to_2d_forw
    kw = dict(output_shape=(N, N), interpolation="cubic")
    single = lambda b, r, s=None: fn(recs[b:b + 1], r.view(1, 1, dim, dim), shifts=None if s is None else s.view(1, 1, 2), **kw)[0, 0]  # noqa: E731
    many_recs = fn(recs, shared[:, :1], **kw)
    assert many_recs.shape == (B, 1, N, N // 2 + 1)
    many_poses = fn(recs[:1], shared, **kw)
    assert many_poses.shape == (1, P, N, N // 2 + 1)
    both_shared = fn(recs, shared, shifts=shifts[:1], **kw)
    both_own = fn(recs, own, shifts=shifts, **kw)
    for b in range(B):
        assert torch.equal(many_recs[b, 0], single(b, shared[0, 0]))
        for p in range(P):
            assert torch.equal(both_shared[b, p], single(b, shared[0, p], shifts[0, p]))
            assert torch.equal(both_own[b, p], single(b, own[b, p], shifts[b, p]))
    for p in range(P):
        assert torch.equal(many_poses[0, p], single(0, shared[0, p]))
    with pytest.raises((ValueError, RuntimeError), match="[Bb]atch size of rotations"):
        fn(recs, own[:2], **kw)


@pytest.mark.parametrize("dim", [2, 3])
def test_backprojection_batching_broadcast_and_accumulation(tp, dim):
    """(themes: tests/2d/back/test_batching_back.py:21-285, tests/3d/back/test_batching_back_2d_to_3d.py:21-302)
    Each batch item accumulates its own slices; shared rotations / shifts broadcast over the
    batch; all poses in one call equal the sum of one-pose calls."""
    N, B, P = 16, 2, 5
    gen = torch.Generator().manual_seed(33)
    proj = _crandn(B, P, N, N // 2 + 1, gen=gen)
    wts = torch.rand(B, P, N, N // 2 + 1, generator=gen).to(DEV)
    make = random_rotations_2d if dim == 2 else random_rotations_3d
    shared = make(P, gen).view(1, P, dim, dim).to(DEV)
    own = make(B * P, gen).view(B, P, dim, dim).to(DEV)
    shifts = ((torch.rand(1, P, 2, generator=gen) * 2 - 1) * 3).to(DEV)
    fn = tp.backproject_2d_forw if dim == 2 else tp.backproject_2d_to_3d_forw
    vol = (B,) + (N,) * (dim - 1) + (N // 2 + 1,)
    d_all, w_all = fn(proj, shared, weights=wts, shifts=shifts)
    assert d_all.shape == vol and w_all.shape == vol and w_all.dtype == torch.float32
    d_sum, w_sum = torch.zeros_like(d_all), torch.zeros_like(w_all)
    for b in range(B):
        for p in range(P):
            d1, w1 = fn(proj[b:b + 1, p:p + 1], shared[:, p:p + 1], weights=wts[b:b + 1, p:p + 1], shifts=shifts[:, p:p + 1])
            d_sum[b] += d1[0]
            w_sum[b] += w1[0]
    assert rel_err(d_all, d_sum) < TOL_ATOMIC and rel_err(w_all, w_sum) < TOL_ATOMIC
    # explicit per-item copies of the shared poses give the same volumes
    d_exp, w_exp = fn(proj, shared.expand(B, -1, -1, -1).contiguous(), weights=wts, shifts=shifts.expand(B, -1, -1).contiguous())
    assert rel_err(d_exp, d_all) < TOL_ATOMIC and rel_err(w_exp, w_all) < TOL_ATOMIC
    # per-item poses: item b only sees its own rotations
    d_own, _ = fn(proj, own)
    for b in range(B):
        d_b, _ = fn(proj[b:b + 1], own[b:b + 1])
        assert rel_err(d_own[b], d_b[0]) < TOL_ATOMIC
    # without weights the second output is an empty tensor, as in the reference
    assert fn(proj, shared)[1].numel() == 0


# ---- back-projection: known answers ----------------------------------------------------------
@pytest.mark.parametrize("dim", [2, 3])
@pytest.mark.parametrize("interp", ["linear", "cubic"])
def test_identity_backprojection_places_the_slice_on_the_central_section(tp, dim, interp):
    """(themes: tests/2d/back/test_basic_backprojection.py:21-88, tests/3d/back/test_basic_backprojection_2d_to_3d.py:53-131 and :291)
    At the identity every sample sits on a lattice point: columns > 0 inside the cutoff receive
    exactly the slice value and weight, nothing leaves the central section, and a second
    identical slice doubles the sums."""
    N = 32
    gen = torch.Generator().manual_seed(5)
    proj = _crandn(1, 1, N, N // 2 + 1, gen=gen)
    wts = torch.rand(1, 1, N, N // 2 + 1, generator=gen).to(DEV)
    fn = tp.backproject_2d_forw if dim == 2 else tp.backproject_2d_to_3d_forw
    data, wrec = fn(proj, _eye(dim), weights=wts, interpolation=interp)
    section_d = data[0] if dim == 2 else data[0, 0]
    section_w = wrec[0] if dim == 2 else wrec[0, 0]
    keep = _inside(N).clone()
    keep[:, 0] = False                       # column 0 also receives its Friedel partners
    assert torch.allclose(section_d[keep], proj[0, 0][keep], atol=1e-6)
    assert torch.allclose(section_w[keep], wts[0, 0][keep], atol=1e-6)
    assert section_d[~_inside(N)].abs().max() == 0
    if dim == 3:
        assert data[0, 1:].abs().max() == 0 and wrec[0, 1:].abs().max() == 0
    assert (wrec >= 0).all()
    twice_d, twice_w = fn(proj.repeat(1, 2, 1, 1), _eye(dim, 2), weights=wts.repeat(1, 2, 1, 1), interpolation=interp)
    assert rel_err(twice_d, 2 * data) < 1e-6 and rel_err(twice_w, 2 * wrec) < 1e-6


@pytest.mark.parametrize("interp", ["linear", "cubic"])
def test_backprojection_undoes_the_shift_of_the_projection(tp, interp):
    """(themes: tests/2d/back/test_basic_backprojection.py:123, tests/3d/back/test_basic_backprojection_2d_to_3d.py:175)
    Back-projection applies the conjugate ramp: inserting a shifted slice with the same shift
    equals inserting the unshifted slice."""
    N = 32
    gen = torch.Generator().manual_seed(8)
    rec = _crandn(1, N, N, N // 2 + 1, gen=gen)
    rot = random_rotations_3d(3, gen).view(1, 3, 3, 3).to(DEV)
    shifts = ((torch.rand(1, 3, 2, generator=gen) * 2 - 1) * 4).to(DEV)
    plain = tp.project_3d_to_2d_forw(rec, rot, interpolation=interp)
    moved = tp.project_3d_to_2d_forw(rec, rot, shifts=shifts, interpolation=interp)
    d_plain, _ = tp.backproject_2d_to_3d_forw(plain, rot, interpolation=interp)
    d_moved, _ = tp.backproject_2d_to_3d_forw(moved, rot, shifts=shifts, interpolation=interp)
    assert rel_err(d_moved, d_plain) < TOL_ATOMIC


# ---- oversampling ----------------------------------------------------------------------------
def _ncc(a, b):
    a, b = a - a.mean(), b - b.mean()
    return float((a * b).sum() / (a.norm() * b.norm()))


@pytest.mark.parametrize("dim", [2, 3])
@pytest.mark.parametrize("factor", [2.0, 3.0])
def test_oversampled_path_agrees_with_the_unpadded_path(tp, dim, factor):
    """(themes: tests/2d/forw/test_oversampling.py:17, tests/3d/forw/test_oversampling_3d_to_2d.py:17)
    Zero-padding in real space by `factor` and projecting with oversampling=factor shows the same
    image as the unpadded path (normalised cross-correlation above 0.99)."""
    n, B = 32, 2
    gen = torch.Generator().manual_seed(12)
    real = torch.randn(B, *([n] * dim), generator=gen).to(DEV)
    quarter = torch.tensor([[0., -1.], [1., 0.]]) if dim == 2 else _rot3(0, 0, math.pi / 2)
    rot = quarter.view(1, 1, dim, dim).to(DEV)
    fn = tp.project_2d_forw if dim == 2 else tp.project_3d_to_2d_forw
    padded = fn(tp.prep.pad_and_fftshift(real, factor, dims=dim), rot, output_shape=(n, n), interpolation="cubic", oversampling=factor)
    plain = fn(tp.prep.pad_and_fftshift(real, 1.0, dims=dim), rot, output_shape=(n, n), interpolation="cubic", oversampling=1.0)
    for b in range(B):
        assert _ncc(torch.fft.irfft2(padded[b, 0], s=(n, n)), torch.fft.irfft2(plain[b, 0], s=(n, n))) > 0.99


@pytest.mark.parametrize("dim", [2, 3])
def test_backprojection_volume_grows_with_oversampling(tp, dim):
    """(themes: tests/2d/back/test_oversampling_back.py:17-101, tests/3d/back/test_oversampling_back_2d_to_3d.py:17-115)
    The reconstruction box is ceil(N * oversampling) made even; data and weights share it."""
    N = 16
    gen = torch.Generator().manual_seed(2)
    proj = _crandn(1, 2, N, N // 2 + 1, gen=gen)
    wts = torch.rand(1, 2, N, N // 2 + 1, generator=gen).to(DEV)
    rot = (random_rotations_2d(2, gen) if dim == 2 else random_rotations_3d(2, gen)).view(1, 2, dim, dim).to(DEV)
    fn = tp.backproject_2d_forw if dim == 2 else tp.backproject_2d_to_3d_forw
    for factor, box in ((1.0, 16), (1.3, 22), (1.5, 24), (2.0, 32), (3.0, 48)):
        data, wrec = fn(proj, rot, weights=wts, oversampling=factor)
        want = (1,) + (box,) * (dim - 1) + (box // 2 + 1,)
        assert data.shape == want and wrec.shape == want, (factor, data.shape)
        assert torch.isfinite(data.abs()).all() and (wrec >= 0).all() and wrec.sum() > 0


# ---- gradients -------------------------------------------------------------------------------
@pytest.mark.parametrize("dim", [2, 3])
@pytest.mark.parametrize("interp", ["linear", "cubic"])
def test_backward_of_projection_is_its_adjoint(tp, dim, interp):
    """(themes: tests/2d/forw/test_gradients.py:22-66, tests/3d/forw/test_gradients_3d_to_2d.py:68 and :331)
    project is real-linear in the reconstruction, so for L(v) = Re<project(v), g> the gradient
    A^T g satisfies Re<v, A^T g> = L(v) -- for any g that is blind to the redundant half of
    column 0 (which the backward pass skips) and a cutoff that keeps every tap inside the
    volume (gathers clamp at the border, scatters drop)."""
    N, P = 16, 6
    gen = torch.Generator().manual_seed(17)
    v = _crandn(1, *([N] * (dim - 1)), N // 2 + 1, gen=gen).to(torch.complex128).requires_grad_(True)
    g = _crandn(1, P, N, N // 2 + 1, gen=gen).to(torch.complex128)
    g[..., N // 2:, 0] = 0
    make = random_rotations_2d if dim == 2 else random_rotations_3d
    rot = make(P, gen, torch.float64).view(1, P, dim, dim).to(DEV)
    shifts = ((torch.rand(1, P, 2, generator=gen, dtype=torch.float64) * 2 - 1) * 3).to(DEV)
    fwd = tp.project_2d_forw if dim == 2 else tp.project_3d_to_2d_forw
    out = fwd(v, rot, shifts=shifts, output_shape=(N, N), interpolation=interp, fourier_radius_cutoff=N / 2 - 3)
    loss = (out.conj() * g).real.sum()
    loss.backward()
    back = (v.detach().conj() * v.grad).real.sum()
    assert abs(loss.item() - back.item()) <= 1e-10 * max(abs(loss.item()), 1.0), (loss.item(), back.item())
    # and the explicit backward entry of the public API returns that same gradient at the default cutoff
    bwd = tp.project_2d_back if dim == 2 else tp.project_3d_to_2d_back
    v2 = v.detach().clone().requires_grad_(True)
    (fwd(v2, rot, shifts=shifts, output_shape=(N, N), interpolation=interp).conj() * g).real.sum().backward()
    assert rel_err(bwd(g, v.detach(), rot, shifts=shifts, interpolation=interp), v2.grad) < 1e-12


@pytest.mark.parametrize("dim", [2, 3])
def test_weight_gradients_of_backprojection(tp, dim):
    """(themes: tests/2d/back/test_gradients_back.py:492, tests/3d/back/test_gradients_back_2d_to_3d.py:541)
    weight_rec is linear in the weights with non-negative tap weights.  Away from column 0 of
    the volume (where back-projection also feeds the Friedel partners, which the weight
    gradient does not follow) the gradient is the exact adjoint: gradcheck in double, and a
    uniform upstream gradient gives each pixel the sum of its tap weights off column 0."""
    N, P = 8, 3
    gen = torch.Generator().manual_seed(23)
    proj = _crandn(1, P, N, N // 2 + 1, gen=gen).to(torch.complex128)
    make = random_rotations_2d if dim == 2 else random_rotations_3d
    rot = make(P, gen, torch.float64).view(1, P, dim, dim).to(DEV)
    wts = torch.rand(1, P, N, N // 2 + 1, generator=gen, dtype=torch.float64).to(DEV).requires_grad_(True)
    fn = tp.backproject_2d_forw if dim == 2 else tp.backproject_2d_to_3d_forw
    pix = torch.ones(N, N // 2 + 1, dtype=torch.float64, device=DEV)
    pix[N // 2:, 0] = 0                       # the redundant half of column 0 is not inserted

    def weight_volume_off_column_0(w):
        return fn(proj, rot, weights=w * pix, interpolation="linear", oversampling=2.0, fourier_radius_cutoff=3.0)[1][..., 1:]

    assert torch.autograd.gradcheck(weight_volume_off_column_0, (wts,), eps=1e-6, atol=1e-7, rtol=1e-6, nondet_tol=1e-9)
    weight_volume_off_column_0(wts).sum().backward()
    grad = wts.grad[0]
    contributes = (_inside(N, 3.0).double() * pix).expand(P, -1, -1)
    assert (grad >= 0).all() and (grad <= 1 + 1e-9).all()
    assert (grad[contributes == 0] == 0).all() and grad.sum() > 0.5 * contributes.sum()
