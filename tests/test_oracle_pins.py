"""Pin the C restatement oracle (oracle/fourier_slice_oracle.c): against the golden vectors
made by the reference's own CPU operators, against those operators directly where
oracle/_ref has been built, and against known answers the reference's tests assert."""
import glob
import math
from pathlib import Path

import pytest
import torch

import oracle
from oracle import port
from cases import SMALL_CASES, make_inputs, random_case, rel_err
from runners import load_golden, run_case

GOLDEN = sorted(glob.glob(str(Path(__file__).parent / "golden" / "*.npz")))

# The oracle follows the reference's fp32 rounding sequence, so it agrees far inside the
# contract tolerances (differences: float vs double cos/sin, summation order of scatters).
PIN_TOL = 2e-6


def test_golden_files_present():
    assert len(GOLDEN) >= 10


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: Path(p).stem)
def test_port_matches_golden(path):
    case, t, want = load_golden(path)
    got = run_case("port", case, t)
    assert set(got) == set(want)
    for k in want:
        assert got[k].shape == want[k].shape, k
        assert rel_err(got[k], want[k]) <= PIN_TOL, (k, rel_err(got[k], want[k]))


@pytest.mark.skipif(not oracle.reference_available(), reason="oracle/_ref not built")
@pytest.mark.parametrize("case", SMALL_CASES, ids=lambda c: c.name)
def test_port_matches_reference_ops(case):
    t = make_inputs(case)
    want = run_case("reference", case, t)
    got = run_case("port", case, t)
    for k in want:
        assert got[k].shape == want[k].shape, k
        assert rel_err(got[k], want[k]) <= PIN_TOL, (k, rel_err(got[k], want[k]))


@pytest.mark.skipif(not oracle.reference_available(), reason="oracle/_ref not built")
@pytest.mark.parametrize("k", range(48))
def test_port_matches_reference_ops_on_randomised_configurations(k):
    """48 seeded random small configurations (odd oversampling factors, tight to unbounded
    cutoffs, every combination of optional arguments and batch broadcasting): the same cases the
    GPU parity test runs against this oracle."""
    case = random_case(k)
    t = make_inputs(case)
    want = run_case("reference", case, t)
    got = run_case("port", case, t)
    assert set(got) == set(want)
    for key in want:
        assert got[key].shape == want[key].shape, key
        assert rel_err(got[key], want[key]) <= PIN_TOL * 2, (case, key, rel_err(got[key], want[key]))


@pytest.mark.skipif(not oracle.reference_available(), reason="oracle/_ref not built")
@pytest.mark.parametrize("case", SMALL_CASES[:4] + SMALL_CASES[9:11], ids=lambda c: c.name)
def test_port_f64_matches_reference_f64(case):
    t = make_inputs(case, cdtype=torch.complex128)
    want = run_case("reference", case, t)
    got = run_case("port", case, t)
    for k in want:
        assert rel_err(got[k], want[k]) <= 1e-13, (k, rel_err(got[k], want[k]))


# ---- known answers (restated from the reference's tests) ----------------------------------
def _mask(N, cutoff=None):
    kr = torch.arange(N).float()
    kr = torch.where(kr <= N // 2, kr, kr - N)
    kc = torch.arange(N // 2 + 1).float()
    c = (N / 2.0) if cutoff is None else cutoff
    return (kr[:, None] ** 2 + kc[None, :] ** 2) <= c * c


@pytest.mark.parametrize("interp", ["linear", "cubic"])
def test_identity_rotation_returns_masked_central_slice(interp):
    # reference: tests/3d/forw/test_basic_projection_3d_to_2d.py:47-94 (atol 1e-5)
    torch.manual_seed(0)
    N = 16
    rec = torch.randn(1, N, N, N // 2 + 1, dtype=torch.complex64)
    rot = torch.eye(3).view(1, 1, 3, 3)
    out = port.project_3d_to_2d_forw(rec, rot, None, [N, N], interp, 1.0)
    want = rec[0, 0] * _mask(N)
    assert torch.allclose(out[0, 0], want, atol=1e-5)


def test_2d_identity_and_peak_rotation():
    # reference: tests/2d/forw/test_basic_projection.py:15-97
    N = 16
    rec = torch.zeros(1, N, N // 2 + 1, dtype=torch.complex64)
    rec[0, 0, 3] = 1.0                      # peak at (kr, kc) = (0, 3)
    for ang, (i, j) in ((0.0, (0, 3)), (math.pi / 2, (N - 3, 0))):
        rot = torch.tensor([[math.cos(ang), -math.sin(ang)], [math.sin(ang), math.cos(ang)]]).view(1, 1, 2, 2)
        out = port.project_2d_forw(rec, rot, None, [N, N], "linear", 1.0)
        # out(k) = rec(R k): the peak is found where R k = (c, r) = (3, 0)
        v = out[0, 0].abs()
        assert v.max().item() == pytest.approx(1.0, abs=1e-5)
        # the rotated peak lands on (i, j) or on its Friedel mate, both are stored for j = 0
        assert v[i, j].item() == pytest.approx(1.0, abs=1e-5) or v[(N - i) % N, j].item() == pytest.approx(1.0, abs=1e-5)


def test_shift_pairs_component_0_with_rows():
    # exp(-2*pi*i*(kr*s0 + kc*s1)/N): shift (1, 0) rotates pixel (1, 0), leaves (0, 1)
    N = 8
    rec = torch.ones(1, N, N // 2 + 1, dtype=torch.complex64)
    rot = torch.eye(2).view(1, 1, 2, 2)
    sh = torch.tensor([[[1.0, 0.0]]])
    out = port.project_2d_forw(rec, rot, sh, [N, N], "linear", 1.0)
    assert torch.allclose(out[0, 0, 1, 0], torch.polar(torch.tensor(1.0), torch.tensor(-2 * math.pi / N)).to(torch.complex64), atol=1e-6)
    assert torch.allclose(out[0, 0, 0, 1], torch.tensor(1.0 + 0j, dtype=torch.complex64), atol=1e-6)


def test_cutoff_is_inclusive_and_default_is_nyquist():
    N = 8
    rec = torch.ones(1, N, N // 2 + 1, dtype=torch.complex64)
    rot = torch.eye(2).view(1, 1, 2, 2)
    out = port.project_2d_forw(rec, rot, None, [N, N], "linear", 1.0, 2.0)
    assert out[0, 0, 0, 2] != 0 and out[0, 0, 2, 0] != 0      # radius exactly 2 is kept
    assert out[0, 0, 1, 2] == 0                                   # r^2 = 5 > 4
    full = port.project_2d_forw(rec, rot, None, [N, N], "linear", 1.0)
    assert full[0, 0, 0, 4] != 0 and full[0, 0, 4, 1] == 0        # default N/2


def test_edge_clamp_replicates_last_column():
    # os = 2 into a volume that is too small: sample c = 6 > Rh-1 = 4 reads column 4
    N, R = 8, 8
    torch.manual_seed(1)
    rec = torch.randn(1, R, R, R // 2 + 1, dtype=torch.complex64)
    rot = torch.eye(3).view(1, 1, 3, 3)
    out = port.project_3d_to_2d_forw(rec, rot, None, [N, N], "linear", 2.0, 100.0)
    assert torch.allclose(out[0, 0, 0, 3], rec[0, 0, 0, 4], atol=1e-6)


def test_backprojection_x0_line_semantics():
    # identity pose, column j = 0 holds (i+1) + 0.1i: rows 1..3 are inserted and mirrored as
    # conjugates, the DC pixel once, the Nyquist row and rows > N/2 are ignored.
    N = 8
    proj = torch.zeros(1, 1, N, N // 2 + 1, dtype=torch.complex64)
    proj[0, 0, :, 0] = torch.arange(1, N + 1).float() + 0.1j
    rot = torch.eye(3).view(1, 1, 3, 3)
    data, w = port.backproject_2d_to_3d_forw(proj, None, rot, None, "linear", 1.0)
    col = data[0, 0, :, 0]
    want = torch.tensor([1 + .1j, 2 + .1j, 3 + .1j, 4 + .1j, 0, 4 - .1j, 3 - .1j, 2 - .1j], dtype=torch.complex64)
    assert torch.allclose(col, want, atol=1e-6)
    assert w.shape == (0,)


@pytest.mark.parametrize("N,os,R", [(6, 1.5, 10), (8, 1.3, 12), (10, 2.0, 20), (6, 1.0, 6)])
def test_rec_boxsize_rule(N, os, R):
    assert port.rec_boxsize(N, os) == R


def test_weights_are_non_negative_and_identical_slices_accumulate():
    # reference: tests/3d/back/test_basic_backprojection_2d_to_3d.py:119-120, 244-287
    torch.manual_seed(2)
    N, P = 8, 5
    one = torch.randn(1, 1, N, N // 2 + 1, dtype=torch.complex64)
    w1 = torch.rand(1, 1, N, N // 2 + 1)
    rot = torch.eye(3).view(1, 1, 3, 3)
    d1, wr1 = port.backproject_2d_to_3d_forw(one, w1, rot, None, "cubic", 1.0)
    dP, wrP = port.backproject_2d_to_3d_forw(one.expand(1, P, -1, -1), w1.expand(1, P, -1, -1),
                                             rot.expand(1, P, -1, -1), None, "cubic", 1.0)
    assert (wrP >= 0).all()
    assert torch.allclose(dP, d1 * P, atol=1e-4)
    assert torch.allclose(wrP, wr1 * P, atol=1e-4)
