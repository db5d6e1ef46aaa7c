"""GPU tests restated from the themes of the reference's own suite (basic / batching /
gradients / oversampling), run against this package's public API.  Inputs are seeded."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tp(cuda_device):
    import torch_projectors_b200
    return torch_projectors_b200


def _rot_z(angle, device="cuda"):
    c, s = math.cos(angle), math.sin(angle)
    return torch.tensor([[c, -s, 0.0], [s, c, 0.0], [0.0, 0.0, 1.0]], device=device).view(1, 1, 3, 3)


def _ignore_redundant_half_column(target, out):
    """The backward passes skip the Friedel-redundant half of the j = 0 column (rows >= N/2),
    as the reference's do; its tests zero those contributions.  Copying the output into the
    target there makes the loss blind to that half-column."""
    N = target.shape[-2]
    target = target.clone()
    target[..., N // 2:, 0] = out.detach()[..., N // 2:, 0]
    return target


def _pad_fftshift_rfftn(vol, factor):
    n = vol.shape[-1]
    pad = (n * factor - n) // 2
    padded = torch.nn.functional.pad(vol, (pad, pad) * 3)
    return torch.fft.rfftn(torch.fft.fftshift(padded, dim=(-3, -2, -1)), dim=(-3, -2, -1), norm="forward").to(torch.complex64)


@pytest.mark.parametrize("interp", ["linear", "cubic"])
def test_rotation_gradient_matches_finite_difference_on_the_angle(tp, interp):
    # reference: tests/3d/forw/test_gradients_3d_to_2d.py:455-508 (central difference on the angle)
    torch.manual_seed(3)
    N = 32
    rec = _pad_fftshift_rfftn(torch.randn(1, N, N, N, device="cuda"), 1)
    target = torch.randn(1, 1, N, N // 2 + 1, dtype=torch.complex64, device="cuda")

    def loss_of(angle_t):
        c, s = torch.cos(angle_t), torch.sin(angle_t)
        zero, one = torch.zeros_like(c), torch.ones_like(c)
        rot = torch.stack([torch.stack([c, -s, zero]), torch.stack([s, c, zero]), torch.stack([zero, zero, one])]).view(1, 1, 3, 3)
        out = tp.project_3d_to_2d_forw(rec, rot, interpolation=interp, fourier_radius_cutoff=10.0)
        # a linear functional of the projection (well conditioned for a difference quotient),
        # blind to the half-column the backward pass skips; float64 sum against rounding noise
        g = target.clone()
        g[..., N // 2:, 0] = 0
        return (out.to(torch.complex128) * g.to(torch.complex128).conj()).real.sum()

    angle = torch.tensor(0.3, device="cuda", requires_grad=True)
    loss_of(angle).backward()
    # small step: trilinear interpolation has a gradient kink wherever a sample crosses a voxel
    # boundary, and every crossing inside the step biases the difference quotient
    eps = 2e-4
    with torch.no_grad():
        fd = (loss_of(torch.tensor(0.3 + eps, device="cuda")) - loss_of(torch.tensor(0.3 - eps, device="cuda"))) / (2 * eps)
    tol = 3e-2 if interp == "linear" else 1e-2
    assert abs(angle.grad.item() - fd.item()) <= tol * abs(fd.item()) + 1e-3, (angle.grad.item(), fd.item())


def test_shift_gradient_matches_autograd_through_a_manual_phase_ramp(tp):
    # reference: tests/3d/forw/test_gradients_3d_to_2d.py:169-290 (atol 1e-4, rtol 1e-2)
    torch.manual_seed(4)
    N = 16
    rec = torch.randn(1, N, N, N // 2 + 1, dtype=torch.complex64, device="cuda")
    rot = _rot_z(0.4)
    target = torch.randn(1, 1, N, N // 2 + 1, dtype=torch.complex64, device="cuda")
    sh = torch.tensor([[[1.5, -2.25]]], device="cuda", requires_grad=True)
    out = tp.project_3d_to_2d_forw(rec, rot, sh)
    target = _ignore_redundant_half_column(target, out)
    ((out - target).abs() ** 2).sum().backward()
    sh2 = sh.detach().clone().requires_grad_(True)
    base = tp.project_3d_to_2d_forw(rec, rot).detach()
    kr = torch.fft.fftfreq(N, 1.0 / N, device="cuda")[:, None]
    kc = torch.arange(N // 2 + 1, device="cuda", dtype=torch.float32)[None, :]
    phase = -2 * math.pi * (kr * sh2[0, 0, 0] + kc * sh2[0, 0, 1]) / N
    # the reference stores +N/2 (not -N/2) at the Nyquist row
    phase = torch.where(kr == -N / 2, -2 * math.pi * ((N / 2) * sh2[0, 0, 0] + kc * sh2[0, 0, 1]) / N, phase)
    manual = base * torch.polar(torch.ones_like(phase), phase)
    ((manual - target).abs() ** 2).sum().backward()
    assert torch.allclose(out.detach(), manual.detach(), atol=1e-4)
    assert torch.allclose(sh.grad, sh2.grad, atol=1e-3, rtol=1e-2)


def test_oversampled_projection_matches_unpadded_projection(tp):
    # reference: tests/3d/forw/test_oversampling_3d_to_2d.py:14-94 (loose atol 1e-1)
    torch.manual_seed(5)
    N = 32
    x = torch.arange(N, device="cuda") - N // 2
    zz, yy, xx = torch.meshgrid(x, x, x, indexing="ij")
    vol = torch.exp(-((xx - 3) ** 2 + (yy + 2) ** 2 + zz ** 2) / 18.0).unsqueeze(0).float()   # smooth blob, compact support
    rot = _rot_z(0.6)
    plain = tp.project_3d_to_2d_forw(_pad_fftshift_rfftn(vol, 1), rot, interpolation="cubic")
    over = tp.project_3d_to_2d_forw(_pad_fftshift_rfftn(vol, 2), rot, output_shape=(N, N), interpolation="cubic", oversampling=2.0)
    # rfftn(norm='forward') of a volume padded 2x per axis is scaled by 1/8 at equal frequencies
    assert torch.allclose(over * 8, plain, atol=1e-1 * plain.abs().max().item())
    assert (over * 8 - plain).abs().max() < 0.05 * plain.abs().max()


def test_identical_slices_accumulate_and_weights_stay_non_negative(tp):
    # reference: tests/3d/back/test_basic_backprojection_2d_to_3d.py:119-120, 244-287
    torch.manual_seed(6)
    N, P = 16, 7
    one = torch.randn(1, 1, N, N // 2 + 1, dtype=torch.complex64, device="cuda")
    w1 = torch.rand(1, 1, N, N // 2 + 1, device="cuda")
    rot = _rot_z(0.2)
    d1, wr1 = tp.backproject_2d_to_3d_forw(one, rot, weights=w1, interpolation="cubic")
    dP, wrP = tp.backproject_2d_to_3d_forw(one.expand(1, P, -1, -1), rot.expand(1, P, -1, -1), weights=w1.expand(1, P, -1, -1), interpolation="cubic")
    assert (wrP >= 0).all()
    assert torch.allclose(dP, d1 * P, atol=1e-4) and torch.allclose(wrP, wr1 * P, atol=1e-4)
    nowt, empty = tp.backproject_2d_to_3d_forw(one, rot)
    assert empty.shape == (0,) and torch.allclose(nowt, tp.backproject_2d_to_3d_forw(one, rot, interpolation="linear")[0])


def test_batched_backprojection_equals_per_item_calls(tp):
    # reference: tests/3d/back/test_batching_back_2d_to_3d.py:20-345 (atol 1e-5)
    torch.manual_seed(7)
    B, P, N = 3, 5, 12
    proj = torch.randn(B, P, N, N // 2 + 1, dtype=torch.complex64, device="cuda")
    w = torch.rand(B, P, N, N // 2 + 1, device="cuda")
    q = torch.randn(P, 4, device="cuda")
    q = q / q.norm(dim=1, keepdim=True)
    a, b, c, d = q.unbind(1)
    rot = torch.stack([1 - 2 * (c * c + d * d), 2 * (b * c - d * a), 2 * (b * d + c * a),
                       2 * (b * c + d * a), 1 - 2 * (b * b + d * d), 2 * (c * d - b * a),
                       2 * (b * d - c * a), 2 * (c * d + b * a), 1 - 2 * (b * b + c * c)], 1).view(1, P, 3, 3)
    sh = torch.rand(1, P, 2, device="cuda") * 4 - 2
    full_d, full_w = tp.backproject_2d_to_3d_forw(proj, rot, weights=w, shifts=sh, oversampling=1.5)
    for k in range(B):
        d_k, w_k = tp.backproject_2d_to_3d_forw(proj[k:k + 1], rot, weights=w[k:k + 1], shifts=sh, oversampling=1.5)
        assert torch.allclose(full_d[k:k + 1], d_k, atol=1e-5) and torch.allclose(full_w[k:k + 1], w_k, atol=1e-5)
    # broadcast (expanded, stride-0) rotations give the same result as one shared rotation set
    exp_d, _ = tp.backproject_2d_to_3d_forw(proj, rot.expand(B, -1, -1, -1), weights=w, shifts=sh.expand(B, -1, -1), oversampling=1.5)
    assert torch.allclose(exp_d, full_d, atol=1e-5)


def test_2d_projection_roundtrip_known_answers(tp):
    # reference: tests/2d/forw/test_basic_projection.py:15-141 (identity and +-90 degree peaks)
    N = 16
    rec = torch.zeros(1, N, N // 2 + 1, dtype=torch.complex64, device="cuda")
    rec[0, 0, 3] = 1.0
    ident = tp.project_2d_forw(rec, torch.eye(2, device="cuda").view(1, 1, 2, 2))
    assert ident[0, 0, 0, 3].abs().item() == pytest.approx(1.0, abs=1e-5) and ident[0, 0].abs().sum().item() == pytest.approx(1.0, abs=1e-4)
    ang = math.pi / 2
    rot = torch.tensor([[math.cos(ang), -math.sin(ang)], [math.sin(ang), math.cos(ang)]], device="cuda").view(1, 1, 2, 2)
    turned = tp.project_2d_forw(rec, rot)[0, 0].abs()
    assert max(turned[N - 3, 0].item(), turned[3, 0].item()) == pytest.approx(1.0, abs=1e-5)
