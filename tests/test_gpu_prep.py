"""The fused pad + fftshift and ifftshift + crop passes of ``prep`` on the GPU against the plain
torch composition (which is what CPU tensors take), their autograd, and the round trip."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tp(cuda_device):
    import torch_projectors_b200
    return torch_projectors_b200


@pytest.mark.parametrize("dims", [2, 3])
@pytest.mark.parametrize("n,factor", [(16, 1.0), (16, 2.0), (10, 1.3), (15, 2.0), (12, 3.0)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_fused_passes_equal_the_torch_composition(tp, dims, n, factor, dtype):
    gen = torch.Generator().manual_seed(n * 7 + dims)
    real = torch.randn(2, 3, *([n] * dims), generator=gen, dtype=dtype)
    want = tp.prep.pad_and_fftshift(real, factor, dims=dims)                # CPU: pad -> fftshift -> rfftn
    got = tp.prep.pad_and_fftshift(real.cuda(), factor, dims=dims)
    assert got.is_cuda and got.shape == want.shape
    tol = 1e-5 if dtype == torch.float32 else 1e-12
    assert (got.cpu() - want).abs().max() <= tol * want.abs().max()
    m = want.shape[-2]
    back_want = tp.prep.ifftshift_and_crop(want, m / n, dims=dims)
    back_got = tp.prep.ifftshift_and_crop(got, m / n, dims=dims)
    assert back_got.shape == back_want.shape == real.shape
    assert (back_got.cpu() - back_want).abs().max() <= tol * 10
    assert (back_got.cpu() - real).abs().max() <= tol * 10                  # round trip


def test_the_padded_array_itself_is_bit_exact(tp):
    from torch_projectors_b200.prep import _CropUnshift, _PadShift
    gen = torch.Generator().manual_seed(1)
    for dims, n, m in ((2, 6, 10), (3, 6, 10), (3, 7, 12), (2, 8, 8)):
        real = torch.randn(4, *([n] * dims), generator=gen).cuda()
        lo = (m - n) // 2
        padded = torch.nn.functional.pad(real, (lo, m - n - lo) * dims)
        axes = tuple(range(-dims, 0))
        want = torch.fft.fftshift(padded, dim=axes)
        got = _PadShift.apply(real, dims, m)
        assert torch.equal(got, want)
        full = torch.randn(4, *([m] * dims), generator=gen).cuda()
        crop = torch.fft.ifftshift(full, dim=axes)[(Ellipsis,) + (slice(lo, lo + n),) * dims]
        assert torch.equal(_CropUnshift.apply(full, dims, n), crop)


@pytest.mark.parametrize("dims", [2, 3])
def test_autograd_through_the_fused_passes(tp, dims):
    gen = torch.Generator().manual_seed(3)
    real = torch.randn(2, *([6] * dims), generator=gen, dtype=torch.float64).cuda().requires_grad_(True)
    assert torch.autograd.gradcheck(lambda x: torch.view_as_real(tp.prep.pad_and_fftshift(x, 2.0, dims=dims)), (real,), eps=1e-6, atol=1e-7)
    rec = tp.prep.pad_and_fftshift(real.detach(), 2.0, dims=dims).requires_grad_(True)
    # irfftn only sees the Hermitian part of its input: check the gradient through the crop on the real side
    full = torch.randn(2, *([12] * dims), generator=gen, dtype=torch.float64).cuda().requires_grad_(True)
    from torch_projectors_b200.prep import _CropUnshift
    assert torch.autograd.gradcheck(lambda x: _CropUnshift.apply(x, dims, 6), (full,), eps=1e-6, atol=1e-7)
    # and the pipeline volume -> projections -> loss back-propagates into the real-space volume
    if dims == 3:
        vol = torch.randn(1, 8, 8, 8, generator=gen).cuda().requires_grad_(True)
        rot = torch.eye(3, device="cuda").view(1, 1, 3, 3)
        out = tp.project_3d_to_2d_forw(tp.prep.pad_and_fftshift(vol, 2.0).to(torch.complex64), rot, output_shape=(8, 8), oversampling=2.0)
        out.abs().pow(2).sum().backward()
        assert vol.grad is not None and torch.isfinite(vol.grad).all() and vol.grad.abs().sum() > 0


def test_large_batches_are_split_over_launches(tp):
    real = torch.randn(70000, 4, 4).cuda()                   # more 2D images than one grid's z extent
    got = tp.prep.pad_and_fftshift(real, 2.0, dims=2)
    want = tp.prep.pad_and_fftshift(real[-3:].cpu(), 2.0, dims=2)
    assert got.shape == (70000, 8, 5) and (got[-3:].cpu() - want).abs().max() < 1e-6
