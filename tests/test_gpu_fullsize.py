"""Parity at the full volume sizes of the two large benchmark workloads, on subsets of poses
the CPU reference finishes in seconds: the box-512 volume of the autograd-step workload (cubic,
forward and all gradients, 32 poses) and the box-400 -> 800^3 back-projection of the sharded
workload (256 slices: the slab-ordered kernel with its real slab count, the persistent
accumulator, and the slab-by-slab final stage that overlaps the fold)."""
import pytest
import torch

from cases import TOL_ATOMIC, TOL_FORWARD, make_rotations, rel_err, rel_err_on_device
from runners import cpu_checker

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tp(cuda_device):
    import torch_projectors_b200
    return torch_projectors_b200


def test_autograd_step_volume_size_subset_against_reference(tp):
    ops, _ = cpu_checker()
    gen = torch.Generator().manual_seed(404)
    R, N, P = 512, 256, 32
    rec = torch.complex(torch.randn(1, R, R, R // 2 + 1, generator=gen), torch.randn(1, R, R, R // 2 + 1, generator=gen))
    rot = make_rotations(3, 1, P, gen, special=False)
    shifts = (torch.rand(1, P, 2, generator=gen) * 2 - 1) * 10.0
    g = torch.complex(torch.randn(1, P, N, N // 2 + 1, generator=gen), torch.randn(1, P, N, N // 2 + 1, generator=gen))
    d_rec = rec.cuda().requires_grad_(True)
    d_rot = rot.cuda().requires_grad_(True)
    d_sh = shifts.cuda().requires_grad_(True)
    # with the plane-locality order the full workload uses (32 poses are below the threshold at which it is derived unasked)
    out = tp.project_3d_to_2d_forw(d_rec, d_rot, d_sh, output_shape=(N, N), interpolation="cubic", oversampling=2.0,
                                   pose_order=tp.plane_locality_order(d_rot.detach()))
    out.backward(g.cuda())
    want = ops.project_3d_to_2d_forw(rec, rot, shifts, [N, N], "cubic", 2.0, None)
    assert rel_err(out, want) <= TOL_FORWARD
    w_rec, w_rot, w_sh = ops.project_3d_to_2d_back(g, rec, rot.clone().requires_grad_(True), shifts.clone().requires_grad_(True),
                                                   "cubic", 2.0, None)
    assert rel_err(d_rot.grad, w_rot) <= TOL_ATOMIC
    assert rel_err(d_sh.grad, w_sh) <= TOL_ATOMIC
    assert rel_err_on_device(d_rec.grad, w_rec) <= TOL_ATOMIC
    # the same gradient with the slices in the order given (32 poses are below the threshold of the order)
    plain = tp.project_3d_to_2d_back(g.cuda(), rec.cuda(), rot.cuda(), shifts.cuda(), interpolation="cubic", oversampling=2.0)
    assert rel_err_on_device(plain, w_rec) <= TOL_ATOMIC


def test_box400_backprojection_subset_against_reference(tp):
    ops, _ = cpu_checker()
    gen = torch.Generator().manual_seed(405)
    N, P = 400, 256
    proj = torch.complex(torch.randn(1, P, N, N // 2 + 1, generator=gen), torch.randn(1, P, N, N // 2 + 1, generator=gen))
    weights = torch.rand(1, P, N, N // 2 + 1, generator=gen)
    rot = make_rotations(3, 1, P, gen, special=True)
    shifts = (torch.rand(1, P, 2, generator=gen) * 2 - 1) * 12.0
    d_want, w_want = ops.backproject_2d_to_3d_forw(proj, weights, rot, shifts, "linear", 2.0, None)
    c = lambda x, lo=0, hi=P: x[:, lo:hi].cuda()  # noqa: E731
    data, wrec = tp.backproject_2d_to_3d_forw(c(proj), c(rot), weights=c(weights), shifts=c(shifts),
                                              interpolation="linear", oversampling=2.0)
    assert data.shape == (1, 800, 800, 401)
    assert rel_err_on_device(data, d_want) <= TOL_ATOMIC
    assert rel_err_on_device(wrec, w_want) <= TOL_ATOMIC
    # accumulate a second time: exactly twice the volumes (streaming use of the plain entry point)
    tp.backproject_2d_to_3d_accumulate_(data, wrec, c(proj), c(rot), c(weights), c(shifts), oversampling=2.0)
    assert rel_err_on_device(data, 2 * d_want) <= TOL_ATOMIC
    del data, wrec
    # the same slices through the persistent interleaved accumulator (slabs of 16-byte voxels, the
    # path the sharded workload runs): two chunks, then the last 96 slices as the final stage, which
    # is scattered slab by slab while finished slabs are folded on a second stream
    vols = tp.sharding.PartialVolumes(1, 800, "cuda")
    kw = dict(interpolation="linear", oversampling=2.0)
    for lo, hi in ((0, 100), (100, 160)):
        vols.add_(c(proj, lo, hi), c(rot, lo, hi), c(weights, lo, hi), c(shifts, lo, hi), **kw)
    vols.add_(c(proj, 160, P), c(rot, 160, P), c(weights, 160, P), c(shifts, 160, P), final=True, **kw)
    seen = []
    vols.flush(after_part=lambda first, stop: seen.append((first, stop)))
    torch.cuda.synchronize()
    n = vols.data.numel()
    assert sum(b - a for a, b in seen) == n and len(seen) >= 8       # every voxel folded once, in many ranges
    assert rel_err_on_device(vols.data, d_want) <= TOL_ATOMIC
    assert rel_err_on_device(vols.weights, w_want) <= TOL_ATOMIC
    # the accumulator is cleared lazily: a further chunk after the fold adds to the folded volumes
    vols.add_(c(proj, 0, 16), c(rot, 0, 16), c(weights, 0, 16), c(shifts, 0, 16), **kw)
    vols.flush()
    d16, w16 = ops.backproject_2d_to_3d_forw(proj[:, :16].contiguous(), weights[:, :16].contiguous(), rot[:, :16].contiguous(),
                                              shifts[:, :16].contiguous(), "linear", 2.0, None)
    assert rel_err_on_device(vols.data, d_want + d16) <= TOL_ATOMIC
    assert rel_err_on_device(vols.weights, w_want + w16) <= TOL_ATOMIC


def test_offsets_beyond_2_to_the_30_in_a_box_1400_volume(tp):
    """Maximum-size edge: a 1400^3 half-volume has 1.37e9 voxels (11 GB), so flat offsets use
    the top of the 31-bit range.  Known answers instead of an oracle: with a quarter turn about x
    (pixel (kr, kc) samples column 20*kc, row 0, plane 20*kr at oversampling 20) a single voxel
    in the last planes is read by exactly one pixel, and a single pixel is back-projected onto
    exactly that voxel."""
    R, N, os_ = 1400, 70, 20.0
    free, _ = torch.cuda.mem_get_info()
    if free < 40 * (1 << 30):
        pytest.skip("needs 40 GB of free device memory")
    rot = torch.tensor([[1.0, 0.0, 0.0], [0.0, 0.0, -1.0], [0.0, 1.0, 0.0]], device="cuda").view(1, 1, 3, 3)
    rec = torch.zeros(1, R, R, R // 2 + 1, dtype=torch.complex64, device="cuda")
    # plane -100 (index R-100), row 0, column 60  <-  pixel kr = -5 (row N-5), kc = 3
    rec[0, R - 100, 0, 60] = 2.0 - 3.0j
    flat = ((R - 100) * R + 0) * (R // 2 + 1) + 60
    assert flat > 1 << 30
    for interp in ("linear", "cubic"):
        out = tp.project_3d_to_2d_forw(rec, rot, output_shape=(N, N), interpolation=interp, oversampling=os_)
        assert out[0, 0, N - 5, 3] == 2.0 - 3.0j
        assert out.abs().sum().item() == pytest.approx(abs(2.0 - 3.0j), rel=1e-6)       # nothing else is non-zero
    grad = torch.zeros(1, 1, N, N // 2 + 1, dtype=torch.complex64, device="cuda")
    grad[0, 0, N - 5, 3] = 1.0 + 0.5j
    grad_rec = tp.project_3d_to_2d_back(grad, rec, rot, interpolation="linear", oversampling=os_)
    assert grad_rec[0, R - 100, 0, 60] == 1.0 + 0.5j and grad_rec.abs().sum().item() == pytest.approx(abs(1.0 + 0.5j), rel=1e-6)
    del grad_rec, rec
    # back-projection of that one pixel (slab-ordered: 16.5 GB of data + weight volumes)
    proj = torch.zeros(1, 1, N, N // 2 + 1, dtype=torch.complex64, device="cuda")
    proj[0, 0, N - 5, 3] = 4.0 + 1.0j
    wts = torch.zeros(1, 1, N, N // 2 + 1, device="cuda")
    wts[0, 0, N - 5, 3] = 0.25
    data, wrec = tp.backproject_2d_to_3d_forw(proj, rot, weights=wts, interpolation="linear", oversampling=os_)
    assert data.shape == (1, R, R, R // 2 + 1)
    assert data[0, R - 100, 0, 60] == 4.0 + 1.0j and wrec[0, R - 100, 0, 60] == 0.25
    assert data.abs().sum().item() == pytest.approx(abs(4.0 + 1.0j), rel=1e-6) and wrec.sum().item() == pytest.approx(0.25, rel=1e-6)
