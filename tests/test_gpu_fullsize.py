"""Parity at the full volume sizes of the large BASELINE configurations, on subsets of poses
small enough for the CPU oracle: the box-512 volume of the autograd-step workload (cubic,
forward and all gradients) and the box-400 -> 800^3 back-projection of the sharded workload
(the slab-ordered kernel with its real slab count)."""
import pytest
import torch

from cases import TOL_ATOMIC, TOL_FORWARD, make_rotations, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tp(cuda_device):
    import torch_projectors_b200
    return torch_projectors_b200


def test_autograd_step_volume_size_subset_against_oracle(tp):
    from oracle import port
    gen = torch.Generator().manual_seed(404)
    R, N, P = 512, 256, 3
    rec = torch.complex(torch.randn(1, R, R, R // 2 + 1, generator=gen), torch.randn(1, R, R, R // 2 + 1, generator=gen))
    rot = make_rotations(3, 1, P, gen, special=False)
    shifts = (torch.rand(1, P, 2, generator=gen) * 2 - 1) * 10.0
    g = torch.complex(torch.randn(1, P, N, N // 2 + 1, generator=gen), torch.randn(1, P, N, N // 2 + 1, generator=gen))
    d_rec = rec.cuda().requires_grad_(True)
    d_rot = rot.cuda().requires_grad_(True)
    d_sh = shifts.cuda().requires_grad_(True)
    out = tp.project_3d_to_2d_forw(d_rec, d_rot, d_sh, output_shape=(N, N), interpolation="cubic", oversampling=2.0)
    out.backward(g.cuda())
    want = port.project_3d_to_2d_forw(rec, rot, shifts, [N, N], "cubic", 2.0)
    assert rel_err(out, want) <= TOL_FORWARD
    w_rec, w_rot, w_sh = port.project_3d_to_2d_back(g, rec, rot, shifts, "cubic", 2.0, None, True, True)
    assert rel_err(d_rot.grad, w_rot) <= TOL_ATOMIC
    assert rel_err(d_sh.grad, w_sh) <= TOL_ATOMIC
    assert rel_err(d_rec.grad, w_rec) <= TOL_ATOMIC


def test_box400_backprojection_subset_against_oracle(tp):
    from oracle import port
    gen = torch.Generator().manual_seed(405)
    N, P = 400, 24
    proj = torch.complex(torch.randn(1, P, N, N // 2 + 1, generator=gen), torch.randn(1, P, N, N // 2 + 1, generator=gen))
    weights = torch.rand(1, P, N, N // 2 + 1, generator=gen)
    rot = make_rotations(3, 1, P, gen, special=True)
    shifts = (torch.rand(1, P, 2, generator=gen) * 2 - 1) * 12.0
    data, wrec = tp.backproject_2d_to_3d_forw(proj.cuda(), rot.cuda(), weights=weights.cuda(), shifts=shifts.cuda(),
                                              interpolation="linear", oversampling=2.0)
    assert data.shape == (1, 800, 800, 401)
    d_want, w_want = port.backproject_2d_to_3d_forw(proj, weights, rot, shifts, "linear", 2.0)
    assert rel_err(data, d_want) <= TOL_ATOMIC
    assert rel_err(wrec, w_want) <= TOL_ATOMIC
    # accumulate a second time: exactly twice the volumes (streaming use of the sharded path)
    tp.backproject_2d_to_3d_accumulate_(data, wrec, proj.cuda(), rot.cuda(), weights.cuda(), shifts.cuda(), oversampling=2.0)
    assert rel_err(data, 2 * d_want) <= TOL_ATOMIC
    # and the same slices through the persistent interleaved accumulator (slabs of 16-byte voxels,
    # the path the sharded workload runs), two chunks folded once
    vols = tp.sharding.PartialVolumes(1, 800, "cuda")
    for lo, hi in ((0, 10), (10, P)):
        vols.add_(proj[:, lo:hi].cuda(), rot[:, lo:hi].cuda(), weights[:, lo:hi].cuda(), shifts[:, lo:hi].cuda(),
                  interpolation="linear", oversampling=2.0)
    vols.flush()
    assert rel_err(vols.data, d_want) <= TOL_ATOMIC
    assert rel_err(vols.weights, w_want) <= TOL_ATOMIC
