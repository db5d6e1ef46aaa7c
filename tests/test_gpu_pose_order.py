"""The optional processing order of the slices (3D operators that read a volume): the order
the library derives from the rotations is a permutation that keeps neighbouring planes
together, and results do not depend on the order at all."""
import pytest
import torch

from cases import TOL_ATOMIC, random_rotations_3d, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tp(cuda_device):
    import torch_projectors_b200
    return torch_projectors_b200


def _normals(rot):
    n = rot[..., :, 2]
    return torch.where(n[..., 2:3] < 0, -n, n)


@pytest.mark.parametrize("B,B_rot,dtype", [(1, 1, torch.float32), (3, 3, torch.float32), (3, 1, torch.float32),
                                           (2, 2, torch.float64)])
def test_order_is_a_permutation_per_batch_item_and_groups_nearby_planes(tp, B, B_rot, dtype):
    P = 3000
    gen = torch.Generator().manual_seed(5)
    rot = random_rotations_3d(B_rot * P, gen).reshape(B_rot, P, 3, 3).to("cuda", dtype)
    order = torch.full((B * P,), -7, dtype=torch.int32, device="cuda")
    tp._abi.pose_order_3d(rot, B, P, order)
    order = order.cpu().long().reshape(B, P)
    for b in range(B):
        assert torch.equal(order[b].sort().values, torch.arange(b * P, (b + 1) * P))
        n = _normals(rot[b if B_rot > 1 else 0].float().cpu())
        walk = n[order[b] - b * P]
        # |cos| of the angle between the planes of consecutive slices: ~0.5 on average for random
        # order, close to 1 when neighbours in the order are neighbours on the sphere
        near = (walk[1:] * walk[:-1]).sum(-1).abs().mean().item()
        rand = (n[1:] * n[:-1]).sum(-1).abs().mean().item()
        assert near > 0.97 and rand < 0.6, (near, rand)


@pytest.mark.parametrize("interp", ["linear", "cubic"])
def test_results_do_not_depend_on_the_processing_order(tp, interp):
    from torch_projectors_b200 import ops
    B, P, N, R = 2, 70, 16, 32
    gen = torch.Generator().manual_seed(11)
    rec = torch.randn(B, R, R, R // 2 + 1, dtype=torch.complex64, generator=gen).cuda()
    rot = random_rotations_3d(B * P, gen).reshape(B, P, 3, 3).cuda()
    sh = ((torch.rand(B, P, 2, generator=gen) * 2 - 1) * 3).cuda()
    gp = torch.randn(B, P, N, N // 2 + 1, dtype=torch.complex64, generator=gen).cuda()
    gw = torch.randn(B, R, R, R // 2 + 1, generator=gen).cuda()
    wts = torch.rand(B, P, N, N // 2 + 1, generator=gen).cuda()
    t = torch.ops.torch_projectors_b200

    def run():
        r = rot.clone().requires_grad_(True)
        s = sh.clone().requires_grad_(True)
        return (t.project_3d_to_2d_forw(rec, r, s, [N, N], interp, 2.0, None),
                *t.project_3d_to_2d_back(gp, rec, r, s, interp, 2.0, None),
                *t.backproject_2d_to_3d_back(rec, gw, gp, wts, r, s, interp, 2.0, None))

    try:
        ops.set_pose_order_thresholds(1 << 60, 64)
        natural = run()
        ops.set_pose_order_thresholds(0, 1)              # every call derives an order
        ordered = run()
    finally:
        ops.set_pose_order_thresholds()
    # the same through the *_ordered operators with one order computed up front and reused
    order = ops.plane_locality_order(rot, B)
    assert order.dtype == torch.int32 and order.numel() == B * P
    r = rot.clone().requires_grad_(True)
    s = sh.clone().requires_grad_(True)
    reused = (t.project_3d_to_2d_forw_ordered(rec, r, s, [N, N], interp, 2.0, None, order),
              *t.project_3d_to_2d_back_ordered(gp, rec, r, s, interp, 2.0, None, order),
              *t.backproject_2d_to_3d_back_ordered(rec, gw, gp, wts, r, s, interp, 2.0, None, order))
    for k in (0, 4, 5):
        assert torch.equal(natural[k], reused[k]), k
    for k in (1, 2, 3, 6, 7):
        assert rel_err(reused[k], natural[k]) < TOL_ATOMIC * 0.1, k
    # gathers write each slice on its own: bit-identical; atomically accumulated outputs agree
    # to rounding (their summation order is not fixed in either run)
    for k in (0, 4, 5):                       # projections, grad_projections, grad_weights
        assert torch.equal(natural[k], ordered[k]), k
    for k in (1, 2, 3, 6, 7):
        assert rel_err(ordered[k], natural[k]) < TOL_ATOMIC * 0.1, k


def test_entries_outside_the_range_leave_their_slice_unwritten(tp):
    P, N, R = 6, 8, 16
    gen = torch.Generator().manual_seed(3)
    rec = torch.randn(1, R, R, R // 2 + 1, dtype=torch.complex64, generator=gen).cuda()
    rot = random_rotations_3d(P, gen).reshape(1, P, 3, 3).cuda()
    want = torch.ops.torch_projectors_b200.project_3d_to_2d_forw(rec, rot, None, [N, N], "linear", 2.0, None)
    out = torch.full_like(want, 123.0)
    order = torch.tensor([5, 4, -1, 2, 1000, 0], dtype=torch.int32, device="cuda")
    tp._abi.project_forw(3, rec, rot, None, P, N, tp._abi.LINEAR, 2.0, N / 2.0, out, order)
    for p in (5, 4, 2, 0):
        assert torch.equal(out[0, p], want[0, p])
    for p in (1, 3):
        assert (out[0, p] == 123.0).all()


def test_public_api_keeps_one_order_for_forward_and_backward(tp):
    """pose_order= of the public function: an order computed once is used by the forward pass and
    saved for the backward pass; None derives one per call; False keeps the given order.  All give
    the same projections (bit for bit) and gradients (to rounding)."""
    from torch_projectors_b200 import ops
    P, N, R = 80, 16, 32
    gen = torch.Generator().manual_seed(12)
    rec = torch.randn(1, R, R, R // 2 + 1, dtype=torch.complex64, generator=gen).cuda()
    rot = random_rotations_3d(P, gen).reshape(1, P, 3, 3).cuda()
    sh = ((torch.rand(1, P, 2, generator=gen) * 2 - 1) * 3).cuda()
    g = torch.randn(1, P, N, N // 2 + 1, dtype=torch.complex64, generator=gen).cuda()
    order = tp.plane_locality_order(rot)
    assert torch.equal(order.sort().values.cpu(), torch.arange(P, dtype=torch.int32))
    results = {}
    try:
        ops.set_pose_order_thresholds(0, 1)
        for name, arg in (("given", order), ("auto", None), ("natural", False)):
            v = rec.clone().requires_grad_(True)
            r = rot.clone().requires_grad_(True)
            s = sh.clone().requires_grad_(True)
            out = tp.project_3d_to_2d_forw(v, r, s, output_shape=(N, N), interpolation="cubic", oversampling=2.0, pose_order=arg)
            out.backward(g)
            results[name] = (out.detach(), v.grad, r.grad, s.grad)
    finally:
        ops.set_pose_order_thresholds()
    for name in ("auto", "natural"):
        assert torch.equal(results[name][0], results["given"][0])
        for a, b in zip(results[name][1:], results["given"][1:]):
            assert rel_err(a, b) < TOL_ATOMIC * 0.1
    # without gradients the call goes straight to the raw operator: the same projections to rounding
    # (with rotation gradients wanted the forward pass is the kernel that also keeps the pixels'
    # derivatives, which sums the taps in another order), bit for bit with that kernel switched off
    with torch.no_grad():
        plain = tp.project_3d_to_2d_forw(rec, rot, sh, output_shape=(N, N), interpolation="cubic", oversampling=2.0, pose_order=order)
    assert rel_err(plain, results["given"][0]) <= 1e-6
    tp.set_save_derivatives(False)
    try:
        out = tp.project_3d_to_2d_forw(rec.clone().requires_grad_(True), rot.clone().requires_grad_(True), sh, output_shape=(N, N),
                                       interpolation="cubic", oversampling=2.0, pose_order=order)
    finally:
        tp.set_save_derivatives(True)
    assert torch.equal(plain, out.detach())
