"""Parity of the CUDA kernels (called through torch ops -> ctypes -> C ABI) with the CPU
oracle and with the golden vectors made by the reference's own CPU operators.

Tolerances (global-normalised max error, see cases.rel_err): 1e-5 for forward projection,
1e-4 for atomically accumulated back-projection and for all gradients."""
import glob
import math
from pathlib import Path

import pytest
import torch

from cases import (Case, MEDIUM_CASES, SMALL_CASES, TOL_ATOMIC, TOL_FORWARD, hermitian_dc_column_,
                   make_inputs, make_rotations, random_case, rel_err)
from runners import load_golden, run_case, tolerance_for

pytestmark = pytest.mark.gpu

GOLDEN = sorted(glob.glob(str(Path(__file__).parent / "golden" / "*.npz")))


@pytest.fixture(scope="module")
def tp(cuda_device):
    import torch_projectors_b200
    return torch_projectors_b200


def _compare(got: dict, want: dict):
    assert set(got) == set(want)
    for k in want:
        assert got[k].shape == want[k].shape, (k, got[k].shape, want[k].shape)
        err = rel_err(got[k], want[k])
        assert err <= tolerance_for(k), f"{k}: rel err {err:.3e} > {tolerance_for(k):.0e}"


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: Path(p).stem)
def test_cuda_matches_reference_golden_vectors(tp, path):
    case, t, want = load_golden(path)
    _compare(run_case("cuda", case, t), want)


@pytest.mark.parametrize("case", SMALL_CASES + MEDIUM_CASES, ids=lambda c: c.name)
def test_cuda_matches_oracle(tp, case):
    t = make_inputs(case)
    _compare(run_case("cuda", case, t), run_case("port", case, t))


def test_gradient_flags_follow_requires_grad(tp):
    case = SMALL_CASES[0]
    t = {k: (v.cuda() if v is not None else None) for k, v in make_inputs(case).items()}
    ops = torch.ops.torch_projectors_b200
    g_rec, g_rot, g_sh = ops.project_3d_to_2d_back(t["proj"], t["rec"], t["rot"], t["shifts"], case.interp, case.os, None)
    assert g_rec.shape == t["rec"].shape and g_rot.shape == (0,) and g_sh.shape == (0,)
    rot_g = t["rot"].clone().requires_grad_(True)
    _, g_rot, g_sh = ops.project_3d_to_2d_back(t["proj"], t["rec"], rot_g, t["shifts"], case.interp, case.os, None)
    assert g_rot.shape == t["rot"].shape and g_sh.shape == (0,)
    assert (g_rot[..., 2] == 0).all()            # column 2 of the 3x3 gradient is identically 0
    data, w = ops.backproject_2d_to_3d_forw(t["proj"], None, t["rot"], t["shifts"], case.interp, case.os, None)
    assert w.shape == (0,) and data.shape[-1] == data.shape[-2] // 2 + 1
    gp, gw, gr, gs = ops.backproject_2d_to_3d_back(t["grad_data"], None, t["proj"], t["weights"], t["rot"], t["shifts"], case.interp, case.os, None)
    assert gw.shape == t["proj"].shape and (gw == 0).all() and gr.shape == (0,) and gs.shape == (0,)


@pytest.mark.parametrize("interp", ["linear", "cubic"])
def test_autograd_through_public_api_3d(tp, interp):
    from oracle import port
    case = Case("ag3", 3, interp, 2, 5, 12, 24, 2.0, None, 1, 2, seed=31)
    t = make_inputs(case)
    rec = t["rec"].cuda().requires_grad_(True)
    rot = t["rot"].cuda().requires_grad_(True)
    sh = t["shifts"].cuda().requires_grad_(True)
    out = tp.project_3d_to_2d_forw(rec, rot, sh, output_shape=(case.N, case.N), interpolation=interp, oversampling=case.os)
    g = t["proj"].cuda()
    out.backward(g)
    want_out = port.project_3d_to_2d_forw(t["rec"], t["rot"], t["shifts"], [case.N, case.N], interp, case.os)
    w_rec, w_rot, w_sh = port.project_3d_to_2d_back(t["proj"], t["rec"], t["rot"], t["shifts"], interp, case.os, None, True, True)
    assert rel_err(out, want_out) <= TOL_FORWARD
    assert rel_err(rec.grad, w_rec) <= TOL_ATOMIC
    assert rel_err(rot.grad, w_rot) <= TOL_ATOMIC
    assert rel_err(sh.grad, w_sh) <= TOL_ATOMIC


@pytest.mark.parametrize("dim", [2, 3])
def test_autograd_through_public_api_backprojection(tp, dim):
    from oracle import port
    case = Case("agb", dim, "linear", 1, 6, 12, 24, 2.0, None, 1, 1, seed=32)
    t = make_inputs(case)
    proj = t["proj"].cuda().requires_grad_(True)
    w = t["weights"].cuda().requires_grad_(True)
    rot = t["rot"].cuda().requires_grad_(True)
    sh = t["shifts"].cuda().requires_grad_(True)
    f = tp.backproject_2d_to_3d_forw if dim == 3 else tp.backproject_2d_forw
    data, wrec = f(proj, rot, weights=w, shifts=sh, interpolation="linear", oversampling=case.os)
    torch.autograd.backward([data, wrec], [t["grad_data"].cuda(), t["grad_weight"].cuda()])
    fo = port.backproject_2d_to_3d_forw if dim == 3 else port.backproject_2d_forw
    bo = port.backproject_2d_to_3d_back if dim == 3 else port.backproject_2d_back
    d_want, w_want = fo(t["proj"], t["weights"], t["rot"], t["shifts"], "linear", case.os)
    gp, gw, gr, gs = bo(t["grad_data"], t["grad_weight"], t["proj"], t["weights"], t["rot"], t["shifts"], "linear", case.os, None, True, True)
    assert rel_err(data, d_want) <= TOL_ATOMIC and rel_err(wrec, w_want) <= TOL_ATOMIC
    assert rel_err(proj.grad, gp) <= TOL_ATOMIC
    assert rel_err(w.grad, gw) <= TOL_ATOMIC
    assert rel_err(rot.grad, gr) <= TOL_ATOMIC
    assert rel_err(sh.grad, gs) <= TOL_ATOMIC


def test_rank_canonicalisation_and_none_gradients(tp):
    # [P,3,3] rotations and [P,2] shifts get a batch axis; an un-batched 3D volume is rejected by
    # the public function as in the reference (torch_projectors/ops.py:153-154, 352-366)
    case = Case("canon", 3, "linear", 1, 3, 8, 8, 1.0, None, 1, 0, seed=33)
    t = make_inputs(case)
    with pytest.raises(ValueError, match="must be a 4D tensor"):
        tp.project_3d_to_2d_forw(t["rec"][0].cuda(), t["rot"][0].cuda())
    rec = t["rec"].cuda().requires_grad_(True)
    rot = t["rot"][0].cuda()
    out = tp.project_3d_to_2d_forw(rec, rot)
    assert out.shape == (1, 3, 8, 5)
    out2d = tp.project_2d_forw(t["rec"][0, 0].cuda(), torch.eye(2, device="cuda"))   # 2D API accepts un-batched input
    assert out2d.shape == (1, 1, 8, 5)
    out.abs().sum().backward()
    assert rec.grad is not None and rec.grad.shape == rec.shape
    same = tp.project_3d_to_2d_forw(t["rec"].cuda(), t["rot"].cuda(), torch.zeros(3, 2, device="cuda"))
    assert torch.allclose(same, out.detach(), atol=1e-6)       # zero shift == no shift


def test_batched_call_equals_per_item_calls_bitwise(tp):
    case = Case("batch", 3, "cubic", 3, 4, 12, 24, 2.0, None, 3, 3, seed=34)
    t = {k: (v.cuda() if v is not None else None) for k, v in make_inputs(case).items()}
    full = tp.project_3d_to_2d_forw(t["rec"], t["rot"], t["shifts"], output_shape=(12, 12), interpolation="cubic", oversampling=2.0)
    for b in range(case.B):
        one = tp.project_3d_to_2d_forw(t["rec"][b:b + 1], t["rot"][b:b + 1], t["shifts"][b:b + 1], output_shape=(12, 12),
                                       interpolation="cubic", oversampling=2.0)
        assert torch.equal(full[b:b + 1], one)
    again = tp.project_3d_to_2d_forw(t["rec"], t["rot"], t["shifts"], output_shape=(12, 12), interpolation="cubic", oversampling=2.0)
    assert torch.equal(full, again)                              # gathers are deterministic


def test_non_contiguous_and_broadcast_poses(tp):
    # expanded (stride-0) and sliced pose tensors are legal inputs
    # (reference: tests/3d/back/test_batching_back_2d_to_3d.py:274, tests/3d/forw/test_basic_projection_3d_to_2d.py:212)
    case = Case("nc", 3, "linear", 2, 4, 8, 16, 2.0, None, 1, 1, seed=35)
    t = {k: (v.cuda() if v is not None else None) for k, v in make_inputs(case).items()}
    a = tp.project_3d_to_2d_forw(t["rec"], t["rot"], t["shifts"], output_shape=(8, 8), oversampling=2.0)
    b = tp.project_3d_to_2d_forw(t["rec"], t["rot"].expand(2, -1, -1, -1), t["shifts"].expand(2, -1, -1), output_shape=(8, 8), oversampling=2.0)
    assert torch.equal(a, b)
    c = tp.project_3d_to_2d_forw(t["rec"], t["rot"][:, :1], t["shifts"][:, :1], output_shape=(8, 8), oversampling=2.0)
    assert torch.equal(a[:, :1], c)
    rec_t = t["rec"].transpose(1, 2)                              # non-contiguous volume
    d = tp.project_3d_to_2d_forw(rec_t, t["rot"], None, output_shape=(8, 8), oversampling=2.0)
    e = tp.project_3d_to_2d_forw(rec_t.contiguous(), t["rot"], None, output_shape=(8, 8), oversampling=2.0)
    assert torch.equal(d, e)


def test_empty_pose_list_and_unsupported_precision(tp):
    rec = torch.zeros(1, 8, 8, 5, dtype=torch.complex64, device="cuda")
    out = tp.project_3d_to_2d_forw(rec, torch.zeros(1, 0, 3, 3, device="cuda"))
    assert out.shape == (1, 0, 8, 5)
    data, _ = tp.backproject_2d_to_3d_forw(torch.zeros(1, 0, 8, 5, dtype=torch.complex64, device="cuda"), torch.zeros(1, 0, 3, 3, device="cuda"))
    assert data.shape == (1, 8, 8, 5) and (data == 0).all()
    with pytest.raises(RuntimeError, match="mixed precisions"):
        tp.project_3d_to_2d_forw(rec, torch.eye(3, dtype=torch.float64, device="cuda").view(1, 1, 3, 3))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        tp.project_3d_to_2d_forw(rec.to(torch.complex32), torch.eye(3, dtype=torch.float16, device="cuda").view(1, 1, 3, 3))
    with pytest.raises(RuntimeError, match="Number of poses in shifts"):
        tp.project_3d_to_2d_forw(rec, torch.eye(3, device="cuda").expand(1, 2, 3, 3), torch.zeros(1, 3, 2, device="cuda"))
    with pytest.raises(RuntimeError, match="interpolation"):
        tp.project_3d_to_2d_forw(rec, torch.eye(3, device="cuda").view(1, 1, 3, 3), interpolation="nearest")


def test_accumulate_equals_one_shot_and_sum_of_chunks(tp):
    # reference usage: chunk results are summed by the caller
    # (tests/3d/back/test_performance_back_2d_to_3d.py:348-382 there, max diff < 5e-4)
    case = Case("acc", 3, "linear", 1, 40, 16, 32, 2.0, None, 1, 1, seed=36, special_poses=False)
    t = {k: (v.cuda() if v is not None else None) for k, v in make_inputs(case).items()}
    d_all, w_all = tp.backproject_2d_to_3d_forw(t["proj"], t["rot"], weights=t["weights"], shifts=t["shifts"], oversampling=2.0)
    d_acc, w_acc = torch.zeros_like(d_all), torch.zeros_like(w_all)
    for lo in range(0, 40, 16):
        sl = slice(lo, lo + 16)
        tp.backproject_2d_to_3d_accumulate_(d_acc, w_acc, t["proj"][:, sl], t["rot"][:, sl], t["weights"][:, sl], t["shifts"][:, sl], oversampling=2.0)
    assert rel_err(d_acc, d_all) <= TOL_ATOMIC and rel_err(w_acc, w_all) <= TOL_ATOMIC
    assert (w_all >= 0).all()
    from torch_projectors_b200 import sharding
    vols = sharding.backproject_2d_to_3d_sharded(t["proj"], t["rot"], t["weights"], t["shifts"], oversampling=2.0, chunk=16)
    assert rel_err(vols.data, d_all) <= TOL_ATOMIC and rel_err(vols.weights, w_all) <= TOL_ATOMIC


@pytest.mark.parametrize("interp", ["linear", "cubic"])
def test_known_answer_identity_rotation(tp, interp):
    # reference: tests/3d/forw/test_basic_projection_3d_to_2d.py:47-94 (atol 1e-5)
    torch.manual_seed(0)
    N = 32
    rec = torch.randn(1, N, N, N // 2 + 1, dtype=torch.complex64, device="cuda")
    out = tp.project_3d_to_2d_forw(rec, torch.eye(3, device="cuda").view(1, 1, 3, 3), interpolation=interp)
    kr = torch.arange(N, device="cuda").float()
    kr = torch.where(kr <= N // 2, kr, kr - N)
    mask = (kr[:, None] ** 2 + torch.arange(N // 2 + 1, device="cuda")[None, :] ** 2) <= (N / 2) ** 2
    assert torch.allclose(out[0, 0], rec[0, 0] * mask, atol=1e-5)


# ---- the benchmark configurations at full size: subsets against the oracle + properties ----
def _cfg2_inputs(P, seed=2):
    gen = torch.Generator().manual_seed(seed)
    vol = torch.randn(128, 128, 128, generator=gen)
    pad = torch.nn.functional.pad(vol, (64, 64) * 3)
    rec = torch.fft.rfftn(torch.fft.fftshift(pad), norm="forward").to(torch.complex64).unsqueeze(0)
    rot = make_rotations(3, 1, P, gen, special=False)
    shifts = (torch.rand(1, P, 2, generator=gen) * 2 - 1) * 8.0
    return rec, rot, shifts


def test_full_size_projection_config(tp):
    """Box-256 2x-oversampled volume, 10,000 poses, 128x128 output, cubic, cutoff 64 (the headline
    projection workload at its full pose count): the first, the last and 256 random poses against
    the CPU reference, plus linearity in the volume."""
    from runners import cpu_checker
    ops, _ = cpu_checker()
    P = 10_000
    rec, rot, shifts = _cfg2_inputs(P)
    kw = dict(output_shape=(128, 128), interpolation="cubic", oversampling=2.0, fourier_radius_cutoff=64.0)
    out = tp.project_3d_to_2d_forw(rec.cuda(), rot.cuda(), shifts.cuda(), **kw)
    pick = torch.unique(torch.cat([torch.tensor([0, P - 1]), torch.randint(0, P, (256,), generator=torch.Generator().manual_seed(8))]))
    want = ops.project_3d_to_2d_forw(rec, rot[:, pick].contiguous(), shifts[:, pick].contiguous(), [128, 128], "cubic", 2.0, 64.0)
    assert rel_err(out[:, pick.cuda()], want) <= TOL_FORWARD
    # linearity in the volume on a subset of the poses: P(a*x + y) = a*P(x) + P(y)
    sub = slice(0, 512)
    rec2 = torch.roll(rec, 3, dims=1).cuda()
    lhs = tp.project_3d_to_2d_forw(2.5 * rec.cuda() + rec2, rot[:, sub].cuda(), shifts[:, sub].cuda(), **kw)
    rhs = 2.5 * out[:, sub] + tp.project_3d_to_2d_forw(rec2, rot[:, sub].cuda(), shifts[:, sub].cuda(), **kw)
    assert rel_err(lhs, rhs) <= TOL_FORWARD


def test_medium_case_directly_against_the_reference_operators(tp):
    """No restatement in between: the CUDA operators against the reference's own CPU operators
    (oracle/_ref, compiled from its sources) on a medium case, all eight operators."""
    import oracle
    if not oracle.reference_available():
        pytest.skip("oracle/_ref is not built on this machine")
    case = Case("direct_ref", 3, "cubic", 2, 12, 32, 64, 2.0, 14.0, 2, 2, shift_range=5.0, seed=31, special_poses=True)
    t = make_inputs(case)
    got = run_case("cuda", case, t)
    want = run_case("reference", case, t)
    assert set(got) == set(want)
    for key in want:
        assert rel_err(got[key], want[key]) <= tolerance_for(key), key


def test_full_size_backprojection_config(tp):
    """128x128 slices into a box-256 volume, linear, with weights (the headline
    back-projection workload): 512 slices against the CPU reference, chunk additivity, linearity."""
    from runners import cpu_checker
    ops, _ = cpu_checker()
    P = 2048
    gen = torch.Generator().manual_seed(3)
    proj = torch.complex(torch.randn(1, P, 128, 65, generator=gen), torch.randn(1, P, 128, 65, generator=gen))
    hermitian_dc_column_(proj)
    weights = torch.rand(1, P, 128, 65, generator=gen)
    rot = make_rotations(3, 1, P, gen, special=False)
    shifts = (torch.rand(1, P, 2, generator=gen) * 2 - 1) * 8.0
    c = lambda x: x.cuda()  # noqa: E731
    d_all, w_all = tp.backproject_2d_to_3d_forw(c(proj), c(rot), weights=c(weights), shifts=c(shifts), oversampling=2.0)
    assert d_all.shape == (1, 256, 256, 129) and w_all.shape == (1, 256, 256, 129)
    n = 512
    d_sub, w_sub = tp.backproject_2d_to_3d_forw(c(proj[:, :n]), c(rot[:, :n]), weights=c(weights[:, :n]), shifts=c(shifts[:, :n]), oversampling=2.0)
    d_want, w_want = ops.backproject_2d_to_3d_forw(proj[:, :n].contiguous(), weights[:, :n].contiguous(), rot[:, :n].contiguous(),
                                                   shifts[:, :n].contiguous(), "linear", 2.0, None)
    assert rel_err(d_sub, d_want) <= TOL_ATOMIC and rel_err(w_sub, w_want) <= TOL_ATOMIC
    d_rest, w_rest = tp.backproject_2d_to_3d_forw(c(proj[:, n:]), c(rot[:, n:]), weights=c(weights[:, n:]), shifts=c(shifts[:, n:]), oversampling=2.0)
    assert rel_err(d_sub + d_rest, d_all) <= TOL_ATOMIC and rel_err(w_sub + w_rest, w_all) <= TOL_ATOMIC
    d_twice, _ = tp.backproject_2d_to_3d_forw(2 * c(proj), c(rot), weights=c(weights), shifts=c(shifts), oversampling=2.0)
    assert rel_err(d_twice, 2 * d_all) <= TOL_ATOMIC


def test_autograd_step_config_reduced(tp):
    """The full-autograd-step workload (cubic, 2x oversampling, all gradients) on a reduced
    volume the oracle finishes in seconds: MSE loss against a target, all three gradients."""
    from oracle import port
    case = Case("step", 3, "cubic", 1, 16, 32, 64, 2.0, None, 1, 1, shift_range=5.0, seed=40, special_poses=False)
    t = make_inputs(case)
    rec = t["rec"].cuda().requires_grad_(True)
    rot = t["rot"].cuda().requires_grad_(True)
    sh = t["shifts"].cuda().requires_grad_(True)
    target = t["proj"].cuda()
    out = tp.project_3d_to_2d_forw(rec, rot, sh, output_shape=(32, 32), interpolation="cubic", oversampling=2.0)
    loss = ((out - target).abs() ** 2).mean()
    loss.backward()
    out_cpu = port.project_3d_to_2d_forw(t["rec"], t["rot"], t["shifts"], [32, 32], "cubic", 2.0)
    g = 2 * (out_cpu - t["proj"]) / out_cpu.numel()           # d mean|o - t|^2 / d conj(o), torch's convention
    w_rec, w_rot, w_sh = port.project_3d_to_2d_back(g, t["rec"], t["rot"], t["shifts"], "cubic", 2.0, None, True, True)
    assert rel_err(rec.grad, w_rec) <= TOL_ATOMIC
    assert rel_err(rot.grad, w_rot) <= TOL_ATOMIC
    assert rel_err(sh.grad, w_sh) <= TOL_ATOMIC


@pytest.mark.parametrize("dim,interp", [(3, "linear"), (3, "cubic"), (2, "linear"), (2, "cubic")])
def test_workspace_path_equals_direct_path_and_oracle(tp, dim, interp):
    """Back-projection through the interleaved workspace (data and weight of a voxel in one
    16-byte slot) gives the same volumes as direct reductions, with and without accumulate."""
    from oracle import port
    from torch_projectors_b200 import _abi
    case = Case("ws", dim, interp, 2, 6, 12, 24, 2.0, None, 1, 2, seed=50 + dim)
    t = {k: (v.cuda() if v is not None else None) for k, v in make_inputs(case).items()}
    code = _abi.CUBIC if interp == "cubic" else _abi.LINEAR
    R = 24
    shape = (2, R, R, R // 2 + 1) if dim == 3 else (2, R, R // 2 + 1)
    n = 2 * (R if dim == 3 else 1) * R * (R // 2 + 1)
    outs = {}
    for use_ws in (False, True):
        data = torch.full(shape, 7.0, dtype=torch.complex64, device="cuda")     # must be overwritten
        wrec = torch.full(shape, 7.0, dtype=torch.float32, device="cuda")
        ws = torch.empty(n * 16, dtype=torch.uint8, device="cuda") if use_ws else None
        _abi.backproject_forw(dim, t["proj"], t["weights"], t["rot"], t["shifts"], code, 2.0, 6.0, data, wrec, False, ws)
        _abi.backproject_forw(dim, t["proj"], t["weights"], t["rot"], t["shifts"], code, 2.0, 6.0, data, wrec, True, ws)
        outs[use_ws] = (data, wrec)
    f = port.backproject_2d_to_3d_forw if dim == 3 else port.backproject_2d_forw
    d_want, w_want = f(t["proj"].cpu(), t["weights"].cpu(), t["rot"].cpu(), t["shifts"].cpu(), interp, 2.0)
    for use_ws in (False, True):
        assert rel_err(outs[use_ws][0], 2 * d_want) <= TOL_ATOMIC
        assert rel_err(outs[use_ws][1], 2 * w_want) <= TOL_ATOMIC


def test_host_streaming_wrappers_match_device_calls(tp):
    """project_3d_to_2d_to_host / backproject_2d_to_3d_from_host (chunked, copies on a second
    stream) give what the plain device calls give."""
    case = Case("stream", 3, "linear", 1, 37, 16, 32, 2.0, None, 1, 1, seed=70, special_poses=False)
    t = make_inputs(case)
    pin = lambda x: x.pin_memory()  # noqa: E731
    out = tp.project_3d_to_2d_to_host(pin(t["rec"]), pin(t["rot"]), pin(t["shifts"]), chunk=8, output_shape=(16, 16),
                                      interpolation="linear", oversampling=2.0)
    torch.cuda.current_stream().synchronize()
    want = tp.project_3d_to_2d_forw(t["rec"].cuda(), t["rot"].cuda(), t["shifts"].cuda(), output_shape=(16, 16), oversampling=2.0)
    assert not out.is_cuda and torch.equal(out, want.cpu())
    vols = tp.backproject_2d_to_3d_from_host(pin(t["proj"]), t["rot"], pin(t["weights"]), t["shifts"], chunk=8, oversampling=2.0)
    d_want, w_want = tp.backproject_2d_to_3d_forw(t["proj"].cuda(), t["rot"].cuda(), weights=t["weights"].cuda(), shifts=t["shifts"].cuda(), oversampling=2.0)
    assert rel_err(vols.data, d_want) <= TOL_ATOMIC and rel_err(vols.weights, w_want) <= TOL_ATOMIC


@pytest.mark.parametrize("interp", ["linear", "cubic"])
def test_persistent_accumulator_matches_oracle_and_partial_volumes_use_it(tp, interp):
    from oracle import port
    case = Case("accum", 3, interp, 2, 12, 16, 32, 2.0, None, 2, 2, weights=True, seed=77)
    t = make_inputs(case)
    c = lambda x: x.cuda()  # noqa: E731
    dw, ww = port.backproject_2d_to_3d_forw(t["proj"], t["weights"], t["rot"], t["shifts"], interp, 2.0)
    acc = tp.new_backprojection_accumulator(2, 32, "cuda")
    for lo, hi in ((0, 5), (5, 12)):
        tp.backproject_2d_to_3d_accumulate_interleaved_(acc, c(t["proj"])[:, lo:hi], c(t["rot"])[:, lo:hi], c(t["weights"])[:, lo:hi],
                                                        c(t["shifts"])[:, lo:hi], interpolation=interp, oversampling=2.0)
    d, w = tp.fold_backprojection_accumulator(acc)
    assert rel_err(d, dw) <= TOL_ATOMIC and rel_err(w, ww) <= TOL_ATOMIC
    # folding again with accumulate adds the same sums once more; the accumulator is unchanged
    tp.fold_backprojection_accumulator(acc, d, w, accumulate=True)
    assert rel_err(d, 2 * dw) <= TOL_ATOMIC and rel_err(w, 2 * ww) <= TOL_ATOMIC
    assert acc[..., 3].abs().max().item() == 0.0          # the padding lane stays zero
    # PartialVolumes: chunks through the accumulator, complete after flush()
    vols = tp.sharding.PartialVolumes(2, 32, "cuda")
    for lo, hi in ((0, 7), (7, 12)):
        vols.add_(c(t["proj"])[:, lo:hi], c(t["rot"])[:, lo:hi], c(t["weights"])[:, lo:hi], c(t["shifts"])[:, lo:hi],
                  interpolation=interp, oversampling=2.0)
    assert vols._pending and vols.data.abs().max().item() == 0.0
    vols.flush()
    assert not vols._pending and rel_err(vols.data, dw) <= TOL_ATOMIC and rel_err(vols.weights, ww) <= TOL_ATOMIC
    vols.flush()                                         # nothing pending: a no-op
    assert rel_err(vols.data, dw) <= TOL_ATOMIC
    # folding range by range (as reduce() does to overlap the collective) gives the same volumes
    parts = tp.sharding.PartialVolumes(2, 32, "cuda")
    parts.add_(c(t["proj"]), c(t["rot"]), c(t["weights"]), c(t["shifts"]), interpolation=interp, oversampling=2.0)
    seen = []
    parts.flush(parts=3, after_part=lambda first, stop: seen.append((first, stop)))
    n = parts.data.numel()
    assert len(seen) == 3 and seen[0][0] == 0 and seen[-1][1] == n and all(a[1] == b[0] for a, b in zip(seen, seen[1:]))
    assert rel_err(parts.data, dw) <= TOL_ATOMIC and rel_err(parts.weights, ww) <= TOL_ATOMIC
    parts.reduce()                                       # one process: nothing pending, nothing to reduce
    assert rel_err(parts.data, dw) <= TOL_ATOMIC
    half = tp.fold_backprojection_accumulator(acc, voxel_range=(0, n // 2))[0]
    assert rel_err(half.flatten()[: n // 2], dw.flatten()[: n // 2]) <= TOL_ATOMIC
    # errors: weights are required, shapes are checked
    with pytest.raises(RuntimeError, match="needs weights"):
        tp.backproject_2d_to_3d_accumulate_interleaved_(acc, c(t["proj"]), c(t["rot"]), None, oversampling=2.0)
    with pytest.raises(RuntimeError, match="accumulator must be"):
        tp.backproject_2d_to_3d_accumulate_interleaved_(acc[:1], c(t["proj"]), c(t["rot"]), c(t["weights"]), oversampling=2.0)


_SLAB_SCRIPT = r"""
import sys, torch
sys.path[:0] = [{root!r}, {root!r} + "/tests", {root!r} + "/torch-projectors_b200"]
import torch_projectors_b200 as tp
from oracle import port
from cases import Case, make_inputs, rel_err, TOL_ATOMIC
for interp, weights in (("linear", True), ("cubic", True), ("linear", False)):
    case = Case("slab", 3, interp, 2, 9, 20, 40, 2.0, None, 1, 2, weights=weights, seed=90)
    t = make_inputs(case)
    c = lambda x: None if x is None else x.cuda()
    d, w = tp.backproject_2d_to_3d_forw(c(t["proj"]), c(t["rot"]), weights=c(t["weights"]), shifts=c(t["shifts"]),
                                        interpolation=interp, oversampling=2.0)
    dw, ww = port.backproject_2d_to_3d_forw(t["proj"], t["weights"], t["rot"], t["shifts"], interp, 2.0)
    assert rel_err(d, dw) <= TOL_ATOMIC, (interp, rel_err(d, dw))
    if weights:
        assert rel_err(w, ww) <= TOL_ATOMIC, (interp, rel_err(w, ww))
    tp.backproject_2d_to_3d_accumulate_(d, w if weights else None, c(t["proj"]), c(t["rot"]), c(t["weights"]), c(t["shifts"]),
                                        interpolation=interp, oversampling=2.0)
    assert rel_err(d, 2 * dw) <= TOL_ATOMIC
    if weights:
        # persistent interleaved accumulator: two chunks added, folded once (slabs of 16-byte voxels)
        acc = tp.new_backprojection_accumulator(2, 40, "cuda")
        for lo, hi in ((0, 4), (4, 9)):
            tp.backproject_2d_to_3d_accumulate_interleaved_(acc, c(t["proj"])[:, lo:hi], c(t["rot"])[:, lo:hi], c(t["weights"])[:, lo:hi],
                                                            c(t["shifts"])[:, lo:hi], interpolation=interp, oversampling=2.0)
        da, wa = tp.fold_backprojection_accumulator(acc)
        assert rel_err(da, dw) <= TOL_ATOMIC and rel_err(wa, ww) <= TOL_ATOMIC, (interp, rel_err(da, dw), rel_err(wa, ww))
        # slab by slab: every slab's pass alone, in reverse order, adds up to the same sums, and a pass
        # writes nothing outside the voxels it owns
        slabs, planes = tp._abi.accumulator_slab_plan(40)
        assert slabs > 4
        acc2 = tp.new_backprojection_accumulator(2, 40, "cuda")
        call = tp.ops.prepare_accumulate_interleaved(acc2, c(t["proj"]), c(t["rot"]), c(t["weights"]), c(t["shifts"]), interpolation=interp, oversampling=2.0)
        per_item = 40 * 40 * 21
        for k in reversed(range(slabs)):
            before = acc2.clone()
            tp._abi.backproject_accumulate_slabs(*call, k, 1)
            changed = (acc2 != before).any(dim=-1).flatten()
            owned = torch.zeros(2 * per_item, dtype=torch.bool, device="cuda")
            for b in range(2):
                for first, stop in tp._abi.accumulator_slab_voxels(40, k, 1):
                    owned[b * per_item + first: b * per_item + stop] = True
            assert not (changed & ~owned).any(), (interp, k)
        assert rel_err(acc2, acc) <= TOL_ATOMIC, (interp, rel_err(acc2, acc))
        # and PartialVolumes with the last chunk as the final stage (fold of finished slab groups on a second stream)
        vols = tp.sharding.PartialVolumes(2, 40, "cuda")
        vols.slab_groups = 5
        vols.add_(c(t["proj"])[:, :4], c(t["rot"])[:, :4], c(t["weights"])[:, :4], c(t["shifts"])[:, :4], interpolation=interp, oversampling=2.0)
        vols.add_(c(t["proj"])[:, 4:], c(t["rot"])[:, 4:], c(t["weights"])[:, 4:], c(t["shifts"])[:, 4:], interpolation=interp, oversampling=2.0, final=True)
        vols.flush()
        torch.cuda.synchronize()
        assert rel_err(vols.data, dw) <= TOL_ATOMIC and rel_err(vols.weights, ww) <= TOL_ATOMIC, (interp, rel_err(vols.data, dw))
print("SLAB-OK")
"""


def test_slab_ordered_backprojection_matches_oracle(tp):
    """The slab-ordered kernel (used for volumes larger than L2) forced onto a small case in a
    fresh process: 40 planes in slabs of 3, every tap written by exactly one slab pass."""
    import os
    import subprocess
    import sys
    root = str(Path(__file__).resolve().parent.parent)
    plane_mb = 40 * 21 * 12 / 1e6
    env = dict(os.environ, B200PROJ_SLAB_MIN_MB="0", B200PROJ_SLAB_MB=str(3.5 * plane_mb))
    r = subprocess.run([sys.executable, "-c", _SLAB_SCRIPT.format(root=root)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "SLAB-OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]



@pytest.mark.parametrize("interp", ["linear", "cubic"])
@pytest.mark.parametrize("geom", [(12, 24, 2.0, 3.0), (16, 24, 1.5, 6.7), (34, 34, 1.0, 2.0), (10, 30, 3.0, None)], ids=str)
def test_all_3d_operators_on_lattice_poses(tp, geom, interp):
    """The 24 axis-aligned rotations, exact and turned by 1e-6 .. 1e-3 rad: every sample on or a hair
    off a voxel, zero-weight taps, taps on the volume's edge planes and on the Friedel column, for all
    eight outputs of the four 3D operators against the oracle."""
    from cases import axis_aligned_rotations
    N, R, os_, cut = geom
    special = axis_aligned_rotations(torch.Generator().manual_seed(N))
    case = Case("lattice", 3, interp, 2, special.shape[0] + 4, N, R, os_, cut, 1, 1, weights=True, seed=2000 + N, shift_range=3.0)
    t = make_inputs(case)
    t["rot"][0, : special.shape[0]] = special
    got = run_case("cuda", case, t)
    want = run_case("port", case, t)
    assert set(got) == set(want)
    for k in want:
        assert rel_err(got[k], want[k]) <= (TOL_FORWARD if k == "fwd" else TOL_ATOMIC), (k, rel_err(got[k], want[k]))


@pytest.mark.parametrize("interp", ["linear", "cubic"])
@pytest.mark.parametrize("geom", [(12, 24, 2.0, 3.0), (16, 24, 1.5, 6.7), (34, 34, 1.0, None)], ids=str)
def test_all_2d_operators_on_lattice_poses(tp, geom, interp):
    """Quarter turns, exact and off by +-1e-6 .. 1e-3 rad, for the four 2D operators."""
    import math
    N, R, os_, cut = geom
    angles = [q * math.pi / 2 + d for q in range(4) for d in (0.0, 1e-6, -1e-5, 1e-4, -1e-3)]
    special = torch.tensor([[[round(math.cos(a), 15), -round(math.sin(a), 15)], [round(math.sin(a), 15), round(math.cos(a), 15)]] for a in angles],
                           dtype=torch.float64).float()
    case = Case("lattice2d", 2, interp, 2, special.shape[0] + 4, N, R, os_, cut, 1, 1, weights=True, seed=2100 + N, shift_range=3.0)
    t = make_inputs(case)
    t["rot"][0, : special.shape[0]] = special
    got = run_case("cuda", case, t)
    want = run_case("port", case, t)
    assert set(got) == set(want)
    for k in want:
        assert rel_err(got[k], want[k]) <= (TOL_FORWARD if k == "fwd" else TOL_ATOMIC), (k, rel_err(got[k], want[k]))


_SLAB_LATTICE_SCRIPT = r"""
import sys, math, torch
sys.path[:0] = [{root!r}, {root!r} + "/tests", {root!r} + "/torch-projectors_b200"]
import torch_projectors_b200 as tp
from oracle import port
from cases import Case, make_inputs, rel_err, TOL_ATOMIC, axis_aligned_rotations
gen = torch.Generator().manual_seed(7)
worst = 0.0
for k, (N, os_, cut, interp, B) in enumerate([(8, 1.0, None, "linear", 1), (12, 2.0, 3.0, "cubic", 2), (16, 1.5, 6.7, "linear", 2),
                                              (20, 3.0, None, "cubic", 1), (26, 2.0, 11.7, "linear", 1), (34, 1.0, 2.0, "cubic", 1)]):
    special = axis_aligned_rotations(gen)
    P = special.shape[0] + 6
    case = Case("lattice", 3, interp, B, P, N, N, os_, cut, 1, 1, weights=True, seed=700 + k)
    t = make_inputs(case)
    t["rot"][0, : special.shape[0]] = special
    c = lambda x: None if x is None else x.cuda()
    raw = math.ceil(N * os_)
    R = raw + raw % 2
    dw, ww = port.backproject_2d_to_3d_forw(t["proj"], t["weights"], t["rot"], t["shifts"], interp, os_, cut)
    d, w = tp.backproject_2d_to_3d_forw(c(t["proj"]), c(t["rot"]), weights=c(t["weights"]), shifts=c(t["shifts"]),
                                        interpolation=interp, oversampling=os_, fourier_radius_cutoff=cut)
    acc = tp.new_backprojection_accumulator(B, R, "cuda")
    tp.backproject_2d_to_3d_accumulate_interleaved_(acc, c(t["proj"]), c(t["rot"]), c(t["weights"]), c(t["shifts"]),
                                                    interpolation=interp, oversampling=os_, fourier_radius_cutoff=cut)
    da, wa = tp.fold_backprojection_accumulator(acc)
    assert tp._abi.accumulator_slab_plan(R) == (R, 1), tp._abi.accumulator_slab_plan(R)
    errs = [rel_err(d, dw), rel_err(w, ww), rel_err(da, dw), rel_err(wa, ww)]
    assert max(errs) <= TOL_ATOMIC, (N, os_, cut, interp, errs)
    worst = max(worst, max(errs))
print("LATTICE-OK", worst)
"""


def test_slab_ordered_backprojection_with_one_plane_slabs_and_lattice_poses(tp):
    """The hardest inputs for the slab-ordered kernel's search: slabs of a single plane (every
    footprint straddles slabs) and the 24 axis-aligned rotations, exact and turned by 1e-6 .. 1e-3 rad
    (whole rows and columns of a slice lie in one plane, samples on or a hair off the lattice, the
    linear estimates of the search have zero slopes), over six geometries; both the plain entry point
    and the interleaved accumulator against the oracle."""
    import os
    import subprocess
    import sys
    root = str(Path(__file__).resolve().parent.parent)
    env = dict(os.environ, B200PROJ_SLAB_MIN_MB="0", B200PROJ_SLAB_MIN_MB_EAGER="0", B200PROJ_SLAB_MB="0.00001")
    r = subprocess.run([sys.executable, "-c", _SLAB_LATTICE_SCRIPT.format(root=root)], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "LATTICE-OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


# ---- complex128 / float64: the same kernels instantiated for double ---------------------------
F64_TOL = 1e-11      # against the fp64 oracle; sums are re-associated, reductions unordered


@pytest.mark.parametrize("case", SMALL_CASES[:6] + SMALL_CASES[9:13] + MEDIUM_CASES[3:5], ids=lambda c: c.name)
def test_double_precision_matches_fp64_oracle(tp, case):
    t = make_inputs(case, cdtype=torch.complex128)
    got = run_case("cuda", case, t)
    want = run_case("port", case, t)
    assert set(got) == set(want)
    for k in want:
        assert got[k].dtype == want[k].dtype, (k, got[k].dtype, want[k].dtype)
        assert rel_err(got[k], want[k]) <= F64_TOL, (k, rel_err(got[k], want[k]))


@pytest.mark.parametrize("interp", ["linear", "cubic"])
def test_gradcheck_projection_in_double_precision(tp, interp):
    # reference: tests/3d/forw/test_gradients_3d_to_2d.py:67-110 -- gradcheck in complex128 with the
    # Friedel-redundant half of the c = 0 line masked (forward reads it, backward does not write it)
    torch.manual_seed(42)
    N = 8
    rec = torch.randn(1, N, N, N // 2 + 1, dtype=torch.complex128, device="cuda", requires_grad=True)
    gen = torch.Generator().manual_seed(1)
    rot = make_rotations(3, 1, 2, gen, special=True, dtype=torch.float64).cuda()
    mask = torch.ones_like(rec)
    mask[0, :, N // 2:, 0] = 0

    def func(r):
        return tp.project_3d_to_2d_forw(r * mask, rot[:, :1], output_shape=(N, N), interpolation=interp)
    assert torch.autograd.gradcheck(func, rec, atol=1e-4, rtol=1e-2)


@pytest.mark.parametrize("interp", ["linear", "cubic"])
def test_gradcheck_backprojection_in_double_precision(tp, interp):
    # reference: tests/3d/back/test_gradients_back_2d_to_3d.py:69-110 -- projections only, identity
    # pose; the column-0 pixels with a distinct Friedel partner are masked, because the forward
    # pass inserts them twice (x = 0 duplicate) while the backward pass reads them once
    torch.manual_seed(42)
    N = 8
    proj = torch.randn(1, 1, N, N // 2 + 1, dtype=torch.complex128, device="cuda", requires_grad=True)
    rot = torch.eye(3, dtype=torch.float64, device="cuda").view(1, 1, 3, 3)
    sh = torch.tensor([[[0.5, -1.25]]], dtype=torch.float64, device="cuda")
    mask = torch.ones_like(proj)
    mask[0, 0, 1:N // 2, 0] = 0

    def func(p):
        return tp.backproject_2d_to_3d_forw(p * mask, rot, shifts=sh, interpolation=interp)[0]
    assert torch.autograd.gradcheck(func, proj, atol=1e-4, rtol=1e-2)


def test_operators_can_be_captured_in_a_cuda_graph(tp):
    """The entry points never synchronise or allocate, so a launch-bound loop of small calls can
    be captured once and replayed: forward projection and back-projection of the small 2D case,
    replayed on new input values, equal the eager results."""
    gen = torch.Generator().manual_seed(9)
    N, R, P = 64, 128, 256
    rec = torch.randn(1, R, R // 2 + 1, dtype=torch.complex64, generator=gen).cuda()
    rot = make_rotations(2, 1, P, gen, special=False).cuda()
    sh = ((torch.rand(1, P, 2, generator=gen) * 2 - 1) * 4).cuda()
    wts = torch.rand(1, P, N, N // 2 + 1, generator=gen).cuda()
    kw = dict(interpolation="linear", oversampling=2.0)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):                      # warm-up outside the capture (library load, allocator)
        for _ in range(2):
            out = tp.project_2d_forw(rec, rot, sh, output_shape=(N, N), **kw)
            tp.backproject_2d_forw(out, rot, weights=wts, shifts=sh, **kw)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        g_out = tp.project_2d_forw(rec, rot, sh, output_shape=(N, N), **kw)
        g_data, g_w = tp.backproject_2d_forw(g_out, rot, weights=wts, shifts=sh, **kw)
    for seed in (1, 2):
        rec.copy_(torch.randn(1, R, R // 2 + 1, dtype=torch.complex64, generator=torch.Generator().manual_seed(seed)))
        graph.replay()
        torch.cuda.synchronize()
        want = tp.project_2d_forw(rec, rot, sh, output_shape=(N, N), **kw)
        want_d, want_w = tp.backproject_2d_forw(want, rot, weights=wts, shifts=sh, **kw)
        assert torch.equal(g_out, want)
        assert rel_err(g_data, want_d) <= TOL_ATOMIC and rel_err(g_w, want_w) <= TOL_ATOMIC


@pytest.mark.parametrize("k", range(48))
def test_randomised_configurations_match_the_oracle(tp, k):
    case = random_case(k)
    t = make_inputs(case)
    _compare(run_case("cuda", case, t), run_case("port", case, t))


@pytest.mark.parametrize("k", range(0, 48, 3))
def test_randomised_configurations_in_double_precision(tp, k):
    case = random_case(k)
    t = make_inputs(case, cdtype=torch.complex128)
    got = run_case("cuda", case, t)
    want = run_case("port", case, t)
    assert set(got) == set(want)
    for key in want:
        assert got[key].dtype == want[key].dtype and got[key].shape == want[key].shape, key
        assert rel_err(got[key], want[key]) <= F64_TOL, (case, key, rel_err(got[key], want[key]))


def test_calls_from_several_threads_on_their_own_streams(tp):
    """The library keeps no shared mutable state between calls (its error text is per thread):
    four host threads, each on its own stream, run forward and backward passes at once and get
    the single-threaded results."""
    import threading
    case = Case("threads", 3, "cubic", 1, 12, 16, 32, 2.0, None, 1, 1, seed=61)
    t = {k: (v.cuda() if v is not None else None) for k, v in make_inputs(case).items()}
    ops = torch.ops.torch_projectors_b200

    def work():
        rot = t["rot"].clone().requires_grad_(True)
        sh = t["shifts"].clone().requires_grad_(True)
        fwd = ops.project_3d_to_2d_forw(t["rec"], rot, sh, [16, 16], "cubic", 2.0, None)
        back = ops.project_3d_to_2d_back(t["proj"], t["rec"], rot, sh, "cubic", 2.0, None)
        bp = ops.backproject_2d_to_3d_forw(t["proj"], t["weights"], rot, sh, "cubic", 2.0, None)
        return [fwd, *back, *bp]

    want = work()
    torch.cuda.synchronize()
    results, errors = {}, []

    def runner(i):
        try:
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.default_stream())
            with torch.cuda.stream(stream):
                for _ in range(5):
                    out = work()
                stream.synchronize()
            results[i] = out
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    threads = [threading.Thread(target=runner, args=(i,)) for i in range(4)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not errors, errors
    for i in range(4):
        assert torch.equal(results[i][0], want[0])                       # gathers are deterministic
        for got, ref in zip(results[i][1:], want[1:]):
            assert rel_err(got, ref) <= TOL_ATOMIC * 0.1
