"""Additions around the operators: packed projections (only the pixels inside the cutoff), the
weighted-average reconstruction straight from the accumulator, and the reduction-rate probe."""
import pytest
import torch

from cases import Case, TOL_ATOMIC, make_inputs, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tp(cuda_device):
    import torch_projectors_b200
    return torch_projectors_b200


@pytest.mark.parametrize("interp,cutoff", [("cubic", None), ("linear", 5.5), ("cubic", 100.0)])
def test_packed_projection_holds_exactly_the_pixels_inside_the_cutoff(tp, interp, cutoff):
    case = Case("packed", 3, interp, 2, 9, 16, 32, 2.0, cutoff, 2, 2, shift_range=3.0, seed=81)
    t = {k: (v.cuda() if v is not None else None) for k, v in make_inputs(case).items()}
    kw = dict(output_shape=(16, 16), interpolation=interp, oversampling=2.0, fourier_radius_cutoff=cutoff)
    dense = tp.project_3d_to_2d_forw(t["rec"], t["rot"], t["shifts"], **kw)
    packed, index = tp.project_3d_to_2d_forw_packed(t["rec"], t["rot"], t["shifts"], **kw)
    # the table marks what the dense kernel leaves non-zero-able: kr^2 + kc^2 <= cutoff^2
    kr = torch.where(torch.arange(16) <= 8, torch.arange(16), torch.arange(16) - 16).float()[:, None]
    kc = torch.arange(9).float()[None, :]
    inside = (kr * kr + kc * kc <= (cutoff if cutoff is not None else 8.0) ** 2).flatten()
    assert torch.equal(index.cpu() >= 0, inside) and packed.shape == (2, 9, int(inside.sum()))
    assert torch.equal(index.cpu()[inside], torch.arange(int(inside.sum()), dtype=torch.int32))
    assert torch.equal(tp.unpack_projections(packed, index, 16), dense)          # bit for bit
    assert dense.flatten(2)[:, :, ~inside.cuda()].abs().max().item() == 0.0 if (~inside).any() else True


def test_packed_host_streaming_matches_the_dense_call(tp):
    case = Case("packed_host", 3, "linear", 1, 37, 16, 32, 2.0, None, 1, 1, seed=82, special_poses=False)
    t = make_inputs(case)
    pin = lambda x: x.pin_memory()  # noqa: E731
    out, index = tp.project_3d_to_2d_to_host(pin(t["rec"]), pin(t["rot"]), pin(t["shifts"]), chunk=8, output_shape=(16, 16),
                                             interpolation="linear", oversampling=2.0, packed=True)
    torch.cuda.current_stream().synchronize()
    want = tp.project_3d_to_2d_forw(t["rec"].cuda(), t["rot"].cuda(), t["shifts"].cuda(), output_shape=(16, 16), oversampling=2.0)
    assert not out.is_cuda and not index.is_cuda and out.shape[-1] == int((index >= 0).sum())
    assert torch.equal(tp.unpack_projections(out, index, 16), want.cpu())


def test_normalized_fold_equals_fold_then_divide(tp):
    from oracle import port
    case = Case("norm", 3, "linear", 2, 12, 16, 32, 2.0, None, 2, 2, weights=True, seed=83)
    t = make_inputs(case)
    c = lambda x: x.cuda()  # noqa: E731
    acc = tp.new_backprojection_accumulator(2, 32, "cuda")
    tp.backproject_2d_to_3d_accumulate_interleaved_(acc, c(t["proj"]), c(t["rot"]), c(t["weights"]), c(t["shifts"]), oversampling=2.0)
    got = tp.fold_backprojection_accumulator_normalized(acc, eps=1e-2)
    d, w = tp.fold_backprojection_accumulator(acc)
    assert rel_err(got, tp.prep.normalize_by_weights(d, w, eps=1e-2)) <= 1e-6
    dw, ww = port.backproject_2d_to_3d_forw(t["proj"], t["weights"], t["rot"], t["shifts"], "linear", 2.0)
    assert rel_err(got, dw / torch.clamp(ww, min=1e-2)) <= TOL_ATOMIC
    with pytest.raises(RuntimeError, match="eps must be positive"):
        tp.fold_backprojection_accumulator_normalized(acc, eps=0.0)


@pytest.mark.parametrize("pattern,per_tap", [(0, 3.0), (1, 3.0), (2, 3.0), (3, 2.0), (4, 2.0), (5, 2.0)])
def test_reduction_rate_probe_issues_every_reduction(tp, pattern, per_tap):
    buf = torch.zeros(1 << 18, dtype=torch.float32, device="cuda")           # 1 MiB
    tp._abi.reduction_rate_probe(pattern, buf, blocks=8, iterations=5)
    torch.cuda.synchronize()
    assert buf.double().sum().item() == 8 * 256 * 5 * per_tap                 # every lane added 1.0 to 3 (v4) or 2 (v2) floats
    with pytest.raises(RuntimeError, match="pattern must be"):
        tp._abi.reduction_rate_probe(9, buf, blocks=1, iterations=1)


@pytest.mark.parametrize("evict_last", [False, True])
def test_streaming_reduction_rate_probe_issues_every_reduction_inside_its_windows(tp, evict_last):
    target = torch.zeros(1 << 18, dtype=torch.float32, device="cuda")         # 1 MiB = 4 windows of 256 KiB
    source = torch.full((1 << 16,), 0.5, dtype=torch.float32, device="cuda")
    tp._abi.reduction_rate_probe_streaming(target, 1 << 18, source, blocks=8, iterations=6, evict_last=evict_last)
    torch.cuda.synchronize()
    slots = target.view(-1, 4).double()
    taps = 8 * 256 * 6
    assert slots[:, 0].sum().item() == taps and slots[:, 3].sum().item() == 0
    assert slots[:, 1].sum().item() == 1.5 * taps == slots[:, 2].sum().item()   # 1 + the streamed 0.5
    per_window = slots[:, 0].view(4, -1).sum(dim=1)
    assert per_window.tolist() == [taps / 4] * 4                               # blocks 2k, 2k+1 work in window k
    with pytest.raises(RuntimeError, match="out of range"):
        tp._abi.reduction_rate_probe_streaming(target, 1 << 21, source, blocks=1, iterations=1)


@pytest.mark.parametrize("interp,fixed_volume", [("cubic", False), ("cubic", True), ("linear", True)])
@pytest.mark.parametrize("with_shifts", [True, False])
@pytest.mark.parametrize("dim,os_", [(3, 2.0), (3, 1.0), (2, 2.0), (2, 1.0)])
def test_saved_derivatives_give_the_gradients_of_the_plain_backward(tp, interp, fixed_volume, with_shifts, dim, os_):
    """With rotation gradients wanted, the forward pass keeps its pixels' derivatives and the backward
    pass gathers nothing (and skips the volume's gradient when the volume is fixed).  Outputs and all
    gradients must equal those of the plain pair of operators (set_save_derivatives(False)) to
    rounding, and the CPU oracle within the gradient tolerance."""
    from oracle import port
    case = Case("saved", dim, interp, 2, 7, 16, 32, os_, 6.5, 1, 2 if with_shifts else 0, shift_range=3.0, seed=91)
    t = make_inputs(case)
    kw = dict(output_shape=(16, 16), interpolation=interp, oversampling=os_, fourier_radius_cutoff=6.5)
    project = tp.project_3d_to_2d_forw if dim == 3 else tp.project_2d_forw
    g = t["proj"].cuda()
    results = {}
    for saving in (True, False):
        tp.set_save_derivatives(saving, min_volume_bytes=0)           # the small test volumes are below the default limit
        try:
            rec = t["rec"].cuda().requires_grad_(not fixed_volume)
            rot = t["rot"].cuda().requires_grad_(True)
            sh = t["shifts"].cuda().requires_grad_(True) if with_shifts else None
            out = project(rec, rot, sh, **kw)
            assert (len(out.grad_fn.saved_tensors) == 5) == saving
            torch.view_as_real(out).backward(torch.view_as_real(g))
            results[saving] = (out.detach(), rec.grad, rot.grad, sh.grad if with_shifts else None)
        finally:
            tp.set_save_derivatives(True)
    for a, b in zip(results[True], results[False]):
        assert (a is None) == (b is None)
        if a is not None:
            assert rel_err(a, b) <= 2e-6, rel_err(a, b)
    assert (results[True][1] is None) == fixed_volume
    back = port.project_3d_to_2d_back if dim == 3 else port.project_2d_back
    want = back(t["proj"], t["rec"], t["rot"], t["shifts"] if with_shifts else None, interp, os_, 6.5,
                need_rot_grad=True, need_shift_grad=with_shifts)
    if not fixed_volume:
        assert rel_err(results[True][1], want[0]) <= TOL_ATOMIC
    assert rel_err(results[True][2], want[1]) <= TOL_ATOMIC
    if with_shifts:
        assert rel_err(results[True][3], want[2]) <= TOL_ATOMIC


@pytest.mark.parametrize("dim", [2, 3])
@pytest.mark.parametrize("interp", ["linear", "cubic"])
@pytest.mark.parametrize("fixed_volume", [True, False])
def test_shift_gradients_alone_need_only_the_saved_projections(tp, dim, interp, fixed_volume):
    """Fixed rotations, shifts to be optimised (with or without the reconstruction): the shift gradients
    come from the gradient and the projections the forward pass made; no derivatives are kept and the
    backward pass gathers nothing."""
    from oracle import port
    case = Case("shiftonly", dim, interp, 2, 6, 16, 32, 2.0, None, 1, 2, shift_range=3.0, seed=94)
    t = make_inputs(case)
    project = tp.project_3d_to_2d_forw if dim == 3 else tp.project_2d_forw
    kw = dict(output_shape=(16, 16), interpolation=interp, oversampling=2.0)
    grads = {}
    for saving in (True, False):
        tp.set_save_derivatives(saving)
        try:
            sh = t["shifts"].cuda().requires_grad_(True)
            rec = t["rec"].cuda().requires_grad_(not fixed_volume)
            out = project(rec, t["rot"].cuda(), sh, **kw)
            kept = out.grad_fn.saved_tensors
            assert len(kept) == (5 if saving else 3) and (not saving or kept[4].numel() == 0)
            torch.view_as_real(out).backward(torch.view_as_real(t["proj"].cuda()))
            grads[saving] = (sh.grad, rec.grad)
        finally:
            tp.set_save_derivatives(True)
    assert rel_err(grads[True][0], grads[False][0]) <= 2e-6
    back = port.project_3d_to_2d_back if dim == 3 else port.project_2d_back
    want = back(t["proj"], t["rec"], t["rot"], t["shifts"], interp, 2.0, None, need_rot_grad=False, need_shift_grad=True)
    assert rel_err(grads[True][0], want[2]) <= TOL_ATOMIC
    assert (grads[True][1] is None) == fixed_volume
    if not fixed_volume:
        assert rel_err(grads[True][1], grads[False][1]) <= 2e-6 and rel_err(grads[True][1], want[0]) <= TOL_ATOMIC


def test_saved_derivatives_are_not_kept_for_small_reconstructions_that_need_a_gradient(tp):
    """Onto a small reconstruction the backward scatter is bound by contention either way, so the plain
    pair stays unless the reconstruction is fixed."""
    case = Case("saved3", 2, "cubic", 1, 8, 16, 32, 2.0, None, 1, 1, seed=93)
    t = make_inputs(case)
    rot = t["rot"].cuda().requires_grad_(True)
    for needs_grad, kept in ((True, 3), (False, 5)):
        out = tp.project_2d_forw(t["rec"].cuda().requires_grad_(needs_grad), rot, t["shifts"].cuda(), output_shape=(16, 16),
                                 interpolation="cubic", oversampling=2.0)
        assert len(out.grad_fn.saved_tensors) == kept


def test_saved_derivatives_respect_the_size_limit_and_the_pose_order(tp):
    case = Case("saved2", 3, "cubic", 1, 80, 16, 32, 2.0, None, 1, 1, shift_range=3.0, seed=92)
    t = make_inputs(case)
    kw = dict(output_shape=(16, 16), interpolation="cubic", oversampling=2.0)
    rec = t["rec"].cuda().requires_grad_(True)
    rot = t["rot"].cuda().requires_grad_(True)
    sh = t["shifts"].cuda().requires_grad_(True)
    tp.set_save_derivatives(True, max_bytes=1000, min_volume_bytes=0)   # too small for 80 x 16 x 9 pixels
    try:
        out = tp.project_3d_to_2d_forw(rec, rot, sh, **kw)
        assert len(out.grad_fn.saved_tensors) == 3
    finally:
        tp.set_save_derivatives(True)
    order = tp.plane_locality_order(rot.detach())
    grads = []
    tp.set_save_derivatives(True, min_volume_bytes=0)
    for po in (order, False):
        for x in (rec, rot, sh):
            x.grad = None
        out = tp.project_3d_to_2d_forw(rec, rot, sh, pose_order=po, **kw)
        assert len(out.grad_fn.saved_tensors) == 5
        torch.view_as_real(out).backward(torch.view_as_real(t["proj"].cuda()))
        grads.append((out.detach().clone(), rec.grad.clone(), rot.grad.clone(), sh.grad.clone()))
    tp.set_save_derivatives(True)
    assert torch.equal(grads[0][0], grads[1][0])                        # the order changes no output
    for a, b in zip(grads[0][1:], grads[1][1:]):
        assert rel_err(a, b) <= 2e-6


_ROWS_SCRIPT = r"""
import sys, torch
sys.path[:0] = [{root!r}, {root!r} + "/tests", {root!r} + "/torch-projectors_b200"]
import torch_projectors_b200 as tp
from cases import Case, make_inputs
out = {{}}
for k, (dim, B, P, N, R, os_, cutoff) in enumerate([(3, 1, 7, 34, 70, 2.0, None), (3, 2, 5, 16, 16, 1.0, 6.5), (2, 1, 9, 64, 128, 2.0, None),
                                                     (2, 3, 4, 12, 12, 1.0, 4.5), (3, 1, 3, 48, 72, 1.5, None)]):
    case = Case(f"rows{{k}}", dim, "linear", B, P, N, R, os_, cutoff, B, B, shift_range=3.0, seed=300 + k)
    t = make_inputs(case)
    f = tp.project_3d_to_2d_forw if dim == 3 else tp.project_2d_forw
    out[k] = f(t["rec"].cuda(), t["rot"].cuda(), t["shifts"].cuda(), output_shape=(N, N), interpolation="linear",
               oversampling=os_, fourier_radius_cutoff=cutoff).cpu()
torch.save(out, {path!r})
"""


def test_two_pixels_per_lane_forward_kernel_is_bit_identical_to_the_one_pixel_kernel(tp, tmp_path):
    """Linear forward projection runs a kernel in which every lane handles two pixels of one column
    (terms that do not depend on the row are formed once).  Its arithmetic per pixel is unchanged, so
    its outputs must equal, bit for bit, those of the one-pixel kernel (selected in a fresh process)."""
    import os
    import subprocess
    import sys
    from pathlib import Path
    root = str(Path(__file__).resolve().parent.parent)
    results = {}
    for flag in ("1", "0"):
        path = str(tmp_path / f"rows{flag}.pt")
        env = dict(os.environ, B200PROJ_LINEAR_ROWS2=flag)
        r = subprocess.run([sys.executable, "-c", _ROWS_SCRIPT.format(root=root, path=path)], env=env, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
        results[flag] = torch.load(path)
    assert results["1"].keys() == results["0"].keys()
    for k in results["1"]:
        assert torch.equal(results["1"][k], results["0"][k]), k


def test_raw_operators_pass_opcheck_schema_and_fake_tensor(tp):
    """torch.library.opcheck on the compiled operators: the schemas tell the truth about aliasing and
    mutation, and the Meta implementations agree with the CUDA ones on shapes, dtypes and strides (what
    tracing relies on).  The operators have no autograd registration (autograd lives in the Python
    functions, as in the reference), so the autograd-related checks are not asked for."""
    ops = torch.ops.torch_projectors_b200
    case = Case("opcheck", 3, "cubic", 2, 5, 8, 16, 2.0, None, 1, 2, seed=91)
    t = {k: (v.cuda() if v is not None else None) for k, v in make_inputs(case).items()}
    rot_g = t["rot"].clone().requires_grad_(True)
    which = ("test_schema", "test_faketensor")
    torch.library.opcheck(ops.project_3d_to_2d_forw.default, (t["rec"], t["rot"], t["shifts"], [8, 8], "cubic", 2.0, None), test_utils=which)
    torch.library.opcheck(ops.project_3d_to_2d_back.default, (t["proj"], t["rec"], rot_g, t["shifts"], "cubic", 2.0, None), test_utils=which)
    torch.library.opcheck(ops.backproject_2d_to_3d_forw.default, (t["proj"], t["weights"], t["rot"], t["shifts"], "linear", 2.0, None), test_utils=which)
    torch.library.opcheck(ops.backproject_2d_to_3d_back.default,
                          (t["grad_data"], t["grad_weight"], t["proj"], t["weights"], rot_g, t["shifts"], "linear", 2.0, None), test_utils=which)
    # the forward projection that keeps its pixels' derivatives, and the backward pass from them
    torch.library.opcheck(ops.project_3d_to_2d_forw_saving.default, (t["rec"], t["rot"], t["shifts"], [8, 8], "cubic", 2.0, None, None), test_utils=which)
    out, der = ops.project_3d_to_2d_forw_saving(t["rec"], t["rot"], t["shifts"], [8, 8], "cubic", 2.0, None, None)
    der = torch.where(torch.isfinite(torch.view_as_real(der)).all(-1), der, torch.zeros_like(der))     # pixels outside the cutoff are not written
    for need_rec in (True, False):
        torch.library.opcheck(ops.project_3d_to_2d_back_saved.default,
                              (t["proj"], out, der, t["rec"], rot_g, t["shifts"], "cubic", 2.0, None, None, need_rec), test_utils=which)
    case2 = Case("opcheck2", 2, "linear", 1, 4, 8, 16, 2.0, None, 1, 0, weights=False, seed=92)
    t2 = {k: (v.cuda() if v is not None else None) for k, v in make_inputs(case2).items()}
    torch.library.opcheck(ops.project_2d_forw.default, (t2["rec"], t2["rot"], None, [8, 8], "linear", 2.0, 3.5), test_utils=which)
    torch.library.opcheck(ops.backproject_2d_forw.default, (t2["proj"], None, t2["rot"], None, "linear", 2.0, None), test_utils=which)
    torch.library.opcheck(ops.project_2d_forw_saving.default, (t2["rec"], t2["rot"], None, [8, 8], "linear", 2.0, 3.5), test_utils=which)


@pytest.mark.parametrize("B,P", [(1, 40_000), (2, 33_000)])
@pytest.mark.parametrize("interp", ["linear", "cubic"])
def test_pose_counts_beyond_one_grid_row(tp, B, P, interp):
    """More than 32,768 poses per call: the slice index is then spread over two grid dimensions
    (one batch item) or recovered by a division (several batch items).  All four operator families
    against the oracle on tiny slices, including the last poses."""
    from runners import run_case, tolerance_for
    case = Case("manyposes", 3, interp, B, P, 4, 8, 2.0, None, B, B, shift_range=1.0, seed=95, special_poses=False)
    t = make_inputs(case)
    got = run_case("cuda", case, t)
    want = run_case("port", case, t)
    # Tens of thousands of slices summed into an 8^3 volume: a sequential fp32 sum (the CPU oracle) drops
    # addends below half an ulp of the running total, so the accumulated volumes are judged against the
    # double-precision oracle on the same inputs (the CUDA sums, spread over lanes and copies, lose less).
    exact = run_case("port", case, {k: (v.to(torch.complex128 if v.is_complex() else torch.float64) if v is not None else None)
                                    for k, v in t.items()}, which=("pb", "bp"))
    for key in want:
        ref = exact[key].to(want[key].dtype) if key in ("bp_data", "bp_weight", "pb_grad_rec") else want[key]
        assert rel_err(got[key], ref) <= tolerance_for(key), key
        # and the tail of the pose-major tensors on its own (a wrong decoding would leave it unwritten or misplaced)
        if got[key].dim() >= 2 and got[key].shape[1] == P:
            assert rel_err(got[key][:, -500:], want[key][:, -500:]) <= tolerance_for(key), key


def test_raw_operator_traces_under_torch_compile(tp):
    """A function around a raw operator is captured as ONE graph (no graph break at the operator:
    its Meta implementation supplies the shapes) and gives the eager result.  The aot_eager backend
    keeps the test independent of code generation for complex tensors."""
    ops = torch.ops.torch_projectors_b200
    case = Case("compile", 3, "linear", 1, 6, 8, 16, 2.0, None, 1, 1, seed=93)
    t = {k: (v.cuda() if v is not None else None) for k, v in make_inputs(case).items()}

    def f(rec, rot, shifts):
        return ops.project_3d_to_2d_forw(rec * 2.0, rot, shifts, [8, 8], "linear", 2.0, None)

    compiled = torch.compile(f, backend="aot_eager", fullgraph=True)
    with torch.no_grad():
        got = compiled(t["rec"], t["rot"], t["shifts"])
        want = f(t["rec"], t["rot"], t["shifts"])
    assert torch.equal(got, want)


@pytest.mark.parametrize("dim,interp,B,P", [(2, "linear", 1, 600), (2, "cubic", 2, 150), (3, "linear", 1, 300), (3, "cubic", 2, 140)])
def test_small_reconstructions_spread_over_workspace_copies(tp, dim, interp, B, P):
    """Reductions onto a reconstruction of less than ~2 MB run at about half rate, so a weighted
    back-projection of many slices onto a small reconstruction spreads the slices over several
    copies of it in the workspace and adds the copies up in the fold.  Same volumes as the oracle,
    with and without accumulate, and the library really asks for more than one copy here."""
    from oracle import port
    from torch_projectors_b200 import _abi
    case = Case("copies", dim, interp, B, P, 8, 16, 2.0, None, 1, B, shift_range=2.0, seed=97, special_poses=False)
    t = make_inputs(case)
    g = {k: (v.cuda() if v is not None else None) for k, v in t.items()}
    code = _abi.CUBIC if interp == "cubic" else _abi.LINEAR
    R = 16
    shape = (B, R, R, R // 2 + 1) if dim == 3 else (B, R, R // 2 + 1)
    one = B * (R if dim == 3 else 1) * R * (R // 2 + 1) * 16
    need = _abi.backproject_workspace_bytes(dim, B, R, P, 8, code, True)
    assert need >= 2 * one and need % one == 0
    f = port.backproject_2d_to_3d_forw if dim == 3 else port.backproject_2d_forw
    d_want, w_want = f(t["proj"], t["weights"], t["rot"], t["shifts"], interp, 2.0)
    for ws_bytes in (need, one, 3 * one):          # all the copies, a single one, an odd number that fits two
        data = torch.full(shape, 5.0, dtype=torch.complex64, device="cuda")
        wrec = torch.full(shape, 5.0, dtype=torch.float32, device="cuda")
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
        _abi.backproject_forw(dim, g["proj"], g["weights"], g["rot"], g["shifts"], code, 2.0, 4.0, data, wrec, False, ws)
        assert rel_err(data, d_want) <= TOL_ATOMIC and rel_err(wrec, w_want) <= TOL_ATOMIC
        _abi.backproject_forw(dim, g["proj"], g["weights"], g["rot"], g["shifts"], code, 2.0, 4.0, data, wrec, True, ws)
        assert rel_err(data, 2 * d_want) <= TOL_ATOMIC and rel_err(wrec, 2 * w_want) <= TOL_ATOMIC
    # and through the public function (the operator layer sizes the workspace itself)
    fn = tp.backproject_2d_to_3d_forw if dim == 3 else tp.backproject_2d_forw
    d, w = fn(g["proj"], g["rot"], weights=g["weights"], shifts=g["shifts"], interpolation=interp, oversampling=2.0)
    assert rel_err(d, d_want) <= TOL_ATOMIC and rel_err(w, w_want) <= TOL_ATOMIC
