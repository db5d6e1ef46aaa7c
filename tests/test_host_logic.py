"""Host-side logic that needs no GPU: the public API's validation (same errors as the
reference's Python layer), the absence of any CPU fallback, and the pose-sharding layer
driven by two gloo ranks with the CPU oracle standing in for the CUDA operators."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import torch_projectors_b200 as tp
from torch_projectors_b200 import sharding

ROOT = Path(__file__).resolve().parent.parent


# ---- validation (reference: torch_projectors/ops.py:19-36, 98-115, 153-172, 246-262) -------
def test_project_2d_validation_messages():
    rot = torch.eye(2).view(1, 1, 2, 2)
    with pytest.raises(ValueError, match="expected boxsize .* to match"):
        tp.project_2d_forw(torch.zeros(8, 6, dtype=torch.complex64), rot)
    with pytest.raises(ValueError, match="Boxsize .* must be even"):
        tp.project_2d_forw(torch.zeros(7, 4, dtype=torch.complex64), rot)
    with pytest.raises(ValueError, match="must be square"):
        tp.project_2d_forw(torch.zeros(8, 5, dtype=torch.complex64), rot, output_shape=(8, 6))
    with pytest.raises(ValueError, match="must be even"):
        tp.project_2d_forw(torch.zeros(8, 5, dtype=torch.complex64), rot, output_shape=(7, 7))


def test_project_3d_validation_messages():
    rot = torch.eye(3).view(1, 1, 3, 3)
    with pytest.raises(ValueError, match="must be a 4D tensor"):
        tp.project_3d_to_2d_forw(torch.zeros(8, 8, 5, dtype=torch.complex64), rot)
    with pytest.raises(ValueError, match="must be even"):
        tp.project_3d_to_2d_forw(torch.zeros(1, 7, 7, 4, dtype=torch.complex64), rot)


def test_backprojection_validation_messages():
    rot = torch.eye(3).view(1, 1, 3, 3)
    with pytest.raises(ValueError, match="Projections must be a 4D tensor"):
        tp.backproject_2d_to_3d_forw(torch.zeros(8, 5, dtype=torch.complex64), rot)
    with pytest.raises(ValueError, match="Weights shape .* must match projections shape"):
        tp.backproject_2d_forw(torch.zeros(1, 1, 8, 5, dtype=torch.complex64), torch.eye(2).view(1, 1, 2, 2),
                               weights=torch.zeros(1, 1, 8, 4))
    with pytest.raises(ValueError, match="real-valued"):
        tp.backproject_2d_forw(torch.zeros(1, 1, 8, 5, dtype=torch.complex64), torch.eye(2).view(1, 1, 2, 2),
                               weights=torch.zeros(1, 1, 8, 5, dtype=torch.complex64))


def test_rotation_batch_mismatch_is_a_value_error():
    rec = torch.zeros(2, 8, 8, 5, dtype=torch.complex64)
    with pytest.raises(ValueError, match="Batch size of rotations"):
        tp.project_3d_to_2d_forw(rec, torch.eye(3).expand(3, 1, 3, 3))


def test_no_cpu_fallback():
    rec = torch.zeros(1, 8, 8, 5, dtype=torch.complex64)
    with pytest.raises((NotImplementedError, RuntimeError)):
        tp.project_3d_to_2d_forw(rec, torch.eye(3).view(1, 1, 3, 3))
    with pytest.raises((NotImplementedError, RuntimeError)):
        tp.backproject_2d_to_3d_forw(torch.zeros(1, 1, 8, 5, dtype=torch.complex64), torch.eye(3).view(1, 1, 3, 3))


def test_product_package_does_not_import_the_oracle():
    pkg = ROOT / "torch-projectors_b200"
    for path in list(pkg.rglob("*.py")) + list(pkg.rglob("*.cu")) + list(pkg.rglob("*.cuh")):
        text = path.read_text()
        assert "import oracle" not in text and "from oracle" not in text and "oracle/" not in text, path


def test_public_names_match_the_reference_api():
    for name in ("project_2d_forw", "project_2d_back", "project_3d_to_2d_forw", "project_3d_to_2d_back",
                 "backproject_2d_forw", "backproject_2d_to_3d_forw", "backproject_2d_to_3d_back"):
        assert callable(getattr(tp, name))
    ns = torch.ops.torch_projectors_b200
    for name in ("project_2d_forw", "project_2d_back", "backproject_2d_forw", "backproject_2d_back",
                 "project_3d_to_2d_forw", "project_3d_to_2d_back", "backproject_2d_to_3d_forw",
                 "backproject_2d_to_3d_back"):
        assert hasattr(ns, name)


# ---- pose sharding ------------------------------------------------------------------------
# ---- the C++ operator layer, as far as it goes without a GPU -----------------------------------
REFERENCE_SCHEMAS = {
    "project_forw": "(Tensor reconstruction, Tensor rotations, Tensor? shifts, int[] output_shape, str interpolation, float oversampling, float? fourier_radius_cutoff) -> Tensor",
    "project_back": "(Tensor grad_projections, Tensor reconstruction, Tensor rotations, Tensor? shifts, str interpolation, float oversampling, float? fourier_radius_cutoff) -> (Tensor, Tensor, Tensor)",
    "backproject_forw": "(Tensor projections, Tensor? weights, Tensor rotations, Tensor? shifts, str interpolation, float oversampling, float? fourier_radius_cutoff) -> (Tensor, Tensor)",
    "backproject_back": "(Tensor grad_data_rec, Tensor? grad_weight_rec, Tensor projections, Tensor? weights, Tensor rotations, Tensor? shifts, str interpolation, float oversampling, float? fourier_radius_cutoff) -> (Tensor, Tensor, Tensor, Tensor)",
}


def test_operators_are_defined_in_cpp_with_the_reference_schemas():
    """The eight raw operators come from the compiled C++ library (not from Python registrations)
    and carry the reference's schema strings (csrc/torch_projectors.cpp:23-36 there)."""
    import torch_projectors_b200  # noqa: F401
    from torch_projectors_b200 import build
    assert build.BINDING_PATH.exists()
    ops = torch.ops.torch_projectors_b200
    for name, kind in (("project_2d_forw", "project_forw"), ("project_3d_to_2d_forw", "project_forw"),
                       ("project_2d_back", "project_back"), ("project_3d_to_2d_back", "project_back"),
                       ("backproject_2d_forw", "backproject_forw"), ("backproject_2d_to_3d_forw", "backproject_forw"),
                       ("backproject_2d_back", "backproject_back"), ("backproject_2d_to_3d_back", "backproject_back")):
        schema = str(getattr(ops, name).default._schema)
        assert schema == f"torch_projectors_b200::{name}{REFERENCE_SCHEMAS[kind]}", schema
        assert torch._C._dispatch_has_kernel_for_dispatch_key(f"torch_projectors_b200::{name}", "CUDA")
        assert not torch._C._dispatch_has_kernel_for_dispatch_key(f"torch_projectors_b200::{name}", "CPU")


def test_cpu_tensors_are_rejected_by_the_dispatcher():
    import torch_projectors_b200 as tp
    rec = torch.zeros(1, 8, 5, dtype=torch.complex64)
    rot = torch.eye(2).view(1, 1, 2, 2)
    with pytest.raises(NotImplementedError, match="CPU"):
        tp.project_2d_forw(rec, rot)
    with pytest.raises(NotImplementedError, match="CPU"):
        tp.backproject_2d_forw(torch.zeros(1, 1, 8, 5, dtype=torch.complex64), rot)


def test_meta_implementations_give_the_output_shapes():
    """Shape-only implementations (Meta key): what tracing the operators needs."""
    import torch_projectors_b200  # noqa: F401
    ops = torch.ops.torch_projectors_b200
    m = dict(device="meta")
    rec = torch.empty(2, 16, 16, 9, dtype=torch.complex64, **m)
    rot = torch.empty(1, 5, 3, 3, **m).requires_grad_(True)
    sh = torch.empty(2, 5, 2, **m)
    assert ops.project_3d_to_2d_forw(rec, rot, sh, [8, 8], "cubic", 2.0, None).shape == (2, 5, 8, 5)
    g = torch.empty(2, 5, 8, 5, dtype=torch.complex64, **m)
    gr, grot, gsh = ops.project_3d_to_2d_back(g, rec, rot, sh, "cubic", 2.0, None)
    assert gr.shape == rec.shape and grot.shape == rot.shape and gsh.shape == (0,)
    w = torch.empty(2, 5, 8, 5, **m)
    d, wr = ops.backproject_2d_to_3d_forw(g, w, rot, sh, "linear", 2.0, None)
    assert d.shape == (2, 16, 16, 9) and wr.shape == (2, 16, 16, 9) and d.dtype == torch.complex64 and wr.dtype == torch.float32
    d2, w2 = ops.backproject_2d_forw(g, None, torch.empty(1, 5, 2, 2, **m), None, "linear", 1.5, None)
    assert d2.shape == (2, 12, 7) and w2.shape == (0,)
    gp, gw, grot, gsh = ops.backproject_2d_to_3d_back(d, wr, g, w, rot, sh, "linear", 2.0, None)
    assert gp.shape == g.shape and gw.shape == w.shape and grot.shape == rot.shape and gsh.shape == (0,)
    assert ops.plane_locality_order(rot, 2).shape == (10,)
    # the variants with an explicit processing order of the slices
    order = torch.empty(10, dtype=torch.int32, **m)
    assert ops.project_3d_to_2d_forw_ordered(rec, rot, sh, [8, 8], "cubic", 2.0, None, order).shape == (2, 5, 8, 5)
    assert ops.project_3d_to_2d_back_ordered(g, rec, rot, sh, "cubic", 2.0, None, None)[0].shape == rec.shape
    assert ops.backproject_2d_to_3d_back_ordered(d, wr, g, w, rot, sh, "linear", 2.0, None, order)[0].shape == g.shape
    # the forward projection that keeps its pixels' derivatives, and its backward pass
    out, der = ops.project_3d_to_2d_forw_saving(rec, rot, sh, [8, 8], "cubic", 2.0, None, order)
    assert out.shape == (2, 5, 8, 5) and der.shape == (3, 2, 5, 8, 5) and der.dtype == torch.complex64
    gr, grot, gsh = ops.project_3d_to_2d_back_saved(g, out, der, rec, rot, sh, "cubic", 2.0, None, order, True)
    assert gr.shape == rec.shape and gr.dtype == torch.complex64 and grot.shape == rot.shape and gsh.shape == (0,)
    assert ops.project_3d_to_2d_back_saved(g, out, der, rec, rot, sh, "cubic", 2.0, None, None, False)[0].shape == (0,)
    rec2, rot2 = torch.empty(2, 16, 9, dtype=torch.complex64, **m), torch.empty(1, 5, 2, 2, **m).requires_grad_(True)
    out2, der2 = ops.project_2d_forw_saving(rec2, rot2, sh, [8, 8], "linear", 2.0, None)
    assert out2.shape == (2, 5, 8, 5) and der2.shape == (2, 2, 5, 8, 5)
    gr2, grot2, _ = ops.project_2d_back_saved(g, out2, der2, rec2, rot2, sh, "linear", 2.0, None, True)
    assert gr2.shape == rec2.shape and grot2.shape == rot2.shape


@pytest.mark.parametrize("P,world", [(10, 1), (10, 2), (10, 3), (7, 8), (0, 4), (200000, 8)])
def test_pose_range_partitions_exactly(P, world):
    spans = [sharding.pose_range(P, r, world) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == P
    for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
        assert a1 == b0
    sizes = [b - a for a, b in spans]
    assert max(sizes) - min(sizes) <= 1


def test_pose_range_rejects_bad_rank():
    with pytest.raises(ValueError):
        sharding.pose_range(10, 2, 2)


def test_partial_volumes_layout_is_one_buffer():
    v = sharding.PartialVolumes(2, 8, "cpu", with_weights=True)
    n = 2 * 8 * 8 * 5
    assert v.flat.numel() == 3 * n and v.data.shape == (2, 8, 8, 5) and v.weights.shape == (2, 8, 8, 5)
    v.data[1, 2, 3, 4] = 1 + 2j
    v.weights[1, 2, 3, 4] = 5.0
    assert v.flat.sum().item() == 8.0
    assert sharding.PartialVolumes(1, 8, "cpu", with_weights=False).weights is None


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gloo_worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path[:0] = [str(ROOT), str(ROOT / "tests"), str(ROOT / "torch-projectors_b200")]
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import port as orc          # CPU stand-in for the CUDA operators (tests only)
        from cases import Case, make_inputs
        case = Case("shard", 3, "linear", 1, 7, 8, 16, 2.0, None, 1, 1, seed=77)
        t = make_inputs(case)
        lo, hi = sharding.pose_range(case.P, rank, world)

        # projection: each rank its pose range, gathered result equals the unsharded call
        def project_fn(rec, rot, shifts, **kw):
            return orc.project_3d_to_2d_forw(rec, rot, shifts, [case.N, case.N], case.interp, case.os)
        full = sharding.project_3d_to_2d_sharded(t["rec"], t["rot"], t["shifts"], gather=True, project_fn=project_fn)
        want = project_fn(t["rec"], t["rot"], t["shifts"])
        assert torch.equal(full, want)
        local = sharding.project_3d_to_2d_sharded(t["rec"], t["rot"], t["shifts"], project_fn=project_fn)
        assert torch.equal(local, want[:, lo:hi])

        # back-projection: local chunks -> partial volumes -> one reduce
        def accumulate_fn(data, wrec, proj, rot, weights, shifts, *, interpolation, oversampling, fourier_radius_cutoff):
            orc.backproject_2d_to_3d_forw(proj, weights, rot, shifts, interpolation, oversampling,
                                          fourier_radius_cutoff, out=(data, wrec))
        vols = sharding.backproject_2d_to_3d_sharded(
            t["proj"][:, lo:hi], t["rot"][:, lo:hi], t["weights"][:, lo:hi], t["shifts"][:, lo:hi],
            interpolation=case.interp, oversampling=case.os, chunk=2, dst=None,
            accumulate_fn=accumulate_fn, rec_boxsize_fn=orc.rec_boxsize)
        d_want, w_want = orc.backproject_2d_to_3d_forw(t["proj"], t["weights"], t["rot"], t["shifts"], case.interp, case.os)
        assert torch.allclose(vols.data, d_want, atol=1e-4)
        assert torch.allclose(vols.weights, w_want, atol=1e-4)

        # reduce to rank 0 only
        vols0 = sharding.backproject_2d_to_3d_sharded(
            t["proj"][:, lo:hi], t["rot"][:, lo:hi], None, None,
            interpolation=case.interp, oversampling=case.os, chunk=8192, dst=0,
            accumulate_fn=accumulate_fn, rec_boxsize_fn=orc.rec_boxsize)
        if rank == 0:
            d0, _ = orc.backproject_2d_to_3d_forw(t["proj"], None, t["rot"], None, case.interp, case.os)
            assert torch.allclose(vols0.data, d0, atol=1e-4)
            assert vols0.weights is None
        Path(tmp, f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


def test_sharded_pipeline_on_two_gloo_ranks(tmp_path):
    world = 2
    mp.spawn(_gloo_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def _gloo_failure_worker(rank, world, port, tmp):
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path[:0] = [str(ROOT), str(ROOT / "tests"), str(ROOT / "torch-projectors_b200")]
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=10))
    vols = sharding.PartialVolumes(1, 8, "cpu", with_weights=True)
    vols.data += 1.0
    dist.barrier()
    if rank == 1:
        # this rank fails on the host before the collective (an exception in its own work) and leaves
        try:
            raise RuntimeError("injected failure before reduce")
        except RuntimeError:
            Path(tmp, "rank1_failed").write_text("left before reduce")
            return
    t0 = time.time()
    try:
        vols.reduce(dst=0)
        outcome = "no error"
    except Exception as e:  # noqa: BLE001
        outcome = f"error {type(e).__name__}"
    Path(tmp, "rank0_outcome").write_text(f"{outcome}|{time.time() - t0:.1f}")


def test_reduce_ends_with_an_error_when_a_rank_left_before_it(tmp_path):
    """Failure on the host, no GPU involved: rank 1 raises in its own work and never joins the
    reduce of the partial volumes; rank 0 must come back from reduce() with an error within the
    process group's timeout instead of waiting for ever."""
    world = 2
    ctx = mp.spawn(_gloo_failure_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=False)
    deadline = 90
    import time
    t0 = time.time()
    while not ctx.join(timeout=1.0) and time.time() - t0 < deadline:
        pass
    for proc in ctx.processes:
        if proc.is_alive():
            proc.terminate()
    assert (tmp_path / "rank1_failed").exists()
    outcome, seconds = (tmp_path / "rank0_outcome").read_text().split("|")
    assert outcome.startswith("error"), outcome
    assert float(seconds) < 60.0


def test_sharding_without_process_group_is_single_rank():
    calls = []

    def project_fn(rec, rot, shifts, **kw):
        calls.append(rot.shape[1])
        return torch.zeros(1, rot.shape[1], 4, 3, dtype=torch.complex64)
    out = sharding.project_3d_to_2d_sharded(torch.zeros(1, 4, 4, 3, dtype=torch.complex64),
                                            torch.eye(3).expand(1, 5, 3, 3), None, project_fn=project_fn)
    assert out.shape[1] == 5 and calls == [5]


# ---- preparation helpers (pure torch, device-agnostic) --------------------------------------
@pytest.mark.parametrize("dims,n,os", [(3, 8, 2.0), (2, 10, 1.5), (3, 6, 1.0)])
def test_pad_fftshift_roundtrip_and_layout(dims, n, os):
    from torch_projectors_b200 import prep
    torch.manual_seed(0)
    real = torch.randn((2,) + (n,) * dims)
    rec = prep.pad_and_fftshift(real, os, dims)
    m = rec.shape[-2]
    assert m % 2 == 0 and m >= n and rec.shape[-1] == m // 2 + 1 and rec.is_complex()
    back = prep.ifftshift_and_crop(rec, m / n, dims)
    assert back.shape == real.shape and torch.allclose(back, real, atol=1e-5)
    # origin at index 0: the DC term is the mean of the padded array
    assert torch.allclose(rec[(slice(None),) + (0,) * dims].real, real.sum(dim=tuple(range(-dims, 0))) / m ** dims, atol=1e-5)


def test_normalize_by_weights():
    from torch_projectors_b200 import prep
    d = torch.tensor([2.0 + 2j, 1.0 + 0j, 5.0 + 0j])
    w = torch.tensor([2.0, 0.0, 1e-6])
    out = prep.normalize_by_weights(d, w, eps=0.5)
    assert torch.allclose(out, torch.tensor([1.0 + 1j, 2.0 + 0j, 10.0 + 0j]))


def test_bench_script_refers_to_no_undefined_name():
    """bench.py cannot run here (no GPU), so at least make sure that every name it loads is defined
    somewhere in it (a function moved or deleted by an edit would otherwise only show on the GPU box)."""
    import ast
    import builtins
    tree = ast.parse((ROOT / "bench.py").read_text())
    defined = set(dir(builtins)) | {"__file__"}
    for n in ast.walk(tree):
        if isinstance(n, (ast.FunctionDef, ast.ClassDef)):
            defined.add(n.name)
        if isinstance(n, (ast.FunctionDef, ast.Lambda)):
            a = n.args
            defined |= {x.arg for x in a.args + a.kwonlyargs + a.posonlyargs} | ({a.vararg.arg} if a.vararg else set()) | ({a.kwarg.arg} if a.kwarg else set())
        if isinstance(n, ast.Import):
            defined |= {x.asname or x.name.split(".")[0] for x in n.names}
        if isinstance(n, ast.ImportFrom):
            defined |= {x.asname or x.name for x in n.names}
        if isinstance(n, ast.ExceptHandler) and n.name:
            defined.add(n.name)
        if isinstance(n, ast.Name) and isinstance(n.ctx, (ast.Store, ast.Del)):
            defined.add(n.id)
    loaded = {n.id for n in ast.walk(tree) if isinstance(n, ast.Name) and isinstance(n.ctx, ast.Load)}
    assert loaded - defined == set(), sorted(loaded - defined)
