"""Two-rank NCCL check of the pose-sharded paths (launched by tests/test_gpu_multi.py with
torch.distributed.run, one process per GPU): sharded projection with gather equals the
single-GPU projection; sharded back-projection through the persistent accumulator, folded and
reduced range by range, equals the single-GPU back-projection of all slices."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path[:0] = [str(ROOT), str(ROOT / "tests"), str(ROOT / "torch-projectors_b200")]


def main():
    import torch_projectors_b200 as tp
    from cases import TOL_ATOMIC, random_rotations_3d, rel_err
    from torch_projectors_b200 import sharding

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    gen = torch.Generator().manual_seed(2024)               # same inputs on every rank
    N, P, R = 16, 37, 32
    rec = torch.randn(1, R, R, R // 2 + 1, dtype=torch.complex64, generator=gen).to(dev)
    rot = random_rotations_3d(P, gen).view(1, P, 3, 3).to(dev)
    sh = ((torch.rand(1, P, 2, generator=gen) * 2 - 1) * 3).to(dev)
    proj = torch.randn(1, P, N, N // 2 + 1, dtype=torch.complex64, generator=gen).to(dev)
    wts = torch.rand(1, P, N, N // 2 + 1, generator=gen).to(dev)
    kw = dict(interpolation="cubic", oversampling=2.0)

    # projection: every rank projects its range of the global pose list, gather gives all slices
    full = tp.project_3d_to_2d_forw(rec, rot, sh, output_shape=(N, N), **kw)
    gathered = sharding.project_3d_to_2d_sharded(rec, rot, sh, gather=True, output_shape=(N, N), **kw)
    assert torch.equal(gathered, full), "gathered projections differ from the single-GPU result"
    lo, hi = sharding.pose_range(P, rank, world)
    local_only = sharding.project_3d_to_2d_sharded(rec, rot, sh, output_shape=(N, N), **kw)
    assert torch.equal(local_only, full[:, lo:hi])

    # back-projection: local slices in chunks through the accumulator; the last chunk is the final
    # stage (scattered slab group by slab group, finished groups folded and reduced meanwhile)
    slabs, _ = tp._abi.accumulator_slab_plan(R)
    assert slabs > 1, "the launcher forces small slabs so that the per-slab path is exercised"
    want_d, want_w = tp.backproject_2d_to_3d_forw(proj, rot, weights=wts, shifts=sh, **kw)
    for dst in (0, None):
        vols = sharding.backproject_2d_to_3d_sharded(proj[:, lo:hi], rot[:, lo:hi], wts[:, lo:hi], sh[:, lo:hi],
                                                     chunk=7, dst=dst, **kw)
        if dst is None or rank == dst:
            assert rel_err(vols.data, want_d) <= TOL_ATOMIC, rel_err(vols.data, want_d)
            assert rel_err(vols.weights, want_w) <= TOL_ATOMIC, rel_err(vols.weights, want_w)
    # without weights: the plain accumulate path, one reduce of the data volume
    want_plain, _ = tp.backproject_2d_to_3d_forw(proj, rot, shifts=sh, **kw)
    vols = sharding.backproject_2d_to_3d_sharded(proj[:, lo:hi], rot[:, lo:hi], None, sh[:, lo:hi], dst=None, **kw)
    assert vols.weights is None and rel_err(vols.data, want_plain) <= TOL_ATOMIC
    dist.barrier()
    if rank == 0:
        print("MULTI-OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
