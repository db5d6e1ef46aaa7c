#!/usr/bin/env python
"""Generate the golden vectors in this folder from the REFERENCE's own CPU operators.

Run in a container that has the reference checkout:

    python oracle/build_ref.py          # compiles the reference's csrc/cpu in place
    python tests/golden/make_golden.py  # writes tests/golden/*.npz

Each ``<case>.npz`` holds the seeded inputs of one tiny case and the outputs of the four
reference operators of that dimensionality (forward projection, its backward,
back-projection, its backward), all computed by ``torch.ops.torch_projectors.*`` on CPU in
complex64/float32.  The files are small (tens of KB) and are committed; the reference
itself is not needed to run the tests that read them.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from cases import Case, make_inputs  # noqa: E402

GOLDEN_CASES = [
    Case("g3_lin_os2", 3, "linear", 1, 4, 8, 16, 2.0, None, 1, 1, seed=100),
    Case("g3_cub_os2", 3, "cubic", 1, 4, 8, 16, 2.0, None, 1, 1, seed=101),
    Case("g3_lin_batch", 3, "linear", 2, 3, 6, 6, 1.0, 2.5, 1, 2, seed=102),
    Case("g3_cub_batch", 3, "cubic", 2, 3, 6, 10, 1.5, None, 2, 1, seed=103),
    Case("g3_cub_overreach", 3, "cubic", 1, 3, 8, 8, 1.5, None, 1, 0, seed=104),
    Case("g3_lin_overreach", 3, "linear", 1, 3, 8, 8, 1.5, None, 1, 1, seed=105),
    Case("g2_lin_os2", 2, "linear", 1, 6, 16, 32, 2.0, None, 1, 1, seed=106),
    Case("g2_cub_os2", 2, "cubic", 1, 6, 16, 32, 2.0, None, 1, 1, seed=107),
    Case("g2_lin_batch", 2, "linear", 3, 4, 12, 12, 1.0, 4.5, 3, 1, seed=108),
    Case("g2_cub_overreach", 2, "cubic", 2, 4, 12, 12, 1.5, None, 1, 2, seed=109),
]


def reference_outputs(ops, case: Case, t: dict) -> dict:
    d = "2d" if case.dim == 2 else "3d_to_2d"
    bd = "2d" if case.dim == 2 else "2d_to_3d"
    rot_g = t["rot"].clone().requires_grad_(True)
    sh_g = t["shifts"].clone().requires_grad_(True) if t["shifts"] is not None else None
    out = {}
    out["fwd"] = getattr(ops, f"project_{d}_forw")(t["rec"], t["rot"], t["shifts"], [case.N, case.N],
                                                   case.interp, case.os, case.cutoff)
    pb = getattr(ops, f"project_{d}_back")(t["proj"], t["rec"], rot_g, sh_g, case.interp, case.os, case.cutoff)
    out["pb_grad_rec"], out["pb_grad_rot"], out["pb_grad_shift"] = pb
    bp = getattr(ops, f"backproject_{bd}_forw")(t["proj"], t["weights"], t["rot"], t["shifts"],
                                                case.interp, case.os, case.cutoff)
    out["bp_data"], out["bp_weight"] = bp
    bb = getattr(ops, f"backproject_{bd}_back")(t["grad_data"], t["grad_weight"] if t["weights"] is not None else None,
                                                t["proj"], t["weights"], rot_g, sh_g, case.interp, case.os, case.cutoff)
    out["bb_grad_proj"], out["bb_grad_weights"], out["bb_grad_rot"], out["bb_grad_shift"] = bb
    return out


def main():
    import oracle
    ops = oracle.reference_ops()
    torch.set_num_threads(1)          # sequential accumulation: reproducible golden files
    for case in GOLDEN_CASES:
        t = make_inputs(case)
        out = reference_outputs(ops, case, t)
        blob = {f"in_{k}": v.numpy() for k, v in t.items() if v is not None}
        blob.update({f"out_{k}": v.detach().numpy() for k, v in out.items()})
        blob["case"] = np.array(repr(case.as_dict()))
        path = HERE / f"{case.name}.npz"
        np.savez_compressed(path, **blob)
        print(f"{path.name}: {path.stat().st_size / 1024:.1f} KB")


if __name__ == "__main__":
    main()
