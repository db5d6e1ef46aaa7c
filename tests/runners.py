"""Run the four operators of a case on one backend and return outputs under the key names
used by the golden files.  Backends: 'port' (C restatement oracle), 'reference' (the
reference's CPU ops from oracle/_ref, where built) and 'cuda' (this package)."""
from __future__ import annotations

import ast

import numpy as np
import torch

from cases import Case


def _ops_for(backend: str):
    if backend == "port":
        from oracle import port
        return port
    if backend == "reference":
        import oracle
        return oracle.reference_ops()
    if backend == "cuda":
        import torch_projectors_b200  # noqa: F401  (registers the ops)
        return torch.ops.torch_projectors_b200
    raise ValueError(backend)


def cpu_checker():
    """(operators, kind) of the strongest CPU checker present: the reference's own CPU operators
    (multi-threaded; oracle/_ref, where built) or else the C restatement of them."""
    import oracle
    if oracle.reference_available():
        try:
            import os
            torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
        except (AttributeError, RuntimeError):
            pass
        return oracle.reference_ops(), "reference"
    from oracle import port
    return port, "port"


def run_case(backend: str, case: Case, t: dict, which=("fwd", "pb", "bp", "bb")) -> dict:
    ops = _ops_for(backend)
    d = "2d" if case.dim == 2 else "3d_to_2d"
    bd = "2d" if case.dim == 2 else "2d_to_3d"
    if backend == "cuda":
        t = {k: (v.cuda() if v is not None else None) for k, v in t.items()}
    rot_g = t["rot"].clone().requires_grad_(True)
    sh_g = t["shifts"].clone().requires_grad_(True) if t["shifts"] is not None else None
    out = {}
    if "fwd" in which:
        out["fwd"] = getattr(ops, f"project_{d}_forw")(t["rec"], t["rot"], t["shifts"], [case.N, case.N],
                                                       case.interp, case.os, case.cutoff)
    if "pb" in which:
        pb = getattr(ops, f"project_{d}_back")(t["proj"], t["rec"], rot_g, sh_g, case.interp, case.os, case.cutoff)
        out["pb_grad_rec"], out["pb_grad_rot"], out["pb_grad_shift"] = pb
    if "bp" in which:
        bp = getattr(ops, f"backproject_{bd}_forw")(t["proj"], t["weights"], t["rot"], t["shifts"],
                                                    case.interp, case.os, case.cutoff)
        out["bp_data"], out["bp_weight"] = bp
    if "bb" in which:
        bb = getattr(ops, f"backproject_{bd}_back")(
            t["grad_data"], t["grad_weight"] if t["weights"] is not None else None,
            t["proj"], t["weights"], rot_g, sh_g, case.interp, case.os, case.cutoff)
        out["bb_grad_proj"], out["bb_grad_weights"], out["bb_grad_rot"], out["bb_grad_shift"] = bb
    return {k: v.detach().cpu() for k, v in out.items()}


def load_golden(path):
    """-> (Case, inputs dict of CPU tensors, outputs dict of CPU tensors)"""
    z = np.load(path, allow_pickle=False)
    case = Case(**ast.literal_eval(str(z["case"])))
    keys = ("rec", "rot", "shifts", "proj", "weights", "grad_data", "grad_weight")
    t = {k: (torch.from_numpy(z[f"in_{k}"]) if f"in_{k}" in z.files else None) for k in keys}
    out = {k[4:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("out_")}
    return case, t, out


# which tolerance class each output belongs to
FORWARD_KEYS = ("fwd",)


def tolerance_for(key: str) -> float:
    from cases import TOL_ATOMIC, TOL_FORWARD
    return TOL_FORWARD if key in FORWARD_KEYS else TOL_ATOMIC
