"""The C-ABI library loads without a GPU, exports every symbol include/b200proj.h declares,
and rejects bad arguments with error codes before touching the device."""
import ctypes as C
import re
from pathlib import Path

import pytest

from torch_projectors_b200 import _abi

HEADER = Path(__file__).resolve().parent.parent / "include" / "b200proj.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(b200proj_\w+)\s*\(", text)))


def test_header_declares_the_eight_operators():
    names = declared_symbols()
    for op in ("project_2d_forw", "project_2d_back", "backproject_2d_forw", "backproject_2d_back",
               "project_3d_to_2d_forw", "project_3d_to_2d_back", "backproject_2d_to_3d_forw",
               "backproject_2d_to_3d_back"):
        assert f"b200proj_{op}" in names


def test_library_exports_every_declared_symbol():
    lib = _abi.load()
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in b200proj.h but not exported"
    # and the binding table covers the operators one to one
    assert set(_abi.EXPORTS) <= set(declared_symbols())


def test_version_and_size_rule_need_no_gpu():
    assert _abi.version() >= 100
    assert _abi.rec_boxsize(6, 1.5) == 10
    assert _abi.rec_boxsize(8, 1.3) == 12
    assert _abi.rec_boxsize(10, 2.0) == 20
    assert _abi.rec_boxsize(128, 2.0) == 256


def _forw(lib, **over):
    a = dict(rec=1, B=1, R=8, rot=1, B_rot=1, shifts=0, B_shift=0, P=1, N=8, interp=0, os=1.0,
             cutoff=4.0, out=1, stream=0)
    a.update(over)
    return lib.b200proj_project_3d_to_2d_forw(a["rec"], a["B"], a["R"], a["rot"], a["B_rot"], a["shifts"],
                                              a["B_shift"], a["P"], a["N"], a["interp"], a["os"],
                                              a["cutoff"], a["out"], 0, a["stream"])


@pytest.mark.parametrize("over,fragment", [
    (dict(interp=7), "interpolation"),
    (dict(N=7), "must be even"),
    (dict(R=9), "must be even"),
    (dict(B_rot=3, B=2), "rotations must be 1 or same"),
    (dict(shifts=1, B_shift=3, B=2), "shifts must be 1 or same"),
    (dict(os=0.0), "oversampling"),
    (dict(os=1.0e9), "beyond 2^30"),
    (dict(rot=0), "NULL"),
    (dict(rec=0), "NULL"),
    (dict(R=4096), "exceeds"),
])
def test_argument_errors_are_reported_without_a_device(over, fragment):
    lib = _abi.load()
    rc = _forw(lib, **over)       # pointers are dummies: validation must fail before any use
    assert rc < 0
    msg = lib.b200proj_last_error().decode()
    assert fragment in msg, msg


def test_backprojection_checks_volume_size_rule():
    lib = _abi.load()
    rc = lib.b200proj_backproject_2d_to_3d_forw(1, 0, 1, 10, 1, 1, 0, 0, 1, 8, 0, 2.0, 4.0, 1, 0, 0, 0, 0, 0)
    assert rc == -1
    assert "does not match" in lib.b200proj_last_error().decode()
    rc = lib.b200proj_backproject_2d_to_3d_forw(1, 1, 1, 16, 1, 1, 0, 0, 1, 8, 0, 2.0, 4.0, 1, 0, 0, 0, 0, 0)
    assert rc == -1 and "given together" in lib.b200proj_last_error().decode()


def test_pose_order_argument_errors_need_no_gpu():
    lib = _abi.load()
    assert lib.b200proj_pose_order_3d(0, 1, 1, 4, 1, 0) == -1 and "NULL" in lib.b200proj_last_error().decode()
    assert lib.b200proj_pose_order_3d(1, 2, 3, 4, 1, 0) == -1 and "rotations must be 1 or same" in lib.b200proj_last_error().decode()
    assert lib.b200proj_pose_order_3d(1, 1, 1, 0, 1, 0) == 0      # no poses: nothing to do


def test_workspace_query_needs_no_gpu():
    # box-256 volumes, 50,000 slices with weights: one 16-byte slot per voxel
    assert _abi.backproject_workspace_bytes(3, 1, 256, 50000, 128, _abi.LINEAR, True) == 256 * 256 * 129 * 16
    assert _abi.backproject_workspace_bytes(3, 1, 256, 50000, 128, _abi.LINEAR, False) == 0     # no weights
    assert _abi.backproject_workspace_bytes(3, 1, 256, 1, 128, _abi.LINEAR, True) == 0          # too few slices


def test_no_alloc_entry_reports_its_limit_without_a_device():
    lib = _abi.load()
    # box 68 > the built-in scratch (box 64): refused before any CUDA call
    rc = lib.b200proj_backproject_2d_to_3d_forw_noalloc(1, 1, 1, 68, 1, 1, 0, 0, 1, 34, 0, 2.0, 17.0, 1, 1, 0, 0)
    assert rc == -2 and "built-in scratch" in lib.b200proj_last_error().decode()
    rc = lib.b200proj_backproject_2d_to_3d_forw_noalloc(1, 0, 1, 64, 1, 1, 0, 0, 1, 32, 0, 2.0, 16.0, 1, 1, 0, 0)
    assert rc == -1 and "required" in lib.b200proj_last_error().decode()


def test_accumulator_and_prep_entries_validate_without_a_device():
    lib = _abi.load()
    assert _abi.accumulator_bytes(1, 800) == 800 * 800 * 401 * 16
    assert _abi.accumulator_bytes(0, 800) == 0
    err = lambda: lib.b200proj_last_error().decode()  # noqa: E731
    # accumulate: weights and accumulator are required, alignment and the size rule are checked
    acc = lib.b200proj_backproject_2d_to_3d_accumulate
    assert acc(1, 0, 1, 16, 1, 1, 0, 0, 1, 8, 0, 2.0, 4.0, 16, 0) == -1 and "required" in err()
    assert acc(1, 1, 1, 16, 1, 1, 0, 0, 1, 8, 0, 2.0, 4.0, 8, 0) == -1 and "16-byte aligned" in err()
    assert acc(1, 1, 1, 10, 1, 1, 0, 0, 1, 8, 0, 2.0, 4.0, 16, 0) == -1 and "does not match" in err()
    assert acc(1, 1, 1, 16, 1, 1, 0, 0, 0, 8, 0, 2.0, 4.0, 16, 0) == 0            # no poses: nothing to launch
    fold = lib.b200proj_accumulator_fold
    assert fold(0, 1, 16, 1, 1, 0, 0) == -1 and "required" in err()
    assert fold(1, 1, 15, 1, 1, 0, 0) == -1 and "even" in err()
    # pad + fftshift / ifftshift + crop
    pad = lib.b200proj_pad_fftshift
    assert pad(0, 1, 3, 8, 16, 1, 0) == -1 and "NULL" in err()
    assert pad(1, 1, 4, 8, 16, 1, 0) == -1 and "dims" in err()
    assert pad(1, 1, 3, 8, 15, 1, 0) == -1 and "even padded box" in err()
    assert pad(1, 1, 3, 20, 16, 1, 0) == -1 and "n <= m" in err()
    assert pad(1, 200, 3, 256, 512, 1, 0) == -2 and "split the batch" in err()
    assert lib.b200proj_ifftshift_crop(1, 1, 2, 16, 20, 1, 0) == -1


def test_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: the header compiles as C99 with no torch, CUDA or C++ in sight."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc on this machine")
    src = tmp_path / "use_header.c"
    src.write_text('#include "b200proj.h"\nint use(void) { return b200proj_version() + B200PROJ_CUBIC + B200PROJ_ERR_LIMIT; }\n')
    r = subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only", f"-I{HEADER.parent}", str(src)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
