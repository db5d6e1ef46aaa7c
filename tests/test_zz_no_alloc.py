"""The allocation-free back-projection entry point (built-in scratch inside the library)
against the regular entry point, through the C ABI.

Collected last on purpose (file name): a run that stops at the first failure has then
already run every other test.  The test does not depend on what ran before it: the entry
point looks up its scratch on first use and clears what it uses on every call."""
import pytest
import torch

from cases import Case, TOL_ATOMIC, make_inputs, rel_err

pytestmark = pytest.mark.gpu


def _run_both(abi, case, code):
    t = {k: (v.cuda() if v is not None else None) for k, v in make_inputs(case).items()}
    R = abi.rec_boxsize(case.N, case.os)
    shape = (case.B, R, R, R // 2 + 1)
    cutoff = case.N / 2.0
    want_d = torch.empty(shape, dtype=torch.complex64, device="cuda")
    want_w = torch.empty(shape, dtype=torch.float32, device="cuda")
    abi.backproject_forw(3, t["proj"], t["weights"], t["rot"], t["shifts"], code, case.os, cutoff, want_d, want_w, False)
    got_d = torch.full(shape, 3.0, dtype=torch.complex64, device="cuda")      # must be overwritten
    got_w = torch.full(shape, 3.0, dtype=torch.float32, device="cuda")
    abi.backproject_2d_to_3d_forw_noalloc(t["proj"], t["weights"], t["rot"], t["shifts"], code, case.os, cutoff, got_d, got_w, False)
    torch.cuda.synchronize()
    return (got_d, got_w), (want_d, want_w), t


def test_no_alloc_entry_matches_regular_entry_twice_in_a_row(cuda_device):
    from torch_projectors_b200 import _abi
    # two different problems back to back: the second must not see the first one's sums
    first = Case("na1", 3, "linear", 1, 48, 32, 64, 2.0, None, 1, 1, shift_range=3.0, seed=61, special_poses=False)
    second = Case("na2", 3, "cubic", 2, 9, 16, 32, 2.0, None, 2, 1, shift_range=2.0, seed=62)
    for case, code in ((first, _abi.LINEAR), (second, _abi.CUBIC)):
        (gd, gw), (wd, ww), _ = _run_both(_abi, case, code)
        assert rel_err(gd, wd) <= TOL_ATOMIC
        assert rel_err(gw, ww) <= TOL_ATOMIC
    # accumulate adds to what the outputs hold
    (gd, gw), (wd, ww), t = _run_both(_abi, first, _abi.LINEAR)
    _abi.backproject_2d_to_3d_forw_noalloc(t["proj"], t["weights"], t["rot"], t["shifts"], _abi.LINEAR, 2.0, 16.0, gd, gw, True)
    assert rel_err(gd, 2 * wd) <= TOL_ATOMIC and rel_err(gw, 2 * ww) <= TOL_ATOMIC


def test_no_alloc_entry_matches_the_cpu_oracle_and_takes_no_device_memory(cuda_device):
    """Against the CPU oracle directly (not only against the regular entry point), and the property
    the entry point exists for: once its first call on the device has been made, further calls
    change neither the free device memory nor what torch's allocator holds."""
    from oracle import port
    from torch_projectors_b200 import _abi
    case = Case("na4", 3, "linear", 1, 24, 32, 64, 2.0, None, 1, 1, shift_range=3.0, seed=64, special_poses=False)
    cpu = make_inputs(case)
    t = {k: (v.cuda() if v is not None else None) for k, v in cpu.items()}
    d = torch.empty((1, 64, 64, 33), dtype=torch.complex64, device="cuda")
    w = torch.empty((1, 64, 64, 33), dtype=torch.float32, device="cuda")
    args = (t["proj"], t["weights"], t["rot"], t["shifts"], _abi.LINEAR, 2.0, 16.0, d, w, False)
    _abi.backproject_2d_to_3d_forw_noalloc(*args)          # first call on the device: set-up happens here
    torch.cuda.synchronize()
    free0, held0, reserved0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    for _ in range(5):
        _abi.backproject_2d_to_3d_forw_noalloc(*args)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0
    assert torch.cuda.memory_allocated() == held0 and torch.cuda.memory_reserved() == reserved0
    d_want, w_want = port.backproject_2d_to_3d_forw(cpu["proj"], cpu["weights"], cpu["rot"], cpu["shifts"], "linear", 2.0)
    assert rel_err(d, d_want) <= TOL_ATOMIC and rel_err(w, w_want) <= TOL_ATOMIC


def test_no_alloc_entry_refuses_volumes_beyond_its_scratch(cuda_device):
    from torch_projectors_b200 import _abi
    case = Case("na3", 3, "linear", 1, 2, 34, 68, 2.0, None, 1, 1, seed=63)      # box 68 > box 64
    t = {k: (v.cuda() if v is not None else None) for k, v in make_inputs(case).items()}
    d = torch.zeros((1, 68, 68, 35), dtype=torch.complex64, device="cuda")
    w = torch.zeros((1, 68, 68, 35), dtype=torch.float32, device="cuda")
    with pytest.raises(RuntimeError, match="exceed the built-in scratch"):
        _abi.backproject_2d_to_3d_forw_noalloc(t["proj"], t["weights"], t["rot"], t["shifts"], _abi.LINEAR, 2.0, 17.0, d, w, False)
    assert (d == 0).all() and (w == 0).all()                                      # nothing was launched
