"""The kernels' voxel-index helpers, run on the HOST (they are compiled for host and device from
one source and exported through ``b200proj_debug_index``).

A sample position at or below -2^31 (a rotation entry of -inf, a diverged optimiser, an
uninitialised pose tensor) saturates to INT_MIN when converted to int, and negating INT_MIN gives
INT_MIN again.  These tests feed the helpers such coordinates on the CPU -- never on a GPU -- and
check that gathers still return an index inside the stored half-volume and scatters drop the tap;
for ordinary coordinates the helpers must equal the reference's int64 arithmetic
(csrc/cpu/common/fftw_sampling.h:96-137 and projection_utils.h:414-493 of warpem/torch-projectors)."""
import ctypes as C

import pytest

INT_MIN, INT_MAX = -2 ** 31, 2 ** 31 - 1
EXTREME = [INT_MIN, INT_MIN + 1, INT_MIN + 2, INT_MIN + 3, -2 ** 30, 2 ** 30, INT_MAX - 3, INT_MAX - 1, INT_MAX]
GATHER_COL_LIN, GATHER_COL_CUB, GATHER_LINE_LIN, GATHER_LINE_CUB, SCATTER_COL, SCATTER_LINE = range(6)


@pytest.fixture(scope="module")
def helper():
    from torch_projectors_b200 import _abi
    lib = _abi.load()
    fn = lib.b200proj_debug_index
    fn.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int)]
    fn.restype = C.c_int

    def call(which, R, coordinate, mirrored=False):
        m = C.c_int(-7)
        r = fn(which, R, coordinate, int(mirrored), C.byref(m))
        return r, bool(m.value)
    return call


def _wrap(r, R):
    return r + R if r < 0 else r


def spec_gather_col(R, c):
    Rh = R // 2 + 1
    return min(abs(c), Rh - 1), c < 0


def spec_gather_line(R, r, mirrored, cubic):
    half = R // 2
    if cubic:
        r = max(-half + 1, min(r, half))
    if mirrored:
        r = -r
    return _wrap(min(half, max(r, -half + 1)), R)


def spec_scatter_col(R, c):
    Rh = R // 2 + 1
    return (abs(c) if abs(c) < Rh else -1), c < 0


def spec_scatter_line(R, r, mirrored):
    half = R // 2
    if mirrored:
        r = -r
    return -1 if (r > half or r < -half + 1) else _wrap(r, R)


@pytest.mark.parametrize("R", [2, 6, 32, 800])
def test_helpers_equal_int64_arithmetic_for_ordinary_coordinates(helper, R):
    span = list(range(-R - 5, R + 6)) + [-10 * R, 10 * R, -2 ** 30, 2 ** 30]
    for c in span:
        for which in (GATHER_COL_LIN, GATHER_COL_CUB):
            assert helper(which, R, c) == spec_gather_col(R, c), (which, R, c)
        assert helper(SCATTER_COL, R, c) == spec_scatter_col(R, c), (R, c)
        for m in (False, True):
            assert helper(GATHER_LINE_LIN, R, c, m)[0] == spec_gather_line(R, c, m, False), (R, c, m)
            assert helper(GATHER_LINE_CUB, R, c, m)[0] == spec_gather_line(R, c, m, True), (R, c, m)
            assert helper(SCATTER_LINE, R, c, m)[0] == spec_scatter_line(R, c, m), (R, c, m)


@pytest.mark.parametrize("R", [2, 32, 800, 2048])
def test_saturated_coordinates_never_index_outside_the_half_volume(helper, R):
    Rh = R // 2 + 1
    for c in EXTREME:
        for which in (GATHER_COL_LIN, GATHER_COL_CUB):
            col, mirrored = helper(which, R, c)
            assert col == Rh - 1 and mirrored == (c < 0), (which, c, col)      # the clamped edge column
        assert helper(SCATTER_COL, R, c)[0] == -1, c                          # dropped
        for m in (False, True):
            for which in (GATHER_LINE_LIN, GATHER_LINE_CUB):
                assert 0 <= helper(which, R, c, m)[0] < R, (which, c, m)
            assert helper(SCATTER_LINE, R, c, m)[0] == -1, (c, m)
