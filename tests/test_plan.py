"""How the tensor-core product of a shape would run is decided on the host, from the shape and the number of SMs
alone (`citlali_gemm_tc_plan`): checked here without a GPU.  The library is compiled if it is not there yet."""
import ctypes

import pytest

from citlali_b200 import ops


def plan(M, N, K, sms=148, force=0):
    try:
        lib = ops.lib()
    except Exception as e:                       # no compiler on this machine
        pytest.skip(f"the kernel library cannot be built here: {e}")
    swapped, bn, splits = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    lib.citlali_gemm_tc_plan(M, N, K, sms, force, ctypes.byref(swapped), ctypes.byref(bn), ctypes.byref(splits))
    return bool(swapped.value), bn.value, splits.value


@pytest.mark.parametrize("M,bn", [(1, 16), (8, 16), (16, 16), (17, 32), (33, 64), (64, 64), (65, 128), (128, 128)])
def test_few_rows_put_the_weights_on_the_wide_side(M, bn):
    swapped, width, splits = plan(M, 4096, 4096)
    assert swapped and width == bn
    assert splits in (1, 2, 4, 8)


def test_k_is_split_by_shape_alone():
    # 148 SMs, two blocks each: 296 places for (tile, split) pairs; a split keeps four K blocks of 64 at least
    assert plan(8, 6144, 4096) == (True, 16, 4)          # 48 tiles: 6 would fit, powers of two only
    assert plan(8, 4096, 4096) == (True, 16, 8)          # 32 tiles
    assert plan(8, 24576, 4096) == (True, 16, 1)         # 192 tiles: no room for a second split
    assert plan(8, 4096, 12288) == (True, 16, 8)
    assert plan(8, 4096, 256) == (True, 16, 1)           # four K blocks: nothing to split
    assert plan(8, 4096, 512) == (True, 16, 2)
    # the same rows in another batch: the split does not depend on M within a width
    assert plan(1, 6144, 4096)[2] == plan(16, 6144, 4096)[2] == 4
    # a forced split replaces the plan's, up to 8 and the number of K blocks
    assert plan(8, 6144, 4096, force=3)[2] == 3
    assert plan(8, 6144, 4096, force=20)[2] == 8
    assert plan(8, 6144, 128, force=8)[2] == 2


def test_many_rows_put_x_on_the_wide_side():
    for M in (512, 2048, 3000):
        swapped, width, splits = plan(M, 6144, 4096)
        assert not swapped and splits == 1 and width in (256, 240, 224, 208, 192)
    # 16 row tiles x 4,096 outputs: 256 columns give 256 tiles (two waves of 148), 240 give 288 (two waves, cheaper tiles)
    assert plan(2048, 4096, 4096) == (False, 240, 1)
    # up to 256 rows one tile of 256 rows of x against narrow weights, K split, when whole tiles would leave SMs idle
    assert plan(200, 4096, 4096)[0] and plan(200, 4096, 4096)[1] == 256
    assert not plan(300, 4096, 4096)[0]
    # a narrow output has one width only
    assert plan(1000, 96, 72) == (False, 128, 1)


def test_the_plan_depends_on_the_number_of_sms():
    assert plan(8, 6144, 4096, sms=148)[2] == 4
    assert plan(8, 6144, 4096, sms=64)[2] == 2           # 128 places for 48 tiles
    assert plan(8, 6144, 4096, sms=20)[2] == 1
