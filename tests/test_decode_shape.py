"""How the decode attention's launch is shaped (host arithmetic only): every block resident at
once, as few tiles of keys per warp as that allows, and no more warps than that needs."""

import itertools

from strata_inference_b200.parts.attention import decode_shape

RES4, RES8 = 1776, 1184        # warps a device of 148 SMs holds: 3 blocks of 4, 1 block of 8 an SM


def _tiles(longest, window):
    return -(-longest // 16) + (1 if 0 < window <= longest else 0)


def test_all_blocks_resident_and_no_warp_idle():
    for units, longest, window in itertools.product(
            (1, 4, 8, 16, 32, 64, 100, 256, 1024), (1, 16, 17, 500, 512, 1024, 4096, 8192), (0, 512, 4096)):
        where = f"units={units} longest={longest} window={window}"
        seen = min(longest, window) if window else longest
        runs, warps = decode_shape(units, seen, window, RES4, RES8)
        assert runs >= 1 and warps in (1, 2, 4, 8) and runs <= 128, where
        resident = RES8 if warps == 8 else RES4
        # one wave: unless a single warp per (row, kv head) is already more than the device holds
        assert runs * warps * units <= resident or runs * warps == 1, where
        tiles = _tiles(seen, window)
        each = -(-tiles // (runs * warps))
        # no warp is left without a tile (a whole block at most, where blocks are wide)
        assert (runs * warps - 1) * each < tiles + each * (warps - 1), where
        # and a warp walks at most about twice the fewest tiles that residency allows (wider
        # blocks, which mean fewer partial results, may cost a tile or two), unless the number
        # of runs is at the kernel's limit
        best = -(-tiles // max(1, RES4 // units))
        assert each <= 2 * best + 1 or runs == 128, where


def test_few_rows_take_wide_blocks_and_one_tile_a_warp():
    # one row, 4 kv heads, a window of 4 096 keys that does not start at a tile's first key
    runs, warps = decode_shape(4, 4096, 4096, RES4, RES8)
    assert warps == 8 and runs * warps >= 257
    # all 8 192 keys: two tiles a warp is what residency allows, and 256 warps are enough for it
    assert decode_shape(4, 8192, 0, RES4, RES8) == (32, 8)
    # many rows: blocks of 4
    runs, warps = decode_shape(32, 8192, 0, RES4, RES8)
    assert warps == 4 and runs * 4 * 32 <= RES4


def test_a_shape_the_wide_kernel_does_not_take():
    runs, warps = decode_shape(4, 8192, 0, RES4, 0)
    assert warps == 4 and runs >= 1
