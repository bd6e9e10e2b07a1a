"""Device step tables through the C ABI, bit-exact against the oracle (src/autokernel/codegen.py:386-431)."""

import numpy as np
import pytest
from helpers import to_device, to_host

import oracle
from tilejax_b200 import ops

pytestmark = pytest.mark.gpu


def check_lengths(lengths, blocks, value0, step, tile_values=None):
    lengths = np.asarray(lengths, np.int32)
    tv = None if tile_values is None else to_device(np.asarray(tile_values, np.int32))
    tile, code, count, first = ops.build_steps(to_device(lengths), blocks, value0, step, tv)
    want_tile, want_code, want_count = oracle.device_step_tables(
        oracle.lengths_runs(lengths, blocks, value0, step, tile_values))
    np.testing.assert_array_equal(to_host(tile), want_tile)
    np.testing.assert_array_equal(to_host(code), want_code)
    assert int(count[0]) == int(want_count[0])
    first = to_host(first)
    n = int(want_count[0])
    assert first[0] == 0 and first[-1] == n
    starts = np.flatnonzero(want_code[:n] & 2)  # each tile's first step
    np.testing.assert_array_equal(first[:-1], starts)
    assert ops.device_status() == 0
    return want_tile, want_code, n


def test_the_reference_ragged_lengths():
    tile, code, n = check_lengths([0, 1, 300, 512], 4, 0, 128)
    assert n == 9 and code[:9].tolist() == [7, 3, 2, 8, 17, 2, 8, 16, 25]
    assert tile.tolist() == [0, 1, 2, 2, 2, 3, 3, 3, 3, 0, 0, 0, 1, 1, 1, 2]


@pytest.mark.parametrize(("tiles", "blocks", "step"), [(64, 256, 16), (1, 1, 16), (3, 33, 128), (1000, 7, 64),
                                                       (8192, 2, 16), (5, 2048, 1)])
def test_random_lengths(tiles, blocks, step):
    rng = np.random.default_rng(tiles * 31 + blocks)
    lengths = rng.integers(0, blocks * step + 2, tiles)  # some past the end, some empty
    lengths[rng.integers(0, tiles, max(1, tiles // 8))] = 0
    check_lengths(lengths, blocks, 0, step)


def test_all_empty_and_all_full():
    check_lengths(np.zeros(17), 9, 0, 16)
    check_lengths(np.full(17, 9 * 16), 9, 0, 16)


def test_tile_values_pick_the_length_each_tile_reads():
    # Tables repeated over an outer loop read the same lengths through tile_values (schedule.py:267).
    check_lengths([40, 0, 100], 8, 0, 16, tile_values=[2, 2, 0, 1, 0])
    check_lengths([40, 0, 100], 8, 32, 16)  # a loop that starts at 32


def test_arbitrary_run_patterns():
    rng = np.random.default_rng(3)
    for tiles, blocks, density in ((37, 19, 0.4), (8, 100, 0.05), (200, 3, 0.7), (4, 64, 0.0), (4, 64, 1.0)):
        run = rng.random((tiles, blocks)) < density
        tile, code, count, _ = ops.build_steps_from_runs(to_device(run.astype(np.uint8)))
        want_tile, want_code, want_count = oracle.device_step_tables(run)
        np.testing.assert_array_equal(to_host(tile), want_tile)
        np.testing.assert_array_equal(to_host(code), want_code)
        assert int(count[0]) == int(want_count[0])


def test_too_many_tiles_is_an_error_not_a_fallback():
    from tilejax_b200._lib import NativeError

    with pytest.raises(NativeError, match="8192 tiles"):
        ops.build_steps(to_device(np.ones(8193, np.int32)), 2, 0, 16)
