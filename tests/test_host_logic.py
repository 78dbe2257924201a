"""Host-side logic that needs no GPU: the random-draw bookkeeping that keeps later tensors' hash parameters in step with
the reference when an intermediate tensor is skipped, and the shape arithmetic helpers."""
import numpy as np

from doksparse_b200 import util
from oracle import port


def _state():
    s = np.random.get_state()
    return s[1].copy(), s[2]


def test_skipped_map_consumes_the_reference_draws():
    for key_size, n_buckets, n_new in ((1, 1024, 700), (3, 64, 40), (2, 1 << 20, 1)):
        np.random.seed(3)
        port.draw_hash_parameters(n_buckets, key_size)
        want = _state()
        np.random.seed(3)
        util.consume_fresh_map_draws(n_buckets, key_size, n_new)
        got = _state()
        assert (want[0] == got[0]).all() and want[1] == got[1]


def test_skipped_map_that_would_rehash_draws_twice():
    np.random.seed(9)
    port.draw_hash_parameters(1024, 2)
    port.draw_hash_parameters(int(900 * 2.0), 2)          # 900 > int(0.75 * 1024): the reference rebuilds at 1800 buckets
    want = _state()
    np.random.seed(9)
    util.consume_fresh_map_draws(1024, 2, 900)
    got = _state()
    assert (want[0] == got[0]).all() and want[1] == got[1]


def test_nothing_stored_draws_nothing():
    np.random.seed(1)
    before = _state()
    util.consume_fresh_map_draws(1024, 2, 0)
    after = _state()
    assert (before[0] == after[0]).all() and before[1] == after[1]


def test_shape_helpers():
    assert util.next_power_of_2(1) == 1 and util.next_power_of_2(10_000_000) == 1 << 24 and util.next_power_of_2(1 << 20) == 1 << 20
    assert list(util.shape_to_stride((4, 3, 2))) == [6, 2, 1]
    assert util.next_prime(14) == 17 and util.next_prime(17) in (17, 19)


def test_sliced_exchange_geometry():
    """Arena layout of the sliced exchange: slices hold the mean plus eight standard deviations of the binomial row
    count plus a constant, never more than the capacity, start on 256-row boundaries, and the regions of a generation
    do not overlap."""
    import math
    import torch
    from doksparse_b200.sharded import CudaShardOps
    key_row, value_row = ((1,), torch.int64), ((2,), torch.float32)
    for world, cap in ((2, 30000), (8, 1 << 25), (4, 100), (16, 1 << 20), (8, 1)):
        g = CudaShardOps.sliced_geometry(world, cap, key_row, value_row)
        rows = g["slice_rows"]
        mean = cap / world
        assert rows % 256 == 0 and rows >= min(cap, math.ceil(mean + 8 * math.sqrt(mean))) and rows <= (cap + 255) // 256 * 256
        assert rows <= max(256, mean + 8 * math.sqrt(mean) + 64 + 256)
        if cap >= 1 << 25:
            assert rows <= 1.005 * mean                         # the slack is a fraction of a percent for large batches
        sizes, offs = g["sizes"], g["offs"]
        assert sizes[0] >= world * rows * 8 and sizes[1] >= world * rows * 8 and sizes[2] >= world * 8
        assert sizes[3] >= world * rows * 8 and sizes[4] >= world * rows
        assert all(o % 256 == 0 for o in offs) and all(offs[i] + sizes[i] == offs[i + 1] for i in range(4))
        assert g["gen_bytes"] == offs[4] + sizes[4]
