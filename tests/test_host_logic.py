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
