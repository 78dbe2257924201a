"""Routing kernels of the sharded map on one GPU against the host restatement (oracle/routing.py), and the
world-size-1 path of ShardedClosedHashmap against a plain map."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import port, routing
from tests.helpers import dev, host

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("value_columns", [3, 12])      # 12 float32 columns: rows too wide for the staged scatter
@pytest.mark.parametrize("world", [2, 8, 64])
@pytest.mark.parametrize("n", [1, 2047, 2048, 2049, 100_003])
def test_partition_matches_host_restatement(world, n, value_columns):
    from doksparse_b200.sharded import CudaShardOps
    np.random.seed(world)
    params = port.draw_hash_parameters(1 << 20, 2)
    ops = CudaShardOps("cuda:0", 1024, params, 2.0, 0.75)
    rng = np.random.default_rng(n)
    keys = rng.integers(0, 2 ** 40, size=(n, 2)).astype(np.int64)
    vals = rng.standard_normal((n, value_columns)).astype(np.float32)
    gk, gv, dest, counts = ops.partition(dev(keys), dev(vals), world)

    o = port.OracleHashmap(n_buckets=8, **params)
    o._keys, o._values = np.zeros((8, 2), np.int64), np.zeros((8, 1), np.float32)
    own = routing.owners(o.hash_uuid(keys)[1], world)
    order, want_dest, want_counts = routing.stable_partition(own, world)
    # every segment starts at a multiple of 16 rows
    padded = (want_counts + 15) // 16 * 16
    np.testing.assert_array_equal(host(counts[0]), want_counts)
    np.testing.assert_array_equal(host(counts[1]), padded)
    starts = np.concatenate([[0], np.cumsum(padded)[:-1]])
    unpadded_starts = np.concatenate([[0], np.cumsum(want_counts)[:-1]])
    want_dest_padded = want_dest + (starts - unpadded_starts)[own]
    np.testing.assert_array_equal(host(dest), want_dest_padded)
    gk_h, gv_h = host(gk), host(gv)
    np.testing.assert_array_equal(gk_h[want_dest_padded], keys)
    np.testing.assert_array_equal(gv_h[want_dest_padded], vals)
    back_v, back_f = ops.unpermute(gv, (gk[:, 0] % 2).to(torch.uint8), dest)
    np.testing.assert_array_equal(host(back_v), vals)
    np.testing.assert_array_equal(host(back_f), keys[:, 0] % 2)


def test_world_size_one_equals_plain_map():
    from doksparse_b200 import CudaClosedHashmap
    from doksparse_b200.sharded import ShardedClosedHashmap
    np.random.seed(0)
    params = port.draw_hash_parameters(1 << 18, 1)
    rng = np.random.default_rng(0)
    keys = rng.permutation(1 << 20)[:100_000].astype(np.int64)[:, None]
    vals = rng.standard_normal((100_000, 2)).astype(np.float32)
    s = ShardedClosedHashmap(1 << 18, device="cuda:0", **params)
    m = CudaClosedHashmap(n_buckets=1 << 18, **params)
    with pytest.raises(RuntimeError):
        s.get(dev(keys))
    s.set(dev(keys), dev(vals))
    m.set(dev(keys), dev(vals))
    q = dev(np.concatenate([keys[:50_000], keys[:1000] + (1 << 21)]))
    sv, sf = s.get(q, fallback_value=-3.0)
    mv, mf = m.get(q, fallback_value=-3.0)
    assert torch.equal(sv, mv) and torch.equal(sf, mf)
    assert torch.equal(s.remove(q[::2]), m.remove_rows(q[::2]))
    assert s.n_elements == m.n_elements == len(s)
