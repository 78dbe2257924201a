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


@pytest.mark.parametrize("world", [2, 8])
def test_peer_scatter_places_rows_in_each_owners_buffer(world):
    """dok_shard_partition_scatter_peer on one GPU: every "owner" gets its own buffer inside an arena from
    dok_peer_alloc and a different start row; rows must land there in batch order (the multi-GPU runs hand the same
    entry point the peers' mapped arenas instead)."""
    from doksparse_b200 import _lib as L
    from doksparse_b200.sharded import CudaShardOps
    lib = L.lib()
    np.random.seed(world)
    params = port.draw_hash_parameters(1 << 20, 1)
    ops = CudaShardOps("cuda:0", 1024, params, 2.0, 0.75)
    rng = np.random.default_rng(5)
    n = 50_000
    keys = rng.integers(0, 2 ** 50, size=(n, 1)).astype(np.int64)
    vals = rng.standard_normal((n, 2)).astype(np.float32)
    tk, tv = dev(keys), dev(vals)
    owners, offsets, counts = ops.partition_count(tk, world)

    o = port.OracleHashmap(n_buckets=8, **params)
    o._keys, o._values = np.zeros((8, 1), np.int64), np.zeros((8, 1), np.float32)
    own = routing.owners(o.hash_uuid(keys)[1], world)
    np.testing.assert_array_equal(host(owners), own)
    want_counts = np.bincount(own, minlength=world)
    np.testing.assert_array_equal(host(counts[:world]), want_counts)

    region_rows = n + 64
    base = ctypes.c_void_p()
    assert lib.dok_peer_alloc(world * region_rows * 16, ctypes.byref(base)) == 0
    try:
        handle = (ctypes.c_uint8 * 64)()
        assert lib.dok_peer_export(base, handle) == 0              # the handle other processes would open
        row0 = [17 * (i + 1) for i in range(world)]
        arr = ctypes.c_void_p * world
        peer_keys = arr(*[base.value + i * region_rows * 16 for i in range(world)])
        peer_vals = arr(*[base.value + i * region_rows * 16 + region_rows * 8 for i in range(world)])
        rows = (ctypes.c_int64 * world)(*row0)
        dest = torch.empty(n, device="cuda:0", dtype=torch.long)
        L.check(lib.dok_shard_partition_scatter_peer(L.ptr(tk), 8, L.ptr(tv), 8, n, world, L.ptr(owners), L.ptr(offsets),
                                                     L.ptr(counts), peer_keys, peer_vals, rows, L.ptr(dest),
                                                     L.stream_ptr(torch.device("cuda:0"))), "scatter_peer")
        arena = torch.as_tensor(CudaShardOps._RawDeviceBytes(base.value, world * region_rows * 16), device="cuda:0")
        torch.cuda.synchronize()
        for i in range(world):
            mine = own == i
            c = int(mine.sum())
            lo = i * region_rows * 16
            got_k = arena[lo + row0[i] * 8: lo + (row0[i] + c) * 8].view(torch.int64)
            got_v = arena[lo + region_rows * 8 + row0[i] * 8: lo + region_rows * 8 + (row0[i] + c) * 8].view(torch.float32).view(c, 2)
            np.testing.assert_array_equal(host(got_k), keys[mine, 0])          # batch order inside the owner
            np.testing.assert_array_equal(host(got_v), vals[mine])
        # dest = position in this rank's own grouped order (padded segment starts), as for the local scatter
        padded = (want_counts + 15) // 16 * 16
        starts = np.concatenate([[0], np.cumsum(padded)[:-1]])
        rank_in_owner = np.zeros(n, dtype=np.int64)
        for i in range(world):
            rank_in_owner[own == i] = np.arange(int((own == i).sum()))
        np.testing.assert_array_equal(host(dest), starts[own] + rank_in_owner)
        # the count words come back through pinned memory
        assert ops.to_host(counts)[:world] == want_counts.tolist()
    finally:
        torch.cuda.synchronize()
        assert lib.dok_peer_free(base) == 0
