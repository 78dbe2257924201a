"""The plain-C restatement (oracle/dok_oracle.c) against the reference's own kernel text compiled for
the host (oracle/_ref): identical flags, values AND identical raw storage arrays, op by op."""
import numpy as np
import pytest

from oracle import port, ref

pytestmark = pytest.mark.skipif(not ref.available(), reason="oracle/_ref not built (no reference checkout)")

COMBOS = [
    (np.int64, 1, np.float32, 1), (np.int64, 1, np.float32, 2), (np.int64, 1, np.float32, 4),
    (np.int64, 1, np.int64, 1), (np.int64, 2, np.float32, 1), (np.int64, 3, np.float32, 1),
    (np.int64, 4, np.float32, 1), (np.int64, 2, np.float64, 1), (np.int32, 2, np.float32, 3),
    (np.int16, 3, np.int32, 2), (np.float32, 3, np.int64, 5), (np.float32, 1, np.float32, 1),
    (np.float64, 2, np.float32, 1),
]


def random_keys(rng, n, dtype, ks, lo=-50, hi=50):
    if np.issubdtype(dtype, np.floating):
        return (rng.uniform(lo, hi, size=(n, ks))).astype(dtype)
    info = np.iinfo(dtype)
    return rng.integers(max(lo, info.min), min(hi, info.max), size=(n, ks)).astype(dtype)


def random_values(rng, n, dtype, vs):
    if np.issubdtype(dtype, np.floating):
        return rng.standard_normal((n, vs)).astype(dtype)
    return rng.integers(-2 ** 31, 2 ** 31, size=(n, vs)).astype(dtype)


def make_pair(n_buckets, kd, ks, vd, vs, seed, key_perm=None):
    np.random.seed(seed)
    params = port.draw_hash_parameters(n_buckets, ks)
    perm = np.arange(ks) if key_perm is None else np.asarray(key_perm)
    r = ref.RefMap(n_buckets, kd, ks, vd, vs, dict(params, key_perm=perm))
    o = port.OracleHashmap(n_buckets=n_buckets, key_perm=perm, **params)
    o._keys = np.zeros((n_buckets, ks), dtype=kd)
    o._values = np.zeros((n_buckets, vs), dtype=vd)
    return r, o


def assert_same_storage(r, o):
    np.testing.assert_array_equal(r.all_uuids, o._uuid)
    live = (r.all_uuids != -1) & (r.all_uuids != -3)
    np.testing.assert_array_equal(r.all_keys[live], o._keys[live])
    np.testing.assert_array_equal(r.all_values[live].view(np.uint8), o._values[live].view(np.uint8))


@pytest.mark.parametrize("kd,ks,vd,vs", COMBOS)
@pytest.mark.parametrize("n_buckets", [37, 256])
def test_op_stream_matches_reference(kd, ks, vd, vs, n_buckets):
    rng = np.random.default_rng(1234 + n_buckets + ks)
    r, o = make_pair(n_buckets, kd, ks, vd, vs, seed=7)
    for step in range(6):
        n = int(n_buckets * 0.3)
        keys, vals = random_keys(rng, n, kd, ks), random_values(rng, n, vd, vs)
        np.testing.assert_array_equal(r.set(keys, vals), o.set_rows(keys, vals))
        assert_same_storage(r, o)
        q = np.concatenate([keys[: n // 2], random_keys(rng, n, kd, ks)])
        rv, rf = r.get(q, fallback=step)
        ov, of = o._kernel_get(q, step)
        np.testing.assert_array_equal(rf, of)
        np.testing.assert_array_equal(rv.view(np.uint8), ov.view(np.uint8))
        dele = q[rng.permutation(len(q))[: n // 2]]
        np.testing.assert_array_equal(r.remove(dele), o.remove_rows(dele))
        assert_same_storage(r, o)


@pytest.mark.parametrize("kd,ks,vd,vs", [(np.int64, 2, np.float32, 1), (np.float32, 3, np.int64, 5)])
def test_hash_and_uuid_match_reference(kd, ks, vd, vs):
    rng = np.random.default_rng(5)
    r, o = make_pair(1024, kd, ks, vd, vs, seed=3, key_perm=list(reversed(range(ks))))
    keys = random_keys(rng, 500, kd, ks, lo=-10 ** 6, hi=10 ** 6)
    rh, ru = r.hash_uuid(keys)
    oh, ou = o.hash_uuid(keys)
    np.testing.assert_array_equal(rh, oh)
    np.testing.assert_array_equal(ru, ou)


def test_full_table_and_wraparound():
    kd, ks, vd, vs = np.int64, 1, np.float32, 1
    r, o = make_pair(16, kd, ks, vd, vs, seed=11)
    keys = np.arange(100, 140, dtype=np.int64)[:, None]
    vals = np.arange(40, dtype=np.float32)[:, None]
    rs, os_ = r.set(keys, vals), o.set_rows(keys, vals)
    np.testing.assert_array_equal(rs, os_)
    assert rs.sum() == 16 and not rs[16:].any()     # a full table refuses silently
    assert_same_storage(r, o)
    np.testing.assert_array_equal(r.get(keys)[1], o._kernel_get(keys)[1])
    np.testing.assert_array_equal(r.remove(keys[::3]), o.remove_rows(keys[::3]))
    rs, os_ = r.set(keys[20:], vals[20:]), o.set_rows(keys[20:], vals[20:])
    np.testing.assert_array_equal(rs, os_)
    assert_same_storage(r, o)


def test_float_keys_in_unit_interval_collapse():
    """The device hash casts float keys by value (closed_hashmap_impl_class.cu:88-107): every key in
    [0,1) truncates to 0, so all such keys share one uuid and one slot."""
    kd, ks, vd, vs = np.float32, 3, np.int64, 5
    r, o = make_pair(256, kd, ks, vd, vs, seed=0)
    rng = np.random.default_rng(0)
    keys = rng.random((100, 3), dtype=np.float32)
    vals = rng.integers(0, 2 ** 62, size=(100, 5))
    r.set(keys, vals), o.set_rows(keys, vals)
    assert_same_storage(r, o)
    assert ((r.all_uuids != -1).sum()) == 1
    fresh = rng.random((50, 3), dtype=np.float32)
    assert r.get(fresh)[1].all() and o._kernel_get(fresh)[1].all()


@pytest.mark.parametrize("sd,nd,vd", [(1, 2, np.float32), (2, 2, np.float32), (2, 3, np.float32), (1, 2, np.float64)])
def test_dok_kernels_match_reference(sd, nd, vd):
    """sparse_dok_count_items / set_items_dense / zero_items of the reference against the oracle's
    materialised-key equivalents."""
    rng = np.random.default_rng(21)
    n_buckets = 512
    r, o = make_pair(n_buckets, np.int64, nd, vd, 1, seed=5)
    dok = ref.RefDok(sd, nd, vd)
    shape = (24,) if sd == 1 else (6, 5)
    size = 9
    for step in range(3):
        # selectors: one contiguous, others broadcast (stride 0) views, like _handle_selectors returns
        sels = []
        for d in range(nd):
            if sd == 2 and d % 2 == 0:
                base = rng.integers(0, size, size=(shape[0], 1))
            elif sd == 2:
                base = rng.integers(0, size, size=(1, shape[1]))
            else:
                base = rng.integers(0, size, size=shape)
            sels.append(np.broadcast_to(base.astype(np.int64), shape))
        src = np.broadcast_to(rng.standard_normal((shape[-1],)).astype(vd), shape)
        keys = np.ascontiguousarray(np.stack([s.reshape(-1) for s in sels], axis=1))
        vals = np.ascontiguousarray(src.reshape(-1, 1))
        assert dok.count_items(r, sels) == o.count_exists(keys)[0]
        dok.set_items_dense(r, sels, src)
        o.set_rows(keys, vals)
        assert_same_storage(r, o)
        assert dok.count_items(r, sels) == o.count_exists(keys)[0] == keys.shape[0]
    n_removed = dok.zero_items(r, sels)
    assert n_removed == int(o.remove_rows(keys).sum())
    assert_same_storage(r, o)
