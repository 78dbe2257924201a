"""The plain-C restatement replays the committed reference-generated streams (tests/golden/map_streams.npz)
and must reproduce every flag, value and the live items bit for bit.  Needs no reference checkout."""
import os

import numpy as np
import pytest

from oracle import port

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "map_streams.npz")


def load_cases():
    data = np.load(GOLDEN)
    names = sorted({k.split("/")[0] for k in data.files})
    return data, names


DATA, NAMES = load_cases()


def make_oracle(name, data=DATA):
    nb, ks, vs = (int(x) for x in data[f"{name}/meta"])
    params = {k: data[f"{name}/param/{k}"] for k in ("prime1", "prime2", "alpha1", "alpha2", "beta1", "beta2")}
    o = port.OracleHashmap(n_buckets=nb, key_perm=data[f"{name}/param/key_perm"], **params)
    return o, nb


@pytest.mark.parametrize("name", NAMES)
def test_port_replays_reference_stream(name):
    o, nb = make_oracle(name)
    step = 0
    while f"{name}/step{step}/set_keys" in DATA.files:
        g = lambda key: DATA[f"{name}/step{step}/{key}"]
        keys, vals = g("set_keys"), g("set_values")
        if o._keys is None:
            o._keys = np.zeros((nb,) + keys.shape[1:], dtype=keys.dtype)
            o._values = np.zeros((nb,) + vals.shape[1:], dtype=vals.dtype)
        np.testing.assert_array_equal(o.set_rows(keys, vals), g("set_stored"))
        gv, gf = o._kernel_get(g("get_keys"), 7)
        np.testing.assert_array_equal(gf, g("get_found"))
        np.testing.assert_array_equal(gv.view(np.uint8), g("get_values").view(np.uint8))
        np.testing.assert_array_equal(o.remove_rows(g("remove_keys")), g("remove_flags"))
        ik, iv, iu = o.items_sorted()
        np.testing.assert_array_equal(iu, g("items_uuid"))
        np.testing.assert_array_equal(ik, g("items_keys").reshape(ik.shape))
        np.testing.assert_array_equal(iv.view(np.uint8), g("items_values").reshape(iv.shape).view(np.uint8))
        step += 1
    assert step == 5


def test_python_bookkeeping_rehash_and_counts():
    """n_elements / n_buckets bookkeeping of the restated Python layer: rehash trigger and size
    (cuda_closed_hashmap.py:363-366), remove on sorted unique rows (:438-454)."""
    np.random.seed(3)
    o = port.OracleHashmap(n_buckets=16)
    keys = np.arange(100, dtype=np.int64)[:, None]
    vals = np.arange(100, dtype=np.float32)[:, None]
    o.set(keys[:10], vals[:10])
    assert (o.n_elements, o.n_buckets) == (10, 16)
    o.set(keys[5:14], vals[5:14])            # 4 new -> 14 > int(0.75*16)=12 -> rehash to int(14*2)=28
    assert (o.n_elements, o.n_buckets) == (14, 28)
    v, f = o.get(keys[:20], fallback_value=-1)
    assert f[:14].all() and not f[14:].any()
    np.testing.assert_array_equal(v[:14, 0], vals[:14, 0])
    assert (v[14:] == -1).all()
    flags = o.remove(np.array([[3], [50], [3], [1]], dtype=np.int64))
    np.testing.assert_array_equal(flags, [True, True, False])      # sorted unique rows: 1, 3, 50
    assert o.n_elements == 12 and o.n_tombstones == 2
    with pytest.raises(RuntimeError):
        port.OracleHashmap(n_buckets=4).get(keys)


def test_duplicates_in_a_batch_last_row_wins_serially():
    np.random.seed(5)
    o = port.OracleHashmap(n_buckets=64)
    keys = np.array([[7], [8], [7], [9], [7]], dtype=np.int64)
    vals = np.array([[1.0], [2.0], [3.0], [4.0], [5.0]], dtype=np.float32)
    o.set(keys, vals)
    assert o.n_elements == 3
    v, f = o.get(np.array([[7], [8], [9]], dtype=np.int64))
    assert f.all()
    np.testing.assert_array_equal(v[:, 0], [5.0, 2.0, 4.0])
