"""Parity of the CUDA hash map (through the C ABI) with the CPU oracle and with the reference-generated
golden streams.  Integer / byte work: everything is compared bit-exactly."""
import os

import numpy as np
import pytest
import torch

from oracle import port
from tests.helpers import TORCH_OF, assert_same_bytes, assert_same_items, dev, host

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "map_streams.npz")


def new_maps(seed, **kwargs):
    from doksparse_b200 import CudaClosedHashmap
    np.random.seed(seed)
    c = CudaClosedHashmap(**kwargs)
    o = port.OracleHashmap(**kwargs)
    return c, o


def both(seed_state, fn_cuda, fn_oracle):
    """Runs the two implementations from the same numpy random state (parameter draws happen lazily)."""
    np.random.set_state(seed_state)
    a = fn_cuda()
    after = np.random.get_state()
    np.random.set_state(seed_state)
    b = fn_oracle()
    np.random.set_state(after)
    return a, b


class Pair:
    """A CUDA map and an oracle map that consume identical numpy random streams."""

    def __init__(self, seed=0, **kwargs):
        from doksparse_b200 import CudaClosedHashmap
        self.c = CudaClosedHashmap(**kwargs)
        self.o = port.OracleHashmap(**kwargs)
        np.random.seed(seed)
        self.state = np.random.get_state()

    def run(self, fn_cuda, fn_oracle):
        a, b = both(self.state, fn_cuda, fn_oracle)
        self.state = np.random.get_state()
        return a, b

    def set(self, keys, values, **kw):
        self.run(lambda: self.c.set(dev(keys), dev(values), **kw), lambda: self.o.set(keys, values))
        self.check_sizes()

    def get(self, keys, fallback=None):
        (cv, cf), (ov, of) = self.run(lambda: self.c.get(dev(keys), fallback), lambda: self.o.get(keys, fallback))
        np.testing.assert_array_equal(host(cf), of)
        assert_same_bytes(host(cv), ov)
        return ov, of

    def remove(self, keys):
        cr, orr = self.run(lambda: self.c.remove(dev(keys)), lambda: self.o.remove(keys))
        if np.issubdtype(keys.dtype, np.floating):
            # float keys are cast by value, so different rows share a uuid (and a slot).  Exactly one row of such a
            # group reports the removal; which one is unspecified on the GPU (the serial oracle reports the first of
            # the sorted rows), so flags are compared per uuid group.
            rows = np.unique(keys.reshape(len(keys), -1), axis=0).reshape((-1,) + keys.shape[1:])
            _, uu = self.o.hash_uuid(rows)
            order = np.argsort(uu, kind="stable")
            bounds = np.flatnonzero(np.diff(uu[order], prepend=uu[order][0] - 1))
            np.testing.assert_array_equal(np.add.reduceat(host(cr)[order].astype(int), bounds),
                                          np.add.reduceat(orr[order].astype(int), bounds))
        else:
            np.testing.assert_array_equal(host(cr), orr)
        self.check_sizes()
        return orr

    def check_sizes(self):
        assert self.c.n_elements == self.o.n_elements
        assert self.c.n_buckets == self.o.n_buckets

    def check_items(self):
        assert_same_items(self.c, self.o)
        assert self.c.n_tombstones <= self.c.n_buckets


def good_parameters(n_buckets, ks, seed):
    """Explicit hash parameters drawn like the reference draws them, rejecting alpha2 == 0 (a draw the reference
    allows and that makes a key element drop out of the uuid)."""
    np.random.seed(seed)
    while True:
        params = port.draw_hash_parameters(n_buckets, ks)
        if (params["alpha2"] != 0).all():
            return params


def rand_keys(rng, n, dtype, ks, lo, hi):
    if np.issubdtype(dtype, np.floating):
        return rng.uniform(lo, hi, size=(n, ks)).astype(dtype)
    return rng.integers(lo, hi, size=(n, ks)).astype(dtype)


def rand_values(rng, n, dtype, vs):
    if np.issubdtype(dtype, np.floating):
        return rng.standard_normal((n, vs)).astype(dtype)
    return rng.integers(-2 ** 31, 2 ** 31, size=(n, vs)).astype(dtype)


# ---------------------------------------------------------------------------------------------------------------

def test_golden_streams_from_the_reference():
    """Replays the streams recorded from the reference's own kernels (tests/golden) on the GPU."""
    from doksparse_b200 import CudaClosedHashmap
    data = np.load(GOLDEN)
    names = sorted({k.split("/")[0] for k in data.files})
    assert len(names) == 7
    for name in names:
        nb, ks, vs = (int(x) for x in data[f"{name}/meta"])
        params = {k: torch.from_numpy(data[f"{name}/param/{k}"]).cuda()
                  for k in ("prime1", "prime2", "alpha1", "alpha2", "beta1", "beta2")}
        c = CudaClosedHashmap(n_buckets=nb, key_perm=data[f"{name}/param/key_perm"].tolist(),
                              rehash_threshold=10.0, **params)     # the recorded streams never rehash
        for step in range(5):
            g = lambda key: data[f"{name}/step{step}/{key}"]
            c.set(dev(g("set_keys")), dev(g("set_values")), assume_unique=bool(step % 2))
            cv, cf = c.get(dev(g("get_keys")), 7)
            np.testing.assert_array_equal(host(cf), g("get_found"))
            assert_same_bytes(host(cv), g("get_values"))
            np.testing.assert_array_equal(host(c.remove_rows(dev(g("remove_keys")))), g("remove_flags"))
            k, v, u = c.items()
            ck, cv_, cu = port.sort_items(host(k), host(v), host(u))
            np.testing.assert_array_equal(cu, g("items_uuid"))
            np.testing.assert_array_equal(ck, g("items_keys").reshape(ck.shape))
            assert_same_bytes(cv_, g("items_values").reshape(cv_.shape))
            assert c.n_elements == len(cu)


UUID_CASES = [
    (np.int64, 1, -2 ** 62, 2 ** 62), (np.int64, 2, -10 ** 9, 10 ** 9), (np.int64, 4, 0, 5000), (np.int64, 8, -100, 100),
    (np.int32, 3, -2 ** 31, 2 ** 31 - 1), (np.int16, 2, -2 ** 15, 2 ** 15 - 1), (np.int8, 2, -128, 127),
    (np.uint8, 3, 0, 255), (np.float32, 3, -1e6, 1e6), (np.float32, 1, 0, 1), (np.float64, 2, -1e12, 1e12),
    (np.float16, 2, -1000, 1000),
]


@pytest.mark.parametrize("kd,ks,lo,hi", UUID_CASES)
def test_uuid_is_bit_identical(kd, ks, lo, hi):
    """The device uuid equals the oracle's restatement of get_uuid (closed_hashmap_impl_class.cu:98-107),
    parameter permutation included."""
    rng = np.random.default_rng(ks * 31 + 1)
    perm = list(rng.permutation(ks))
    p = Pair(seed=ks, n_buckets=4096, key_perm=perm)
    keys = rand_keys(rng, 5000, kd, ks, lo, hi)
    vals = np.zeros((5000, 1), dtype=np.float32)
    p.set(keys, vals)
    np.testing.assert_array_equal(host(p.c.device_uuid(dev(keys))), p.o.hash_uuid(keys)[1])


COMBOS = [
    (np.int64, 1, np.float32, 1, -2 ** 62, 2 ** 62), (np.int64, 1, np.float32, 2, 0, 10 ** 7),
    (np.int64, 1, np.float32, 4, 0, 10 ** 7), (np.int64, 1, np.int64, 1, 0, 10 ** 7),
    (np.int64, 2, np.float32, 1, 0, 5000), (np.int64, 3, np.float32, 1, 0, 300), (np.int64, 4, np.float32, 1, 0, 80),
    (np.int64, 2, np.float64, 1, 0, 5000), (np.int32, 2, np.float32, 3, -5000, 5000), (np.int16, 3, np.int32, 2, -150, 150),
    (np.float32, 3, np.int64, 5, -300, 300), (np.float64, 2, np.float32, 1, -5000, 5000),
    (np.int64, 1, np.uint8, 3, 0, 10 ** 7), (np.int64, 2, np.float16, 5, 0, 5000), (np.int64, 1, np.float64, 31, 0, 10 ** 7),
]


@pytest.mark.parametrize("kd,ks,vd,vs,lo,hi", COMBOS)
def test_operation_stream_matches_oracle(kd, ks, vd, vs, lo, hi):
    """set / get / remove with automatic rehashing, duplicates inside batches (last row wins), tombstone reuse:
    flags, values, remove flags, n_elements, n_buckets and the live items all equal the serial oracle.
    Tables start at 2^16 buckets: the reference draws alpha and beta below 2 * n_buckets, and with small tables the
    uuid (a product of small integers) of different multi-element keys coincides often; what happens to such keys
    depends on the slot layout, in the reference as well as here, so parity is only defined without them."""
    rng = np.random.default_rng(7 + ks + vs)
    p = Pair(seed=11 + vs, n_buckets=2 ** 16)
    for step in range(6):
        n = 30_000 + 20_000 * step
        keys, vals = rand_keys(rng, n, kd, ks, lo, hi), rand_values(rng, n, vd, vs)
        if step % 3 == 2:                                # force duplicates inside the batch
            keys[n // 2:] = keys[: n - n // 2]
        p.set(keys, vals)
        q = np.concatenate([keys[::2], rand_keys(rng, n, kd, ks, lo, hi)])
        p.get(q, fallback=None if step % 2 else 3)
        p.remove(q[rng.permutation(len(q))[: len(q) // 3]])
        p.check_items()
    assert p.c.n_buckets > 2 ** 16          # the stream grew the table at least once


def test_tiny_tables_wraparound_and_full():
    """8..64 bucket tables driven to 100 % load: probe wrap-around, tombstones are reused.  A full table stores no
    further row, like the reference (closed_hashmap_impl_class.cu:426, which drops them without a word); here the
    refused rows are counted on the device and reported once, at the next host-side read of n_elements."""
    from doksparse_b200._lib import DokError
    for nb in (8, 13, 64):
        rng = np.random.default_rng(nb)
        p = Pair(seed=nb, n_buckets=nb, rehash_threshold=100.0, **good_parameters(nb, 1, seed=nb))
        p.c._tombstone_threshold = None              # the reference's behaviour: tombstones stay (the default cleans up)
        keys = rng.permutation(10 * nb)[: 2 * nb].astype(np.int64)[:, None]
        vals = rng.standard_normal((2 * nb, 2)).astype(np.float32)
        first, second = keys[:nb], keys[nb:]
        p.set(first, vals[:nb])
        p.check_items()
        assert host(p.c._uuid != -1).all()                     # 100 % load
        ov, of = p.get(keys)
        assert of[:nb].all() and not of[nb:].any()
        # a full table: further distinct keys are not stored
        p.c.set(dev(second), dev(vals[nb:]), assume_unique=True)
        cv, cf = p.c.get(dev(second))
        assert not host(cf).any()
        assert p.c.last_set_failed == nb
        with pytest.raises(DokError, match="table was full"):
            p.c.n_elements
        assert p.c.last_set_failed == 0 and p.c.n_elements == nb      # reported once; nothing was added
        removed = p.remove(first[::2])
        assert removed.all()
        assert p.c.n_tombstones == len(first[::2])
        p.set(second[: nb // 4], vals[nb: nb + nb // 4])        # lands in tombstones
        p.check_items()
        assert p.c.n_tombstones == p.o.n_tombstones


def test_config1_shape_float_keys_collapse():
    """BASELINE config 1 as written: float32[3] keys in [0,1) -> int64[5] values, 2^21 buckets.  The value cast of
    the device hash sends every key to the same uuid, so one slot is live, every lookup hits and returns the last
    stored row, and n_elements counts distinct ROWS like the reference."""
    n = 200_000
    rng = np.random.default_rng(0)
    keys = rng.random((n, 3), dtype=np.float32)
    vals = rng.integers(0, 2 ** 63 - 1, size=(n, 5), dtype=np.int64)
    p = Pair(seed=0, n_buckets=2 ** 21)
    p.set(keys, vals)
    assert p.c.n_elements == n and int(host(p.c.nonempty_mask).sum()) == 1
    q = np.concatenate([keys[: n // 2], rng.random((n // 2, 3), dtype=np.float32)])
    ov, of = p.get(q)
    assert of.all() and (ov == vals[-1]).all()
    # all rows share the one slot: exactly one row of the removal batch reports it (which one is unspecified when the
    # rows race; the serial reference reports the first of the sorted unique rows)
    dele = keys[rng.permutation(n)[: n // 4]]
    removed = host(p.c.remove(dev(dele)))
    o_removed = p.o.remove(dele)
    assert removed.sum() == o_removed.sum() == 1 and removed.shape == o_removed.shape
    p.check_sizes()
    _, of = p.get(q)
    assert not of.any()
    p.check_items()


def test_config1_injective_float_keys():
    """Config 1 with keys floor(U(0, 2^24)) stored as float32 (the value cast is then injective): a million-row
    set, a half-present get, removal of a quarter and a re-get, all against the oracle."""
    n = 1_000_000
    rng = np.random.default_rng(1)
    keys = np.floor(rng.uniform(0, 2 ** 24, size=(n, 3))).astype(np.float32)
    vals = rng.integers(0, 2 ** 63 - 1, size=(n, 5), dtype=np.int64)
    p = Pair(seed=1, n_buckets=2 ** 21)
    p.set(keys, vals)
    fresh = np.floor(rng.uniform(0, 2 ** 24, size=(n // 2, 3))).astype(np.float32)
    q = np.concatenate([keys[: n // 2], fresh])
    p.get(q)
    p.remove(keys[rng.permutation(n)[: n // 4]])
    ov, of = p.get(q)
    assert 0.3 < of.mean() < 0.45
    p.check_items()


def test_duplicates_last_row_wins_across_blocks():
    """100k rows over 1000 distinct keys: thousands of CUDA blocks race for the same slots; the result must be the
    serial one (last row of the batch per key) and no row may be torn."""
    rng = np.random.default_rng(3)
    n = 100_000
    keys = rng.integers(0, 1000, size=(n, 2)).astype(np.int64)
    keys[:, 1] = keys[:, 0] * 7
    vals = np.repeat(np.arange(n, dtype=np.float32)[:, None], 6, axis=1)     # a torn row would mix two indices
    p = Pair(seed=3, n_buckets=4096)
    p.set(keys, vals)
    uniq = np.unique(keys, axis=0)
    ov, of = p.get(uniq)
    assert of.all() and (ov == ov[:, :1]).all()
    p.check_items()
    p.set(keys[::-1].copy(), vals)          # all keys now present: overwrite path, again last row wins
    p.get(uniq)
    p.check_items()


def test_mixed_churn_skewed_keys_high_load():
    """BASELINE config 4 at reduced size: int64 ids with a heavy-tailed (Pareto, shape 0.99) distribution -> float32[4],
    table driven to ~0.85 load with rehash_threshold 0.95, then batches of 70 % get / 20 % set / 10 % remove.  Batches
    are full of repeated ids, so this exercises last-row-wins, tombstone reuse and long chains; everything observable
    equals the serial oracle after every batch.  (The NUMBER of tombstones may differ: which tombstone a set reuses
    depends on the slot layout.)"""
    rng = np.random.default_rng(4)
    nb = 1 << 16
    p = Pair(seed=44, n_buckets=nb, rehash_threshold=0.95)
    fill = rng.permutation(1 << 22)[: int(0.85 * nb)].astype(np.int64)[:, None]
    p.set(fill, rng.standard_normal((len(fill), 4)).astype(np.float32))
    assert p.c.n_buckets == nb

    def skewed(n):
        return (rng.pareto(0.99, size=n) * 50).astype(np.int64)[:, None] % (1 << 22)

    for batch in range(6):
        p.get(np.concatenate([skewed(14_000), fill[rng.integers(0, len(fill), 14_000)]]))
        sk = skewed(8_000)
        p.set(sk, rng.standard_normal((len(sk), 4)).astype(np.float32))
        p.remove(np.concatenate([skewed(2_000), fill[rng.integers(0, len(fill), 2_000)]]))
        p.check_items()
        assert p.c.n_buckets == nb and p.c.n_tombstones > 0
    probes, hit_rate = p.c.probe_stats(dev(fill))
    assert probes >= 1.0 and 0.5 < hit_rate <= 1.0


def test_key_perm_views_share_storage():
    """A shallow clone with another key_perm sees the same slots with permuted key columns
    (cuda_closed_hashmap.py:213-231, closed_hashmap_impl_class.cu:54-63, 144-150)."""
    rng = np.random.default_rng(4)
    p = Pair(seed=4, n_buckets=1024)
    keys = rng.integers(0, 50, size=(300, 3)).astype(np.int64)
    vals = rng.standard_normal((300, 1)).astype(np.float32)
    p.set(keys, vals)
    view = p.c.clone(False)
    view.key_perm = [2, 0, 1]
    perm = np.array([2, 0, 1])
    # column i of the view's key is storage column perm[i]: a key (a,b,c) of the original is (c,a,b) in the view
    v1, f1 = p.c.get(dev(keys))
    v2, f2 = view.get(dev(keys[:, perm]))
    assert host(f1).all() and host(f2).all()
    assert_same_bytes(host(v1), host(v2))
    np.testing.assert_array_equal(host(view.keys()), host(p.c.keys())[:, perm])
    newk = rng.integers(100, 150, size=(50, 3)).astype(np.int64)
    newv = rng.standard_normal((50, 1)).astype(np.float32)
    view.set(dev(newk[:, perm]), dev(newv))
    v3, f3 = p.c.get(dev(newk))
    assert host(f3).all()
    assert_same_bytes(host(v3), newv)
    assert p.c.n_elements == view.n_elements


def test_api_surface_and_errors():
    from doksparse_b200 import CudaClosedHashmap
    m = CudaClosedHashmap()
    assert m.n_buckets == 1024 and m._empty_marker == -1 and m._removed_marker == -3
    assert m.keys() is None and m.values() is None and m._keys is None and m._values is None
    assert (host(m._uuid) == -1).all() and len(m) == 0
    keys = torch.arange(10, device="cuda")[:, None]
    with pytest.raises(RuntimeError, match="store something first"):
        m.get(keys)
    with pytest.raises(RuntimeError, match="store something first"):
        m.remove(keys)
    assert m.set(keys, torch.ones(10, 2, device="cuda")) is None
    m[keys + 10] = torch.zeros(10, 2, device="cuda")
    values, found = m[torch.arange(30, device="cuda")[:, None]]
    assert values.shape == (30, 2) and found.dtype == torch.bool and found.sum().item() == 20
    assert m.key_shape == (1,) and m.value_shape == (2,) and m.key_type == torch.long and m.value_type == torch.float32
    assert m._keys.shape == (1024, 1) and m._values.shape == (1024, 2) and m._uuid.shape == (1024,)
    e_v, e_f = m.get(keys[:0])
    assert e_v.shape == (0, 2) and e_f.shape == (0,)
    assert m.remove(keys[:0]).shape == (0,)
    m.set(keys[:0], torch.ones(0, 2, device="cuda"))
    with pytest.raises(AssertionError):
        m.get(keys.int())
    with pytest.raises(AssertionError):
        m.set(keys, torch.ones(10, 3, device="cuda"))
    del m[keys]
    assert m.n_elements == 10 and abs(m.load_factor - 10 / 1024) < 1e-12
    # in-place edits through the public storage views reach the table
    m._values.mul_(0).add_(5)
    assert (host(m.values()) == 5).all()
    d = m.clone(deepclone=True)
    d.remove(keys + 10)
    assert d.n_elements == 0 and m.n_elements == 10
    m.rehash(5000)
    assert m.n_buckets == 5000 and m.n_elements == 10 and m.n_tombstones == 0
    assert (host(m.get(keys + 10)[0]) == 5).all()


def test_large_roundtrip_properties():
    """Size-independent properties at 2^24 rows (no oracle): every stored key is found with its value, absent keys
    are not, removed keys disappear, counters are exact."""
    from doksparse_b200 import CudaClosedHashmap
    n = 1 << 24
    g = torch.Generator(device="cuda").manual_seed(0)
    keys = torch.randperm(1 << 26, device="cuda", generator=g)[:n][:, None] * 64 + 5
    vals = torch.stack([keys[:, 0].float(), (keys[:, 0] % 977).float()], dim=1)
    np.random.seed(0)
    m = CudaClosedHashmap(n_buckets=1 << 25)
    m.set(keys, vals)
    assert m.n_elements == n and m.n_buckets == 1 << 25
    v, f = m.get(keys)
    assert bool(f.all()) and torch.equal(v, vals)
    v, f = m.get(keys + 1, fallback_value=-2.0)
    assert not bool(f.any()) and bool((v == -2).all())
    flags = m.remove_rows(keys[: n // 2])
    assert bool(flags.all()) and m.n_elements == n - n // 2
    v, f = m.get(keys)
    assert int(f.sum().item()) == n - n // 2 and not bool(f[: n // 2].any())
    m.set(keys[: n // 4], vals[: n // 4], assume_unique=True)
    assert m.n_elements == n - n // 2 + n // 4
    k2, v2, u2 = m.items()
    assert k2.shape[0] == m.n_elements
    assert torch.equal(torch.sort(k2[:, 0]).values, torch.sort(torch.cat([keys[: n // 4, 0], keys[n // 2:, 0]])).values)


def test_tombstone_aware_maintenance():
    """With a tombstone threshold the table is rebuilt in place once live + tombstone slots exceed it: tombstones go;
    contents, size and hash parameters stay.  With None (the reference's behaviour) tombstones only accumulate."""
    from doksparse_b200 import CudaClosedHashmap
    rng = np.random.default_rng(3)
    nb = 1 << 16
    pool = rng.permutation(1 << 20)[:60000].astype(np.int64)[:, None]
    values = rng.standard_normal((60000, 2)).astype(np.float32)
    tables, first_prime = {}, {}
    for name, threshold in (("plain", None), ("maintained", 0.4)):
        np.random.seed(4)
        table = CudaClosedHashmap(n_buckets=nb, device="cuda:0", rehash_threshold=0.9, tombstone_threshold=threshold)
        live = {}
        for lo in range(0, 60000, 10000):                     # a sliding window: insert 10 k, remove the 10 k before
            k, v = pool[lo:lo + 10000], values[lo:lo + 10000]
            table.set(dev(k), dev(v))
            first_prime.setdefault(name, int(table.prime2[0]))
            live.update({int(a): tuple(b) for a, b in zip(k[:, 0], v)})
            if lo >= 10000:
                old = pool[lo - 10000:lo]
                flags = table.remove_rows(dev(old))
                assert bool(flags.all())
                for a in old[:, 0]:
                    del live[int(a)]
            assert table.n_buckets == nb and table.n_elements == len(live)
            assert table.n_tombstones <= table.tombstone_bound
        keys, vals, _ = table.items()
        got = {int(a): tuple(b) for a, b in zip(host(keys)[:, 0], host(vals))}
        assert got == live
        tables[name] = table
    # a rebuild keeps the hash parameters and draws nothing from the random state
    assert int(tables["plain"].prime2[0]) == first_prime["plain"]
    assert int(tables["maintained"].prime2[0]) == first_prime["maintained"] == first_prime["plain"]
    assert tables["maintained"].n_tombstones < tables["plain"].n_tombstones
    assert tables["maintained"].n_elements + tables["maintained"].n_tombstones <= 0.4 * nb + 10000


def test_default_maintenance_keeps_a_churned_table_from_running_out_of_empty_slots():
    """Insert / remove churn at high load uses up the empty slots of a table that never rebuilds (the reference's
    behaviour, tombstone_threshold=None): in the end a miss walks the whole table.  The default rebuilds in place
    before that, with identical answers."""
    from doksparse_b200 import CudaClosedHashmap
    rng = np.random.default_rng(5)
    nb = 1 << 12
    params = good_parameters(nb, 1, seed=9)
    plain = CudaClosedHashmap(n_buckets=nb, device="cuda:0", rehash_threshold=2.0, tombstone_threshold=None, **params)
    kept = CudaClosedHashmap(n_buckets=nb, device="cuda:0", rehash_threshold=2.0, **params)
    base = np.unique(rng.integers(0, 1 << 30, size=4000))[:3000].astype(np.int64)[:, None]
    for t in (plain, kept):
        t.set(dev(base), dev(np.ones((3000, 1), np.float32)))
    for step in range(100):                                 # 500 fresh keys in, the same 500 out again
        fresh = np.unique(rng.integers(0, 1 << 30, size=700))[:500].astype(np.int64)[:, None] + (1 << 31) + (step << 32)
        for t in (plain, kept):
            t.set(dev(fresh), dev(np.full((500, 1), step, np.float32)))
            assert bool(t.remove_rows(dev(fresh)).all())
    assert plain.n_tombstones + plain.n_elements >= 0.99 * nb          # no empty slot left to stop a miss
    assert kept.n_tombstones + kept.n_elements <= 0.95 * nb + 500
    probe = dev(rng.integers(0, 1 << 30, size=(2000, 1)).astype(np.int64) + (1 << 50))
    (pv, pf), (kv, kf) = plain.get(probe), kept.get(probe)
    assert not pf.any() and not kf.any()
    assert plain.probe_stats(probe)[0] > 4 * kept.probe_stats(probe)[0]           # groups walked per miss
    (pv, pf), (kv, kf) = plain.get(dev(base)), kept.get(dev(base))
    assert pf.all() and kf.all() and torch.equal(pv, kv)


def test_state_dict_round_trip(tmp_path):
    """A map rebuilt from its state_dict answers like the original (same uuids: same parameters), whatever the slot
    layout did in between; tombstones are gone."""
    from doksparse_b200 import CudaClosedHashmap
    rng = np.random.default_rng(8)
    np.random.seed(8)
    table = CudaClosedHashmap(n_buckets=1 << 15, device="cuda:0")
    keys = np.unique(rng.integers(0, 1 << 40, size=(12000, 2), dtype=np.int64), axis=0)
    values = rng.standard_normal((len(keys), 3)).astype(np.float32)
    table.set(dev(keys), dev(values))
    table.remove_rows(dev(keys[:3000]))
    path = tmp_path / "map.pt"
    torch.save(table.state_dict(), path)
    again = CudaClosedHashmap.from_state_dict(torch.load(path), device="cuda:0")
    assert again.n_elements == table.n_elements == len(keys) - 3000 and again.n_buckets == table.n_buckets
    assert again.n_tombstones == 0 < table.n_tombstones
    queries = dev(np.concatenate([keys[::3], keys[:10] + 1]))
    for a, b in zip(table.get(queries, -1.0), again.get(queries, -1.0)):
        assert torch.equal(a, b)
    ka, va, ua = (host(x) for x in table.items())
    kb, vb, ub = (host(x) for x in again.items())
    for x, y in zip(port.sort_items(ka, va, ua), port.sort_items(kb, vb, ub)):
        np.testing.assert_array_equal(x, y)
    empty = CudaClosedHashmap.from_state_dict(CudaClosedHashmap(n_buckets=64, device="cuda:0").state_dict())
    assert empty.n_elements == 0 and empty.n_buckets == 64
