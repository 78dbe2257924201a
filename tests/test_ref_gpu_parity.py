"""This library against the reference's OWN kernels running on the same GPU (oracle/_ref/refgpu_map_*.so: the
reference's kernel text compiled by nvcc, which is what CuPy does for it at run time).  Same explicit hash
parameters, same seeded batches, bit-exact comparison of everything a caller can observe.  Set batches hold
pairwise different keys: with equal keys in one launch the reference kernels race and store duplicates."""
import numpy as np
import pytest
import torch

from oracle import port, ref_gpu
from tests.helpers import host

pytestmark = pytest.mark.gpu

CASES = [  # key dtype, key size, value dtype, value size, key range
    (torch.int64, 1, torch.float32, 2, (0, 2 ** 62)),
    (torch.int64, 1, torch.float32, 4, (0, 2 ** 34)),
    (torch.int64, 2, torch.float32, 1, (0, 100000)),
    (torch.int32, 2, torch.float32, 3, (-2 ** 20, 2 ** 20)),
    (torch.float32, 3, torch.int64, 5, (0, 2 ** 12)),          # integral floats: the value-cast stays injective
]


def sorted_items(keys, values, uuid):
    return port.sort_items(host(keys), host(values), host(uuid))


def unique_rows(rng, n, key_size, lo, hi):
    rows = np.unique(rng.integers(lo, hi, size=(int(n * 1.2), key_size), dtype=np.int64), axis=0)
    assert len(rows) >= n
    return rows[rng.permutation(len(rows))[:n]]


@pytest.mark.parametrize("kd,ks,vd,vs,key_range", CASES)
def test_same_results_as_reference_kernels_on_the_gpu(kd, ks, vd, vs, key_range):
    if not ref_gpu.available(kd, ks, vd, vs):
        pytest.skip("reference GPU kernels not built (oracle: make refgpu)")
    from doksparse_b200 import CudaClosedHashmap
    device = torch.device("cuda:0")
    rng = np.random.default_rng(2024 + ks + vs)
    nb = 1 << 18
    np.random.seed(11 + ks)
    params = port.draw_hash_parameters(nb, ks)
    while 0 in np.asarray(params["alpha2"]):                   # alpha2 = 0 makes every key alias: redraw
        params = port.draw_hash_parameters(nb, ks)
    mine = CudaClosedHashmap(n_buckets=nb, device=device, **params)
    theirs = ref_gpu.RefGpuMap(nb, kd, ks, vd, vs, params, device)

    def tk(rows):
        return torch.from_numpy(rows).to(device).to(kd).contiguous()

    def tv(n):
        if vd.is_floating_point:
            return torch.from_numpy(rng.standard_normal((n, vs))).to(device).to(vd).contiguous()
        return torch.from_numpy(rng.integers(-2 ** 62, 2 ** 62, size=(n, vs), dtype=np.int64)).to(device).contiguous()

    lo, hi = key_range
    pool = unique_rows(rng, 120000, ks, lo, hi)
    stored = pool[:60000]
    for part in np.array_split(np.arange(len(stored)), 3):     # three set batches, the last one half overwrites
        rows = stored[part]
        k, v = tk(rows), tv(len(rows))
        mine.set(k, v)
        assert bool(theirs.set(k, v).all())
    again = stored[rng.permutation(len(stored))[:20000]]
    k, v = tk(np.concatenate([again, pool[60000:70000]])), tv(30000)
    mine.set(k, v)
    assert bool(theirs.set(k, v).all())

    def compare_tables():
        a, b = sorted_items(*mine.items()), sorted_items(*theirs.items())
        for x, y in zip(a, b):
            np.testing.assert_array_equal(x.reshape(len(x), -1).view(np.uint8), y.reshape(len(y), -1).view(np.uint8))

    compare_tables()
    assert mine.n_elements == 70000

    queries = tk(np.concatenate([pool[40000:100000], unique_rows(rng, 5000, ks, lo, hi)]))
    for fallback in (None, 7):
        mv, mf = mine.get(queries, fallback)
        rv, rf = theirs.get(queries, fallback)
        assert torch.equal(mf, rf)
        assert torch.equal(mv.view(torch.uint8), rv.view(torch.uint8))

    doomed = tk(pool[50000:90000][rng.permutation(40000)])     # half present, half absent, no repeats
    assert torch.equal(mine.remove_rows(doomed), theirs.remove(doomed))
    compare_tables()
    mv, mf = mine.get(queries)
    rv, rf = theirs.get(queries)
    assert torch.equal(mf, rf) and torch.equal(mv.view(torch.uint8), rv.view(torch.uint8))

    k, v = tk(pool[80000:120000]), tv(40000)                   # re-insert over tombstones
    mine.set(k, v)
    assert bool(theirs.set(k, v).all())
    compare_tables()
    assert mine.n_elements == int(((theirs.all_uuids != -1) & (theirs.all_uuids != -3)).sum())
