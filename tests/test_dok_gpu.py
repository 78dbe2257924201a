"""SparseDOKTensor on the GPU against the CPU oracle: construction, fused __getitem__ / __setitem__, from_dense,
to_sparse_coo, views.  Values are moved, never computed, so every comparison is bit-exact."""
import numpy as np
import pytest
import torch

from doksparse_b200.selectors import normalise_selectors
from doksparse_b200.util import next_power_of_2
from oracle import port
from tests.helpers import assert_same_items, dev, host

pytestmark = pytest.mark.gpu


def random_coo(rng, shape, nnz, dtype=np.float32):
    flat = rng.choice(int(np.prod(shape)), size=nnz, replace=False)
    idx = np.stack(np.unravel_index(flat, shape)).astype(np.int64)
    vals = rng.standard_normal(nnz).astype(dtype)
    vals[vals == 0] = 1
    return idx, vals


class DokPair:
    """A CUDA SparseDOKTensor and an oracle map driven from the same numpy random state."""

    def __init__(self, shape, idx=None, vals=None, seed=0, dtype=torch.float32):
        from doksparse_b200 import SparseDOKTensor
        self.shape = tuple(shape)
        np.random.seed(seed)
        if idx is None:
            self.t = SparseDOKTensor(size=self.shape, dtype=dtype, device="cuda:0")
            after = np.random.get_state()
            np.random.seed(seed)
            self.o = port.OracleHashmap(n_buckets=32)
        else:
            self.t = SparseDOKTensor(size=self.shape, indices=dev(idx), values=dev(vals))
            after = np.random.get_state()
            np.random.seed(seed)
            self.o = port.OracleHashmap(n_buckets=next_power_of_2(len(vals)))
            self.o.set(np.ascontiguousarray(idx.T), vals[:, None])
        self.state = np.random.get_state()
        assert all((a == b).all() if isinstance(a, np.ndarray) else a == b for a, b in zip(after, self.state))
        self.np_dtype = np.float32 if dtype == torch.float32 else np.float64

    def cpu_selectors(self, sel):
        out, scalars = normalise_selectors(sel, self.shape, "cpu")
        return [o.numpy() for o in out], scalars

    def getitem(self, sel_cpu, sel_gpu):
        got = self.t[sel_gpu]
        sels, scalars = self.cpu_selectors(sel_cpu)
        want = port.oracle_getitem(self.o, sels, self.np_dtype)
        for i in reversed(scalars):
            if i < want.ndim and want.shape[i] == 1:
                want = want.squeeze(i)
        assert tuple(got.shape) == want.shape
        np.testing.assert_array_equal(host(got).view(np.uint8), np.ascontiguousarray(want).view(np.uint8))
        return want

    def setitem(self, sel_cpu, sel_gpu, value_cpu, value_gpu):
        np.random.set_state(self.state)
        self.t[sel_gpu] = value_gpu
        after = np.random.get_state()
        np.random.set_state(self.state)
        sels, _ = self.cpu_selectors(sel_cpu)
        port.oracle_set_items_dense(self.o, sels, np.asarray(value_cpu, dtype=self.np_dtype))
        self.state = np.random.get_state()
        np.random.set_state(after)
        self.check()

    def check(self):
        m = self.t.storage()
        assert m.n_elements == self.o.n_elements
        assert m.n_buckets == self.o.n_buckets
        assert_same_items(m, self.o)


def both_devices(x):
    return x, (x.cuda() if isinstance(x, torch.Tensor) else x)


def test_readme_identity_matrix():
    """README.md:27-39 of the reference: t[idx, idx] = 1 on an empty 100x100 tensor is the identity."""
    from doksparse_b200 import SparseDOKTensor
    for value in (1, 1.0, torch.tensor(1.0, device="cuda:0")):
        t = SparseDOKTensor(size=(100, 100), dtype=torch.float, device="cuda:0")
        idx = torch.arange(100, device="cuda:0")
        t[idx, idx] = value
        assert torch.equal(t.to_dense(), torch.eye(100, device="cuda:0"))
        assert t._nnz() == 100


def test_readme_indexing_shapes():
    """README.md:74-102: the 1-D forms and their output shapes."""
    from doksparse_b200 import SparseDOKTensor
    idx = torch.arange(10, device="cuda:0")[None]
    t = SparseDOKTensor(size=(10,), indices=idx, values=torch.arange(10.0, device="cuda:0") + 1)
    assert t[0].shape == () and t[0].item() == 1.0
    assert t[[3, 6, 9]].tolist() == [4.0, 7.0, 10.0]
    assert t[np.arange(5)].shape == (5,)
    assert t[torch.randint(10, size=(2, 2))].shape == (2, 2)
    assert t[torch.arange(10) < 5].tolist() == [1.0, 2.0, 3.0, 4.0, 5.0]
    assert t[0:5].shape == (5,)


def test_getitem_matches_oracle_2d():
    rng = np.random.default_rng(0)
    shape = (60, 70)
    idx, vals = random_coo(rng, shape, 1500)
    p = DokPair(shape, idx, vals)
    p.check()
    I = torch.from_numpy(rng.integers(0, 60, 400))
    J = torch.from_numpy(rng.integers(0, 70, 400))
    hits = p.getitem((I, J), (I.cuda(), J.cuda()))
    assert 0 < (hits != 0).sum() < 400
    p.getitem((I[:20, None], J[None, :30]), (I[:20, None].cuda(), J[None, :30].cuda()))
    p.getitem((slice(5, 25), J[:7]), (slice(5, 25), J[:7].cuda()))
    p.getitem((J[:7] % 60, slice(None)), (J[:7].cuda() % 60, slice(None)))
    p.getitem((3, slice(None)), (3, slice(None)))
    p.getitem((slice(None), 4), (slice(None), 4))
    p.getitem((slice(None),), (slice(None),))
    mask = torch.from_numpy(rng.random(60) < 0.3)
    p.getitem((mask, slice(10, 20)), (mask.cuda(), slice(10, 20)))
    dense = p.t.to_dense()
    assert torch.equal(p.t[:, :], dense)
    assert torch.equal(p.t[I.cuda(), J.cuda()], dense[I.cuda(), J.cuda()])


def test_getitem_matches_oracle_4d_config3_shape():
    """The advanced-indexing form of BASELINE config 3 at reduced extents: t[idx0[:,None,None], :s, idx2[None,:,None], mask]."""
    rng = np.random.default_rng(1)
    shape = (64, 32, 16, 8)
    idx, vals = random_coo(rng, shape, 40_000)
    p = DokPair(shape, idx, vals, seed=1)
    i0 = torch.from_numpy(rng.integers(0, 64, 12))
    i2 = torch.from_numpy(rng.integers(0, 16, 10))
    mask = torch.tensor([True, False, True, True, False, False, True, False])
    sel_cpu = (i0[:, None, None], slice(None, 6), i2[None, :, None], mask)
    sel_gpu = (i0.cuda()[:, None, None], slice(None, 6), i2.cuda()[None, :, None], mask.cuda())
    out = p.getitem(sel_cpu, sel_gpu)
    assert out.shape == (12, 10, 4, 6)
    assert (out != 0).any()


def test_setitem_matches_oracle_including_rehash_and_overcount():
    rng = np.random.default_rng(2)
    shape = (200, 300)
    p = DokPair(shape, seed=2)
    I = torch.from_numpy(rng.integers(0, 200, 500))
    J = torch.from_numpy(rng.integers(0, 300, 500))
    p.setitem((I, J), (I.cuda(), J.cuda()), 1.0, torch.tensor(1.0, device="cuda:0"))      # empty map: seed + rehash
    assert p.t.storage().n_buckets > 32
    V = torch.from_numpy(rng.standard_normal(500).astype(np.float32))
    p.setitem((I, J), (I.cuda(), J.cuda()), V.numpy(), V.cuda())                          # all present: overwrite
    I2 = torch.from_numpy(rng.integers(0, 200, 3000))
    J2 = torch.from_numpy(rng.integers(0, 300, 3000))
    I2[1500:] = I2[:1500]
    J2[1500:] = J2[:1500]                                                                # duplicates: last wins, count over-counts
    V2 = torch.from_numpy(rng.standard_normal(3000).astype(np.float32))
    p.setitem((I2, J2), (I2.cuda(), J2.cuda()), V2.numpy(), V2.cuda())
    assert p.t.storage().n_elements > int(host(p.t.storage().nonempty_mask).sum())        # the reference's over-count
    p.setitem((slice(10, 14), J[:6]), (slice(10, 14), J[:6].cuda()), 0.0, 0.0)            # zeros are stored, not erased
    row = torch.from_numpy(rng.standard_normal(6).astype(np.float32))
    p.setitem((slice(20, 24), J[:6]), (slice(20, 24), J[:6].cuda()), row.numpy()[None, :].repeat(4, 0), row.cuda())
    p.getitem((I2, J2), (I2.cuda(), J2.cuda()))


def test_from_dense_and_coo_roundtrip():
    from doksparse_b200 import SparseDOKTensor
    rng = np.random.default_rng(3)
    for shape, density, dtype in [((512, 384), 0.01, torch.float32), ((40, 50, 6), 0.2, torch.float64),
                                  ((3000,), 0.5, torch.float32), ((64, 64), 0.05, torch.int64), ((32, 32), 0.0, torch.float32)]:
        dense = torch.from_numpy(rng.standard_normal(shape)).to(dtype)
        if dtype == torch.int64:
            dense = torch.from_numpy(rng.integers(-5, 5, shape))
        dense = dense * torch.from_numpy(rng.random(shape) < density)
        dense[dense == 0] = 0                                   # no negative zeros in the expected result
        d = dense.cuda()
        np.random.seed(9)
        t = SparseDOKTensor.from_dense(d)
        nnz = int((d != 0).sum().item())
        assert t._nnz() == nnz and t.dtype == dtype
        # same table size as the reference path (ctor from the COO form, same numpy seed)
        np.random.seed(9)
        ref_path = SparseDOKTensor.from_sparse_coo(d.to_sparse())
        assert ref_path.storage().n_buckets == t.storage().n_buckets
        if nnz:      # an empty tensor never draws its hash parameters
            assert torch.equal(ref_path.storage().prime2, t.storage().prime2)
        coo = t.to_sparse_coo()
        assert coo._nnz() == nnz and (nnz == 0 or not coo.is_coalesced())
        assert torch.equal(coo.to_dense(), d)
        assert torch.equal(t.to_dense(), d)
        assert torch.equal(torch.sparse_coo_tensor(t.indices(), t.values(), shape).to_dense(), d)
        k1, v1, _ = t.storage().items()
        k2, v2, _ = ref_path.storage().items()
        a = port.sort_items(host(k1), host(v1), np.zeros(len(k1), dtype=np.int64))
        b = port.sort_items(host(k2), host(v2), np.zeros(len(k2), dtype=np.int64))
        np.testing.assert_array_equal(a[0], b[0])
        np.testing.assert_array_equal(a[1].view(np.uint8), b[1].view(np.uint8))
    neg_zero = torch.tensor([0.0, -0.0, 1.0, float("nan")], device="cuda:0")
    t = SparseDOKTensor.from_dense(neg_zero)
    assert t._nnz() == 2                                        # -0.0 == 0 is not stored, NaN is


def test_constructor_matches_oracle_and_counts():
    rng = np.random.default_rng(5)
    shape = (50, 40, 30)
    idx, vals = random_coo(rng, shape, 5000)
    p = DokPair(shape, idx, vals, seed=5)
    p.check()
    assert p.t.storage().n_buckets == 8192
    sel = (torch.from_numpy(idx[0, :100]), torch.from_numpy(idx[1, :100]), torch.from_numpy(idx[2, :100]))
    assert p.t.count_items(tuple(s.cuda() for s in sel)) == 100
    assert p.t.zero_items(tuple(s.cuda() for s in sel)) == 100
    assert p.t._nnz() == 4900 and p.t.count_items(tuple(s.cuda() for s in sel)) == 0


def test_views_clone_and_unary():
    from doksparse_b200 import SparseDOKTensor
    rng = np.random.default_rng(6)
    shape = (30, 20)
    idx, vals = random_coo(rng, shape, 200)
    np.random.seed(6)
    t = SparseDOKTensor(size=shape, indices=dev(idx), values=dev(vals))
    dense = t.to_dense()
    assert torch.equal(t.T.to_dense(), dense.T) and t.T.shape == (20, 30)
    I = torch.from_numpy(rng.integers(0, 30, 64)).cuda()
    J = torch.from_numpy(rng.integers(0, 20, 64)).cuda()
    assert torch.equal(t.T[J, I], dense[I, J])
    t.T[J[:5], I[:5]] = torch.tensor(9.0, device="cuda:0")       # a view writes the shared storage
    assert bool((t[I[:5], J[:5]] == 9).all())
    c = t.clone()
    c[I[:5], J[:5]] = torch.tensor(0.5, device="cuda:0")
    assert bool((t[I[:5], J[:5]] == 9).all())
    assert torch.equal(t.abs().to_dense(), t.to_dense().abs())
    idx3, vals3 = random_coo(rng, (6, 5, 4), 50)
    np.random.seed(1)     # a seed whose parameter draws for these small tables are not degenerate (alpha2 != 0)
    t3 = SparseDOKTensor(size=(6, 5, 4), indices=dev(idx3), values=dev(vals3))
    assert torch.equal(t3.permute(2, 0, 1).to_dense(), t3.to_dense().permute(2, 0, 1))
    assert torch.equal(t3.flatten().to_dense(), t3.to_dense().flatten())
    assert torch.equal(t3.reshape(10, 12).to_dense(), t3.to_dense().reshape(10, 12))
    assert torch.equal(torch.add(t3, t3).to_dense(), 2 * t3.to_dense())      # __torch_function__ COO fallback


def test_sparse_gather_and_sparse_assignment():
    """__spgetitem__ and assignment of sparse values (the reference's get_items / set_items_sparse), against the dense
    semantics they stand for: the gather holds exactly the stored selected positions; the assignment replaces the
    selection by the source (absent source positions become absent)."""
    from doksparse_b200 import SparseDOKTensor
    rng = np.random.default_rng(11)
    shape = (200, 300)
    idx, vals = random_coo(rng, shape, 9000)
    np.random.seed(11)
    t = SparseDOKTensor(shape, torch.from_numpy(idx).cuda(), torch.from_numpy(vals).cuda())
    rows = torch.from_numpy(rng.permutation(200)[:40]).cuda()
    cols = torch.from_numpy(rng.permutation(300)[:70]).cuda()
    sel = (rows[:, None], cols[None, :])

    gathered = t.__spgetitem__(sel)
    assert tuple(gathered.shape) == (40, 70)
    dense_selection = t[sel]
    assert torch.equal(gathered.to_dense(), dense_selection)
    n_hits = t.count_items(sel)
    assert gathered._nnz() == n_hits == int((dense_selection != 0).sum())
    assert gathered.storage().n_buckets == int(n_hits * 2.0)
    miss = t.__spgetitem__((torch.tensor([0, 1]).cuda(), torch.tensor([0, 0]).cuda()))
    assert tuple(miss.shape) == (2,) and torch.equal(miss.to_dense(), t[torch.tensor([0, 1]).cuda(), torch.tensor([0, 0]).cuda()])

    for as_torch_coo in (False, True):
        src_idx, src_vals = random_coo(rng, (40, 70), 500)
        src = SparseDOKTensor((40, 70), torch.from_numpy(src_idx).cuda(), torch.from_numpy(src_vals).cuda())
        want = t.to_dense()
        want[rows[:, None], cols[None, :]] = src.to_dense()
        live_outside = int((want != 0).sum()) - 500
        t[sel] = src.to_sparse_coo() if as_torch_coo else src
        assert torch.equal(t.to_dense(), want)
        assert torch.equal(t[sel], src.to_dense())
        assert t._nnz() == live_outside + 500                          # n_elements: what stayed plus nnz(src)
        assert t.storage().n_buckets == int(np.ceil((live_outside + 500) * 2.0 * 2))


def test_flatten_and_reshape_rekey_in_one_pass():
    """flatten / reshape through the fused re-key kernel, against the dense semantics, for plain tensors, permuted
    views and an empty tensor; the random draws stay in step with the reference's two-tensor route."""
    from doksparse_b200 import SparseDOKTensor
    from doksparse_b200.util import consume_fresh_map_draws
    rng = np.random.default_rng(21)
    shape = (12, 10, 16)
    idx, vals = random_coo(rng, shape, 700)
    np.random.seed(21)
    t = SparseDOKTensor(shape, torch.from_numpy(idx).cuda(), torch.from_numpy(vals).cuda())
    dense = t.to_dense()
    flat = t.flatten()
    assert tuple(flat.shape) == (1920,) and flat._nnz() == 700 and flat.storage().n_buckets == 1024
    assert torch.equal(flat.to_dense(), dense.flatten())
    for new_shape in ((40, 48), (2, 6, 10, 16), (1920, 1)):
        r = t.reshape(*new_shape)
        assert tuple(r.shape) == new_shape and r._nnz() == 700 and r.storage().n_buckets == 1024
        assert torch.equal(r.to_dense(), dense.reshape(new_shape))
    view = t.permute(2, 0, 1)
    assert torch.equal(view.reshape(16, 120).to_dense(), dense.permute(2, 0, 1).reshape(16, 120))
    assert torch.equal(view.flatten().to_dense(), dense.permute(2, 0, 1).flatten())
    empty = SparseDOKTensor((4, 6), device="cuda:0")
    assert empty.reshape(3, 8)._nnz() == 0 and tuple(empty.reshape(3, 8).shape) == (3, 8)

    # draws: reshape to 2-D consumes what a flattened tensor plus the reshaped one would
    np.random.seed(5)
    a = t.reshape(40, 48)
    after_reshape = np.random.get_state()[1][:8].copy(), np.random.get_state()[2]
    np.random.seed(5)
    consume_fresh_map_draws(1024, 1, 700)
    consume_fresh_map_draws(1024, 2, 700)
    expected = np.random.get_state()[1][:8].copy(), np.random.get_state()[2]
    assert (after_reshape[0] == expected[0]).all() and after_reshape[1] == expected[1]
