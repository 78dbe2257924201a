"""BASELINE configurations 2, 3 and 4 at their FULL sizes, checked through properties that do not need the CPU oracle
(which would take minutes at these sizes): every answer is compared with a model kept as sorted tensors on the GPU
(membership by searchsorted), conversions must round-trip, counts must add up.  Seeded synthetic inputs with the
configurations' shapes, sizes and distributions."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def lookup_model(sorted_ids, sorted_values, query_ids):
    """(values, found) of query ids against a sorted model."""
    pos = torch.searchsorted(sorted_ids, query_ids).clamp_(max=sorted_ids.numel() - 1)
    found = sorted_ids[pos] == query_ids
    values = torch.where(found, sorted_values[pos], torch.zeros((), device=query_ids.device, dtype=sorted_values.dtype))
    return values, found


def bounded_zipf(gen, n, support, s):
    """n samples from P(k) ~ (k + 1)^-s, k in [0, support): inverse CDF on a tabulated support (<= 2^22 entries), the
    tail beyond the table drawn log-uniformly, which is what the power law with s close to 1 amounts to."""
    table = min(support, 1 << 22)
    w = torch.arange(1, table + 1, device=DEV, dtype=torch.float64).pow_(-s)
    cdf = torch.cumsum(w, 0)
    head_mass = float(cdf[-1])
    tail_mass = 0.0
    if support > table:
        tail_mass = (support ** (1 - s) - table ** (1 - s)) / (1 - s) if s != 1 else float(np.log(support / table))
    u = torch.rand(n, generator=gen, device=DEV, dtype=torch.float64) * (head_mass + tail_mass)
    k = torch.searchsorted(cdf, u.clamp(max=head_mass * (1 - 1e-12)))
    in_tail = u > head_mass
    if tail_mass > 0:
        t = (u - head_mass) / tail_mass
        if s != 1:
            kt = (table ** (1 - s) + t * (support ** (1 - s) - table ** (1 - s))).pow_(1 / (1 - s))
        else:
            kt = table * torch.exp(t * np.log(support / table))
        k = torch.where(in_tail, kt.long().clamp_(table, support - 1), k)
    return k


def test_config2_two_dimensional_dok_full_size():
    from doksparse_b200 import SparseDOKTensor
    g = torch.Generator(device=DEV).manual_seed(0)
    n_rows = n_cols = 100_000
    lin = torch.unique(torch.randint(0, n_rows * n_cols, (10_600_000,), generator=g, device=DEV))
    lin = lin[torch.randperm(lin.numel(), generator=g, device=DEV)[:10_000_000]]
    assert lin.numel() == 10_000_000
    values = torch.randn(lin.numel(), generator=g, device=DEV)
    np.random.seed(0)
    t = SparseDOKTensor((n_rows, n_cols), torch.stack([lin // n_cols, lin % n_cols]), values)
    assert t.storage().n_buckets == 1 << 24 and t._nnz() == 10_000_000

    order = torch.argsort(lin)
    ids, vals = lin[order], values[order]
    i = torch.randint(0, n_rows, (4_000_000,), generator=g, device=DEV)
    j = torch.randint(0, n_cols, (4_000_000,), generator=g, device=DEV)
    out = t[i, j]
    want, found = lookup_model(ids, vals, i * n_cols + j)
    assert out.shape == (4_000_000,) and torch.equal(out, want)
    assert 2000 < int(found.sum()) < 6000                       # ~0.1 % hits

    i2 = torch.randint(0, n_rows, (4_000_000,), generator=g, device=DEV)
    j2 = torch.randint(0, n_cols, (4_000_000,), generator=g, device=DEV)
    new_ids = i2 * n_cols + j2
    _, present = lookup_model(ids, vals, new_ids)
    t[i2, j2] = 1.0
    distinct_new = torch.unique(new_ids[~present]).numel()
    live = int(t.storage().nonempty_mask.sum())
    assert live == 10_000_000 + distinct_new
    # the reference counts every absent ROW as new (duplicates over-count) and rehashes to twice that
    counted = 10_000_000 + int((~present).sum())
    assert t.storage().n_elements == counted
    assert t.storage().n_buckets == 28_000_000       # ceil((10 M stored + 4 M selected) * 2), sparse_dok_tensor_impl.py:461-462
    assert torch.equal(t[i2, j2], torch.ones(4_000_000, device=DEV))
    assert torch.equal(t[i, j], torch.where(torch.isin(i * n_cols + j, new_ids), torch.ones((), device=DEV), want))


def test_config3_four_dimensional_dok_full_size():
    from doksparse_b200 import SparseDOKTensor
    g = torch.Generator(device=DEV).manual_seed(0)
    shape = (4096, 2048, 512, 8)
    inner = shape[1] * shape[2] * shape[3]
    n_draw = 64_000_000          # the heavy rows lose many draws to duplicates
    d0 = bounded_zipf(g, n_draw, shape[0], 1.1)                  # row skew
    rest = torch.randint(0, inner, (n_draw,), generator=g, device=DEV)
    lin = torch.unique(d0 * inner + rest)
    del d0, rest
    assert lin.numel() >= 50_000_000
    lin = lin[torch.randperm(lin.numel(), generator=g, device=DEV)[:50_000_000]]
    values = torch.randn(lin.numel(), generator=g, device=DEV)
    idx = torch.stack([lin // inner, (lin // (shape[2] * shape[3])) % shape[1], (lin // shape[3]) % shape[2], lin % shape[3]])
    np.random.seed(0)
    t = SparseDOKTensor(shape, idx, values)
    del idx
    assert t.storage().n_buckets == 1 << 26 and t._nnz() == 50_000_000       # load 0.745, below the rehash threshold
    order = torch.argsort(lin)
    ids, vals = lin[order], values[order]
    del order

    idx0 = torch.randint(0, shape[0], (256,), generator=g, device=DEV)
    idx2 = torch.randint(0, shape[2], (128,), generator=g, device=DEV)
    mask = torch.tensor([True, False, True, True, False, False, True, False], device=DEV)
    out = t[idx0[:, None, None], :64, idx2[None, :, None], mask]
    assert out.shape == (256, 128, 4, 64)
    m = mask.nonzero().flatten()
    q = (idx0[:, None, None, None] * shape[1] + torch.arange(64, device=DEV)[None, None, None, :]) * shape[2]
    q = (q + idx2[None, :, None, None]) * shape[3] + m[None, None, :, None]
    want, found = lookup_model(ids, vals, q.reshape(-1))
    assert torch.equal(out.reshape(-1), want) and int(found.sum()) > 0

    coo = t.to_sparse_coo().coalesce()
    back = ((coo.indices()[0] * shape[1] + coo.indices()[1]) * shape[2] + coo.indices()[2]) * shape[3] + coo.indices()[3]
    assert torch.equal(back, ids) and torch.equal(coo.values(), vals)
    del coo, back, t

    block = torch.randn(8192, 8192, generator=g, device=DEV) * (torch.rand(8192, 8192, generator=g, device=DEV) < 0.01)
    np.random.seed(1)
    d = SparseDOKTensor.from_dense(block)
    assert d._nnz() == int((block != 0).sum()) and d.storage().n_buckets == 1 << 20
    assert torch.equal(d.to_dense(), block)


def test_config4_mixed_churn_full_size():
    """capacity 2^28 at load 0.9, 20 batches of 64 M operations (70 % get, 20 % set, 10 % remove) on Zipf(0.99) ids;
    the model is a sorted tensor of live ids, the value of an id is a function of the id."""
    from doksparse_b200 import CudaClosedHashmap
    g = torch.Generator(device=DEV).manual_seed(0)
    cap = 1 << 28
    n_fill = int(0.9 * cap)

    def value_of(ids):
        return torch.stack([(ids & 0xFFFF).float(), ((ids >> 16) & 0xFFFF).float(), ((ids >> 32) & 0xFF).float(),
                            (ids % 1000).float()], dim=1)

    np.random.seed(0)
    table = CudaClosedHashmap(n_buckets=cap, device=DEV, rehash_threshold=0.95)
    live = torch.arange(n_fill, device=DEV, dtype=torch.long) * 61 + 7          # distinct ids below 2^34
    for lo in range(0, n_fill, 1 << 26):
        part = live[lo:lo + (1 << 26)]
        table.set(part[:, None].contiguous(), value_of(part), assume_unique=True)
    assert table.n_elements == n_fill and table.n_buckets == cap
    removed_total, nb = 0, cap
    for batch in range(20):
        ids = bounded_zipf(g, 64_000_000, 1 << 34, 0.99)
        gets, sets, rems = ids[:44_800_000], ids[44_800_000:57_600_000], ids[57_600_000:]
        values, found = table.get(gets[:, None].contiguous())
        pos = torch.searchsorted(live, gets).clamp_(max=live.numel() - 1)
        want_found = live[pos] == gets
        assert torch.equal(found, want_found)
        assert torch.equal(values[found], value_of(gets[found]))
        assert not values[~found].any()
        del values, found, pos, want_found
        # the reference's rehash rule (cuda_closed_hashmap.py:363-366) on the model
        pos = torch.searchsorted(live, sets).clamp_(max=live.numel() - 1)
        n_new = torch.unique(sets[live[pos] != sets]).numel()
        if live.numel() + n_new > int(0.95 * nb):
            nb = int((live.numel() + n_new) * 2.0)
            removed_total = 0                                                        # a rehash drops the tombstones
        table.set(sets[:, None].contiguous(), value_of(sets))                       # duplicate-heavy
        live = torch.unique(torch.cat([live, sets]))
        assert table.n_elements == live.numel() and table.n_buckets == nb
        flags = table.remove(rems[:, None].contiguous())                            # reference API: sorted unique rows
        urem = torch.unique(rems)
        pos = torch.searchsorted(live, urem).clamp_(max=live.numel() - 1)
        present = live[pos] == urem
        assert torch.equal(flags, present)
        keep = torch.ones(live.numel(), device=DEV, dtype=torch.bool)
        keep[pos[present]] = False
        live = live[keep]
        removed_total += int(present.sum())
        assert table.n_elements == live.numel()
    assert table.n_tombstones <= removed_total
    k, v, _ = table.items()
    order = torch.argsort(k[:, 0])
    assert torch.equal(k[order, 0], live) and torch.equal(v[order], value_of(live))
