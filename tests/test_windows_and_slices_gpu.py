"""Two launch forms that change nothing a caller can observe:

* passes over windows of the slot array (what tables beyond the TLB's reach get): forced here on small tables by
  shrinking the window, and compared with the CPU oracle and with the single-pass results;
* sliced batches (row counts read on the device) and the sliced exchange built on them: several ranks are emulated
  in ONE process on one GPU -- every rank's arena is a local allocation, the fence is a host-side maximum -- and the
  union of the shards is compared with one serial oracle table fed the ranks' batches in rank order."""
import numpy as np
import pytest
import torch

from oracle import port
from tests.helpers import assert_same_bytes, assert_same_items, dev, host
from tests.test_map_gpu import Pair, good_parameters, rand_keys, rand_values

pytestmark = pytest.mark.gpu


@pytest.fixture
def tiny_windows():
    from doksparse_b200 import _lib as L
    L.check(L.lib().dok_set_window_bytes(0, 64 * 1024), "dok_set_window_bytes")       # every table: 64 KiB windows
    yield
    L.check(L.lib().dok_set_window_bytes(72 << 30, 58 << 30), "dok_set_window_bytes")


@pytest.mark.parametrize("kdtype,ks,vdtype,vs", [(np.int64, 1, np.float32, 2), (np.int64, 2, np.float32, 1),
                                                 (np.float32, 3, np.int64, 5), (np.int32, 2, np.float64, 30)])
def test_windowed_passes_match_the_oracle(tiny_windows, kdtype, ks, vdtype, vs):
    from doksparse_b200 import _lib as L
    rng = np.random.default_rng(ks * 100 + vs)
    pair = Pair(seed=5, n_buckets=1 << 16, rehash_threshold=0.9)
    lo, hi = (0, 2 ** 20) if np.issubdtype(kdtype, np.floating) else (-2 ** 30, 2 ** 30)
    stored = rand_keys(rng, 20000, kdtype, ks, lo, hi)
    pair.set(stored, rand_values(rng, len(stored), vdtype, vs))
    assert L.lib().dok_table_passes(pair.c._c_table()) > 4, "the fixture did not force several passes"
    for step in range(4):
        fresh = rand_keys(rng, 6000, kdtype, ks, lo, hi)
        batch = np.concatenate([stored[rng.integers(0, len(stored), 6000)], fresh, fresh[:500]])     # duplicates too
        pair.set(batch, rand_values(rng, len(batch), vdtype, vs))
        pair.get(np.concatenate([batch[::3], rand_keys(rng, 3000, kdtype, ks, lo, hi)]), fallback=7)
        pair.remove(batch[rng.integers(0, len(batch), 3000)])
        stored = np.concatenate([stored, fresh])
    pair.check_items()
    pair.c.rehash(1 << 17)          # k_reinsert in passes
    pair.o.rehash(1 << 17)
    assert pair.c.n_elements == pair.o.n_elements


def test_windowed_dok_tensor_paths(tiny_windows):
    from doksparse_b200 import SparseDOKTensor
    rng = np.random.default_rng(3)
    dense = (rng.random((300, 500)) < 0.05) * rng.standard_normal((300, 500))
    dense = torch.from_numpy(dense.astype(np.float32)).cuda()
    np.random.seed(1)
    t = SparseDOKTensor.from_dense(dense)
    assert torch.equal(t.to_dense(), dense)
    i, j = torch.randint(0, 300, (5000,), device="cuda"), torch.randint(0, 500, (5000,), device="cuda")
    assert torch.equal(t[i, j], dense[i, j])
    t[i[:1000], j[:1000]] = torch.tensor(2.5, device="cuda")
    dense[i[:1000], j[:1000]] = 2.5
    assert torch.equal(t.to_dense(), dense)
    flat = t.flatten()
    assert torch.equal(flat.to_dense(), dense.flatten())


def test_sliced_operations_equal_plain_ones():
    """get / set / remove over slices with device-side counts against the same rows passed as plain batches."""
    from doksparse_b200 import CudaClosedHashmap
    rng = np.random.default_rng(11)
    params = good_parameters(1 << 16, 1, seed=3)
    plain = CudaClosedHashmap(n_buckets=1 << 16, **params)
    sliced = CudaClosedHashmap(n_buckets=1 << 16, **params)
    n_slices, rows = 3, 1024
    for step in range(3):
        counts = [[1024, 0, 517], [1, 1000, 1023], [0, 0, 300]][step]
        keys = rng.integers(0, 6000, size=(n_slices * rows, 1)).astype(np.int64)          # duplicates within and across slices
        vals = rng.standard_normal((n_slices * rows, 2)).astype(np.float32)
        used = np.concatenate([np.arange(s * rows, s * rows + c) for s, c in enumerate(counts)]).astype(np.int64)
        k, v, c = dev(keys), dev(vals), torch.tensor(counts, device="cuda")
        if step == 0:
            sliced._allocate(k.shape[1:], k.dtype, v.shape[1:], v.dtype)
        abort = torch.zeros(1, device="cuda", dtype=torch.long)
        sliced.set_sliced(k, v, n_slices, rows, c, abort)
        plain.set(k[used], v[used])
        assert sliced.n_elements == plain.n_elements
        out_v = torch.full((n_slices * rows, 2), -9.0, device="cuda")
        out_f = torch.zeros(n_slices * rows, device="cuda", dtype=torch.bool)
        probe = dev(rng.integers(0, 7000, size=(n_slices * rows, 1)).astype(np.int64))
        sliced.get_sliced(probe, n_slices, rows, c, abort, 5.0, out_v, out_f)
        want_v, want_f = plain.get(probe[used], 5.0)
        assert torch.equal(out_f[used], want_f) and torch.equal(out_v[used], want_v)
        untouched = np.setdiff1d(np.arange(n_slices * rows), used)
        assert (out_v[untouched] == -9.0).all() and not out_f[untouched].any()             # unused rows are not written
        flags = torch.zeros(n_slices * rows, device="cuda", dtype=torch.bool)
        sliced.remove_sliced(probe, n_slices, rows, c, abort, flags)
        want = plain.remove_rows(probe[used])
        assert int(flags[used].sum()) == int(want.sum()) and sliced.n_elements == plain.n_elements
        # a raised abort word turns every call into a no-op
        abort.fill_(1)
        before = sliced.n_elements
        sliced.set_sliced(k, v + 1, n_slices, rows, c, abort)
        sliced.remove_sliced(k, n_slices, rows, c, abort, flags)
        assert sliced.n_elements == before
    a, b = sliced.items(), plain.items()
    sa, sb = port.sort_items(*(host(x) for x in a)), port.sort_items(*(host(x) for x in b))
    for x, y in zip(sa, sb):
        assert_same_bytes(x, y)


class EmulatedRanks:
    """`world` ranks of the sliced exchange in one process: same kernels and arena layout as the real thing, local
    allocations instead of CUDA IPC mappings, one stream instead of fences."""

    def __init__(self, world, n_buckets, capacity, params, value_columns):
        from doksparse_b200.sharded import CudaShardOps
        self.world = world
        key_row, value_row = ((1,), torch.int64), ((value_columns,), torch.float32)
        self.ops = [CudaShardOps("cuda:0", n_buckets, params, 2.0, 0.75) for _ in range(world)]
        geometry = CudaShardOps.sliced_geometry(world, capacity, key_row, value_row)
        self.geometry = geometry
        bases = [o.sliced_alloc(geometry) for o in self.ops]
        assert all(bases)
        for r, o in enumerate(self.ops):
            o.sliced_attach(geometry, bases, r, group=False, own_base=bases[r], ipc=False)
            o.ensure_allocated(key_row, value_row)
        self.seq = 0

    def close(self):
        for o in self.ops:
            o.sliced_close()

    def _fence(self, tokens):
        """what the all-reduce does: every rank sees the maximum"""
        from doksparse_b200 import _lib as L
        top = torch.stack(tokens).max(dim=0).values
        for o, t in zip(self.ops, tokens):
            t.copy_(top)
            L.check(L.lib().dok_shard_token_finish(L.ptr(t), L.ptr(o._sx["status"]), L.stream_ptr(o.device)), "finish")

    def step(self, kind, batches, fallback=None, force=False):
        """batches[r] = (keys,) or (keys, values) of rank r -> per-rank results, or None when the step overflowed"""
        gen = self.seq % self.geometry["generations"]
        self.seq += 1
        tokens = [torch.zeros(3, device="cuda", dtype=torch.long) for _ in self.ops]
        dests = []
        for o, b, t in zip(self.ops, batches, tokens):
            dests.append(o.sliced_send(b[0], b[1] if kind == "set" else None, gen, want_dest=(kind != "set"), force_overflow=force))
            o.sliced_fence(t, 1)
        self._fence(tokens)
        out = []
        for o, t in zip(self.ops, tokens):
            if kind == "set":
                o.sliced_apply_set(gen, t[0:1], False)
            else:
                o.sliced_apply_lookup(gen, t[0:1], kind == "get", fallback)
        torch.cuda.synchronize()
        if int(tokens[0][0]) != 0:
            for o in self.ops:
                o.sliced_reset_status()
            return None
        if kind == "set":
            return [None] * self.world
        for o, d in zip(self.ops, dests):
            out.append(o.sliced_results(gen, d, kind == "get"))
        return out


@pytest.mark.parametrize("world,value_columns,routing_blocks", [(2, 2, 0), (4, 1, 0), (8, 3, 0), (4, 2, 1), (8, 1, 2)])
def test_emulated_ranks_equal_one_serial_table(world, value_columns, routing_blocks):
    """routing_blocks > 0: the partition passes run with that many blocks, each walking several tiles"""
    from doksparse_b200 import _lib as L
    params = good_parameters(1 << 15, 1, seed=world)
    cap = 6000
    L.check(L.lib().dok_set_routing_blocks(routing_blocks), "dok_set_routing_blocks")
    ranks = EmulatedRanks(world, 1 << 15, cap, params, value_columns)
    single = port.OracleHashmap(n_buckets=(1 << 15) * world, **params)
    rng = np.random.default_rng(world)
    try:
        for step in range(6):
            sizes = [[cap, 0, 1, 3000, 2049, 777, 5000, 4096][(step + r) % 8] for r in range(world)]
            keys = [rng.integers(0, 20000, size=(n, 1)).astype(np.int64) for n in sizes]
            vals = [rng.standard_normal((n, value_columns)).astype(np.float32) for n in sizes]
            qs = [rng.integers(0, 25000, size=(n // 2 + 3, 1)).astype(np.int64) for n in sizes]
            doomed = [np.unique(rng.integers(0, 25000, size=(n // 4 + 1, 1)).astype(np.int64), axis=0) for n in sizes]
            assert ranks.step("set", [(dev(k), dev(v)) for k, v in zip(keys, vals)]) is not None
            for k, v in zip(keys, vals):
                if len(k):
                    single.set(k, v)
            got = ranks.step("get", [(dev(q),) for q in qs], fallback=-3.0)
            for (gv, gf), q in zip(got, qs):
                wv, wf = single.get(q, fallback_value=-3.0)
                np.testing.assert_array_equal(host(gf), wf)
                assert_same_bytes(host(gv), wv)
            removed = ranks.step("remove", [(dev(d),) for d in doomed])
            # a stored key is reported by exactly one of the rows asking for it, in whichever rank's batch
            every = np.concatenate(doomed)[:, 0]
            distinct, inverse = np.unique(every, return_inverse=True)
            was_stored = single.get(distinct[:, None], fallback_value=0.0)[1].astype(np.int64)
            reports = np.bincount(inverse, weights=np.concatenate([host(rf) for _, rf in removed]).astype(np.float64),
                                  minlength=len(distinct)).astype(np.int64)
            np.testing.assert_array_equal(reports, was_stored)
            single.remove_rows(distinct[:, None])
            assert sum(o.local.n_elements for o in ranks.ops) == single.n_elements
        # an overflow anywhere makes every rank skip the operation: nothing changes
        before = [o.local.n_elements for o in ranks.ops]
        assert ranks.step("set", [(dev(keys[0]), dev(vals[0]))] * world, force=True) is None
        assert [o.local.n_elements for o in ranks.ops] == before
        skew = np.zeros((cap, 1), dtype=np.int64)                                   # every row to one owner: a real overflow
        assert ranks.step("set", [(dev(skew), dev(np.zeros((cap, value_columns), np.float32)))] * world) is None
        assert [o.local.n_elements for o in ranks.ops] == before
        assert ranks.step("get", [(dev(q),) for q in qs]) is not None              # the status word was reset
    finally:
        ranks.close()
        L.check(L.lib().dok_set_routing_blocks(0), "dok_set_routing_blocks")
