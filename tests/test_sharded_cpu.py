"""The collective logic of ShardedClosedHashmap with two CPU ranks over gloo.  The CUDA kernels are replaced by
the host restatement in oracle/routing.py; what is tested is the routing: split sizes, the two exchanges, result
order, and that the union of the shards equals one big serial table fed the ranks' batches in rank order."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import port, routing

WORLD = 2


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def batches(rank, step):
    rng = np.random.default_rng(1000 * step + rank)
    n = [700, 0, 1300][(step + rank) % 3]            # ragged, sometimes empty
    keys = rng.integers(0, 4000, size=(n, 1)).astype(np.int64)
    vals = np.stack([keys[:, 0] * 10 + rank, np.full(n, step)], axis=1).astype(np.float32)
    return keys, vals


def params():
    np.random.seed(42)
    return port.draw_hash_parameters(1 << 14, 1)


def worker(rank, port_no, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port_no))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        from doksparse_b200.sharded import ShardedClosedHashmap
        p = params()
        m = ShardedClosedHashmap(1 << 14, ops=routing.OracleShardOps(1 << 14, p), **p)
        log = []
        for step in range(4):
            keys, vals = batches(rank, step)
            m.set(torch.from_numpy(keys), torch.from_numpy(vals))
            q = np.concatenate([keys[::2], keys[:5] + 100000]) if len(keys) else np.zeros((0, 1), dtype=np.int64)
            v, f = m.get(torch.from_numpy(q), fallback_value=-1.0)
            r = m.remove(torch.from_numpy(q[::3].copy()))
            log.append((v.numpy(), f.numpy(), r.numpy(), m.n_elements))
        out[rank] = (log, m.ops.local.n_elements)
    finally:
        dist.destroy_process_group()


def test_two_rank_routing_equals_one_table():
    port_no = free_port()
    manager = mp.Manager()
    out = manager.dict()
    mp.spawn(worker, args=(port_no, out), nprocs=WORLD, join=True)
    assert sorted(out.keys()) == [0, 1]

    # the same stream on ONE serial table: per step the ranks' batches are applied in rank order
    p = params()
    single = port.OracleHashmap(n_buckets=1 << 16, **p)
    for step in range(4):
        per_rank = [batches(rank, step) for rank in range(WORLD)]
        allk = np.concatenate([k for k, _ in per_rank])
        allv = np.concatenate([v for _, v in per_rank])
        single.set(allk, allv)
        gets, removes = [], []
        for rank in range(WORLD):
            keys, _ = per_rank[rank]
            q = np.concatenate([keys[::2], keys[:5] + 100000]) if len(keys) else np.zeros((0, 1), dtype=np.int64)
            gets.append(single.get(q, fallback_value=-1.0) if len(q) else (np.zeros((0, 2), np.float32), np.zeros(0, bool)))
        for rank in range(WORLD):
            keys, _ = per_rank[rank]
            q = np.concatenate([keys[::2], keys[:5] + 100000]) if len(keys) else np.zeros((0, 1), dtype=np.int64)
            removes.append(single.remove_rows(q[::3].copy()))
        for rank in range(WORLD):
            v, f, r, n_el = out[rank][0][step]
            np.testing.assert_array_equal(f, gets[rank][1])
            np.testing.assert_array_equal(v, gets[rank][0])
            np.testing.assert_array_equal(r, removes[rank])
            assert n_el == single.n_elements
    assert sum(out[rank][1] for rank in range(WORLD)) == single.n_elements
    assert all(out[rank][1] > 0 for rank in range(WORLD))          # both shards took part


def test_owner_function_is_balanced_and_stable():
    uu = np.random.default_rng(0).integers(0, 2 ** 62, size=20000)
    for world in (2, 4, 8):
        own = routing.owners(uu, world)
        counts = np.bincount(own, minlength=world)
        assert counts.min() > 0.9 * len(uu) / world
        order, dest, c = routing.stable_partition(own, world)
        assert (np.diff(own[order]) >= 0).all() and (c == counts).all()
        for s in range(world):
            assert (np.diff(order[own[order] == s]) > 0).all()         # order within a shard is preserved
        assert (order[dest] == np.arange(len(uu))).all()
