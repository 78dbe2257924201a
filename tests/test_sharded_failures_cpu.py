"""Failure handling of the sharded map's collective logic, with CPU ranks over gloo and the host stand-in for the
kernels (oracle/routing.py).  Every failure is made on the host -- a rank that raises and never joins, ranks that
submit different operations, a batch of the wrong dtype, an exchange arena that cannot be set up -- and must end in an
exception (or in the slower exchange) on every rank within a timeout, never in a hang.  No GPU is involved."""
import datetime
import os
import socket
import time

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


def params():
    np.random.seed(42)
    return port.draw_hash_parameters(1 << 12, 1)


def make_map(ops_class=routing.OracleShardOps, **kwargs):
    from doksparse_b200.sharded import ShardedClosedHashmap
    p = params()
    return ShardedClosedHashmap(1 << 12, ops=ops_class(1 << 12, p), **p, **kwargs)


def rows(rank, n=300):
    rng = np.random.default_rng(rank)
    keys = rng.integers(0, 2000, size=(n, 1)).astype(np.int64)
    return torch.from_numpy(keys), torch.from_numpy(np.stack([keys[:, 0], keys[:, 0] + rank], axis=1).astype(np.float32))


def run_ranks(worker, timeout_s=10):
    port_no = free_port()
    manager = mp.Manager()
    out = manager.dict()
    mp.spawn(worker, args=(port_no, out, timeout_s), nprocs=WORLD, join=True)
    return dict(out)


def init(rank, port_no, timeout_s):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port_no))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD, timeout=datetime.timedelta(seconds=timeout_s))


# --------------------------------------------------------------------------------------------------------------

def _mismatched_kinds(rank, port_no, out, timeout_s):
    from doksparse_b200._lib import DokError
    init(rank, port_no, timeout_s)
    try:
        m = make_map()
        keys, values = rows(rank)
        m.set(keys, values)
        try:
            if rank == 0:
                m.get(keys)
            else:
                m.remove(keys)
            out[rank] = "no error"
        except DokError as exc:
            out[rank] = str(exc)
        # the ranks are still in step: a matching pair of calls works
        v, f = m.get(keys)
        out[f"after{rank}"] = bool(f.all()) and m.n_elements > 0
    finally:
        dist.destroy_process_group()


def test_ranks_submitting_different_operations_fail_on_every_rank():
    out = run_ranks(_mismatched_kinds)
    for rank in range(WORLD):
        assert "different operations" in out[rank], out[rank]
        assert out[f"after{rank}"] is True


def _wrong_dtype(rank, port_no, out, timeout_s):
    init(rank, port_no, timeout_s)
    try:
        m = make_map()
        keys, values = rows(rank)
        m.set(keys, values)
        caught = []
        for bad in (lambda: m.get(keys.to(torch.int32)), lambda: m.remove(torch.cat([keys, keys], dim=1)),
                    lambda: m.set(keys, values.double()), lambda: m.set(keys, values[:, :1]),
                    lambda: m.run([("get", keys), ("set", keys.to(torch.int16), values)])):
            try:
                bad()
                caught.append("no error")
            except AssertionError:
                caught.append("assert")
        out[rank] = caught
        # nothing was launched or exchanged for the refused calls: the ranks are still in step
        v, f = m.get(keys)
        out[f"after{rank}"] = bool(f.all())
    finally:
        dist.destroy_process_group()


def test_batches_of_another_dtype_or_width_are_refused_before_anything_is_launched():
    out = run_ranks(_wrong_dtype)
    for rank in range(WORLD):
        assert out[rank] == ["assert"] * 5, out[rank]
        assert out[f"after{rank}"] is True


def _absent_rank(rank, port_no, out, timeout_s):
    init(rank, port_no, timeout_s)
    m = make_map()
    keys, values = rows(rank)
    m.set(keys, values)
    if rank == 1:
        # injected failure: this rank raises before the next exchange and never joins it
        out[rank] = "left"
        time.sleep(0.5)
        os._exit(0)
    t0 = time.time()
    try:
        m.set(keys, values)
        out[rank] = "no error"
    except Exception as exc:                               # gloo reports the lost peer or the timeout
        out[rank] = f"{type(exc).__name__} after {time.time() - t0:.1f} s"
    out["seconds"] = time.time() - t0
    os._exit(0)                                            # the group cannot be torn down collectively any more


def test_a_rank_that_never_joins_ends_the_exchange_with_an_error_not_a_hang():
    out = run_ranks(_absent_rank, timeout_s=8)
    assert out[1] == "left"
    assert out[0] != "no error", out[0]
    assert out["seconds"] < 60


class NoArenaOps(routing.OracleShardOps):
    """device side whose exchange arena cannot be set up (what CudaShardOps.sliced_setup reports when an allocation or
    a peer mapping fails on any rank)"""
    supports_sliced = True
    setups = 0

    def sliced_setup(self, group, world, rank, capacity_rows, key_row, value_row):
        type(self).setups += 1
        flag = torch.tensor([0 if rank == 1 else 1])
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)           # one rank failed: nobody uses the arena
        return bool(flag.item())

    def ensure_allocated(self, key_row, value_row):
        pass


def _no_arena(rank, port_no, out, timeout_s):
    init(rank, port_no, timeout_s)
    try:
        m = make_map(ops_class=NoArenaOps, peer_capacity_rows=1000)
        keys, values = rows(rank)
        m.set(keys, values)
        results = m.run([("set", keys, values + 1), ("get", keys), ("remove", keys[:50])])
        v, f = results[1]
        out[rank] = (m._sliced_on, NoArenaOps.setups, bool(f.all()), int(results[2].sum()) > 0)
    finally:
        dist.destroy_process_group()


def test_a_failed_arena_setup_leaves_the_exact_exchange_in_use_on_every_rank():
    out = run_ranks(_no_arena)
    for rank in range(WORLD):
        assert out[rank] == (False, 1, True, True), out[rank]
