"""Worker of tests/test_sharded_multi_gpu.py (one process per GPU, launched by torch.distributed.run).

The same operation stream goes through two sharded maps, one exchanging rows with NCCL all-to-all and one storing
them straight into fixed slices of the peers' memory (operation by operation and as pipelined submissions that the
host never waits for), and -- gathered on rank 0 -- through ONE serial CPU oracle table that receives the ranks'
batches in rank order.  Everything a caller can observe must agree bit for bit.  Batches larger than the slices, and
a skewed batch whose rows all go to one owner, take the overflow route: skipped by every rank on the device and
repeated over the all-to-all exchange.  argv[1] = value columns (default 2)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from doksparse_b200.sharded import ShardedClosedHashmap  # noqa: E402
from oracle import port  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    value_columns = int(sys.argv[1]) if len(sys.argv) > 1 else 2
    np.random.seed(7)
    params = port.draw_hash_parameters(1 << 17, 1)
    nb = 1 << 17
    cap = 30000
    via_nccl = ShardedClosedHashmap(nb, device=device, **params)
    via_peer = ShardedClosedHashmap(nb, device=device, peer_capacity_rows=cap, **params)
    single = port.OracleHashmap(n_buckets=nb * world, **params) if rank == 0 else None
    rng = np.random.default_rng(100 + rank)

    def gather(obj):
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    for step in range(7):
        n = [9000, 0, 12000, 5, 40000, 7000, 15000][(step + rank) % 7]     # 40000 rows exceed the capacity: all-to-all
        keys = rng.integers(0, 50000, size=(n, 1), dtype=np.int64)          # duplicates within and across ranks
        if step == 5 and rank == 0:
            keys[:] = 12345                              # fits the capacity, but every row goes to ONE owner: slice overflow
        values = rng.standard_normal((n, value_columns)).astype(np.float32)
        queries = rng.integers(0, 60000, size=(n // 2 + 3, 1), dtype=np.int64)
        doomed = np.unique(rng.integers(0, 60000, size=(n // 5 + 1, 1), dtype=np.int64), axis=0)
        tk, tv = torch.from_numpy(keys).to(device), torch.from_numpy(values).to(device)
        tq, td = torch.from_numpy(queries).to(device), torch.from_numpy(doomed).to(device)
        results = []
        for table in (via_nccl, via_peer):
            if table is via_peer and step % 2 == 1:      # every other step as pipelined submissions
                if step % 4 == 1:
                    _, (gv, gf), rm = table.run([("set", tk, tv), ("get", tq, -3.0), ("remove", td)])
                else:                                    # two submissions that are not waited for in between
                    _, (gv, gf) = table.run([("set", tk, tv), ("get", tq, -3.0)], wait=False)
                    (rm,) = table.run([("remove", td)], wait=False)
                    table.wait()
            else:
                table.set(tk, tv)
                gv, gf = table.get(tq, fallback_value=-3.0)
                rm = table.remove(td)
            results.append((gv.cpu().numpy(), gf.cpu().numpy(), rm.cpu().numpy(), table.n_elements))
        a, b = results
        assert np.array_equal(a[1], b[1]) and np.array_equal(a[0].view(np.uint8), b[0].view(np.uint8)), f"get differs, step {step}"
        assert a[3] == b[3], f"n_elements differ, step {step}"
        everything = gather((keys, values, queries, doomed, b[0], b[1], a[2], b[2]))
        if rank == 0:
            for k, v, *_ in everything:
                if len(k):
                    single.set(k, v)
            wanted = [single.get(e[2], fallback_value=-3.0) for e in everything]
            for e, (want_v, want_f) in zip(everything, wanted):
                assert np.array_equal(e[5], want_f), f"found flags differ from the single table, step {step}"
                assert np.array_equal(e[4].view(np.uint8), want_v.view(np.uint8)), f"values differ from the single table, step {step}"
            # removals: every key that was stored is reported by exactly ONE of the rows that ask for it (in whichever
            # rank's batch), a key that was not stored by none; which row reports is unspecified across ranks
            all_doomed = np.concatenate([e[3] for e in everything])
            distinct, inverse = np.unique(all_doomed[:, 0], return_inverse=True)
            was_stored = single.get(distinct[:, None], fallback_value=0.0)[1].astype(np.int64)
            for which in (6, 7):                         # the all-to-all exchange, the sliced exchange
                reports = np.bincount(inverse, weights=np.concatenate([e[which] for e in everything]).astype(np.float64),
                                      minlength=len(distinct)).astype(np.int64)
                assert np.array_equal(reports, was_stored), f"remove reports differ from the single table, step {step}"
            single.remove_rows(distinct[:, None])
            assert single.n_elements == b[3]
    assert via_peer._sliced_on, "the sliced exchange was not in use"
    # a shard checkpoint restored into a fresh map brings the sliced exchange up again and answers like the old one
    restored = ShardedClosedHashmap(nb, device=device, peer_capacity_rows=cap, **params)
    restored.load_state_dict(via_peer.state_dict())
    assert restored._sliced_on
    probe = torch.from_numpy(rng.integers(0, 60000, size=(5000 + rank, 1), dtype=np.int64)).to(device)
    (v1, f1), (v2, f2) = via_peer.get(probe, -1.0), restored.get(probe, -1.0)
    assert torch.equal(f1, f2) and torch.equal(v1, v2), "restored shard answers differently"
    # ranks that submit different operations find out on every rank instead of hanging
    from doksparse_b200._lib import DokError
    for table in (via_nccl, via_peer):
        try:
            if rank == 0:
                table.get(probe)
            else:
                table.remove(probe)
            raise AssertionError("mismatched operations went unnoticed")
        except DokError as exc:
            assert "different operations" in str(exc)
    restored.close()
    via_peer.close()
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("multi-gpu parity ok")


if __name__ == "__main__":
    main()
