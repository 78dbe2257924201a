"""Extra legs of bench.py on one GPU: BASELINE.json configs 1' (the throughput variant of config 1), 2, 3 and 4 at
their full sizes, each with its operation rates and the fraction of the HBM byte roofline of its byte model
(bytes per operation as in bench.algorithmic_bytes; streaming passes = bytes read + bytes written).  Seeded synthetic
inputs with the configurations' shapes, sizes and value distributions; none of this is in the timed headline.

The reference's own kernels are not run on these configurations: 2, 3 and the 2^31-key table exceed its 32-bit
indices, and at config 4's load of 0.9 its bucket hash -- a value in [0, prime1), prime1 between n_buckets and
2 * n_buckets, folded with `% n_buckets` (closed_hashmap_impl_class.cu:87-96, cuda_closed_hashmap.py:66-76), which
doubles the key density of the first prime1 - n_buckets buckets -- overfills that part of the table, so that one probe
cluster spans a large share of it and the pre-fill alone did not finish within a quarter of an hour on a B200."""
import time

import numpy as np

M62 = (1 << 62) - 1


def _mix62(x):
    x = (x * 0x2545F4914F6CDD1D) & M62
    x = x ^ (x >> 29)
    x = (x * 0x1B03738712FAD5C9) & M62
    x = x ^ (x >> 32)
    return x


def _timed(torch, fn, reps, warm=1):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


def _rate(rows, ms, bytes_per_row, peak):
    return {"ms": ms, "mops": rows / (ms * 1e-3) / 1e6, "bytes_per_op": bytes_per_row,
            "frac": bytes_per_row * rows / (ms * 1e-3) / 1e9 / peak}


def bounded_zipf(torch, gen, n, support, s, device):
    """n samples from P(k) ~ (k + 1)^-s, k in [0, support): inverse CDF on a tabulated head (<= 2^22 entries), the tail
    beyond the table drawn from the continuous power law."""
    table = min(support, 1 << 22)
    w = torch.arange(1, table + 1, device=device, dtype=torch.float64).pow_(-s)
    cdf = torch.cumsum(w, 0)
    head_mass = float(cdf[-1])
    tail_mass = 0.0
    if support > table:
        tail_mass = (support ** (1 - s) - table ** (1 - s)) / (1 - s) if s != 1 else float(np.log(support / table))
    u = torch.rand(n, generator=gen, device=device, dtype=torch.float64) * (head_mass + tail_mass)
    k = torch.searchsorted(cdf, u.clamp(max=head_mass * (1 - 1e-12)))
    if tail_mass > 0:
        t = (u - head_mass) / tail_mass
        kt = (table ** (1 - s) + t * (support ** (1 - s) - table ** (1 - s))).pow_(1 / (1 - s))
        k = torch.where(u > head_mass, kt.long().clamp_(table, support - 1), k)
    return k


# ---------------------------------------------------------------------------------------------------------------
# config 1': float32[3] keys (integers below 2^24, so that the kernels' value cast is injective) -> int64[5]
# ---------------------------------------------------------------------------------------------------------------

C1_KEYS_LOG2, C1_BATCH_LOG2 = 26, 25


def c1_keys(torch, idx):
    m = _mix62(idx)
    return torch.stack([(m & 0xFFFFFF), ((m >> 24) & 0xFFFFFF), ((m >> 48) & 0x3FFF)], dim=1).float().contiguous()


def c1_values(torch, idx):
    return (idx[:, None] * torch.arange(1, 6, device=idx.device)[None, :]).contiguous()


def c1_batches(torch, device):
    n_keys, q = 1 << C1_KEYS_LOG2, 1 << C1_BATCH_LOG2
    g = torch.Generator(device=device).manual_seed(1)
    hit = (torch.arange(q // 2, device=device) * 7919 + 13) % n_keys
    absent = (1 << 40) + torch.arange(q // 2, device=device)
    perm = torch.randperm(q, device=device, generator=g)
    idx = torch.cat([hit, absent])[perm]
    doomed = (torch.arange(1 << 23, device=device) * 104729 + 5) % n_keys
    return idx, absent, doomed


def config1_prime(torch, device, peak):
    from doksparse_b200 import CudaClosedHashmap
    from bench import algorithmic_bytes
    n_keys, q = 1 << C1_KEYS_LOG2, 1 << C1_BATCH_LOG2
    np.random.seed(1)
    table = CudaClosedHashmap(n_buckets=1 << (C1_KEYS_LOG2 + 1), device=device, rehash_threshold=0.95)
    for lo in range(0, n_keys, 1 << 24):
        idx = torch.arange(lo, lo + (1 << 24), device=device)
        table.set_rows(c1_keys(torch, idx), c1_values(torch, idx), assume_unique=True)
    assert table.n_elements == n_keys
    idx, absent, doomed = c1_batches(torch, device)
    keys, values = c1_keys(torch, idx), c1_values(torch, idx)
    absent_keys, doomed_keys = c1_keys(torch, absent), c1_keys(torch, doomed)
    got, found = table.get(keys)
    ok = bool(torch.equal(found, idx < (1 << 40))) and bool(torch.equal(got[found], values[found]))
    get_ms = _timed(torch, lambda: table.get(keys), 5)

    def set_and_undo():
        table.set_rows(keys, values)
    set_ms = _timed(torch, set_and_undo, 1, warm=0)                # first: half the rows are inserts
    undo_ms = _timed(torch, lambda: table.remove_rows(absent_keys), 1, warm=0)
    remove_ms = _timed(torch, lambda: table.remove_rows(doomed_keys), 1, warm=0)
    ok = ok and table.n_elements == n_keys - (1 << 23)
    # the drop-in calls, with the reference's bookkeeping (row-wise unique on float keys, host read of n_elements)
    t0 = time.perf_counter(); table.set(keys, values); torch.cuda.synchronize(); api_set_ms = (time.perf_counter() - t0) * 1e3
    t0 = time.perf_counter(); table.remove(absent_keys); torch.cuda.synchronize(); api_remove_ms = (time.perf_counter() - t0) * 1e3
    return {"what": f"float32[3] -> int64[5], 2^{C1_KEYS_LOG2} keys in 2^{C1_KEYS_LOG2 + 1} buckets of 64 bytes, batches of 2^{C1_BATCH_LOG2}",
            "results_ok": ok,
            "get_50pct_hits": _rate(q, get_ms, algorithmic_bytes("get", 12, 40, 0.5), peak),
            "set_50pct_inserts_kernel_only": _rate(q, set_ms, algorithmic_bytes("set", 12, 40), peak),
            "remove_kernel_only": _rate(1 << 23, remove_ms, algorithmic_bytes("remove", 12, 40), peak),
            "remove_of_inserted_kernel_only_ms": undo_ms,
            "set_drop_in_ms": api_set_ms, "remove_drop_in_ms": api_remove_ms}


# ---------------------------------------------------------------------------------------------------------------
# config 2: 2-D DOK tensor, 10 M nnz; config 3: 4-D DOK tensor, 50 M nnz
# ---------------------------------------------------------------------------------------------------------------

def config2(torch, device, peak):
    from doksparse_b200 import SparseDOKTensor
    g = torch.Generator(device=device).manual_seed(0)
    n_rows = n_cols = 100_000
    lin = torch.unique(torch.randint(0, n_rows * n_cols, (10_600_000,), generator=g, device=device))
    lin = lin[torch.randperm(lin.numel(), generator=g, device=device)[:10_000_000]]
    values = torch.randn(lin.numel(), generator=g, device=device)
    indices = torch.stack([lin // n_cols, lin % n_cols])
    np.random.seed(0)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    t = SparseDOKTensor((n_rows, n_cols), indices, values)
    torch.cuda.synchronize()
    build_ms = (time.perf_counter() - t0) * 1e3
    i = torch.randint(0, n_rows, (4_000_000,), generator=g, device=device)
    j = torch.randint(0, n_cols, (4_000_000,), generator=g, device=device)
    get_ms = _timed(torch, lambda: t[i, j], 10, warm=2)
    i2 = torch.randint(0, n_rows, (4_000_000,), generator=g, device=device)
    j2 = torch.randint(0, n_cols, (4_000_000,), generator=g, device=device)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    t[i2, j2] = 1.0                                           # the reference rehashes to 28,000,000 buckets here
    torch.cuda.synchronize()
    set_rehash_ms = (time.perf_counter() - t0) * 1e3
    buckets = t.storage().n_buckets
    set_ms = _timed(torch, lambda: t.__setitem__((i2, j2), 1.0), 5, warm=1)       # steady state: all rows present
    return {"what": "100000 x 100000 float32 DOK tensor, 10 M nnz, 4 M-element selectors",
            "constructor": _rate(10_000_000, build_ms, 84, peak),
            "getitem_fused": _rate(4_000_000, get_ms, 52, peak),
            "setitem_with_rehash_ms": set_rehash_ms, "n_buckets_after_setitem": buckets,
            "setitem_fused_steady": _rate(4_000_000, set_ms, 84, peak)}


def config3(torch, device, peak):
    from doksparse_b200 import SparseDOKTensor
    g = torch.Generator(device=device).manual_seed(0)
    shape = (4096, 2048, 512, 8)
    inner = shape[1] * shape[2] * shape[3]
    d0 = bounded_zipf(torch, g, 64_000_000, shape[0], 1.1, device)
    rest = torch.randint(0, inner, (64_000_000,), generator=g, device=device)
    lin = torch.unique(d0 * inner + rest)
    del d0, rest
    lin = lin[torch.randperm(lin.numel(), generator=g, device=device)[:50_000_000]]
    values = torch.randn(lin.numel(), generator=g, device=device)
    idx = torch.stack([lin // inner, (lin // (shape[2] * shape[3])) % shape[1], (lin // shape[3]) % shape[2], lin % shape[3]])
    del lin
    np.random.seed(0)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    t = SparseDOKTensor(shape, idx, values)
    torch.cuda.synchronize()
    build_ms = (time.perf_counter() - t0) * 1e3
    nnz = idx.shape[1]
    del idx, values
    idx0 = torch.randint(0, shape[0], (256,), generator=g, device=device)
    idx2 = torch.randint(0, shape[2], (128,), generator=g, device=device)
    mask = torch.tensor([True, False, True, True, False, False, True, False], device=device)
    out = t[idx0[:, None, None], :64, idx2[None, :, None], mask]
    elements = out.numel()
    get_ms = _timed(torch, lambda: t[idx0[:, None, None], :64, idx2[None, :, None], mask], 10, warm=2)
    coo_ms = _timed(torch, lambda: t.to_sparse_coo(), 3, warm=1)
    coo_bytes = 8 * t.storage().n_buckets + nnz * 2 * 36          # tags read, (4 indices + value) read and written
    del t, out
    block = torch.randn(8192, 8192, generator=g, device=device) * (torch.rand(8192, 8192, generator=g, device=device) < 0.01)
    np.random.seed(1)
    dense_ms = _timed(torch, lambda: SparseDOKTensor.from_dense(block), 5, warm=1)
    dense_nnz = int((block != 0).sum())
    dense_bytes = block.numel() * 4 + dense_nnz * 84
    return {"what": "4096 x 2048 x 512 x 8 float32 DOK tensor, 50 M nnz (row skew Zipf 1.1)",
            "constructor": _rate(nnz, build_ms, 116, peak),
            "getitem_advanced_fused": {**_rate(elements, get_ms, 36, peak), "shape": [256, 128, 4, 64]},
            "to_sparse_coo": {"ms": coo_ms, "model_bytes": coo_bytes, "frac": coo_bytes / (coo_ms * 1e-3) / 1e9 / peak,
                              "model_ms_at_8TBs": coo_bytes / 8e12 * 1e3},
            "from_dense_8192x8192_1pct": {"ms": dense_ms, "nnz": dense_nnz, "model_bytes": dense_bytes,
                                           "frac": dense_bytes / (dense_ms * 1e-3) / 1e9 / peak,
                                           "model_ms_at_8TBs": dense_bytes / 8e12 * 1e3}}


# ---------------------------------------------------------------------------------------------------------------
# config 4: churn at load 0.9 on Zipf(0.99) ids
# ---------------------------------------------------------------------------------------------------------------

C4_CAP = 1 << 28


def c4_value_of(torch, ids):
    return torch.stack([(ids & 0xFFFF).float(), ((ids >> 16) & 0xFFFF).float(), ((ids >> 32) & 0xFF).float(),
                        (ids % 1000).float()], dim=1)


def config4(torch, device, peak, batches=20):
    from doksparse_b200 import CudaClosedHashmap
    from bench import algorithmic_bytes
    g = torch.Generator(device=device).manual_seed(0)
    n_fill = int(0.9 * C4_CAP)
    np.random.seed(0)
    table = CudaClosedHashmap(n_buckets=C4_CAP, device=device, rehash_threshold=0.95)
    live = torch.arange(n_fill, device=device, dtype=torch.long) * 61 + 7
    for lo in range(0, n_fill, 1 << 26):
        part = live[lo:lo + (1 << 26)]
        table.set(part[:, None].contiguous(), c4_value_of(torch, part), assume_unique=True)
    del live
    per_batch = {"get_ms": [], "set_ms": [], "remove_kernel_ms": [], "remove_drop_in_ms": [], "tombstones_after_batch": [],
                 "n_elements_after_batch": [], "n_buckets_after_batch": [], "mean_probe_groups": []}
    for batch in range(batches):
        ids = bounded_zipf(torch, g, 64_000_000, 1 << 34, 0.99, device)
        gets = ids[:44_800_000, None].contiguous()
        sets = ids[44_800_000:57_600_000, None].contiguous()
        rems = ids[57_600_000:, None].contiguous()
        set_values = c4_value_of(torch, sets[:, 0])
        del ids
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        ev[0].record()
        table.get(gets)
        ev[1].record()
        table.set(sets, set_values)                      # drop-in call: duplicate-heavy batch, exact rehash rule
        ev[2].record()
        flags = table.remove(rems)                       # drop-in call: flags for the sorted unique rows
        ev[3].record()
        torch.cuda.synchronize()
        per_batch["get_ms"].append(ev[0].elapsed_time(ev[1]))
        per_batch["set_ms"].append(ev[1].elapsed_time(ev[2]))
        per_batch["remove_drop_in_ms"].append(ev[2].elapsed_time(ev[3]))
        per_batch["tombstones_after_batch"].append(table.n_tombstones)
        per_batch["n_elements_after_batch"].append(table.n_elements)
        per_batch["n_buckets_after_batch"].append(table.n_buckets)
        if batch in (0, batches - 1):
            per_batch["mean_probe_groups"].append(table.probe_stats(gets[: 1 << 22])[0])
        del flags
    # kernel-only removal of a batch that is in the table (the drop-in call above spends its time in the row sort)
    rems_u = rems.unique(dim=0)
    table.set_rows(rems_u, c4_value_of(torch, rems_u[:, 0]))
    per_batch["remove_kernel_ms"] = _timed(torch, lambda: table.remove_rows(rems_u), 1, warm=0)
    mean = lambda xs: float(np.mean(xs))
    return {"what": "int64 Zipf(0.99) ids over 2^34 -> float32[4], 2^28 buckets pre-filled to load 0.9, "
                    f"{batches} batches of 44.8 M get + 12.8 M set + 6.4 M remove (drop-in calls)",
            "get": _rate(44_800_000, mean(per_batch["get_ms"]), algorithmic_bytes("get", 8, 16, 0.8), peak),
            "set_drop_in": _rate(12_800_000, mean(per_batch["set_ms"]), algorithmic_bytes("set", 8, 16), peak),
            "remove_drop_in": _rate(6_400_000, mean(per_batch["remove_drop_in_ms"]), algorithmic_bytes("remove", 8, 16), peak),
            "remove_kernel_only": _rate(int(rems_u.shape[0]), per_batch["remove_kernel_ms"], algorithmic_bytes("remove", 8, 16), peak),
            "tombstones_after_batch": per_batch["tombstones_after_batch"],
            "n_elements_after_batch": per_batch["n_elements_after_batch"],
            "n_buckets_after_batch": per_batch["n_buckets_after_batch"],
            "mean_probe_groups_first_last": per_batch["mean_probe_groups"]}


def run_all(torch, device, peak):
    out = {}
    for name, fn in (("config1_prime", config1_prime), ("config2", config2), ("config3", config3), ("config4", config4)):
        try:
            out[name] = fn(torch, device, peak)
        except Exception as exc:                                # the headline line must still be printed
            out[name] = {"error": f"{type(exc).__name__}: {exc}"}
        torch.cuda.empty_cache()
    return out
