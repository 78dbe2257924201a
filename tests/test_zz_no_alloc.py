"""dok_map_count_new_static, the entry point for hosts that cannot allocate device memory (they bind the C ABI
without an allocator behind it, or must not pay the device-wide synchronisation of cudaMalloc / cudaFree in their
request loop).  Its scratch tag set is a fixed array inside the library, shared by all calls, so the test runs it
twice in a row with different batches and checks each count against dok_map_count_new with a caller-supplied
buffer.  Counts are integers: exact equality.  Collected last on purpose."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def count_new(m, keys, static):
    from doksparse_b200 import _lib as L
    lib = L.lib()
    keys = keys.contiguous()
    n = keys.shape[0]
    cnt = torch.zeros(L.N_COUNTERS, device="cuda:0", dtype=torch.long)
    st = L.stream_ptr(torch.device("cuda:0"))
    if static:
        rc = lib.dok_map_count_new_static(m._c_table(), m._c_hash(), L.ptr(keys), n, L.ptr(cnt), st)
    else:
        scratch = torch.empty(2 * n, device="cuda:0", dtype=torch.long)
        rc = lib.dok_map_count_new(m._c_table(), m._c_hash(), L.ptr(keys), n, L.ptr(scratch), 2 * n, L.ptr(cnt), st)
    return rc, int(cnt[L.CNT_CLAIMED_EMPTY].item())


def test_static_scratch_matches_caller_scratch_twice_in_a_row():
    from doksparse_b200 import CudaClosedHashmap, _lib as L
    np.random.seed(3)
    m = CudaClosedHashmap(n_buckets=1 << 18)
    g = torch.Generator(device="cuda:0").manual_seed(0)
    stored = torch.randint(0, 1 << 40, (100_000, 1), device="cuda:0", generator=g)
    m.set(stored, torch.zeros(100_000, 2, device="cuda:0"))
    max_rows = L.lib().dok_static_scratch_max_rows()
    assert max_rows == 1 << 19

    # first call: half stored keys, half new ones with many repeats (distinct new keys are what is counted)
    fresh = torch.randint(1 << 41, (1 << 41) + 5000, (60_000, 1), device="cuda:0", generator=g)
    batch1 = torch.cat([stored[:60_000], fresh])[torch.randperm(120_000, device="cuda:0", generator=g)]
    rc_a, a = count_new(m, batch1, static=True)
    rc_b, b = count_new(m, batch1, static=False)
    assert rc_a == 0 and rc_b == 0
    assert a == b == int(fresh.unique().numel())

    # second call right behind it, smaller and with other keys: leftovers of the first call must not be seen
    fresh2 = torch.randint(1 << 42, (1 << 42) + 300, (7_000, 1), device="cuda:0", generator=g)
    batch2 = torch.cat([fresh2, stored[500:1500]])
    rc_c, c = count_new(m, batch2, static=True)
    rc_d, d = count_new(m, batch2, static=False)
    assert rc_c == 0 and rc_d == 0
    assert c == d == int(fresh2.unique().numel())

    # the fixed capacity is enforced before anything is launched
    too_many = torch.zeros(max_rows + 1, 1, device="cuda:0", dtype=torch.long)
    rc, _ = count_new(m, too_many, static=True)
    assert rc == 3      # DOK_TOO_LARGE
    rc, full = count_new(m, torch.arange(max_rows, device="cuda:0")[:, None] + (1 << 50), static=True)
    assert rc == 0 and full == max_rows


def test_static_calls_take_no_device_memory_and_run_on_any_stream():
    """What the entry point is for: after the first call on a device (which looks up the scratch array's address)
    further calls leave the device's free memory untouched, on the default stream and on another one."""
    from doksparse_b200 import CudaClosedHashmap, _lib as L
    lib = L.lib()
    np.random.seed(4)
    m = CudaClosedHashmap(n_buckets=1 << 16)
    g = torch.Generator(device="cuda:0").manual_seed(1)
    stored = torch.randint(0, 1 << 40, (20_000, 1), device="cuda:0", generator=g)
    m.set(stored, torch.zeros(20_000, 2, device="cuda:0"))
    batch = torch.cat([stored[:5000], torch.arange(9000, device="cuda:0")[:, None] + (1 << 45)]).contiguous()
    cnt = torch.zeros(L.N_COUNTERS, device="cuda:0", dtype=torch.long)          # everything is allocated up front
    side = torch.cuda.Stream(device="cuda:0")
    table, params = m._c_table(), m._c_hash()
    assert lib.dok_map_count_new_static(table, params, L.ptr(batch), batch.shape[0], L.ptr(cnt), L.stream_ptr(torch.device("cuda:0"))) == 0
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(0)
    reserved_before = torch.cuda.memory_reserved(0)
    for rep in range(4):
        stream = side if rep % 2 else torch.cuda.current_stream()
        with torch.cuda.stream(stream):
            assert lib.dok_map_count_new_static(table, params, L.ptr(batch), batch.shape[0], L.ptr(cnt),
                                                ctypes.c_void_p(stream.cuda_stream)) == 0
        stream.synchronize()              # calls share the scratch array: one at a time
    free_after, _ = torch.cuda.mem_get_info(0)
    assert free_after >= free_before and torch.cuda.memory_reserved(0) == reserved_before
    assert int(cnt[L.CNT_CLAIMED_EMPTY].item()) == 5 * 9000
