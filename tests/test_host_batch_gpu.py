"""HostBatch (pinned host buffers in and out, chunked over three streams) gives what the oracle gives for the same
operation stream; chunk sizes that do and do not divide the batch, duplicates across chunk borders."""
import numpy as np
import pytest
import torch

from oracle import port
from tests.helpers import assert_same_bytes, assert_same_items, host

pytestmark = pytest.mark.gpu


def pinned(a):
    return torch.from_numpy(np.ascontiguousarray(a)).pin_memory()


@pytest.mark.parametrize("chunk_rows", [1000, 4096, 1 << 20])
def test_host_batches_match_oracle(chunk_rows):
    from doksparse_b200 import CudaClosedHashmap
    from doksparse_b200.host_batch import HostBatch
    rng = np.random.default_rng(77)
    np.random.seed(5)
    state = np.random.get_state()
    cuda_map = CudaClosedHashmap(n_buckets=1 << 16, device="cuda:0")
    np.random.set_state(state)
    oracle_map = port.OracleHashmap(n_buckets=1 << 16)
    pipe = HostBatch(cuda_map, "cuda:0", chunk_rows=chunk_rows)

    for round_ in range(4):
        n = 9000 + 37 * round_
        keys = rng.integers(0, 6000, size=(n, 2), dtype=np.int64)          # many duplicates, also across chunks
        values = rng.standard_normal((n, 3)).astype(np.float32)
        state = np.random.get_state()
        pipe.set(pinned(keys), pinned(values))
        pipe.join()
        np.random.set_state(state)
        oracle_map.set(keys, values)
        torch.cuda.synchronize()
        assert_same_items(cuda_map, oracle_map)

        queries = rng.integers(0, 8000, size=(n + 11, 2), dtype=np.int64)
        out_values = torch.empty(n + 11, 3).pin_memory()
        out_found = torch.empty(n + 11, dtype=torch.bool).pin_memory()
        pipe.get(pinned(queries), out_values, out_found)
        pipe.join()
        torch.cuda.synchronize()
        want_values, want_found = oracle_map.get(queries)
        np.testing.assert_array_equal(out_found.numpy(), want_found)
        assert_same_bytes(out_values.numpy()[want_found], want_values[want_found])
        assert not out_values.numpy()[~want_found].any()

        doomed = np.unique(rng.integers(0, 8000, size=(3000, 2), dtype=np.int64), axis=0)   # distinct rows
        doomed = doomed[rng.permutation(len(doomed))]
        flags = torch.empty(len(doomed), dtype=torch.bool).pin_memory()
        pipe.remove_rows(pinned(doomed), flags)
        pipe.join()
        torch.cuda.synchronize()
        _, present = oracle_map.get(doomed)
        oracle_map.remove(doomed)
        np.testing.assert_array_equal(flags.numpy(), present)
        assert_same_items(cuda_map, oracle_map)
        assert cuda_map.n_elements == oracle_map.n_elements


def test_run_pipelines_several_operations():
    from doksparse_b200 import CudaClosedHashmap
    from doksparse_b200.host_batch import HostBatch
    rng = np.random.default_rng(5)
    np.random.seed(9)
    state = np.random.get_state()
    cuda_map = CudaClosedHashmap(n_buckets=1 << 16, device="cuda:0")
    np.random.set_state(state)
    oracle_map = port.OracleHashmap(n_buckets=1 << 16)
    pipe = HostBatch(cuda_map, "cuda:0", chunk_rows=3000)
    for round_ in range(3):
        n = 10000
        keys = rng.integers(0, 9000, size=(n, 1), dtype=np.int64)
        values = rng.standard_normal((n, 2)).astype(np.float32)
        queries = rng.integers(0, 12000, size=(n, 1), dtype=np.int64)
        doomed = np.unique(rng.integers(0, 12000, size=(2500, 1), dtype=np.int64), axis=0)
        out_values = torch.empty(n, 2).pin_memory()
        out_found = torch.empty(n, dtype=torch.bool).pin_memory()
        flags = torch.empty(len(doomed), dtype=torch.bool).pin_memory()
        state = np.random.get_state()
        pipe.run([("set", pinned(keys), pinned(values)), ("get", pinned(queries), out_values, out_found, -2.0),
                  ("remove_rows", pinned(doomed), flags)])
        pipe.join()
        torch.cuda.synchronize()
        np.random.set_state(state)
        oracle_map.set(keys, values)
        want_values, want_found = oracle_map.get(queries, -2.0)
        want_flags = oracle_map.remove_rows(doomed)
        np.testing.assert_array_equal(out_found.numpy(), want_found)
        assert_same_bytes(out_values.numpy(), want_values)
        np.testing.assert_array_equal(flags.numpy(), want_flags)
        assert_same_items(cuda_map, oracle_map)
