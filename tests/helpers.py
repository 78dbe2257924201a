"""Shared pieces of the GPU parity tests: the CUDA path and the CPU oracle are driven with the same seeded
inputs and the same numpy random seed (so both draw the same hash parameters), and compared on everything a
user can observe."""
import numpy as np
import torch

from oracle import port

TORCH_OF = {np.dtype(np.int64): torch.int64, np.dtype(np.int32): torch.int32, np.dtype(np.int16): torch.int16,
            np.dtype(np.int8): torch.int8, np.dtype(np.uint8): torch.uint8, np.dtype(np.float16): torch.float16,
            np.dtype(np.float32): torch.float32, np.dtype(np.float64): torch.float64}


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


def assert_same_items(cuda_map, oracle_map):
    """Live {(key, value, uuid)} sets are equal (slot order is layout-dependent, so compare sorted)."""
    k, v, u = cuda_map.items()
    ck, cv, cu = port.sort_items(host(k), host(v), host(u))
    ok, ov, ou = oracle_map.items_sorted()
    np.testing.assert_array_equal(cu, ou)
    np.testing.assert_array_equal(ck, ok.reshape(ck.shape))
    np.testing.assert_array_equal(cv.view(np.uint8), ov.reshape(cv.shape).view(np.uint8))


def assert_same_bytes(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    assert a.shape == b.shape and a.dtype == b.dtype
    np.testing.assert_array_equal(a.view(np.uint8), b.view(np.uint8))
