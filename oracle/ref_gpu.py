"""TEST INFRASTRUCTURE ONLY -- never imported by the product package.

The reference's own get / set / remove kernels on the GPU (oracle/_ref/refgpu_map_*.so, built by `make refgpu`
from the reference's kernel text with nvcc, since CuPy -- which compiles that text at run time in the reference --
is not available).  `RefGpuMap` keeps the reference storage layout (three contiguous tensors) and mirrors what the
reference launcher does around each kernel (closed_hashmap_impl.py:50-278: output allocation, fallback pre-fill,
zeroed flag vectors).  Hash parameters are explicit.  The Python bookkeeping of the reference map (pre-get, unique,
rehash; cuda_closed_hashmap.py:321-384) is NOT part of it: kernels only.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_NAMES = {torch.int64: "i64", torch.int32: "i32", torch.int16: "i16", torch.float32: "f32", torch.float64: "f64"}
_PARAMS = ("prime1", "prime2", "alpha1", "alpha2", "beta1", "beta2", "key_perm")


def lib_path(key_dtype, key_size, value_dtype, value_size):
    return os.path.join(_HERE, "_ref", f"refgpu_map_{_NAMES[key_dtype]}x{key_size}_{_NAMES[value_dtype]}x{value_size}.so")


def available(key_dtype=torch.int64, key_size=1, value_dtype=torch.float32, value_size=2):
    return key_dtype in _NAMES and value_dtype in _NAMES and os.path.exists(lib_path(key_dtype, key_size, value_dtype, value_size))


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


class RefGpuMap:
    # the reference indexes buckets and value elements with 32-bit ints
    # (closed_hashmap_impl_class.cu:184, 198, 231; closed_hashmap_impl.cu:72)
    MAX_ELEMENTS = 2 ** 31 - 1

    def __init__(self, n_buckets, key_dtype, key_size, value_dtype, value_size, params, device):
        self.lib = ctypes.CDLL(lib_path(key_dtype, key_size, value_dtype, value_size))
        for name in ("refgpu_get", "refgpu_set", "refgpu_remove"):
            getattr(self.lib, name).restype = ctypes.c_int
        assert self.lib.refgpu_key_size() == key_size and self.lib.refgpu_value_size() == value_size
        assert n_buckets * max(key_size, value_size) <= self.MAX_ELEMENTS, "beyond the reference's int indices"
        self.device = torch.device(device)
        self.n_buckets, self.key_size, self.value_size = int(n_buckets), key_size, value_size
        self.all_keys = torch.zeros(n_buckets, key_size, device=self.device, dtype=key_dtype)
        self.all_values = torch.zeros(n_buckets, value_size, device=self.device, dtype=value_dtype)
        self.all_uuids = torch.full((n_buckets,), -1, device=self.device, dtype=torch.long)
        self.params = {}
        for k in _PARAMS:
            v = params.get(k)
            if v is None and k == "key_perm":
                v = list(range(key_size))
            self.params[k] = torch.as_tensor(v, dtype=torch.long).reshape(-1).to(self.device).contiguous()
            assert self.params[k].numel() == key_size

    def _hash_args(self):
        return [_p(self.params[k]) for k in _PARAMS]

    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _check(self, keys, n_limit_factor):
        assert keys.is_contiguous() and keys.device == self.device and keys.dtype == self.all_keys.dtype
        assert keys.shape[1:] == (self.key_size,)
        assert keys.shape[0] * n_limit_factor <= self.MAX_ELEMENTS, "beyond the reference's int offsets"

    def get(self, keys, fallback=None):
        self._check(keys, self.value_size)
        n = keys.shape[0]
        fb = torch.zeros(self.value_size, device=self.device, dtype=self.all_values.dtype) if fallback is None else \
            torch.as_tensor(fallback, dtype=self.all_values.dtype).broadcast_to((self.value_size,)).to(self.device).contiguous()
        values = torch.empty(n, self.value_size, device=self.device, dtype=self.all_values.dtype)
        values[:] = fb[None]
        found = torch.zeros(n, device=self.device, dtype=torch.bool)
        with torch.cuda.device(self.device):
            rc = self.lib.refgpu_get(*self._hash_args(), _p(keys), _p(values), _p(self.all_keys), _p(self.all_values),
                                     _p(self.all_uuids), _p(fb), _p(found), ctypes.c_longlong(n),
                                     ctypes.c_longlong(self.n_buckets), self._stream())
        assert rc == 0, f"reference get launch failed: cudaError {rc}"
        return values, found

    def set(self, keys, values):
        self._check(keys, max(self.key_size, self.value_size))
        assert values.is_contiguous() and values.dtype == self.all_values.dtype and values.shape == (keys.shape[0], self.value_size)
        n = keys.shape[0]
        stored = torch.zeros(n, device=self.device, dtype=torch.bool)
        with torch.cuda.device(self.device):
            rc = self.lib.refgpu_set(*self._hash_args(), _p(keys), _p(values), _p(self.all_keys), _p(self.all_values),
                                     _p(self.all_uuids), _p(stored), ctypes.c_longlong(n),
                                     ctypes.c_longlong(self.n_buckets), self._stream())
        assert rc == 0, f"reference set launch failed: cudaError {rc}"
        return stored

    def remove(self, keys):
        self._check(keys, 1)
        n = keys.shape[0]
        removed = torch.zeros(n, device=self.device, dtype=torch.bool)
        with torch.cuda.device(self.device):
            rc = self.lib.refgpu_remove(*self._hash_args(), _p(keys), _p(self.all_keys), _p(self.all_values),
                                        _p(self.all_uuids), _p(removed), ctypes.c_longlong(n),
                                        ctypes.c_longlong(self.n_buckets), self._stream())
        assert rc == 0, f"reference remove launch failed: cudaError {rc}"
        return removed

    # ---- the reference's Python bookkeeping around the kernels, restated (cuda_closed_hashmap.py:321-384, 423-454):
    # `set` first looks the batch up, counts the distinct absent rows with a row-wise unique and reads n_elements on
    # the host for the rehash decision; `remove` de-duplicates the batch with a row-wise unique and returns flags for
    # the sorted unique rows.  Rehashing itself is not restated: callers size the table so that it never triggers.
    def api_set(self, keys, values, rehash_threshold=0.75):
        if not hasattr(self, "n_elements"):
            self.n_elements = torch.zeros((), device=self.device, dtype=torch.long)
        _, found = self.get(keys)
        n_new = keys[~found].unique(dim=0).shape[0]
        assert int(self.n_elements.item()) + n_new <= int(rehash_threshold * self.n_buckets), "would rehash"
        self.set(keys, values)
        self.n_elements += n_new

    def api_remove(self, keys):
        unique_keys = keys.unique(dim=0)
        removed = self.remove(unique_keys)
        if hasattr(self, "n_elements"):
            self.n_elements -= removed.sum()
        return removed

    def items(self):
        """(keys, values, uuid) of the live buckets in bucket order."""
        live = (self.all_uuids != -1) & (self.all_uuids != -3)
        return self.all_keys[live], self.all_values[live], self.all_uuids[live]
