"""TEST INFRASTRUCTURE ONLY -- never imported by the product package.

ctypes front end of oracle/_ref: the reference's own kernel text compiled for the host
(oracle/Makefile, ref_map_driver.cpp, ref_dok_driver.cpp).  The shared objects exist only where
the reference checkout was present at build time; `available()` says whether they do.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_REF_DIR = os.path.join(_HERE, "_ref")

_NAMES = {np.dtype(np.int64): "i64", np.dtype(np.int32): "i32", np.dtype(np.int16): "i16",
          np.dtype(np.float32): "f32", np.dtype(np.float64): "f64"}


def map_combo_name(key_dtype, key_size, value_dtype, value_size):
    return f"{_NAMES[np.dtype(key_dtype)]}x{key_size}_{_NAMES[np.dtype(value_dtype)]}x{value_size}"


def map_lib_path(combo):
    return os.path.join(_REF_DIR, f"ref_map_{combo}.so")


def dok_lib_path(selector_ndim, ndim, value_dtype):
    return os.path.join(_REF_DIR, f"ref_dok_s{selector_ndim}_n{ndim}_{_NAMES[np.dtype(value_dtype)]}.so")


def available(combo="i64x1_f32x1"):
    return os.path.exists(map_lib_path(combo))


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


class RefMap:
    """The reference kernels on the reference storage layout (three contiguous arrays), driven with
    explicit hash parameters. Mirrors the launcher closed_hashmap_impl.py:50-278 (output allocation and
    pre-fills included)."""

    def __init__(self, n_buckets, key_dtype, key_size, value_dtype, value_size, params, n_threads=1):
        combo = map_combo_name(key_dtype, key_size, value_dtype, value_size)
        self.lib = ctypes.CDLL(map_lib_path(combo))
        assert self.lib.ref_key_size() == key_size and self.lib.ref_value_size() == value_size
        self.n_buckets = n_buckets
        self.key_size, self.value_size = key_size, value_size
        self.all_keys = np.zeros((n_buckets, key_size), dtype=key_dtype)
        self.all_values = np.zeros((n_buckets, value_size), dtype=value_dtype)
        self.all_uuids = np.full(n_buckets, -1, dtype=np.int64)
        self.params = {k: np.ascontiguousarray(np.asarray(v, dtype=np.int64)) for k, v in params.items()}
        self.n_threads = n_threads

    def _hash_args(self):
        p = self.params
        return [_p(p[k]) for k in ("prime1", "prime2", "alpha1", "alpha2", "beta1", "beta2", "key_perm")]

    def get(self, keys, fallback=None):
        keys = np.ascontiguousarray(keys)
        n = keys.shape[0]
        fb = np.zeros(self.value_size, dtype=self.all_values.dtype) if fallback is None else \
            np.ascontiguousarray(np.broadcast_to(np.asarray(fallback, dtype=self.all_values.dtype), (self.value_size,)))
        values = np.empty((n, self.value_size), dtype=self.all_values.dtype)
        values[:] = fb[None]
        found = np.zeros(n, dtype=np.uint8)
        self.lib.ref_get(*self._hash_args(), _p(keys), _p(values), _p(self.all_keys), _p(self.all_values),
                         _p(self.all_uuids), _p(fb), _p(found), ctypes.c_longlong(n),
                         ctypes.c_longlong(self.n_buckets), ctypes.c_int(self.n_threads))
        return values, found.astype(bool)

    def set(self, keys, values):
        keys, values = np.ascontiguousarray(keys), np.ascontiguousarray(values)
        n = keys.shape[0]
        stored = np.zeros(n, dtype=np.uint8)
        self.lib.ref_set(*self._hash_args(), _p(keys), _p(values), _p(self.all_keys), _p(self.all_values),
                         _p(self.all_uuids), _p(stored), ctypes.c_longlong(n), ctypes.c_longlong(self.n_buckets),
                         ctypes.c_int(self.n_threads))
        return stored.astype(bool)

    def remove(self, keys):
        keys = np.ascontiguousarray(keys)
        n = keys.shape[0]
        removed = np.zeros(n, dtype=np.uint8)
        self.lib.ref_remove(*self._hash_args(), _p(keys), _p(self.all_keys), _p(self.all_values),
                            _p(self.all_uuids), _p(removed), ctypes.c_longlong(n),
                            ctypes.c_longlong(self.n_buckets), ctypes.c_int(self.n_threads))
        return removed.astype(bool)

    def hash_uuid(self, keys):
        keys = np.ascontiguousarray(keys)
        n = keys.shape[0]
        h, u = np.zeros(n, dtype=np.int64), np.zeros(n, dtype=np.int64)
        self.lib.ref_hash_uuid(*self._hash_args(), _p(keys), _p(h), _p(u), ctypes.c_longlong(n))
        return h, u

    # ---- argument blocks for the fused DOK kernels -----------------------------------------------
    def kernel_args_block(self):
        """CudaClosedHashmap._kernel_args(as_list=False), cuda_closed_hashmap.py:131-155."""
        p = self.params
        head = np.concatenate([p[k] for k in ("prime1", "prime2", "alpha1", "alpha2", "beta1", "beta2", "key_perm")])
        tail = np.asarray([self.all_keys.ctypes.data, self.all_values.ctypes.data, self.all_uuids.ctypes.data,
                           self.n_buckets, -1, -3], dtype=np.int64)
        return np.ascontiguousarray(np.concatenate([head, tail]))


def accessor_args(*arrays, stride=None):
    """util.get_tensor_accessor_argument_array, sparse_dok/util.py:295-310: one int64 row
    [data_ptr, sizes..., strides...] per array; strides in ELEMENTS."""
    nd = arrays[0].ndim
    out = np.zeros((len(arrays), 1 + 2 * nd), dtype=np.int64)
    for r, a in enumerate(arrays):
        out[r, 0] = a.ctypes.data
        out[r, 1:1 + nd] = a.shape
        out[r, 1 + nd:] = [s // a.itemsize for s in a.strides] if stride is None else stride
    return np.ascontiguousarray(out)


def contiguous_stride(shape):
    """util.shape_to_stride, sparse_dok/util.py:289-293."""
    out, acc = [], 1
    for s in reversed(shape):
        out.append(acc)
        acc *= s
    return tuple(reversed(out))


class RefDok:
    """sparse_dok_count_items / zero_items / set_items_dense on a RefMap whose keys are int64[ndim] and
    whose values are value_dtype[1]."""

    def __init__(self, selector_ndim, ndim, value_dtype):
        self.lib = ctypes.CDLL(dok_lib_path(selector_ndim, ndim, value_dtype))
        assert self.lib.refdok_selector_ndim() == selector_ndim and self.lib.refdok_ndim() == ndim

    def _common(self, refmap, selectors, extra=()):
        shape = selectors[0].shape
        real = accessor_args(selectors[0], stride=contiguous_stride(shape))
        acc = accessor_args(*selectors, *extra)
        return refmap.kernel_args_block(), acc, real, int(np.prod(shape))

    def count_items(self, refmap, selectors):
        args, acc, real, n = self._common(refmap, selectors)
        counts = np.zeros(1, dtype=np.int64)
        self.lib.refdok_count_items(_p(args), _p(acc), _p(real), _p(counts), ctypes.c_longlong(n))
        return int(counts[0])

    def zero_items(self, refmap, selectors):
        args, acc, real, n = self._common(refmap, selectors)
        counts = np.zeros(1, dtype=np.int64)
        self.lib.refdok_zero_items(_p(args), _p(acc), _p(real), _p(counts), ctypes.c_longlong(n))
        return int(counts[0])

    def set_items_dense(self, refmap, selectors, src):
        args, acc, real, n = self._common(refmap, selectors, extra=(src,))
        self.lib.refdok_set_items_dense(_p(args), _p(acc), _p(real), ctypes.c_longlong(n))
