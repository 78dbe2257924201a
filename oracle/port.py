"""TEST INFRASTRUCTURE ONLY -- never imported by the product package.

numpy/ctypes front end of the plain-C restatement (oracle/dok_oracle.c) plus a restatement of
the reference's Python-side bookkeeping, so that a test can replay an operation stream on the
oracle and on the CUDA path and compare what a user can observe.

`OracleHashmap` follows sparse_dok/components/cuda_closed_hashmap.py of the reference:
  __init__ :21-64, lazy parameters :66-113, keys/values/uuid :157-172,233-234,
  set :321-384, get :386-421, remove :423-454, rehash :456-468.
`oracle_set_items_dense` / `oracle_getitem` follow
  sparse_dok/components/cuda/sparse_dok_tensor_impl.py:412-474 and
  sparse_dok/components/sparse_dok_tensor.py:302-315.
"""
import ctypes
import math
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle_port.so")
MAX_KEY_SIZE = 8

DTYPE_CODES = {
    np.dtype(np.int8): 0, np.dtype(np.uint8): 1, np.dtype(np.int16): 2, np.dtype(np.int32): 3,
    np.dtype(np.int64): 4, np.dtype(np.float16): 5, np.dtype(np.float32): 7, np.dtype(np.float64): 8,
}
BF16_CODE = 6  # carried as uint16 bit patterns with key_dtype_code=6


def build(force=False):
    """Compiles dok_oracle.c with gcc (seconds). Building the checker is not using it."""
    src = os.path.join(_HERE, "dok_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "port", "CC=gcc"])
    return _LIB_PATH


class _CMap(ctypes.Structure):
    _fields_ = [
        ("key_size", ctypes.c_int32), ("key_dtype", ctypes.c_int32),
        ("value_row_bytes", ctypes.c_int32), ("_pad", ctypes.c_int32),
        ("prime1", ctypes.c_int64 * MAX_KEY_SIZE), ("prime2", ctypes.c_int64 * MAX_KEY_SIZE),
        ("alpha1", ctypes.c_int64 * MAX_KEY_SIZE), ("alpha2", ctypes.c_int64 * MAX_KEY_SIZE),
        ("beta1", ctypes.c_int64 * MAX_KEY_SIZE), ("beta2", ctypes.c_int64 * MAX_KEY_SIZE),
        ("key_perm", ctypes.c_int64 * MAX_KEY_SIZE),
        ("n_buckets", ctypes.c_int64),
        ("keys", ctypes.c_void_p), ("values", ctypes.c_void_p), ("uuid", ctypes.c_void_p),
    ]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        P, I64, I = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
        MP = ctypes.POINTER(_CMap)
        _lib.orc_get.argtypes = [MP, P, I64, P, P, P, I]
        _lib.orc_get.restype = I64
        _lib.orc_set.argtypes = [MP, P, P, I64, P, I]
        _lib.orc_set.restype = I64
        _lib.orc_remove.argtypes = [MP, P, I64, P, I]
        _lib.orc_remove.restype = I64
        _lib.orc_count_exists.argtypes = [MP, P, I64, P, I]
        _lib.orc_count_exists.restype = I64
        _lib.orc_hash_uuid.argtypes = [MP, P, I64, P, P]
        _lib.orc_hash_uuid.restype = None
        assert _lib.orc_sizeof_map() == ctypes.sizeof(_CMap)
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def next_prime(n):
    import sympy
    return int(sympy.nextprime(int(n)))


def draw_hash_parameters(n_buckets, key_size):
    """The reference's lazy parameter draws in the order `set` evaluates them
    (cuda_closed_hashmap.py:350-357 -> :75-76, :87-88, :94, :100, :106, :112), from the global
    numpy random state."""
    prime1 = [np.random.randint(n_buckets, n_buckets * 2) for _ in range(key_size)]
    prime1 = [next_prime(p) for p in prime1]
    prime2 = [np.random.randint(0, 2 ** 60, dtype="int64") for _ in range(key_size)]
    prime2 = [next_prime(p) for p in prime2]
    alpha1 = [np.random.randint(p) - 1 for p in prime1]
    alpha2 = [np.random.randint(p) - 1 for p in prime1]
    beta1 = [np.random.randint(p) - 1 for p in prime1]
    beta2 = [np.random.randint(p) - 1 for p in prime1]
    as_arr = lambda v: np.asarray(v, dtype=np.int64)
    return dict(prime1=as_arr(prime1), prime2=as_arr(prime2), alpha1=as_arr(alpha1), alpha2=as_arr(alpha2),
                beta1=as_arr(beta1), beta2=as_arr(beta2))


class OracleHashmap:
    EMPTY, REMOVED = -1, -3

    def __init__(self, n_buckets=1024, prime1=None, prime2=None, alpha1=None, alpha2=None, beta1=None,
                 beta2=None, key_size=None, key_perm=None, rehash_factor=2.0, rehash_threshold=0.75,
                 n_threads=1, key_dtype_code=None):
        self.n_buckets = int(n_buckets)
        self._uuid = np.full(self.n_buckets, self.EMPTY, dtype=np.int64)
        self._keys = None
        self._values = None
        self._params = dict(prime1=prime1, prime2=prime2, alpha1=alpha1, alpha2=alpha2, beta1=beta1, beta2=beta2)
        self._params = {k: (None if v is None else np.asarray(v, dtype=np.int64).copy()) for k, v in self._params.items()}
        self._key_size = key_size
        self._key_perm = None if key_perm is None else np.asarray(key_perm, dtype=np.int64).copy()
        self._n_elements = 0
        self._rehash_factor = rehash_factor
        self._rehash_threshold = rehash_threshold
        self.n_threads = n_threads
        self._key_dtype_code = key_dtype_code

    # -- parameters ------------------------------------------------------------------------
    def _materialise_parameters(self):
        ks = int(np.prod(self._keys.shape[1:])) if self._keys is not None else self._key_size
        if any(v is None for v in self._params.values()):
            # each missing parameter is drawn when first touched, in evaluation order
            p = self._params
            # the reference's call pattern: a list of randints first, the primes after
            if p["prime1"] is None:
                raw = [np.random.randint(self.n_buckets, self.n_buckets * 2) for _ in range(ks)]
                p["prime1"] = np.asarray([next_prime(r) for r in raw], dtype=np.int64)
            if p["prime2"] is None:
                raw = [np.random.randint(0, 2 ** 60, dtype="int64") for _ in range(ks)]
                p["prime2"] = np.asarray([next_prime(r) for r in raw], dtype=np.int64)
            for name in ("alpha1", "alpha2", "beta1", "beta2"):
                if p[name] is None:
                    p[name] = np.asarray([np.random.randint(int(q)) - 1 for q in p["prime1"]], dtype=np.int64)
        if self._key_perm is None:
            self._key_perm = np.arange(ks, dtype=np.int64)
        assert self._key_perm.shape[0] == ks

    @property
    def params(self):
        self._materialise_parameters()
        return dict(self._params, key_perm=self._key_perm)

    def _cmap(self):
        self._materialise_parameters()
        m = _CMap()
        ks = int(np.prod(self._keys.shape[1:]))
        assert ks <= MAX_KEY_SIZE
        m.key_size = ks
        m.key_dtype = self._key_dtype_code if self._key_dtype_code is not None else DTYPE_CODES[self._keys.dtype]
        m.value_row_bytes = int(np.prod(self._values.shape[1:], dtype=np.int64)) * self._values.dtype.itemsize
        for name in ("prime1", "prime2", "alpha1", "alpha2", "beta1", "beta2"):
            arr = getattr(m, name)
            for i in range(ks):
                arr[i] = int(self._params[name][i])
        for i in range(ks):
            m.key_perm[i] = int(self._key_perm[i])
        m.n_buckets = self.n_buckets
        m.keys, m.values, m.uuid = self._keys.ctypes.data, self._values.ctypes.data, self._uuid.ctypes.data
        return m

    # -- storage views ---------------------------------------------------------------------
    @property
    def nonempty_mask(self):
        return (self._uuid != self.EMPTY) & (self._uuid != self.REMOVED)

    def keys(self):
        if self._keys is None:
            return None
        self._materialise_parameters()
        return self._keys.reshape(self.n_buckets, -1)[self.nonempty_mask][:, self._key_perm]

    def values(self):
        return None if self._values is None else self._values[self.nonempty_mask]

    def uuid(self):
        return self._uuid[self.nonempty_mask]

    @property
    def n_elements(self):
        return int(self._n_elements)

    @property
    def n_tombstones(self):
        return int((self._uuid == self.REMOVED).sum())

    # -- operations ------------------------------------------------------------------------
    def _kernel_get(self, keys, fallback=None):
        keys = np.ascontiguousarray(keys)
        n = keys.shape[0]
        values = np.empty((n,) + self._values.shape[1:], dtype=self._values.dtype)
        found = np.zeros(n, dtype=np.uint8)
        fb = None if fallback is None else np.ascontiguousarray(
            np.broadcast_to(np.asarray(fallback, dtype=self._values.dtype), self._values.shape[1:]))
        m = self._cmap()
        lib().orc_get(ctypes.byref(m), _ptr(keys), n, _ptr(values), _ptr(fb), _ptr(found), self.n_threads)
        return values, found.astype(bool)

    def set(self, new_keys, new_values):
        assert new_keys.shape[0] == new_values.shape[0]
        if self._keys is None:
            self._keys = np.zeros((self.n_buckets,) + new_keys.shape[1:], dtype=new_keys.dtype)
            self._values = np.zeros((self.n_buckets,) + new_values.shape[1:], dtype=new_values.dtype)
        else:
            assert new_keys.dtype == self._keys.dtype and new_keys.shape[1:] == self._keys.shape[1:]
            assert new_values.dtype == self._values.dtype and new_values.shape[1:] == self._values.shape[1:]
        new_keys, new_values = np.ascontiguousarray(new_keys), np.ascontiguousarray(new_values)
        if new_keys.shape[0] == 0:
            return None
        _, is_found = self._kernel_get(new_keys)
        n_missing = int((~is_found).sum())
        n_new = np.unique(new_keys[~is_found].reshape(n_missing, -1), axis=0).shape[0] if n_missing else 0
        if self._n_elements + n_new > int(self._rehash_threshold * self.n_buckets):
            self.rehash(int((self._n_elements + n_new) * self._rehash_factor))
        stored = np.zeros(new_keys.shape[0], dtype=np.uint8)
        m = self._cmap()
        lib().orc_set(ctypes.byref(m), _ptr(new_keys), _ptr(new_values), new_keys.shape[0], _ptr(stored), self.n_threads)
        self._n_elements += n_new
        self.last_is_stored = stored.astype(bool)
        return None

    def get(self, keys, fallback_value=None):
        if self._keys is None or self._values is None:
            raise RuntimeError("store something first")
        if keys.shape[0] == 0:
            return np.empty((0,) + self._values.shape[1:], dtype=self._values.dtype), np.empty(0, dtype=bool)
        assert keys.dtype == self._keys.dtype and keys.shape[1:] == self._keys.shape[1:]
        return self._kernel_get(keys, fallback_value)

    def remove(self, keys):
        if self._keys is None or self._values is None:
            raise RuntimeError("store something first")
        if keys.shape[0] == 0:
            return np.zeros(0, dtype=bool)
        assert keys.dtype == self._keys.dtype and keys.shape[1:] == self._keys.shape[1:]
        flat = np.ascontiguousarray(keys).reshape(keys.shape[0], -1)
        unique_keys = np.ascontiguousarray(np.unique(flat, axis=0)).reshape((-1,) + self._keys.shape[1:])
        removed = np.zeros(unique_keys.shape[0], dtype=np.uint8)
        m = self._cmap()
        lib().orc_remove(ctypes.byref(m), _ptr(unique_keys), unique_keys.shape[0], _ptr(removed), self.n_threads)
        self._n_elements -= int(removed.sum())
        return removed.astype(bool)

    def remove_rows(self, keys):
        """kernel only (no dedup): flags aligned to the rows given; serial order."""
        keys = np.ascontiguousarray(keys)
        removed = np.zeros(keys.shape[0], dtype=np.uint8)
        m = self._cmap()
        lib().orc_remove(ctypes.byref(m), _ptr(keys), keys.shape[0], _ptr(removed), self.n_threads)
        self._n_elements -= int(removed.sum())
        return removed.astype(bool)

    def count_exists(self, keys):
        keys = np.ascontiguousarray(keys)
        flags = np.zeros(keys.shape[0], dtype=np.uint8)
        m = self._cmap()
        total = lib().orc_count_exists(ctypes.byref(m), _ptr(keys), keys.shape[0], _ptr(flags), self.n_threads)
        return int(total), flags.astype(bool)

    def set_rows(self, keys, values):
        """kernel only (closed_hashmap_set without the Python bookkeeping)."""
        keys, values = np.ascontiguousarray(keys), np.ascontiguousarray(values)
        stored = np.zeros(keys.shape[0], dtype=np.uint8)
        m = self._cmap()
        lib().orc_set(ctypes.byref(m), _ptr(keys), _ptr(values), keys.shape[0], _ptr(stored), self.n_threads)
        return stored.astype(bool)

    def hash_uuid(self, keys):
        keys = np.ascontiguousarray(keys)
        h = np.zeros(keys.shape[0], dtype=np.int64)
        u = np.zeros(keys.shape[0], dtype=np.int64)
        m = self._cmap()
        lib().orc_hash_uuid(ctypes.byref(m), _ptr(keys), keys.shape[0], _ptr(h), _ptr(u))
        return h, u

    def rehash(self, n_buckets):
        keys = np.ascontiguousarray(self.keys()).reshape((-1,) + self._keys.shape[1:])
        values = np.ascontiguousarray(self.values())
        self.__init__(n_buckets=n_buckets, key_perm=self._key_perm, rehash_factor=self._rehash_factor,
                      rehash_threshold=self._rehash_threshold, n_threads=self.n_threads,
                      key_dtype_code=self._key_dtype_code)
        self.set(keys, values)

    def items_sorted(self):
        """{(key row, value row, uuid)} of the live slots as three arrays sorted by (uuid, key bytes):
        the layout-independent view two implementations are compared on."""
        k, v, u = self.keys(), self.values(), self.uuid()
        return sort_items(k, v, u)


def sort_items(k, v, u):
    if len(u) == 0:
        return np.ascontiguousarray(k).reshape(0, 0), np.ascontiguousarray(v).reshape(0, 0), u
    k = np.ascontiguousarray(k).reshape(len(u), -1)
    v = np.ascontiguousarray(v).reshape(len(u), -1)
    order = np.lexsort(tuple(k[:, j] for j in reversed(range(k.shape[1]))) + (u,))
    return k[order], v[order], u[order]


# ---- DOK layer ---------------------------------------------------------------------------------

def oracle_getitem(hashmap, selectors, dtype):
    """selectors: list of ndim int64 arrays already normalised and broadcast to one shape.
    Dense output with zero fill (sparse_dok_tensor.py:304-312)."""
    shape = selectors[0].shape
    keys = np.stack([np.broadcast_to(s, shape).reshape(-1) for s in selectors], axis=1).astype(np.int64)
    if hashmap._values is None:
        return np.zeros(shape, dtype=dtype)
    values, _ = hashmap.get(np.ascontiguousarray(keys), fallback_value=0)
    return values.reshape(shape)


def oracle_set_items_dense(hashmap, selectors, src):
    """sparse_dok_tensor_impl.py:412-474 with keys materialised on the host: seed an empty map with the
    first element, count existing, rehash on (n_elements + nSel) > n_buckets*threshold to
    ceil((n_elements + nSel)*factor), insert-or-assign every selector element in linear order (zeros are
    stored), n_elements += nSel - n_existing."""
    shape = selectors[0].shape
    keys = np.ascontiguousarray(
        np.stack([np.broadcast_to(s, shape).reshape(-1) for s in selectors], axis=1).astype(np.int64))
    vals = np.ascontiguousarray(np.broadcast_to(src, shape).reshape(-1, 1))
    n_sel = keys.shape[0]
    if n_sel == 0:
        return
    if hashmap._keys is None:
        hashmap.set(keys[:1], vals[:1])
    n_existing, _ = hashmap.count_exists(keys)
    n_new = n_sel - n_existing
    if (hashmap.n_elements + n_sel) > hashmap.n_buckets * hashmap._rehash_threshold:
        hashmap.rehash(math.ceil((hashmap.n_elements + n_sel) * hashmap._rehash_factor))
    hashmap.set_rows(keys, vals)
    hashmap._n_elements += n_new
