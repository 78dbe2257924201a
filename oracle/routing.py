"""TEST INFRASTRUCTURE ONLY -- never imported by the product package.

Host restatement of the batch routing of the sharded map (doksparse_b200/csrc/shard_api.cu), which has no
counterpart in the single-GPU reference: owner shard of a uuid, stable partition by owner, and an `ops` test
double that lets ShardedClosedHashmap's collective logic run on CPU ranks (gloo) over OracleHashmap shards.
"""
import numpy as np
import torch

from . import port

_M = (1 << 64) - 1
SHARD_SALT = 0x9E3779B97F4A7C15


def mix64(h):
    h &= _M
    h ^= h >> 33
    h = (h * 0xFF51AFD7ED558CCD) & _M
    h ^= h >> 33
    h = (h * 0xC4CEB9FE1A85EC53) & _M
    h ^= h >> 33
    return h


def owner_of(uuid, n_shards):
    """mulhi64(mix64(uuid ^ salt), n_shards)"""
    return (mix64((int(uuid) & _M) ^ SHARD_SALT) * n_shards) >> 64


def owners(uuids, n_shards):
    return np.asarray([owner_of(u, n_shards) for u in uuids], dtype=np.int64)


def stable_partition(owner, n_shards):
    """-> (order, dest_index, counts): order[j] = source row of grouped row j; dest_index[i] = grouped position of row i"""
    order = np.argsort(owner, kind="stable")
    dest = np.empty_like(order)
    dest[order] = np.arange(len(order))
    counts = np.bincount(owner, minlength=n_shards).astype(np.int64)
    return order, dest, counts


class OracleShardOps:
    """CPU stand-in for CudaShardOps: same interface, torch CPU tensors in and out, OracleHashmap inside."""

    def __init__(self, n_buckets, params, rehash_factor=2.0, rehash_threshold=0.75):
        self.params = {k: np.asarray(v, dtype=np.int64) for k, v in params.items()}
        self.local = port.OracleHashmap(n_buckets=n_buckets, rehash_factor=rehash_factor,
                                        rehash_threshold=rehash_threshold, **self.params)
        self._router = None

    def _uuids(self, keys):
        k = keys.numpy()
        if self._router is None:
            r = port.OracleHashmap(n_buckets=8, **self.params)
            r._keys = np.zeros((8,) + k.shape[1:], dtype=k.dtype)
            r._values = np.zeros((8, 1), dtype=np.float32)
            self._router = r
        return self._router.hash_uuid(np.ascontiguousarray(k))[1]

    def partition(self, keys, values, world, want_dest=True):
        owner = owners(self._uuids(keys), world)
        order, dest, counts = stable_partition(owner, world)
        order_t = torch.from_numpy(order)
        counts_t = torch.from_numpy(counts)
        # the host stand-in does not pad segments (gloo needs no alignment): exact and padded counts coincide
        return (keys[order_t], None if values is None else values[order_t], torch.from_numpy(dest),
                torch.stack([counts_t, counts_t]))

    def unpermute(self, grouped_values, grouped_flags, dest, out_values=None, out_flags=None):
        v = None if grouped_values is None else grouped_values[dest]
        f = None if grouped_flags is None else grouped_flags[dest]
        if v is not None and out_values is not None:
            out_values[:] = v
            v = out_values
        if f is not None and out_flags is not None:
            out_flags[:] = f
            f = out_flags
        return v, f

    def local_get(self, keys, segments, fallback_value):
        assert sum(rows for _, rows in segments) == keys.shape[0]
        v, f = self.local.get(keys.numpy(), fallback_value)
        return torch.from_numpy(v), torch.from_numpy(f)

    def local_set(self, keys, values, segments, assume_unique):
        for start, rows in segments:            # sources in rank order
            if rows:
                self.local.set(keys[start:start + rows].numpy(), values[start:start + rows].numpy())

    def local_remove(self, keys, segments):
        return torch.from_numpy(self.local.remove_rows(keys.numpy()))

    def local_n_elements(self):
        return torch.tensor(self.local.n_elements)

    def to_host(self, words):
        return words.reshape(-1).tolist()

    def ready(self):
        return self.local._keys is not None

    def empty(self, shape, dtype):
        return torch.empty(shape, dtype=dtype)
