"""ShardedClosedHashmap: one logical CudaClosedHashmap spread over the ranks of a torch.distributed group
(one process per GPU).  The reference is single-GPU; this path has no counterpart there, and its contract is
the single-table semantics: a batch applied through the shards leaves the union of the shards equal to one big
table that received the ranks' batches concatenated in rank order.

Per batch and rank:
  1. stable partition of the local rows by owner shard, owner = mulhi(mix(uuid ^ salt), world)  (CUDA kernels)
  2. exchange of the per-owner row counts (exact and padded to 16 rows)        (all_to_all_single, 2*world int64)
  3. exchange of key rows (and value rows for set)                          (all_to_all_single, NCCL over NVLink)
  4. the owner runs the local get / set / remove on what it received -- rows arrive grouped by source rank, in
     the source's order, so "last row wins" on the owner is "last row wins" of the concatenated batch
  5. for get / remove: results travel back with the mirrored split sizes     (all_to_all_single)
  6. inverse permutation to the caller's row order                           (CUDA kernel)
The uuid parameters used for routing are fixed at construction and identical on every rank; each shard is an
ordinary CudaClosedHashmap and rehashes locally on its own load.

The collective and bookkeeping logic talks to the device through a small `ops` object so that it can be
exercised with CPU ranks (gloo) in the tests, where a test double stands in for the CUDA kernels.  The product
default, `CudaShardOps`, has no CPU path.
"""
import ctypes

import numpy as np
import torch
import torch.distributed as dist

from . import _lib as L
from .cuda_closed_hashmap import CudaClosedHashmap


class CudaShardOps:
    """Device side of the sharded map: routing kernels of libdoksparse.so and a local CudaClosedHashmap."""

    def __init__(self, device, n_buckets, params, rehash_factor, rehash_threshold):
        self.device = torch.device(device)
        self.local = CudaClosedHashmap(n_buckets=n_buckets, device=self.device, rehash_factor=rehash_factor,
                                       rehash_threshold=rehash_threshold, **params)
        self._routing = {k: torch.as_tensor(v).cpu().tolist() for k, v in params.items()}
        self._hp = None

    def _routing_hash(self, keys):
        if self._hp is None:
            hp = L.HashParams()
            ks = int(np.prod(keys.shape[1:]))
            hp.key_size = ks
            hp.key_dtype = L.DTYPE_CODES[keys.dtype]
            for name in ("alpha2", "beta2", "prime2", "alpha1", "beta1", "prime1"):
                arr = getattr(hp, name)
                for i in range(ks):
                    arr[i] = self._routing[name][i]
            for i in range(ks):
                hp.key_perm[i] = i
            self._hp = hp
        return ctypes.byref(self._hp)

    def partition(self, keys, values, world):
        """-> (grouped_keys, grouped_values or None, dest_index, counts[2, world] on the device): rows per owner, and
        the same rounded up to multiples of 16 rows.  Owner o's segment starts at the sum of the ROUNDED counts before
        it, so that every segment is 16-byte aligned for the exchange (NCCL moves unaligned segments ~2.6x slower);
        the rows of the gap are never used by the receiver."""
        lib = L.lib()
        n = keys.shape[0]
        keys = keys.contiguous()
        with torch.cuda.device(self.device):
            st = L.stream_ptr(self.device)
            tiles = lib.dok_partition_tiles(n)
            cap = lib.dok_partition_capacity(n, world)
            offsets = torch.empty(world * tiles + 1, device=self.device, dtype=torch.long)
            counts = torch.empty(2 * world, device=self.device, dtype=torch.long)
            L.check(lib.dok_shard_partition_count(self._routing_hash(keys), L.ptr(keys), n, world, L.ptr(offsets),
                                                  L.ptr(counts), st), "dok_shard_partition_count")
            grouped_keys = torch.empty((cap,) + tuple(keys.shape[1:]), device=self.device, dtype=keys.dtype)
            grouped_values, vb = None, 0
            if values is not None:
                values = values.contiguous()
                grouped_values = torch.empty((cap,) + tuple(values.shape[1:]), device=self.device, dtype=values.dtype)
                vb = int(np.prod(values.shape[1:])) * values.element_size()
            dest = torch.empty(n, device=self.device, dtype=torch.long)
            L.check(lib.dok_shard_partition_scatter(self._routing_hash(keys), L.ptr(keys), L.ptr(values), vb, n, world,
                                                    L.ptr(offsets), L.ptr(counts), L.ptr(grouped_keys),
                                                    L.ptr(grouped_values), L.ptr(dest), st), "dok_shard_partition_scatter")
        return grouped_keys, grouped_values, dest, counts.view(2, world)

    def unpermute(self, grouped_values, grouped_flags, dest):
        lib = L.lib()
        n = dest.shape[0]
        out_v = out_f = None
        vb = 0
        with torch.cuda.device(self.device):
            if grouped_values is not None:
                out_v = torch.empty((n,) + tuple(grouped_values.shape[1:]), device=self.device, dtype=grouped_values.dtype)
                vb = int(np.prod(grouped_values.shape[1:])) * grouped_values.element_size()
            if grouped_flags is not None:
                out_f = torch.empty(n, device=self.device, dtype=grouped_flags.dtype)
            L.check(lib.dok_shard_unpermute(L.ptr(grouped_values), L.ptr(grouped_flags), L.ptr(dest), vb, n, L.ptr(out_v),
                                            L.ptr(out_f), L.stream_ptr(self.device)), "dok_shard_unpermute")
        return out_v, out_f

    # local table ops on the rows this rank owns.  `segments` = [(start, rows)] per source rank inside the received
    # buffer (starts are aligned, the gaps hold nothing); sources are processed in rank order, which is what makes
    # "last row wins" global.
    def local_get(self, keys, segments, fallback_value):
        values = torch.empty((keys.shape[0],) + tuple(self.local.value_shape), device=self.device, dtype=self.local.value_type)
        found = torch.zeros(keys.shape[0], device=self.device, dtype=torch.bool)
        for start, rows in segments:
            if rows:
                v, f = self.local.get(keys[start:start + rows], fallback_value)
                values[start:start + rows] = v
                found[start:start + rows] = f
        return values, found

    def local_set(self, keys, values, segments, assume_unique):
        for start, rows in segments:
            if rows:
                self.local.set(keys[start:start + rows], values[start:start + rows], assume_unique=assume_unique)

    def local_remove(self, keys, segments):
        flags = torch.zeros(keys.shape[0], device=self.device, dtype=torch.bool)
        for start, rows in segments:
            if rows:
                flags[start:start + rows] = self.local.remove_rows(keys[start:start + rows])
        return flags

    def local_n_elements(self):
        return self.local._n_elements

    def ready(self):
        return self.local._keys is not None

    def empty(self, shape, dtype):
        return torch.empty(shape, device=self.device, dtype=dtype)


class ShardedClosedHashmap:
    """get / set / remove over a table sharded by hash across the ranks of `group`.

    Every rank calls each method collectively with ITS OWN batch (any size, also empty).  Results are returned in
    the caller's row order.  `prime1..beta2` must be given explicitly (lists or tensors of key_size entries) and be
    identical on all ranks: they define the uuid, which decides the owner shard.
    """

    def __init__(self, n_buckets_per_shard, prime1, prime2, alpha1, alpha2, beta1, beta2, group=None, device=None,
                 rehash_factor=2.0, rehash_threshold=0.75, ops=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > L.MAX_SHARDS:
            raise L.DokError(f"at most {L.MAX_SHARDS} shards")
        params = dict(prime1=prime1, prime2=prime2, alpha1=alpha1, alpha2=alpha2, beta1=beta1, beta2=beta2)
        if ops is None:
            if device is None:
                device = torch.device("cuda", torch.cuda.current_device())
            ops = CudaShardOps(device, n_buckets_per_shard, params, rehash_factor, rehash_threshold)
        self.ops = ops
        self._value_shape = None
        self._value_dtype = None

    # ------------------------------------------------------------------ exchange plumbing
    def _exchange_counts(self, counts):
        """counts[2, world] (device; rows and padded rows per owner) -> (send_padded, recv_rows, recv_padded) as host
        lists; one synchronisation per batch."""
        send = counts.t().contiguous()                       # [world, 2]: what goes to each owner
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        both = torch.stack([send, recv]).cpu().tolist()
        return [int(c[1]) for c in both[0]], [int(c[0]) for c in both[1]], [int(c[1]) for c in both[1]]

    def _all_to_all_rows(self, rows, send, recv):
        """rows grouped by destination -> rows grouped by source."""
        if self.world == 1:
            return rows
        out = self.ops.empty((sum(recv),) + tuple(rows.shape[1:]), rows.dtype)
        dist.all_to_all_single(out, rows, output_split_sizes=recv, input_split_sizes=send, group=self.group)
        return out

    def _route(self, keys, values=None):
        """-> (owned_keys, owned_values, segments, dest, send, recv); segments = [(start, rows)] per source rank."""
        if self.world == 1:        # one shard owns everything: no partition, no exchange, no permutation
            return keys, values, [(0, keys.shape[0])], None, None, None
        grouped_keys, grouped_values, dest, counts = self.ops.partition(keys, values, self.world)
        send, recv_rows, recv = self._exchange_counts(counts)
        assert keys.shape[0] <= sum(send) <= grouped_keys.shape[0], "partition lost rows"
        owned_keys = self._all_to_all_rows(grouped_keys[:sum(send)], send, recv)
        owned_values = None if values is None else self._all_to_all_rows(grouped_values[:sum(send)], send, recv)
        starts = [sum(recv[:i]) for i in range(self.world)]
        return owned_keys, owned_values, list(zip(starts, recv_rows)), dest, send, recv

    # ------------------------------------------------------------------ operations
    def set(self, keys, values, assume_unique=False):
        """Collective insert-or-assign.  `assume_unique` promises pairwise different keys across ALL ranks' batches."""
        if self._value_shape is None:
            self._value_shape, self._value_dtype = tuple(values.shape[1:]), values.dtype
        owned_keys, owned_values, segments, _, _, _ = self._route(keys, values)
        self.ops.local_set(owned_keys, owned_values, segments, assume_unique)

    def get(self, keys, fallback_value=None):
        """Collective lookup -> (values[n, *value_shape], is_found[n]) in the caller's row order."""
        if self._value_shape is None:
            raise RuntimeError("store something first")
        owned_keys, _, segments, dest, send, recv = self._route(keys)
        if self.ops.ready() and owned_keys.shape[0]:
            owned_values, owned_found = self.ops.local_get(owned_keys, segments, fallback_value)
        else:
            # this shard holds nothing yet (or received nothing): every row it was asked about is a miss
            owned_values = self.ops.empty((owned_keys.shape[0],) + self._value_shape, self._value_dtype)
            fill = 0 if fallback_value is None else fallback_value
            if owned_values.numel():
                owned_values[:] = torch.as_tensor(fill, dtype=self._value_dtype)
            owned_found = self.ops.empty((owned_keys.shape[0],), torch.bool)
            owned_found[:] = False
        if dest is None:
            return owned_values, owned_found
        back_values = self._all_to_all_rows(owned_values, recv, send)
        back_found = self._all_to_all_rows(owned_found.view(torch.uint8), recv, send)
        out_values, out_found = self.ops.unpermute(back_values, back_found, dest)
        return out_values, out_found.view(torch.bool)

    def remove(self, keys):
        """Collective removal -> is_removed[n] aligned to the caller's rows (equal keys report once)."""
        if self._value_shape is None:
            raise RuntimeError("store something first")
        owned_keys, _, segments, dest, send, recv = self._route(keys)
        if self.ops.ready() and owned_keys.shape[0]:
            owned_flags = self.ops.local_remove(owned_keys, segments)
        else:
            owned_flags = self.ops.empty((owned_keys.shape[0],), torch.bool)
            owned_flags[:] = False
        if dest is None:
            return owned_flags
        back = self._all_to_all_rows(owned_flags.view(torch.uint8), recv, send)
        _, out = self.ops.unpermute(None, back, dest)
        return out.view(torch.bool)

    @property
    def n_elements(self):
        """Live rows over all shards (collective)."""
        n = self.ops.local_n_elements().clone().reshape(1)
        if self.world > 1:
            dist.all_reduce(n, group=self.group)
        return int(n.item())

    def __len__(self):
        return self.n_elements
