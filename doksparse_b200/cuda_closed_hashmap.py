"""CudaClosedHashmap: the reference's batched GPU hash map
(sparse_dok/components/cuda_closed_hashmap.py) with the same constructor, methods, attributes and
error behaviour, on top of libdoksparse.so.

What is kept from the reference
  * key identity is the 64-bit uuid; uuids are bit-identical for identical parameters and keys;
  * parameters are drawn lazily from the global numpy random state with the reference's calls and
    in the reference's order (:66-113, :350-357), so a seeded run draws the same parameters;
  * set / get / remove / rehash bookkeeping: n_elements, n_buckets, rehash trigger and new size
    (:363-366), `remove` dedups with `unique(dim=0)` and returns flags for the sorted unique rows
    (:438-454), `set` returns None (:384), RuntimeError("store something first") (:391-392).
What is different (the slot layout is not part of the contract)
  * `_uuid`, `_values` and `_keys` are strided views (reference shapes) of ONE interleaved slot array: tag, value
    and key row of a slot share a 128-byte line, the unit that a random access costs on B200;
  * the start slot comes from a mixer of the uuid and of alpha1/beta1, not from the reference's first hash
    (prime1 is still drawn, to keep the random stream aligned with the reference);
  * duplicates inside one `set` batch resolve deterministically to the last row.
"""
import ctypes

import numpy as np
import torch
from torch import Tensor

from . import _lib as L
from .util import next_prime


class CudaClosedHashmap:
    def __init__(
        self,
        n_buckets=1024,
        device="cuda:0",
        prime1=None,
        prime2=None,
        alpha1=None,
        alpha2=None,
        beta1=None,
        beta2=None,
        key_size=None,
        key_perm=None,
        rehash_factor=2.0,
        rehash_threshold=0.75,
        tombstone_threshold="auto",
    ):
        self._empty_marker = -1
        self._removed_marker = -3
        self._n_buckets = int(n_buckets)
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise L.DokError("CudaClosedHashmap needs a CUDA device: there is no CPU path")
        L.lib()  # fail loudly now if the extension is missing
        # before the first `set` only the tags exist (cuda_closed_hashmap.py:40)
        self._slots = None           # uint8 storage of the slot array
        self._key_shape = None
        self._key_dtype = None
        self._uuid_only = torch.full((self._n_buckets,), self._empty_marker, device=self.device, dtype=torch.long)
        # state that shallow clones (views) must see together: the duplicate-resolution stamps with their epoch,
        # and the host-side upper bound of n_elements that lets `set` skip a device synchronisation
        self._shared = {"stamp": None, "epoch": 0, "bound": 0, "snapshots": []}
        self._value_shape = None
        self._value_dtype = None

        self._key_size = key_size
        as_param = lambda v: v if v is None or isinstance(v, Tensor) else self._as_param(np.asarray(v).reshape(-1).tolist())
        self._prime1, self._prime2 = as_param(prime1), as_param(prime2)
        self._alpha1, self._alpha2 = as_param(alpha1), as_param(alpha2)
        self._beta1, self._beta2 = as_param(beta1), as_param(beta2)
        self._n_elements = torch.zeros(size=(), device=self.device, dtype=torch.long)
        # rows that a set could not store because the table was full (the reference drops them silently,
        # closed_hashmap_impl_class.cu:426; here they are counted on the device and reported at the next point where
        # the host synchronises anyway: n_elements, state_dict, the exact-count path of set)
        self._n_failed = torch.zeros(size=(), device=self.device, dtype=torch.long)
        self._rehash_factor = rehash_factor
        self._rehash_threshold = rehash_threshold
        # Tombstone-aware maintenance (no counterpart in the reference, whose rehash looks at live items only,
        # cuda_closed_hashmap.py:365: under insert / remove churn its empty slots run out, miss lookups walk ever longer
        # chains, and with none left they walk the whole table).  A removal that leaves live + tombstone slots above
        # t * n_buckets rebuilds the table IN PLACE: same size, same hash parameters (nothing is drawn from the random
        # state), same contents, no tombstones -- invisible to the caller except through `n_tombstones` and `_uuid`.
        # "auto" (the default): t = 0.95, and only once the tombstones are worth a rebuild (2 % of the buckets).
        # None: never (the reference's behaviour).  A number: that t, for any number of tombstones.
        self._tombstone_threshold = tombstone_threshold
        self._n_tombstones = torch.zeros(size=(), device=self.device, dtype=torch.long)   # upper bound, on the device
        self._tombstone_host_bound = 0                                                  # looser bound, on the host

        self._key_perm = None
        if key_perm is not None:
            if not isinstance(key_perm, Tensor):
                key_perm = torch.tensor(key_perm, dtype=torch.long, device=self.device)
            self._key_perm = key_perm.to(device=self.device, dtype=torch.long)
        self._hp = None       # cached ctypes dok_hash_params
        self._table = None

    # ------------------------------------------------------------------ parameters (lazy, reference order)
    def _current_key_size(self):
        assert self._slots is not None or self._key_size is not None
        if self._slots is not None:
            return int(np.prod(self._key_shape))
        return int(self._key_size)

    def _as_param(self, values):
        return torch.tensor([int(v) for v in values], device=self.device, dtype=torch.long)

    @property
    def prime1(self):
        if self._prime1 is None:
            raw = [np.random.randint(self.n_buckets, self.n_buckets * 2) for _ in range(self._current_key_size())]
            self._prime1 = self._as_param(next_prime(r) for r in raw)
        return self._prime1

    @property
    def prime2(self):
        if self._prime2 is None:
            raw = [np.random.randint(0, 2 ** 60, dtype="int64") for _ in range(self._current_key_size())]
            self._prime2 = self._as_param(next_prime(r) for r in raw)
        return self._prime2

    def _draw_below_prime1(self):
        return self._as_param(np.random.randint(int(p)) - 1 for p in self.prime1.cpu())

    @property
    def alpha1(self):
        if self._alpha1 is None:
            self._alpha1 = self._draw_below_prime1()
        return self._alpha1

    @property
    def alpha2(self):
        if self._alpha2 is None:
            self._alpha2 = self._draw_below_prime1()
        return self._alpha2

    @property
    def beta1(self):
        if self._beta1 is None:
            self._beta1 = self._draw_below_prime1()
        return self._beta1

    @property
    def beta2(self):
        if self._beta2 is None:
            self._beta2 = self._draw_below_prime1()
        return self._beta2

    @property
    def key_perm(self):
        if self._key_perm is None:
            assert self._slots is not None
            self._key_perm = torch.arange(int(np.prod(self.key_shape)), device=self.device)
        else:
            assert self._key_perm.shape[0] == np.prod(self.key_shape)
        return self._key_perm

    @key_perm.setter
    def key_perm(self, new):
        if not isinstance(new, Tensor):
            new = torch.tensor([int(i) for i in new], device=self.device, dtype=torch.long)
        new = new.to(device=self.device, dtype=torch.long)
        assert new.shape == self.key_perm.shape
        self._key_perm = new
        self._hp = None

    def _materialise_parameters(self):
        # evaluation order of the reference's kernel call (cuda_closed_hashmap.py:350-357)
        return (self.prime1, self.prime2, self.alpha1, self.alpha2, self.beta1, self.beta2, self.key_perm)

    # ------------------------------------------------------------------ storage
    def _allocate(self, key_shape, key_dtype, value_shape, value_dtype):
        value_bytes = int(np.prod(value_shape, dtype=np.int64)) * torch.empty((), dtype=value_dtype).element_size()
        key_size = int(np.prod(key_shape, dtype=np.int64))
        if key_dtype not in L.DTYPE_CODES:
            raise L.DokError(f"unsupported key dtype {key_dtype}")
        if not (1 <= key_size <= L.MAX_KEY_SIZE):
            raise L.DokError(f"keys may have 1..{L.MAX_KEY_SIZE} elements, got {key_size}")
        if not (1 <= value_bytes <= L.MAX_VALUE_BYTES):
            raise L.DokError(f"value rows may have 1..{L.MAX_VALUE_BYTES} bytes, got {value_bytes}")
        key_bytes = key_size * torch.empty((), dtype=key_dtype).element_size()
        lay = L.LayoutInfo()
        L.check(L.lib().dok_table_layout(value_bytes, key_bytes, self._n_buckets, ctypes.byref(lay)), "dok_table_layout")
        self._layout = lay
        self._value_bytes, self._key_bytes = value_bytes, key_bytes
        self._value_shape, self._value_dtype = torch.Size(value_shape), value_dtype
        self._key_shape, self._key_dtype = torch.Size(key_shape), key_dtype
        self._slots = torch.empty(lay.total_bytes, device=self.device, dtype=torch.uint8)
        self._uuid_only = None
        self._shared["stamp"] = None
        self._hp = None
        with torch.cuda.device(self.device):
            L.check(L.lib().dok_map_init(self._c_table(), L.stream_ptr(self.device)), "dok_map_init")

    def _begin_bulk_insert(self, key_shape, key_dtype, value_shape, value_dtype, n_new):
        """What `set` does to a never-used map before its kernel runs, for a batch known to hold `n_new` pairwise
        different new keys: allocate, draw the parameters, grow if the reference's trigger fires (which re-draws them,
        cuda_closed_hashmap.py:365-366, 456-468), account for the new elements.  The caller then inserts the rows."""
        assert self._slots is None
        self._allocate(key_shape, key_dtype, value_shape, value_dtype)
        if n_new == 0:
            return
        self._materialise_parameters()
        if n_new > int(self._rehash_threshold * self.n_buckets):
            self.__init__(n_buckets=int(n_new * self._rehash_factor), device=self.device, key_perm=self._key_perm,
                          rehash_factor=self._rehash_factor, rehash_threshold=self._rehash_threshold,
                          tombstone_threshold=self._tombstone_threshold)
            self._allocate(key_shape, key_dtype, value_shape, value_dtype)
            self._materialise_parameters()
        self._n_elements += n_new
        self._shared["bound"] = n_new

    def _slot_view(self, dtype, inner_shape, byte_offset):
        """[n_buckets, *inner_shape] strided view of one field of the slot array."""
        es = torch.empty((), dtype=dtype).element_size()
        strides, acc = [], 1
        for extent in reversed(tuple(inner_shape)):
            strides.append(acc)
            acc *= int(extent)
        strides = (self._layout.slot_bytes // es,) + tuple(reversed(strides))
        return self._slots.view(dtype).as_strided((self._n_buckets,) + tuple(inner_shape), strides, byte_offset // es)

    @property
    def _uuid(self):
        """[n_buckets] int64 tags: uuid, -1 empty, -3 removed (a strided view of the slot array)."""
        if self._slots is None:
            return self._uuid_only
        return self._slot_view(torch.int64, (), 0)

    @property
    def _values(self):
        """[n_buckets, *value_shape] view of the value field of the slots (None before the first set)."""
        if self._slots is None:
            return None
        return self._slot_view(self._value_dtype, self._value_shape, self._layout.value_offset)

    @property
    def _keys(self):
        """[n_buckets, *key_shape] view of the key rows, storage-column order (None before the first set)."""
        if self._slots is None:
            return None
        return self._slot_view(self._key_dtype, self._key_shape, self._layout.key_offset)

    def _next_epoch(self):
        """Epoch of the next general set: larger than every epoch stamped on this table before.  The stamps live in
        the slots when the layout has room for them, else in a separate array allocated on first use."""
        sh = self._shared
        if self._layout.stamp_offset < 0 and sh["stamp"] is None:
            sh["stamp"] = torch.zeros(self._layout.n_slots, device=self.device, dtype=torch.long)
        if sh["epoch"] >= L.MAX_EPOCH - 1:
            raise L.DokError("stamp epochs exhausted: rehash() the map to start over")
        sh["epoch"] += 1
        return sh["epoch"]

    def _c_table(self):
        t = L.Table()
        t.slots = self._slots.data_ptr()
        stamp = self._shared["stamp"]
        t.stamp = stamp.data_ptr() if stamp is not None else None
        t.n_buckets = self._n_buckets
        t.slot_bytes = self._layout.slot_bytes
        t.value_bytes = self._value_bytes
        t.key_bytes = self._key_bytes
        self._table = t   # keeps the struct alive for the duration of the call
        return ctypes.byref(t)

    def _c_hash(self):
        if self._hp is None:
            self._materialise_parameters()
            hp = L.HashParams()
            ks = int(np.prod(self.key_shape))
            hp.key_size = ks
            hp.key_dtype = L.DTYPE_CODES[self._key_dtype]
            names = ("alpha2", "beta2", "prime2", "alpha1", "beta1", "prime1")
            host = {name: getattr(self, name).cpu().tolist() for name in names}
            perm = self.key_perm.cpu().tolist()
            assert all(len(v) == ks for v in host.values()) and len(perm) == ks
            for name in names:
                arr = getattr(hp, name)
                for i in range(ks):
                    arr[i] = host[name][i]
            for i in range(ks):
                hp.key_perm[i] = perm[i]
                assert abs(host["prime1"][i]) >= 2 and abs(host["prime2"][i]) >= 2, "primes must have magnitude >= 2"
            if 0 in host["alpha2"]:
                import warnings
                warnings.warn("alpha2 contains 0: the uuid ignores that key element, so keys differing only there "
                              "are told apart only by their first hash (the reference draws alpha2 from [-1, prime1-2])")
            self._hp = hp
        return ctypes.byref(self._hp)

    def _counters(self):
        return torch.zeros(L.N_COUNTERS, device=self.device, dtype=torch.long)

    # The rehash decision of `set` needs n_elements on the host, which the reference gets with a blocking .item()
    # per call.  Here the host keeps an UPPER BOUND instead: after every mutation the device count is copied to
    # pinned memory without waiting, and the bound is the newest copy that has landed plus the sizes of the set
    # batches enqueued after it.  Only when that bound crosses the threshold is the exact value fetched.
    def _after_mutation(self, added):
        sh = self._shared
        sh["bound"] += added
        snaps = sh["snapshots"]
        for s in snaps:
            s[2] += added                       # rows that may have been inserted after that snapshot was taken
        ring = sh.get("ring")
        if ring is None:
            ring = sh["ring"] = torch.zeros(8, dtype=torch.long, pin_memory=True)
        free = set(range(ring.numel())) - {s[1] for s in snaps}
        if not free:
            return                              # eight copies still in flight: skip this one, the bound stays valid
        slot = free.pop()
        with torch.cuda.device(self.device):
            ring[slot:slot + 1].copy_(self._n_elements.reshape(1), non_blocking=True)
            event = torch.cuda.Event()
            event.record()
        snaps.append([event, slot, 0])

    def _element_bound(self):
        sh = self._shared
        snaps = sh["snapshots"]
        newest = None
        while snaps and snaps[0][0].query():
            newest = snaps.pop(0)
        if newest is not None:
            sh["bound"] = min(sh["bound"], int(sh["ring"][newest[1]]) + newest[2])
        return sh["bound"]

    def _room_for(self, rows, limit):
        """bound + rows <= limit?  When the bound is too high only because the host runs ahead of the device, wait
        for the count copies still in flight to land -- oldest first, each an event on the stream -- instead of for the
        whole stream: the device keeps the work that is queued behind them."""
        bound = self._element_bound()
        snaps = self._shared["snapshots"]
        while bound + rows > limit and snaps:
            snaps[0][0].synchronize()
            bound = self._element_bound()
        return bound + rows <= limit

    # ------------------------------------------------------------------ compaction
    def items(self, keys=True, values=True, uuid=True, transposed_keys=False):
        """(keys, values, uuid) of the live slots in slot order, from one pass over the tags."""
        assert self._slots is not None
        lib = L.lib()
        with torch.cuda.device(self.device):
            st = L.stream_ptr(self.device)
            tiles = lib.dok_compact_tiles(self._n_buckets)
            offsets = torch.empty(tiles + 1, device=self.device, dtype=torch.long)
            L.check(lib.dok_map_compact_count(self._c_table(), L.ptr(offsets), st), "dok_map_compact_count")
            count = int(offsets[-1].item())
            ks = int(np.prod(self.key_shape))
            k = v = u = None
            if keys:
                shape = (ks, count) if transposed_keys else (count, ks)
                k = torch.empty(shape, device=self.device, dtype=self._key_dtype)
            if values:
                v = torch.empty((count,) + tuple(self._value_shape), device=self.device, dtype=self._value_dtype)
            if uuid:
                u = torch.empty(count, device=self.device, dtype=torch.long)
            if count:
                L.check(lib.dok_map_compact_scatter(self._c_table(), self._c_hash(), L.ptr(offsets), L.ptr(k),
                                                    int(transposed_keys), L.ptr(v), L.ptr(u), st),
                        "dok_map_compact_scatter")
        return k, v, u

    def count_live(self):
        """Live slots, counted by the compaction's first pass (one read of the tags, tile sums, one scan) instead of
        a mask tensor plus a reduction."""
        if self._slots is None:
            return 0
        lib = L.lib()
        with torch.cuda.device(self.device):
            tiles = lib.dok_compact_tiles(self._n_buckets)
            offsets = torch.empty(tiles + 1, device=self.device, dtype=torch.long)
            L.check(lib.dok_map_compact_count(self._c_table(), L.ptr(offsets), L.stream_ptr(self.device)), "dok_map_compact_count")
            return int(offsets[-1].item())

    @property
    def nonempty_mask(self):
        return (self._uuid != self._empty_marker) & (self._uuid != self._removed_marker)

    def keys(self):
        if self._slots is None:
            return None
        return self.items(values=False, uuid=False)[0]

    def values(self):
        if self._slots is None:
            return None
        return self.items(keys=False, uuid=False)[1]

    def uuid(self):
        if self._slots is None:
            return self._uuid_only[:0]
        return self.items(keys=False, values=False)[2]

    def set_values(self, selectors, new_values):
        masked_values = self._values[self.nonempty_mask]
        masked_values[selectors] = new_values
        self._values[self.nonempty_mask] = masked_values

    def permute_keys(self, ordering):
        assert self._slots is not None, "hashmap is empty"
        assert len(self.key_shape) == 1, "keys are not one dimensional"
        assert len(ordering) == self.key_shape[0]
        assert len(set(ordering)) == len(ordering), "duplicates are not allowed"
        self._materialise_parameters()
        self._keys.copy_(self._keys[:, ordering].clone())
        for name in ("_alpha1", "_alpha2", "_beta1", "_beta2", "_prime1", "_prime2"):
            setattr(self, name, getattr(self, name)[ordering])
        self._hp = None

    def clone(self, deepclone=False):
        self._materialise_parameters()
        cp = (lambda x: x.clone()) if deepclone else (lambda x: x)
        new = CudaClosedHashmap(
            n_buckets=self.n_buckets, device=self.device,
            prime1=cp(self.prime1), prime2=cp(self.prime2), alpha1=cp(self.alpha1), alpha2=cp(self.alpha2),
            beta1=cp(self.beta1), beta2=cp(self.beta2), key_perm=cp(self._key_perm),
            rehash_factor=self._rehash_factor, rehash_threshold=self._rehash_threshold,
            tombstone_threshold=self._tombstone_threshold,
        )
        new._n_tombstones = cp(self._n_tombstones)
        new._tombstone_host_bound = self._tombstone_host_bound
        if self._slots is not None:
            new._slots = cp(self._slots)
            new._uuid_only = None
            new._layout = self._layout
            new._value_bytes, new._key_bytes = self._value_bytes, self._key_bytes
            new._value_shape, new._value_dtype = self._value_shape, self._value_dtype
            new._key_shape, new._key_dtype = self._key_shape, self._key_dtype
        else:
            new._uuid_only = cp(self._uuid_only)
        new._n_elements = cp(self._n_elements)
        new._n_failed = cp(self._n_failed)
        if deepclone:
            # in-slot stamps were copied with the slots: continue their epochs; a separate array is copied too
            new._shared = {"stamp": None if self._shared["stamp"] is None else self._shared["stamp"].clone(),
                           "epoch": self._shared["epoch"], "bound": self._shared["bound"], "snapshots": []}
        else:
            new._shared = self._shared   # a view writes the same slots: same stamps, epoch and bound
        return new

    # ------------------------------------------------------------------ sizes
    @property
    def n_elements(self):
        n, failed = torch.stack([self._n_elements, self._n_failed]).tolist()      # one synchronisation for both
        self._shared["snapshots"].clear()
        self._shared["bound"] = n
        if failed:
            self._n_failed.zero_()
            raise L.DokError(f"{failed} rows of earlier set calls were not stored: the table was full "
                             f"({self._n_buckets} buckets); rehash() to a larger size and set them again")
        return n

    @property
    def last_set_failed(self):
        """Rows that set calls could not store so far (table full); reading it synchronises."""
        return int(self._n_failed.item())

    @property
    def n_buckets(self):
        return self._n_buckets

    @property
    def load_factor(self):
        return self.n_elements / self.n_buckets

    @property
    def n_tombstones(self):
        return int((self._uuid == self._removed_marker).sum().item())

    @property
    def key_shape(self):
        assert self._slots is not None
        return self._key_shape

    @property
    def value_shape(self):
        assert self._slots is not None
        return self._value_shape

    @property
    def key_type(self):
        return self._key_dtype

    @property
    def value_type(self):
        return self._value_dtype

    def __len__(self):
        return self.n_elements

    # ------------------------------------------------------------------ python-side hashes of the reference
    def _keys_as_long_bits(self, keys):
        n_keys = keys.shape[0]
        keys = keys.reshape(n_keys, -1).clone()
        if keys.dtype == torch.float:
            keys = keys.view(dtype=torch.int32).long()
            keys[keys == -2 ** 31] = 0
        elif keys.dtype == torch.half:
            keys = keys.view(dtype=torch.int16).long()
            keys[keys == -2 ** 15] = 0
        elif keys.dtype == torch.double:
            keys = keys.view(dtype=torch.int64)
            keys[keys == -2 ** 63] = 0
        else:
            keys = keys.to(torch.long)
        return keys

    def get_hash(self, keys):
        """Python-side first hash of the reference (cuda_closed_hashmap.py:278-300; bit-casts floats, unlike the
        kernels).  Diagnostic only: this library does not place rows with it."""
        keys = self._keys_as_long_bits(keys)
        terms = (self.alpha1[None] * keys + self.beta1[None]) % self.prime1[None]
        if self._key_perm is not None:
            terms = terms[:, self._key_perm]
        return terms.prod(dim=-1).abs() % self.n_buckets

    def get_uuid(self, keys):
        """Python-side second hash of the reference (cuda_closed_hashmap.py:302-319).  `device_uuid` returns what
        the kernels use."""
        keys = self._keys_as_long_bits(keys)
        return ((self.alpha2[None] * keys + self.beta2[None]) % self.prime2[None]).prod(dim=-1).abs()

    def test_uniformity(self, keys):
        hash_codes = self.get_hash(keys)
        logits = (torch.bincount(hash_codes, minlength=self.n_buckets) + 1).log()
        logp = torch.log_softmax(logits, dim=-1)
        return (-(logp * logp.exp()).sum(dim=-1)).exp() / self.n_buckets

    def device_uuid(self, keys):
        """uuid of each key row exactly as the kernels compute it (value cast of the key elements)."""
        assert self._slots is not None
        keys = keys.contiguous()
        out = torch.empty(keys.shape[0], device=self.device, dtype=torch.long)
        with torch.cuda.device(self.device):
            L.check(L.lib().dok_map_uuid(self._c_table(), self._c_hash(), L.ptr(keys), keys.shape[0], L.ptr(out), None,
                                         L.stream_ptr(self.device)), "dok_map_uuid")
        return out

    # ------------------------------------------------------------------ set
    def _launch_set(self, keys, values, assume_unique):
        lib = L.lib()
        n = keys.shape[0]
        cnt = self._counters()
        with torch.cuda.device(self.device):
            st = L.stream_ptr(self.device)
            if assume_unique:
                L.check(lib.dok_map_set_unique(self._c_table(), self._c_hash(), L.ptr(keys), L.ptr(values), n, None,
                                               L.ptr(cnt), st), "dok_map_set_unique")
            else:
                epoch = self._next_epoch()
                scratch = torch.empty(n + 1, device=self.device, dtype=torch.long)
                L.check(lib.dok_map_set(self._c_table(), self._c_hash(), L.ptr(keys), L.ptr(values), n, L.ptr(scratch),
                                        epoch, None, L.ptr(cnt), st), "dok_map_set")
        return cnt

    def _count_new(self, keys):
        """Number of distinct new keys of a batch (cuda_closed_hashmap.py:350-363).  Integer keys: distinct absent
        uuids, counted on the device with a scratch tag set.  Floating keys: distinct absent ROWS like the
        reference, because the value cast makes different rows share a uuid."""
        lib = L.lib()
        n = keys.shape[0]
        cnt = self._counters()
        with torch.cuda.device(self.device):
            st = L.stream_ptr(self.device)
            if keys.dtype in L.FLOAT_DTYPES:
                found = torch.empty(n, device=self.device, dtype=torch.bool)
                L.check(lib.dok_map_count_exists(self._c_table(), self._c_hash(), L.ptr(keys), n, L.ptr(found),
                                                 L.ptr(cnt), st), "dok_map_count_exists")
                return int(keys[~found].unique(dim=0).shape[0])
            slots = 2 * n
            scratch = torch.empty(slots, device=self.device, dtype=torch.long)
            L.check(lib.dok_map_count_new(self._c_table(), self._c_hash(), L.ptr(keys), n, L.ptr(scratch), slots,
                                          L.ptr(cnt), st), "dok_map_count_new")
        return int(cnt[L.CNT_CLAIMED_EMPTY].item())

    def set(self, new_keys, new_values, assume_unique=False):
        """Insert-or-assign a batch.  `assume_unique=True` promises pairwise different keys and runs one kernel
        instead of two.  Returns None like the reference."""
        assert new_keys.shape[0] == new_values.shape[0]
        if self._slots is None:
            assert new_keys.device == new_values.device == self.device
            self._allocate(new_keys.shape[1:], new_keys.dtype, new_values.shape[1:], new_values.dtype)
        else:
            assert new_keys.dtype == self._key_dtype
            assert new_keys.device == self.device
            assert new_keys.shape[1:] == self._key_shape
            assert new_values.dtype == self._value_dtype
            assert new_values.device == self.device
            assert new_values.shape[1:] == self._value_shape
        new_keys = new_keys.contiguous()
        new_values = new_values.contiguous()
        n = new_keys.shape[0]
        if n == 0:
            return
        self._materialise_parameters()
        limit = int(self._rehash_threshold * self.n_buckets)
        row_counted = new_keys.dtype in L.FLOAT_DTYPES
        fast = not row_counted and self._room_for(n, limit)
        if not fast and not row_counted:
            # the bound may only be stale (the host runs ahead of the device): fetch the exact count before paying
            # for a pass that counts the distinct new keys
            fast = self.n_elements + n <= limit
        if fast:
            # whatever the number of new keys is, the reference would not rehash: insert and count on the device
            cnt = self._launch_set(new_keys, new_values, assume_unique)
            self._account_set(cnt, n)
            return
        n_new = self._count_new(new_keys)
        n_elements = self.n_elements
        if n_elements + n_new > limit:
            self.rehash(int((n_elements + n_new) * self._rehash_factor))
        cnt = self._launch_set(new_keys, new_values, assume_unique)
        self._n_tombstones -= cnt[L.CNT_REUSED_REMOVED]
        self._n_failed += cnt[L.CNT_FAILED]
        self._n_elements += n_new
        self._shared["snapshots"].clear()
        self._shared["bound"] = n_elements + n_new

    def set_rows(self, keys, values, assume_unique=False):
        """Kernel only, like `remove_rows`: insert-or-assign without the reference's bookkeeping around it -- no count
        of the distinct new keys, no rehash decision, no host synchronisation.  New slots are counted on the device.
        The caller guarantees room (rows that find the table full are counted in `last_set_failed`)."""
        assert keys.shape[0] == values.shape[0]
        if self._slots is None:
            self._allocate(keys.shape[1:], keys.dtype, values.shape[1:], values.dtype)
        assert keys.dtype == self._key_dtype and keys.shape[1:] == self._key_shape and keys.device == self.device
        assert values.dtype == self._value_dtype and values.shape[1:] == self._value_shape and values.device == self.device
        if keys.shape[0] == 0:
            return
        self._materialise_parameters()
        cnt = self._launch_set(keys.contiguous(), values.contiguous(), assume_unique)
        self._account_set(cnt, keys.shape[0])

    def _account_set(self, cnt, rows):
        """Device-side bookkeeping after a set launch that cannot have triggered a rehash."""
        self._n_elements += cnt[L.CNT_CLAIMED_EMPTY] + cnt[L.CNT_REUSED_REMOVED]
        self._n_tombstones -= cnt[L.CNT_REUSED_REMOVED]
        self._n_failed += cnt[L.CNT_FAILED]
        self._after_mutation(rows)

    # ------------------------------------------------------------------ sliced batches (the inbox of a sharded map)
    # keys / values / outputs hold n_slices * slice_rows rows; only the first counts[s] rows of slice s are in use, and
    # the counts (device int64[n_slices]) are read by the kernels, so nothing here waits for them.  `abort` (device
    # int64[1] or None): non-zero when the kernels run = do nothing.
    def _sliced_check(self, keys, n_slices, slice_rows, counts):
        assert self._slots is not None, "store something first"
        assert keys.dtype == self._key_dtype and keys.device == self.device and keys.is_contiguous()
        assert keys.shape == (n_slices * slice_rows,) + tuple(self._key_shape)
        assert counts.dtype == torch.long and counts.shape == (n_slices,) and counts.is_contiguous()

    def get_sliced(self, keys, n_slices, slice_rows, counts, abort, fallback_value, values, is_found):
        self._sliced_check(keys, n_slices, slice_rows, counts)
        fb, _keep = self._fallback_ptr(fallback_value)
        with torch.cuda.device(self.device):
            L.check(L.lib().dok_map_get_sliced(self._c_table(), self._c_hash(), L.ptr(keys), n_slices, slice_rows,
                                               L.ptr(counts), L.ptr(abort), L.ptr(values), L.ptr(is_found), fb, None,
                                               L.stream_ptr(self.device)), "dok_map_get_sliced")

    def remove_sliced(self, keys, n_slices, slice_rows, counts, abort, is_removed):
        self._sliced_check(keys, n_slices, slice_rows, counts)
        cnt = self._counters()
        with torch.cuda.device(self.device):
            L.check(L.lib().dok_map_remove_sliced(self._c_table(), self._c_hash(), L.ptr(keys), n_slices, slice_rows,
                                                  L.ptr(counts), L.ptr(abort), L.ptr(is_removed), L.ptr(cnt),
                                                  L.stream_ptr(self.device)), "dok_map_remove_sliced")
        self._n_elements -= cnt[L.CNT_HITS]
        self._n_tombstones += cnt[L.CNT_HITS]
        self._tombstone_host_bound += n_slices * slice_rows
        self._after_mutation(0)

    def set_sliced(self, keys, values, n_slices, slice_rows, counts, abort, assume_unique=False):
        """Insert-or-assign of a sliced batch.  As long as the table cannot reach its rehash threshold even if every
        row of every slice were new, everything stays on the device.  Otherwise the counts are read (a synchronisation
        of this rank only) and the slices go through `set` one after the other, which may rehash."""
        self._sliced_check(keys, n_slices, slice_rows, counts)
        assert values.dtype == self._value_dtype and values.is_contiguous()
        assert values.shape == (n_slices * slice_rows,) + tuple(self._value_shape)
        self._materialise_parameters()
        rows = n_slices * slice_rows
        limit = int(self._rehash_threshold * self.n_buckets)
        fast = self._room_for(rows, limit)
        if not fast:
            torch.cuda.current_stream(self.device).synchronize()
            fast = self.n_elements + rows <= limit
        if fast:
            cnt = self._counters()
            with torch.cuda.device(self.device):
                epoch, scratch = 0, None
                if not assume_unique:
                    epoch = self._next_epoch()
                    scratch = torch.empty(rows + 1, device=self.device, dtype=torch.long)
                L.check(L.lib().dok_map_set_sliced(self._c_table(), self._c_hash(), L.ptr(keys), L.ptr(values), n_slices,
                                                   slice_rows, L.ptr(counts), L.ptr(abort), L.ptr(scratch), epoch,
                                                   int(bool(assume_unique)), L.ptr(cnt), L.stream_ptr(self.device)),
                        "dok_map_set_sliced")
            self._account_set(cnt, rows)
            return
        if abort is not None and int(abort.item()) != 0:
            return
        for s, c in enumerate(counts.tolist()):
            if c:
                self.set(keys[s * slice_rows:s * slice_rows + c], values[s * slice_rows:s * slice_rows + c],
                         assume_unique=assume_unique)

    def _fallback_ptr(self, fallback_value):
        """-> (host pointer for the C ABI or None, the host tensor that must stay alive for the call)"""
        if fallback_value is None:
            return None, None
        if not isinstance(fallback_value, torch.Tensor):
            fallback_value = torch.tensor(fallback_value, dtype=self._value_dtype)
        host = torch.broadcast_to(fallback_value.to(dtype=self._value_dtype, device="cpu"), self.value_shape).contiguous()
        return ctypes.c_void_p(host.data_ptr()), host

    # ------------------------------------------------------------------ get
    def get(self, keys, fallback_value=None, values=None, is_found=None):
        """`values` / `is_found`: optional preallocated outputs (contiguous, [n, *value_shape] and bool [n]), like the
        `values=` argument of the reference launcher (closed_hashmap_impl.py:63)."""
        if self._slots is None:
            raise RuntimeError("store something first")
        if keys.shape[0] == 0:
            return (torch.empty(0, *self.value_shape, device=self.device, dtype=self._value_dtype),
                    torch.empty(0, device=self.device, dtype=torch.bool))
        assert keys.dtype == self._key_dtype
        assert keys.device == self.device
        assert keys.shape[1:] == self.key_shape
        fb, _keep = self._fallback_ptr(fallback_value)
        keys = keys.contiguous()
        n = keys.shape[0]
        if values is None:
            values = torch.empty(n, *self.value_shape, device=self.device, dtype=self._value_dtype)
        else:
            assert values.dtype == self._value_dtype and values.is_cuda and values.is_contiguous()
            assert values.shape == (n, *self.value_shape)
        if is_found is None:
            is_found = torch.empty(n, device=self.device, dtype=torch.bool)
        else:
            assert is_found.dtype == torch.bool and is_found.shape == (n,) and is_found.is_contiguous()
        with torch.cuda.device(self.device):
            L.check(L.lib().dok_map_get(self._c_table(), self._c_hash(), L.ptr(keys), n, L.ptr(values), L.ptr(is_found),
                                        fb, None, L.stream_ptr(self.device)), "dok_map_get")
        return values, is_found

    def probe_stats(self, keys):
        """(mean probe length, hit rate) of a lookup batch."""
        keys = keys.contiguous()
        n = keys.shape[0]
        values = torch.empty(n, *self.value_shape, device=self.device, dtype=self._value_dtype)
        cnt = self._counters()
        with torch.cuda.device(self.device):
            L.check(L.lib().dok_map_get_probe_stats(self._c_table(), self._c_hash(), L.ptr(keys), n, L.ptr(values), None,
                                                    L.ptr(cnt), L.stream_ptr(self.device)), "dok_map_get_probe_stats")
        cnt = cnt.cpu()
        return cnt[L.CNT_PROBES].item() / max(n, 1), cnt[L.CNT_HITS].item() / max(n, 1)

    # ------------------------------------------------------------------ remove
    def remove_rows(self, keys, is_removed=None):
        """Kernel only: flags aligned to the rows given (no dedup, no sort).  Equal rows report once.
        `is_removed`: optional preallocated bool[n] output."""
        keys = keys.contiguous()
        n = keys.shape[0]
        if is_removed is None:
            is_removed = torch.empty(n, device=self.device, dtype=torch.bool)
        else:
            assert is_removed.dtype == torch.bool and is_removed.shape == (n,) and is_removed.is_contiguous()
        cnt = self._counters()
        with torch.cuda.device(self.device):
            L.check(L.lib().dok_map_remove(self._c_table(), self._c_hash(), L.ptr(keys), n, L.ptr(is_removed), L.ptr(cnt),
                                           L.stream_ptr(self.device)), "dok_map_remove")
        self._n_elements -= cnt[L.CNT_HITS]
        self._n_tombstones += cnt[L.CNT_HITS]
        self._tombstone_host_bound += n
        self._after_mutation(0)
        self._maintain()
        return is_removed

    def _maintain(self):
        """Rebuild in place when live + tombstone slots exceed the tombstone threshold.  The host first looks at its
        own upper bounds (no synchronisation) and reads the device counts only when they cross."""
        if self._tombstone_threshold is None or self._slots is None:
            return
        auto = self._tombstone_threshold == "auto"
        limit = (0.95 if auto else self._tombstone_threshold) * self.n_buckets
        least = max(1, int(0.02 * self.n_buckets)) if auto else 1
        if self._tombstone_host_bound < least or self._element_bound() + self._tombstone_host_bound <= limit:
            return
        tombstones = int(self._n_tombstones.item())
        self._tombstone_host_bound = tombstones
        if tombstones >= least and self.n_elements + tombstones > limit:
            try:
                self.rebuild()
            except torch.OutOfMemoryError:
                import warnings
                warnings.warn("no room for a second slot array: the table keeps its tombstones "
                              f"({tombstones} of {self.n_buckets} buckets)")
                self._tombstone_host_bound = 0

    def rebuild(self):
        """The same table without its tombstones: a fresh slot array of the same geometry, every live slot re-inserted
        with the SAME hash parameters (one kernel, dok_map_reinsert).  Lookups, sizes and parameters are unchanged;
        shallow clones made before keep the old slot array (as after a rehash in the reference)."""
        if self._slots is None:
            return
        old_slots, old_stamp = self._slots, self._shared["stamp"]
        source = L.Table()
        source.slots = old_slots.data_ptr()
        source.stamp = old_stamp.data_ptr() if old_stamp is not None else None
        source.n_buckets = self._n_buckets
        source.slot_bytes = self._layout.slot_bytes
        source.value_bytes, source.key_bytes = self._value_bytes, self._key_bytes
        fresh = torch.empty(self._layout.total_bytes, device=self.device, dtype=torch.uint8)     # may raise: nothing changed yet
        self._slots = fresh
        self._shared["stamp"] = None
        self._shared["epoch"] = 0
        cnt = self._counters()
        with torch.cuda.device(self.device):
            st = L.stream_ptr(self.device)
            L.check(L.lib().dok_map_init(self._c_table(), st), "dok_map_init")
            L.check(L.lib().dok_map_reinsert(ctypes.byref(source), self._c_table(), self._c_hash(), L.ptr(cnt), st),
                    "dok_map_reinsert")
        old_slots.record_stream(torch.cuda.current_stream(self.device))
        self._n_failed += cnt[L.CNT_FAILED]
        self._n_tombstones.zero_()
        self._tombstone_host_bound = 0

    @property
    def tombstone_bound(self):
        """Upper bound of the tombstone slots, from the device counters (exact unless DOK assignments reused some)."""
        return int(self._n_tombstones.item())

    def remove(self, keys):
        if self._slots is None:
            raise RuntimeError("store something first")
        if keys.shape[0] == 0:
            return torch.zeros(0, device=keys.device, dtype=torch.bool)
        assert keys.dtype == self._key_dtype
        assert keys.device == self.device
        assert keys.shape[1:] == self.key_shape
        if int(np.prod(self._key_shape)) == 1 and keys.dtype not in L.FLOAT_DTYPES:
            # one integer column: a flat radix-sort unique gives the rows of `unique(dim=0)` in the same (sorted) order
            # without the lexicographic row sort
            unique_keys = torch.unique(keys.reshape(-1)).reshape((-1,) + tuple(self._key_shape))
        else:
            unique_keys = keys.unique(dim=0)
        return self.remove_rows(unique_keys)

    # ------------------------------------------------------------------ rehash
    def rehash(self, n_buckets):
        """New table of `n_buckets` with new random parameters holding the live items (cuda_closed_hashmap.py:456-468).
        One kernel walks the old slots and inserts every live one into the new table (dok_map_reinsert): no
        compaction, no pre-get, no unique.  Like the reference's recursive `set`, a table that the live items fill
        beyond the rehash threshold grows once more (and draws its parameters again)."""
        if self._slots is None:
            self.__init__(n_buckets=n_buckets, device=self.device, key_perm=self._key_perm,
                          rehash_factor=self._rehash_factor, rehash_threshold=self._rehash_threshold,
                          tombstone_threshold=self._tombstone_threshold)
            return
        live = self.count_live()
        old_slots, old_stamp = self._slots, self._shared["stamp"]          # kept alive until the kernel has run
        source = L.Table()
        source.slots = old_slots.data_ptr()
        source.stamp = old_stamp.data_ptr() if old_stamp is not None else None
        source.n_buckets = self._n_buckets
        source.slot_bytes = self._layout.slot_bytes
        source.value_bytes, source.key_bytes = self._value_bytes, self._key_bytes
        geometry = (self._key_shape, self._key_dtype, self._value_shape, self._value_dtype)
        self.__init__(
            n_buckets=n_buckets, device=self.device, key_perm=self._key_perm,
            rehash_factor=self._rehash_factor, rehash_threshold=self._rehash_threshold,
            tombstone_threshold=self._tombstone_threshold,
        )
        self._begin_bulk_insert(*geometry, live)
        if live:
            cnt = self._counters()
            with torch.cuda.device(self.device):
                L.check(L.lib().dok_map_reinsert(ctypes.byref(source), self._c_table(), self._c_hash(), L.ptr(cnt),
                                                 L.stream_ptr(self.device)), "dok_map_reinsert")
            old_slots.record_stream(torch.cuda.current_stream(self.device))

    # ------------------------------------------------------------------ persistence
    def state_dict(self):
        """Everything needed to rebuild the map, independent of the slot layout: the live (key, value) rows from one
        compaction pass, the hash parameters (so that uuids, and with them the owner shards of a sharded map, stay
        the same) and the sizing options.  Tombstones are not kept.  The reference has no checkpoint format."""
        if self._slots is not None:
            self._materialise_parameters()
        state = {"format": 1, "n_buckets": self.n_buckets, "rehash_factor": self._rehash_factor,
                 "rehash_threshold": self._rehash_threshold, "tombstone_threshold": self._tombstone_threshold,
                 "key_perm": None if self._key_perm is None else self._key_perm.cpu(), "keys": None, "values": None}
        for name in ("prime1", "prime2", "alpha1", "alpha2", "beta1", "beta2"):
            v = getattr(self, "_" + name)
            state[name] = None if v is None else v.cpu()
        if self._slots is not None:
            keys, values, _ = self.items(uuid=False)
            state["keys"] = keys.reshape((-1,) + tuple(self.key_shape)).cpu()
            state["values"] = values.cpu()
            state["n_elements"] = self.n_elements            # may over-count like the reference's DOK assignments do
        return state

    @classmethod
    def from_state_dict(cls, state, device="cuda:0"):
        assert state.get("format") == 1
        table = cls(n_buckets=state["n_buckets"], device=device, rehash_factor=state["rehash_factor"],
                    rehash_threshold=state["rehash_threshold"], tombstone_threshold=state.get("tombstone_threshold"),
                    key_perm=state["key_perm"],
                    **{name: state[name] for name in ("prime1", "prime2", "alpha1", "alpha2", "beta1", "beta2")})
        if state["keys"] is not None:
            keys, values = state["keys"].to(table.device), state["values"].to(table.device)
            if keys.shape[0]:      # items() gives key columns in the caller's order, like rehash relies on
                table.set(keys, values, assume_unique=True)
            else:
                table._allocate(keys.shape[1:], keys.dtype, values.shape[1:], values.dtype)
            table._n_elements.fill_(int(state["n_elements"]))
            table._shared["bound"] = int(state["n_elements"])
            table._shared["snapshots"].clear()
        return table

    def __getitem__(self, keys):
        return self.get(keys)

    def __setitem__(self, keys, values):
        return self.set(keys, values)

    def __delitem__(self, keys):
        return self.remove(keys)
