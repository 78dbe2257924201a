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

With `peer_capacity_rows > 0` (ranks of one node) steps 2, 3 and 5 are replaced by the peer exchange: the counts of
all ranks are gathered, the partition kernel stores each row straight into its owner's memory over NVLink (every rank
maps the others' exchange arenas), a one-element all-reduce on the stream orders the stores before the owners' reads,
and answers are delivered into the asker's memory the same way.  `run([...])` submits several operations at once and
overlaps the sending of one with the table work of the one before.  Batches that do not fit the arena take the
all-to-all path; `close()` releases the arena.

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
        self._pinned = None
        self._peer = None
        self._copy_stream = None
        self._in_flight = []

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

    # ------------------------------------------------------------------ peer exchange (NVLink, no exchange pass)
    supports_peer = True

    class _RawDeviceBytes:
        """Lets torch wrap device memory it did not allocate (the exchange arena, a peer's mapping of its arena)."""

        def __init__(self, ptr, nbytes):
            self.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (int(ptr), False), "version": 3}

    def peer_setup(self, group, world, rank, capacity_rows, key_row, value_row):
        """Collective.  Allocates this rank's exchange arena, maps every peer's, and returns True when all ranks
        succeeded (otherwise the arena is dropped everywhere and the NCCL exchange stays in use).
        key_row / value_row = (row shape, dtype).  Arena = two generations (alternating per batch) of
        {inbox keys | inbox values | result values | result flags}, each for capacity_rows rows."""
        lib = L.lib()
        self._peer = None
        (kshape, kdtype), (vshape, vdtype) = key_row, value_row
        kb = int(np.prod(kshape)) * torch.empty((), dtype=kdtype).element_size()
        vb = int(np.prod(vshape)) * torch.empty((), dtype=vdtype).element_size()
        cap = int(capacity_rows)
        up = lambda x: (x + 255) // 256 * 256
        sizes = [up(cap * kb), up(cap * vb), up(cap * vb), up(cap)]
        gen_bytes = sum(sizes)
        offs = [sum(sizes[:i]) for i in range(4)]
        ok, base, handle = 1, ctypes.c_void_p(), (ctypes.c_uint8 * 64)()
        with torch.cuda.device(self.device):
            if lib.dok_peer_alloc(2 * gen_bytes, ctypes.byref(base)) != 0 or lib.dok_peer_export(base, handle) != 0:
                ok = 0
        handles = [None] * world
        dist.all_gather_object(handles, (ok, bytes(handle)), group=group)
        ok = min(h[0] for h in handles)
        bases = [None] * world
        if ok:
            with torch.cuda.device(self.device):
                for r in range(world):
                    if r == rank:
                        bases[r] = base.value
                        continue
                    p = ctypes.c_void_p()
                    buf = (ctypes.c_uint8 * 64).from_buffer_copy(handles[r][1])
                    if lib.dok_peer_open(buf, ctypes.byref(p)) != 0:
                        ok = 0
                        break
                    bases[r] = p.value
        flag = torch.tensor([ok], device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag.item()) == 0:
            with torch.cuda.device(self.device):
                for r in range(world):
                    if bases[r] is not None and r != rank:
                        lib.dok_peer_close(ctypes.c_void_p(bases[r]))
                if base.value:
                    lib.dok_peer_free(base)
            return False
        views = [torch.as_tensor(self._RawDeviceBytes(bases[r], 2 * gen_bytes), device=self.device) for r in range(world)]
        # a second communicator for the fences of the apply stage: collectives of one communicator run in issue order,
        # and a fence that waits for table work must not hold up the count gather of the next operation's send stage
        group_apply = None
        if group is None or group is dist.group.WORLD:
            group_apply = dist.new_group(backend="nccl")
        self._peer = dict(group_apply=group_apply, world=world, rank=rank, cap=cap, kb=kb, vb=vb, kshape=tuple(kshape), kdtype=kdtype,
                          vshape=tuple(vshape), vdtype=vdtype, gen_bytes=gen_bytes, offs=offs, bases=bases, views=views,
                          own_base=base, token=torch.zeros(1, device=self.device),
                          token_apply=torch.zeros(1, device=self.device), group=group)
        return True

    def peer_close(self):
        """Collective in effect: call it on every rank, after all of them have finished using the exchange."""
        p, self._peer = getattr(self, "_peer", None), None
        if not p:
            return
        lib = L.lib()
        torch.cuda.synchronize(self.device)
        with torch.cuda.device(self.device):
            for r in range(p["world"]):
                if r != p["rank"]:
                    lib.dok_peer_close(ctypes.c_void_p(p["bases"][r]))
            lib.dok_peer_free(p["own_base"])

    def _peer_region(self, rank, generation, which, rows=None, row0=0):
        """Typed view of region `which` (0 inbox keys, 1 inbox values, 2 result values, 3 result flags) of `rank`'s
        arena, generation 0 / 1, rows [row0, row0 + rows)."""
        p = self._peer
        rows = p["cap"] - row0 if rows is None else rows
        width, shape, dtype = [(p["kb"], p["kshape"], p["kdtype"]), (p["vb"], p["vshape"], p["vdtype"]),
                               (p["vb"], p["vshape"], p["vdtype"]), (1, (), torch.bool)][which]
        lo = generation * p["gen_bytes"] + p["offs"][which] + row0 * width
        flat = p["views"][rank][lo:lo + rows * width]
        return flat.view(dtype).view((rows,) + tuple(shape))

    def peer_fence(self, apply_side=False):
        """Every rank's earlier work on its stream (stores into peers' arenas included) is complete before any rank's
        later work starts: a one-element all-reduce, ordered on the stream, not blocking the host.  `apply_side`
        fences travel on the second communicator when there is one."""
        p = self._peer
        group = p["group_apply"] if (apply_side and p["group_apply"] is not None) else p["group"]
        token = p["token_apply"] if apply_side else p["token"]
        dist.all_reduce(token, group=group)

    def can_pipeline(self):
        return self._peer is not None and self._peer["group_apply"] is not None

    def partition_count(self, keys, world):
        """First pass of the partition -> (owners, tile offsets, counts[2 * world] on the device)."""
        lib = L.lib()
        n = keys.shape[0]
        with torch.cuda.device(self.device):
            tiles = lib.dok_partition_tiles(n)
            offsets = torch.empty(world * tiles + 1, device=self.device, dtype=torch.long)
            counts = torch.empty(2 * world, device=self.device, dtype=torch.long)
            owners = torch.empty(n, device=self.device, dtype=torch.uint8)
            L.check(lib.dok_shard_partition_count(self._routing_hash(keys), L.ptr(keys), n, world, L.ptr(owners),
                                                  L.ptr(offsets), L.ptr(counts), L.stream_ptr(self.device)),
                    "dok_shard_partition_count")
        return owners, offsets, counts

    def scatter_to_peers(self, keys, values, world, owners, offsets, counts, generation, row0, want_dest):
        """Second pass with the owners' inboxes as destinations; row0[o] = first row of this rank's segment there."""
        lib = L.lib()
        p = self._peer
        n = keys.shape[0]
        gen = generation * p["gen_bytes"]
        arr_p = ctypes.c_void_p * world
        peer_keys = arr_p(*[p["bases"][o] + gen + p["offs"][0] for o in range(world)])
        peer_values = arr_p(*[p["bases"][o] + gen + p["offs"][1] for o in range(world)])
        rows = (ctypes.c_int64 * world)(*[int(r) for r in row0])
        dest = torch.empty(n, device=self.device, dtype=torch.long) if want_dest else None
        vb = 0 if values is None else p["vb"]
        with torch.cuda.device(self.device):
            L.check(lib.dok_shard_partition_scatter_peer(L.ptr(keys), p["kb"], L.ptr(values), vb, n, world, L.ptr(owners),
                                                         L.ptr(offsets), L.ptr(counts), peer_keys,
                                                         peer_values if values is not None else None, rows, L.ptr(dest),
                                                         L.stream_ptr(self.device)), "dok_shard_partition_scatter_peer")
        return dest

    def partition(self, keys, values, world, want_dest=True):
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
            owners = torch.empty(n, device=self.device, dtype=torch.uint8)
            L.check(lib.dok_shard_partition_count(self._routing_hash(keys), L.ptr(keys), n, world, L.ptr(owners),
                                                  L.ptr(offsets), L.ptr(counts), st), "dok_shard_partition_count")
            grouped_keys = torch.empty((cap,) + tuple(keys.shape[1:]), device=self.device, dtype=keys.dtype)
            kb = int(np.prod(keys.shape[1:])) * keys.element_size()
            grouped_values, vb = None, 0
            if values is not None:
                values = values.contiguous()
                grouped_values = torch.empty((cap,) + tuple(values.shape[1:]), device=self.device, dtype=values.dtype)
                vb = int(np.prod(values.shape[1:])) * values.element_size()
            dest = torch.empty(n, device=self.device, dtype=torch.long) if want_dest else None
            L.check(lib.dok_shard_partition_scatter(L.ptr(keys), kb, L.ptr(values), vb, n, world, L.ptr(owners),
                                                    L.ptr(offsets), L.ptr(counts), L.ptr(grouped_keys),
                                                    L.ptr(grouped_values), L.ptr(dest), st), "dok_shard_partition_scatter")
        return grouped_keys, grouped_values, dest, counts.view(2, world)

    def unpermute(self, grouped_values, grouped_flags, dest, out_values=None, out_flags=None):
        """out[i] = grouped[dest[i]]; writes into out_values / out_flags (contiguous, dest.shape[0] rows) when given."""
        lib = L.lib()
        n = dest.shape[0]
        vb = 0
        with torch.cuda.device(self.device):
            if grouped_values is not None:
                if out_values is None:
                    out_values = torch.empty((n,) + tuple(grouped_values.shape[1:]), device=self.device, dtype=grouped_values.dtype)
                assert out_values.is_contiguous() and out_values.shape[0] == n
                vb = int(np.prod(grouped_values.shape[1:])) * grouped_values.element_size()
            if grouped_flags is not None:
                if out_flags is None:
                    out_flags = torch.empty(n, device=self.device, dtype=grouped_flags.dtype)
                assert out_flags.is_contiguous() and out_flags.shape[0] == n
            L.check(lib.dok_shard_unpermute(L.ptr(grouped_values), L.ptr(grouped_flags), L.ptr(dest), vb, n,
                                            L.ptr(out_values) if grouped_values is not None else None,
                                            L.ptr(out_flags) if grouped_flags is not None else None,
                                            L.stream_ptr(self.device)), "dok_shard_unpermute")
        return (out_values if grouped_values is not None else None), (out_flags if grouped_flags is not None else None)

    # local table ops on the rows this rank owns.  `segments` = [(start, rows)] per source rank inside the received
    # buffer (starts are aligned, the gaps hold nothing); sources are processed in rank order, which is what makes
    # "last row wins" global.
    def local_get(self, keys, segments, fallback_value):
        values = torch.empty((keys.shape[0],) + tuple(self.local.value_shape), device=self.device, dtype=self.local.value_type)
        found = torch.empty(keys.shape[0], device=self.device, dtype=torch.bool)
        for start, rows in segments:
            if rows:      # the kernel writes straight into the segment's rows of the result buffers
                self.local.get(keys[start:start + rows], fallback_value, values=values[start:start + rows],
                               is_found=found[start:start + rows])
        return values, found

    def local_set(self, keys, values, segments, assume_unique):
        for start, rows in segments:
            if rows:
                self.local.set(keys[start:start + rows], values[start:start + rows], assume_unique=assume_unique)

    def local_remove(self, keys, segments):
        flags = torch.empty(keys.shape[0], device=self.device, dtype=torch.bool)
        for start, rows in segments:
            if rows:
                flags[start:start + rows] = self.local.remove_rows(keys[start:start + rows])
        return flags

    def local_answer(self, keys, values, flags, fallback_value, remote):
        """get (values given) or remove (values None) of one source's rows, answers delivered into `values` /
        `flags`.  For another rank's rows (`remote`) those are views of the asker's memory: the kernel then answers
        into local buffers and a bulk copy on a side stream carries them over NVLink while the next source's rows are
        being probed -- row-sized stores from the probing kernel itself use the link far worse."""
        if not remote:
            self._answer(keys, values, flags, fallback_value)
            return
        local_values = None if values is None else torch.empty_like(values)
        local_flags = torch.empty_like(flags)
        self._answer(keys, local_values, local_flags, fallback_value)
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=self.device)
        answered = torch.cuda.Event()
        answered.record()
        with torch.cuda.stream(self._copy_stream):
            self._copy_stream.wait_event(answered)
            if values is not None:
                values.copy_(local_values, non_blocking=True)
            flags.copy_(local_flags, non_blocking=True)
        self._in_flight.append((local_values, local_flags))

    def answers_delivered(self):
        """The current stream waits for the bulk copies of local_answer; their source buffers may then be reused."""
        if self._in_flight:
            done = torch.cuda.Event()
            done.record(self._copy_stream)
            torch.cuda.current_stream(self.device).wait_event(done)
            self._in_flight = []

    def _answer(self, keys, values, flags, fallback_value):
        if self.local._slots is None:              # this shard holds nothing yet: every row is a miss
            if values is not None:
                values[:] = torch.as_tensor(0 if fallback_value is None else fallback_value, dtype=values.dtype)
            flags[:] = False
        elif values is not None:
            self.local.get(keys, fallback_value, values=values, is_found=flags)
        else:
            self.local.remove_rows(keys, is_removed=flags)

    def local_n_elements(self):
        return self.local._n_elements

    def to_host(self, words):
        """Small int64 device tensor -> list of ints on the host, through a kernel store into pinned memory (a copy
        would wait behind bulk device-to-host transfers that other streams have in flight)."""
        n = words.numel()
        if self._pinned is None or self._pinned.numel() < n:
            self._pinned = torch.empty(max(n, 4 * L.MAX_SHARDS), dtype=torch.long, pin_memory=True)
        flat = words.contiguous().reshape(-1)
        with torch.cuda.device(self.device):
            L.check(L.lib().dok_words_to_pinned(L.ptr(flat), ctypes.c_void_p(self._pinned.data_ptr()), n,
                                                L.stream_ptr(self.device)), "dok_words_to_pinned")
            done = torch.cuda.Event()
            done.record()
        done.synchronize()
        return self._pinned[:n].tolist()

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
                 rehash_factor=2.0, rehash_threshold=0.75, ops=None, pipeline_chunks=2, peer_capacity_rows=0):
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
        self.pipeline_chunks = max(1, int(pipeline_chunks))     # must be the same on every rank
        # Peer exchange (ranks of ONE node, NVLink): with peer_capacity_rows > 0 (the same on every rank) the rows of
        # a batch are stored straight into the owners' memory by the partition kernel, and answers straight into the
        # askers', instead of travelling through all-to-all passes.  A batch that does not fit the capacity (rows
        # received by any owner, or rows of any rank's own batch, padding included) takes the all-to-all path.
        self._peer_capacity = int(peer_capacity_rows) if (self.world > 1 and self.world <= 16) else 0
        self._peer_on = False
        self._peer_seq = 0
        self._streams = None
        self._last_applied = None
        self._value_shape = None
        self._value_dtype = None

    # ------------------------------------------------------------------ exchange plumbing
    def _exchange_counts(self, counts):
        """counts[2, world] (device; rows and padded rows per owner) -> (send_padded, recv_rows, recv_padded) as host
        lists; one synchronisation per batch."""
        send = counts.t().contiguous()                       # [world, 2]: what goes to each owner
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        flat = self.ops.to_host(torch.stack([send, recv]))          # [2, world, 2] flattened
        w = self.world
        send_h = [flat[2 * i:2 * i + 2] for i in range(w)]
        recv_h = [flat[2 * w + 2 * i:2 * w + 2 * i + 2] for i in range(w)]
        return [int(c[1]) for c in send_h], [int(c[0]) for c in recv_h], [int(c[1]) for c in recv_h]

    def _all_to_all_rows(self, rows, send, recv, async_op=False):
        """rows grouped by destination -> rows grouped by source.  With async_op the exchange is only enqueued:
        returns (out, work) and the caller waits on `work` before touching `out`."""
        if self.world == 1:
            return (rows, None) if async_op else rows
        out = self.ops.empty((sum(recv),) + tuple(rows.shape[1:]), rows.dtype)
        work = dist.all_to_all_single(out, rows, output_split_sizes=recv, input_split_sizes=send, group=self.group,
                                      async_op=async_op)
        return (out, work) if async_op else out

    def _route(self, keys, values=None, want_dest=True, async_op=False):
        """-> (owned_keys, owned_values, segments, dest, send, recv[, works]); segments = [(start, rows)] per source
        rank.  With async_op the key / value exchanges are in flight on return and `works` must be waited for."""
        if self.world == 1:        # one shard owns everything: no partition, no exchange, no permutation
            out = (keys, values, [(0, keys.shape[0])], None, None, None)
            return out + ([],) if async_op else out
        grouped_keys, grouped_values, dest, counts = self.ops.partition(keys, values, self.world, want_dest=want_dest)
        send, recv_rows, recv = self._exchange_counts(counts)
        assert keys.shape[0] <= sum(send) <= grouped_keys.shape[0], "partition lost rows"
        works = []
        owned_keys, w = self._all_to_all_rows(grouped_keys[:sum(send)], send, recv, async_op=True)
        works.append(w)
        owned_values = None
        if values is not None:
            owned_values, w = self._all_to_all_rows(grouped_values[:sum(send)], send, recv, async_op=True)
            works.append(w)
        starts = [sum(recv[:i]) for i in range(self.world)]
        out = (owned_keys, owned_values, list(zip(starts, recv_rows)), dest, send, recv)
        if async_op:
            return out + (works,)
        for w in works:
            w.wait()
        return out

    def _chunk_bounds(self, n, pipelined):
        """The same number of chunks on every rank (the calls are collective), whatever each rank's batch size."""
        c = self.pipeline_chunks if (pipelined and self.world > 1) else 1
        return [(n * i // c, n * (i + 1) // c) for i in range(c)]

    # ------------------------------------------------------------------ peer exchange
    def _peer_plan(self, keys):
        """First partition pass and the gathered count matrix -> plan, or None when this batch must take the
        all-to-all path (the decision is made from the same matrix on every rank, so all ranks agree)."""
        w, r = self.world, self.rank
        keys = keys.contiguous()
        owners, offsets, counts = self.ops.partition_count(keys, w)
        matrix = self.ops.empty((w, 2 * w), torch.long)
        dist.all_gather_into_tensor(matrix, counts, group=self.group)
        flat = self.ops.to_host(matrix)
        exact = [[int(flat[s * 2 * w + o]) for o in range(w)] for s in range(w)]        # [source][owner]
        padded = [[int(flat[s * 2 * w + w + o]) for o in range(w)] for s in range(w)]
        cap = self._peer_capacity
        if max(sum(exact[s][o] for s in range(w)) for o in range(w)) > cap or max(sum(row) for row in padded) > cap:
            return None
        gen = self._peer_seq & 1
        self._peer_seq += 1
        # Inboxes are filled without gaps: the sources' segments follow each other in rank order at their exact row
        # counts (stores need no alignment, unlike the all-to-all), so an owner can apply everything it received
        # with one launch, in which row order is (source rank, row): the order that makes "last row wins" global.
        # Result regions keep the padded starts of the asker's grouped order, which is what dest_index refers to.
        starts, run = [], 0
        for s in range(w):
            starts.append(run)
            run += exact[s][r]
        return dict(keys=keys, owners=owners, offsets=offsets, counts=counts, exact=exact, padded=padded, gen=gen,
                    row0=[sum(exact[s][o] for s in range(r)) for o in range(w)],
                    segments=[(starts[s], exact[s][r]) for s in range(w)], inbox_rows=run)

    # An operation over the peer exchange has two stages.  SEND: rows into the owners' inboxes (partition + stores
    # over NVLink).  APPLY: the owner's table work on what it received, answers into the askers' result regions, the
    # inverse permutation.  A fence (one-element all-reduce on the stream) separates them.
    def _peer_send(self, plan, values, want_dest):
        plan["dest"] = self.ops.scatter_to_peers(plan["keys"], values, self.world, plan["owners"], plan["offsets"],
                                                 plan["counts"], plan["gen"], plan["row0"], want_dest=want_dest)

    def _peer_apply_set(self, plan, assume_unique):
        owned_keys = self.ops._peer_region(self.rank, plan["gen"], 0, rows=plan["inbox_rows"])
        owned_values = self.ops._peer_region(self.rank, plan["gen"], 1, rows=plan["inbox_rows"])
        self.ops.local_set(owned_keys, owned_values, [(0, plan["inbox_rows"])], assume_unique)     # one launch

    def _peer_apply_lookup(self, plan, with_values, fallback_value):
        w, r, ops = self.world, self.rank, self.ops
        gen, padded = plan["gen"], plan["padded"]
        owned_keys = ops._peer_region(r, gen, 0, rows=plan["inbox_rows"])
        if with_values:
            # lookups commute: other ranks' rows first, source by source, so that the copy of their answers over NVLink
            # runs while the next source's rows (and last this rank's own) are probed
            for s in [s for s in range(w) if s != r] + [r]:
                start, rows = plan["segments"][s]
                if not rows:
                    continue
                at = sum(padded[s][o] for o in range(r))    # my segment in source s's grouped order
                ops.local_answer(owned_keys[start:start + rows], ops._peer_region(s, gen, 2, rows=rows, row0=at),
                                 ops._peer_region(s, gen, 3, rows=rows, row0=at), fallback_value, remote=(s != r))
        else:
            # removals source by source in rank order, one launch each: among equal keys of different ranks the
            # earlier rank reports the removal, and one launch over everything would leave that to the race
            for s, (start, rows) in enumerate(plan["segments"]):
                if rows:
                    at = sum(padded[s][o] for o in range(r))
                    ops.local_answer(owned_keys[start:start + rows], None, ops._peer_region(s, gen, 3, rows=rows, row0=at),
                                     None, remote=(s != r))
        ops.answers_delivered()
        ops.peer_fence(apply_side=True)
        n_mine = sum(padded[r])
        res_flags = ops._peer_region(r, gen, 3, rows=n_mine).view(torch.uint8)
        res_values = ops._peer_region(r, gen, 2, rows=n_mine) if with_values else None
        out_values, out_flags = ops.unpermute(res_values, res_flags, plan["dest"])
        return out_values, out_flags.view(torch.bool)

    def _peer_lookup(self, plan, with_values, fallback_value):
        """get / remove over the peer exchange, one operation at a time."""
        self._peer_send(plan, None, want_dest=True)
        self.ops.peer_fence()
        return self._peer_apply_lookup(plan, with_values, fallback_value)

    def run(self, operations, wait=True):
        """Several operations as one software pipeline: [("get", keys[, fallback_value]), ("set", keys, values[,
        assume_unique]), ("remove", keys)] -> list of results (get: (values, is_found); set: None; remove: flags).
        Collective: every rank passes the same sequence of operation kinds.  The operations are applied in order, as if
        called one after the other; what overlaps is the SEND stage of operation k + 1 (it only reads the caller's
        batch: partition, count gather, stores into the owners' other inbox generation over NVLink) with the APPLY
        stage of operation k (table work in HBM), on two streams.  Without the peer exchange the operations simply
        run one after the other.  Results are ready for the caller's current stream when the call returns -- unless
        `wait=False`: then the call only enqueues, the next submission's first send may overlap this one's last table
        work, and the caller calls `wait()` before it uses results or reuses / frees the input tensors (which must
        already be complete on the current stream at the time of the call)."""
        if not operations:
            return []
        if not self._peer_on or not self.ops.can_pipeline():
            return [self._run_one(op) for op in operations]
        ops = self.ops
        device = ops.device
        if self._streams is None:
            # the send stage runs at high priority: its kernels are short, and behind the big grids of the table work
            # they would otherwise only start when those have handed out all their blocks
            self._streams = (torch.cuda.Stream(device=device, priority=-1), torch.cuda.Stream(device=device))
        s_send, s_apply = self._streams
        main = torch.cuda.current_stream(device)
        start = torch.cuda.Event()
        start.record(main)
        s_send.wait_event(start)
        s_apply.wait_event(start)
        results = [None] * len(operations)

        def send(i):
            """-> plan with the fence still to come, or None when the batch must take the all-to-all path"""
            kind, keys = operations[i][0], operations[i][1]
            with torch.cuda.stream(s_send):
                plan = self._peer_plan(keys)
                if plan is not None:
                    values = operations[i][2].contiguous() if kind == "set" else None
                    self._peer_send(plan, values, want_dest=(kind != "set"))
                    if plan["dest"] is not None:
                        plan["dest"].record_stream(s_apply)
            return plan

        def fence(plan, applied):
            """all ranks' sends of this operation and applies of the previous one are complete past this point"""
            with torch.cuda.stream(s_send):
                if applied is not None:
                    s_send.wait_event(applied)
                ops.peer_fence()
                sent = torch.cuda.Event()
                sent.record(s_send)
            return sent

        def apply(i, plan, sent):
            kind = operations[i][0]
            with torch.cuda.stream(s_apply):
                s_apply.wait_event(sent)
                if kind == "set":
                    self._peer_apply_set(plan, operations[i][3] if len(operations[i]) > 3 else False)
                elif kind == "get":
                    results[i] = self._peer_apply_lookup(plan, True, operations[i][2] if len(operations[i]) > 2 else None)
                else:
                    results[i] = self._peer_apply_lookup(plan, False, None)[1]
                for t in (results[i] if isinstance(results[i], tuple) else (results[i],)):
                    if t is not None:
                        t.record_stream(main)
                applied = torch.cuda.Event()
                applied.record(s_apply)
            return applied

        def drain():
            for s in (s_send, s_apply):
                ev = torch.cuda.Event()
                ev.record(s)
                main.wait_event(ev)

        assert all(op[0] in ("get", "set", "remove") for op in operations)
        applied = self._last_applied          # table work of an earlier submission that was not waited for
        plan = send(0)
        sent = fence(plan, applied) if plan is not None else None
        for i in range(len(operations)):
            if plan is None:
                # this batch does not fit the arena: everything so far completes, then the all-to-all path
                drain()
                self._last_applied = None
                results[i] = self._run_one(operations[i], peer=False)
                back = torch.cuda.Event()
                back.record(main)
                s_send.wait_event(back)
                s_apply.wait_event(back)
                applied = None
                nxt = send(i + 1) if i + 1 < len(operations) else None
            else:
                applied = apply(i, plan, sent)                                # enqueued; the table work takes a while
                nxt = send(i + 1) if i + 1 < len(operations) else None       # runs meanwhile (the host waits for counts)
            if i + 1 < len(operations):
                plan = nxt
                sent = fence(plan, applied) if plan is not None else None
        self._last_applied = applied
        if wait:
            drain()
            self._last_applied = None
        return results

    def _settle(self):
        """Operations called one at a time run on the caller's stream: anything still in flight from a submission
        that was not waited for must be ordered before them."""
        if self._last_applied is not None:
            self.wait()

    def wait(self):
        """The caller's current stream waits for everything submitted with run(..., wait=False)."""
        if self._streams is not None:
            main = torch.cuda.current_stream(self.ops.device)
            for s in self._streams:
                ev = torch.cuda.Event()
                ev.record(s)
                main.wait_event(ev)
        self._last_applied = None

    def _run_one(self, op, peer=True):
        kind = op[0]
        saved, self._peer_on = self._peer_on, self._peer_on and peer
        try:
            if kind == "set":
                return self.set(op[1], op[2], assume_unique=op[3] if len(op) > 3 else False)
            if kind == "get":
                return self.get(op[1], op[2] if len(op) > 2 else None)
            return self.remove(op[1])
        finally:
            self._peer_on = saved

    # ------------------------------------------------------------------ operations
    def set(self, keys, values, assume_unique=False):
        """Collective insert-or-assign.  `assume_unique` promises pairwise different keys across ALL ranks' batches."""
        self._settle()
        if self._value_shape is None:
            self._value_shape, self._value_dtype = tuple(values.shape[1:]), values.dtype
            if self._peer_capacity and getattr(self.ops, "supports_peer", False):
                self._peer_on = self.ops.peer_setup(self.group, self.world, self.rank, self._peer_capacity,
                                                    (tuple(keys.shape[1:]), keys.dtype), (self._value_shape, self._value_dtype))
        if self._peer_on:
            plan = self._peer_plan(keys)
            if plan is not None:
                self._peer_send(plan, values.contiguous(), want_dest=False)
                self.ops.peer_fence()
                self._peer_apply_set(plan, assume_unique)
                return
        owned_keys, owned_values, segments, _, _, _ = self._route(keys, values, want_dest=False)
        self.ops.local_set(owned_keys, owned_values, segments, assume_unique)

    def state_dict(self):
        """This rank's shard (see CudaClosedHashmap.state_dict) plus the sharding it belongs to.  Every rank saves its
        own; a map rebuilt with the same world size and parameters routes every key to the shard that holds it."""
        return {"world": self.world, "rank": self.rank, "shard": self.ops.local.state_dict(),
                "value_shape": self._value_shape, "value_dtype": self._value_dtype}

    def load_state_dict(self, state):
        """Replaces this rank's shard by a saved one (same world size and rank)."""
        assert state["world"] == self.world and state["rank"] == self.rank, "a shard belongs to its rank"
        self.ops.local = CudaClosedHashmap.from_state_dict(state["shard"], device=self.ops.device)
        self._value_shape, self._value_dtype = state["value_shape"], state["value_dtype"]

    def close(self):
        """Releases the peer exchange arena (every rank, after the last operation)."""
        if self._peer_on:
            self._peer_on = False
            self.ops.peer_close()

    def _lookup(self, keys, local_op, with_values, fallback_value=None):
        """Shared body of get and remove.  For get the batch is cut into `pipeline_chunks` pieces that move through
        partition -> key exchange -> local op -> result exchange -> inverse permutation as a software pipeline: the
        exchanges are enqueued asynchronously, so the key exchange of piece i + 1 and the result exchange of piece
        i - 1 run while the table is probed for piece i.  remove goes through in one piece: cutting it would let a
        later rank's first piece overtake an earlier rank's second, and which of two equal keys reports the removal
        is defined by rank order."""
        n = keys.shape[0]
        out_values = self.ops.empty((n,) + self._value_shape, self._value_dtype) if with_values else None
        out_flags = self.ops.empty((n,), torch.bool)
        bounds = self._chunk_bounds(n, pipelined=with_values)
        routed, returned = [], []

        def probe(i):
            owned_keys, _, segments, dest, send, recv, works = routed[i]
            for w in works:
                if w is not None:
                    w.wait()
            if self.ops.ready() and owned_keys.shape[0]:
                res = local_op(owned_keys, segments)
                owned_values, owned_flags = res if with_values else (None, res)
            else:
                # this shard holds nothing yet (or received nothing): every row it was asked about is a miss
                owned_values = None
                if with_values:
                    owned_values = self.ops.empty((owned_keys.shape[0],) + self._value_shape, self._value_dtype)
                    fill = 0 if fallback_value is None else fallback_value
                    if owned_values.numel():
                        owned_values[:] = torch.as_tensor(fill, dtype=self._value_dtype)
                owned_flags = self.ops.empty((owned_keys.shape[0],), torch.bool)
                owned_flags[:] = False
            if dest is None:
                returned.append((owned_values, owned_flags, None, []))
                return
            works = []
            back_values = None
            if with_values:
                back_values, w = self._all_to_all_rows(owned_values, recv, send, async_op=True)
                works.append(w)
            back_flags, w = self._all_to_all_rows(owned_flags.view(torch.uint8), recv, send, async_op=True)
            works.append(w)
            returned.append((back_values, back_flags, dest, works))

        for i, (lo, hi) in enumerate(bounds):
            routed.append(self._route(keys[lo:hi], async_op=True))
            if i >= 1:
                probe(i - 1)
        probe(len(bounds) - 1)
        for (lo, hi), (values, flags, dest, works) in zip(bounds, returned):
            for w in works:
                if w is not None:
                    w.wait()
            if dest is None:
                if with_values:
                    out_values[lo:hi] = values
                out_flags[lo:hi] = flags
            else:
                self.ops.unpermute(values, flags, dest, out_values[lo:hi] if with_values else None,
                                   out_flags[lo:hi].view(torch.uint8))
        return out_values, out_flags

    def get(self, keys, fallback_value=None):
        """Collective lookup -> (values[n, *value_shape], is_found[n]) in the caller's row order."""
        if self._value_shape is None:
            raise RuntimeError("store something first")
        self._settle()
        if self.world == 1:
            if not self.ops.ready():
                return self._lookup(keys, None, True, fallback_value)
            return self.ops.local_get(keys, [(0, keys.shape[0])], fallback_value)
        if self._peer_on:
            plan = self._peer_plan(keys)
            if plan is not None:
                return self._peer_lookup(plan, True, fallback_value)
        return self._lookup(keys, lambda k, seg: self.ops.local_get(k, seg, fallback_value), True, fallback_value)

    def remove(self, keys):
        """Collective removal -> is_removed[n] aligned to the caller's rows (equal keys report once)."""
        if self._value_shape is None:
            raise RuntimeError("store something first")
        self._settle()
        if self.world == 1 and self.ops.ready():
            return self.ops.local_remove(keys, [(0, keys.shape[0])])
        if self._peer_on:
            plan = self._peer_plan(keys)
            if plan is not None:
                return self._peer_lookup(plan, False, None)[1]
        return self._lookup(keys, lambda k, seg: self.ops.local_remove(k, seg), False)[1]

    @property
    def n_elements(self):
        """Live rows over all shards (collective)."""
        self._settle()
        n = self.ops.local_n_elements().clone().reshape(1)
        if self.world > 1:
            dist.all_reduce(n, group=self.group)
        return int(n.item())

    def __len__(self):
        return self.n_elements
