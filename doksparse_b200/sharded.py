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
        self._sx = None
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

    # ------------------------------------------------------------------ sliced exchange (NVLink, no host in the loop)
    supports_sliced = True

    class _RawDeviceBytes:
        """Lets torch wrap device memory it did not allocate (the exchange arena, a peer's mapping of its arena)."""

        def __init__(self, ptr, nbytes):
            self.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (int(ptr), False), "version": 3}

    # Generations of the arena, used in turn by consecutive operations.  Two would do for correctness (the send of
    # operation k + 1 overlaps the apply of operation k), but then the fence of operation k must wait for every rank's
    # apply of k - 1, which turns every apply into a barrier across the ranks; with four, a fence waits for the apply of
    # three operations back, and the ranks drift freely within a step.
    GENERATIONS = 4

    @staticmethod
    def sliced_geometry(world, capacity_rows, key_row, value_row, slack_sigmas=8.0):
        """Arena layout for batches of up to `capacity_rows` rows per rank.  A slice holds the rows one source sends
        to one owner: capacity / world on average; with a uniform owner hash the count is binomial, so a slack of a
        few standard deviations (plus a constant for tiny batches) makes an overflow a non-event, and a batch that
        overflows all the same (skewed keys) is repeated over the exact exchange.  One generation =
        {inbox keys | inbox values | inbox counts | result values | result flags}, each for world slices; inbox slice s
        holds what source rank s sent here, result slice o what owner rank o answered."""
        (kshape, kdtype), (vshape, vdtype) = key_row, value_row
        kb = int(np.prod(kshape)) * torch.empty((), dtype=kdtype).element_size()
        vb = int(np.prod(vshape)) * torch.empty((), dtype=vdtype).element_size()
        cap = max(int(capacity_rows), 1)
        mean = cap / world
        rows = int(np.ceil(mean + slack_sigmas * np.sqrt(mean) + 64))
        rows = min(rows, cap)
        rows = (rows + 255) // 256 * 256                   # slices start 16-byte aligned whatever the row width
        up = lambda x: (x + 255) // 256 * 256
        sizes = [up(world * rows * kb), up(world * rows * vb), up(world * 8), up(world * rows * vb), up(world * rows)]
        return dict(world=world, cap=cap, slice_rows=rows, kb=kb, vb=vb, kshape=tuple(kshape), kdtype=kdtype,
                    vshape=tuple(vshape), vdtype=vdtype, sizes=sizes, offs=[sum(sizes[:i]) for i in range(5)],
                    gen_bytes=sum(sizes), generations=CudaShardOps.GENERATIONS)

    def sliced_alloc(self, geometry):
        """This rank's arena (all generations); returns its base address or None."""
        base = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            if L.lib().dok_peer_alloc(geometry["generations"] * geometry["gen_bytes"], ctypes.byref(base)) != 0:
                return None
        return base.value

    def sliced_attach(self, geometry, bases, rank, group=None, group_apply=None, own_base=None, ipc=True):
        """`bases[r]` = address of rank r's arena as THIS process sees it (its own allocation, a CUDA IPC mapping of a
        peer's, or -- when several ranks are emulated in one process -- another local allocation)."""
        g = dict(geometry)
        w, rows = g["world"], g["slice_rows"]
        views = [torch.as_tensor(self._RawDeviceBytes(b, g["generations"] * g["gen_bytes"]), device=self.device) for b in bases]
        g.update(bases=list(bases), views=views, rank=rank, group=group, group_apply=group_apply, own_base=own_base, ipc=ipc,
                 status=torch.zeros(1, device=self.device, dtype=torch.long),
                 token_apply=torch.zeros(1, device=self.device),
                 answer_values=torch.empty((w * rows,) + g["vshape"], device=self.device, dtype=g["vdtype"]),
                 answer_flags=torch.empty(w * rows, device=self.device, dtype=torch.bool))
        for gen in range(g["generations"]):                    # counts start at zero
            self._sx = g
            self._region(rank, gen, 2).zero_()
        self._sx = g

    def sliced_setup(self, group, world, rank, capacity_rows, key_row, value_row):
        """Collective.  Allocates this rank's arena, maps every peer's (CUDA IPC) and returns True when all ranks
        succeeded; otherwise everything is released again and the exact exchange stays in use."""
        lib = L.lib()
        self._sx = None
        geometry = self.sliced_geometry(world, capacity_rows, key_row, value_row)
        base = self.sliced_alloc(geometry)
        ok, handle = int(base is not None), (ctypes.c_uint8 * 64)()
        if ok:
            with torch.cuda.device(self.device):
                ok = int(lib.dok_peer_export(ctypes.c_void_p(base), handle) == 0)
        handles = [None] * world
        dist.all_gather_object(handles, (ok, bytes(handle)), group=group)
        ok = min(h[0] for h in handles)
        bases = [None] * world
        if ok:
            with torch.cuda.device(self.device):
                for r in range(world):
                    if r == rank:
                        bases[r] = base
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
                if base:
                    lib.dok_peer_free(ctypes.c_void_p(base))
            return False
        # a second communicator for the fences of the apply stage: collectives of one communicator run in issue order,
        # and a fence that waits for table work must not hold up the fence of the next operation's send stage
        group_apply = dist.new_group(backend="nccl") if (group is None or group is dist.group.WORLD) else None
        self.sliced_attach(geometry, bases, rank, group=group, group_apply=group_apply, own_base=base)
        return True

    def sliced_close(self):
        """Collective in effect: call it on every rank, after all of them have finished using the exchange."""
        p, self._sx = getattr(self, "_sx", None), None
        if not p or p.get("own_base") is None:
            return
        lib = L.lib()
        torch.cuda.synchronize(self.device)
        with torch.cuda.device(self.device):
            for r in range(p["world"]):
                if r != p["rank"] and p["ipc"]:
                    lib.dok_peer_close(ctypes.c_void_p(p["bases"][r]))
            lib.dok_peer_free(ctypes.c_void_p(p["own_base"]))

    def _region_ptr(self, rank, generation, which, row0=0):
        p = self._sx
        width = [p["kb"], p["vb"], 8, p["vb"], 1][which]
        return p["bases"][rank] + generation * p["gen_bytes"] + p["offs"][which] + row0 * width

    def _region(self, rank, generation, which, rows=None, row0=0):
        """Typed view of region `which` (0 inbox keys, 1 inbox values, 2 inbox counts, 3 result values, 4 result
        flags) of `rank`'s arena, generation 0 .. GENERATIONS - 1, rows [row0, row0 + rows)."""
        p = self._sx
        cache = p.setdefault("region_cache", {})
        hit = cache.get((rank, generation, which, rows, row0))
        if hit is not None:
            return hit
        asked = (rank, generation, which, rows, row0)
        total = p["world"] if which == 2 else p["world"] * p["slice_rows"]
        rows = total - row0 if rows is None else rows
        width, shape, dtype = [(p["kb"], p["kshape"], p["kdtype"]), (p["vb"], p["vshape"], p["vdtype"]), (8, (), torch.long),
                               (p["vb"], p["vshape"], p["vdtype"]), (1, (), torch.bool)][which]
        lo = generation * p["gen_bytes"] + p["offs"][which] + row0 * width
        flat = p["views"][rank][lo:lo + rows * width]
        cache[asked] = view = flat.view(dtype).view((rows,) + tuple(shape))
        return view

    # Blocks per SM of the partition passes while the table kernels of another operation are running: with one block
    # per tile the (high-priority) send stage takes three quarters of every SM's threads for as long as it runs and
    # the table work stands still, so nothing overlaps; a few blocks per SM walking the tiles keep NVLink busy and
    # leave the rest of the SM to the probing (2 ranks, 2^25 rows each: 6.6 ms per step uncapped, 5.3 with 2 to 4
    # blocks per SM, 8.0 with 1.5 -- a grid that is not a whole number of waves is worse than none).
    OVERLAPPED_ROUTING_BLOCKS_PER_SM = 3

    def sliced_send(self, keys, values, generation, want_dest, force_overflow=False, overlapped=False):
        """SEND stage: owner of every row, then every row into its owner's inbox slice for this rank and this rank's
        row counts into the owners' count words -- plain stores, over NVLink for other ranks' memory.  A slice that
        would overflow raises the sticky status word instead, and nothing is stored.  -> dest_index (or None).
        overlapped: table kernels of an earlier operation are in flight; the partition passes then run on a small
        grid (see OVERLAPPED_ROUTING_BLOCKS_PER_SM)."""
        lib = L.lib()
        if overlapped:
            sms = torch.cuda.get_device_properties(self.device).multi_processor_count
            L.check(lib.dok_set_routing_blocks(int(self.OVERLAPPED_ROUTING_BLOCKS_PER_SM * sms)), "dok_set_routing_blocks")
        try:
            return self._sliced_send(keys, values, generation, want_dest, force_overflow)
        finally:
            if overlapped:
                L.check(lib.dok_set_routing_blocks(0), "dok_set_routing_blocks")

    def _sliced_send(self, keys, values, generation, want_dest, force_overflow):
        lib = L.lib()
        p = self._sx
        w, rows, r = p["world"], p["slice_rows"], p["rank"]
        n = keys.shape[0]
        owners, offsets, counts = self.partition_count(keys, w)
        arr_p = ctypes.c_void_p * w
        slice_keys = arr_p(*[self._region_ptr(o, generation, 0, r * rows) for o in range(w)])
        slice_values = arr_p(*[self._region_ptr(o, generation, 1, r * rows) for o in range(w)])
        count_dst = arr_p(*[self._region_ptr(o, generation, 2, r) for o in range(w)])
        dest = torch.empty(n, device=self.device, dtype=torch.long) if want_dest else None
        with torch.cuda.device(self.device):
            st = L.stream_ptr(self.device)
            L.check(lib.dok_shard_partition_check_slices(L.ptr(counts), w, rows, int(bool(force_overflow)),
                                                         L.ptr(p["status"]), st), "dok_shard_partition_check_slices")
            L.check(lib.dok_shard_partition_scatter_sliced(
                L.ptr(keys), p["kb"], L.ptr(values), 0 if values is None else p["vb"], n, w, L.ptr(owners), L.ptr(offsets),
                L.ptr(counts), slice_keys, slice_values if values is not None else None, count_dst, rows,
                L.ptr(p["status"]), L.ptr(dest), st), "dok_shard_partition_scatter_sliced")
        return dest

    def sliced_fence(self, token, signature=0):
        """Closes a SEND stage.  token (device int64[3]) becomes the maximum over all ranks of {sticky status,
        signature, -signature}: a non-zero token[0] tells every rank, on the device, that this operation (or an earlier
        one) overflowed somewhere, or that the ranks did not submit the same operation (token[1] != -token[2]), and
        must not be applied.  Being a collective ordered on the stream, it also orders every rank's stores before any
        rank's reads.  The host does not wait."""
        p = self._sx
        lib = L.lib()
        with torch.cuda.device(self.device):
            L.check(lib.dok_shard_token_prepare(L.ptr(p["status"]), int(signature), L.ptr(token), L.stream_ptr(self.device)),
                    "dok_shard_token_prepare")
            if p["world"] > 1 and p["group"] is not False:
                dist.all_reduce(token, op=dist.ReduceOp.MAX, group=p["group"])
            L.check(lib.dok_shard_token_finish(L.ptr(token), L.ptr(p["status"]), L.stream_ptr(self.device)),
                    "dok_shard_token_finish")

    def sliced_apply_fence(self):
        """Closes the answer deliveries of an APPLY stage (second communicator when there is one)."""
        p = self._sx
        if p["world"] > 1 and p["group"] is not False:
            dist.all_reduce(p["token_apply"], group=p["group_apply"] if p["group_apply"] is not None else p["group"])

    def sliced_reset_status(self):
        self._sx["status"].zero_()

    def can_pipeline(self):
        return getattr(self, "_sx", None) is not None

    def generations(self):
        return self._sx["generations"]

    def sliced_apply_set(self, generation, abort, assume_unique):
        p = self._sx
        self.local.set_sliced(self._region(p["rank"], generation, 0), self._region(p["rank"], generation, 1), p["world"],
                              p["slice_rows"], self._region(p["rank"], generation, 2), abort, assume_unique)

    def sliced_apply_lookup(self, generation, abort, with_values, fallback_value):
        """get (with_values) or remove of what this rank received, source by source, answers into the askers' result
        regions: this rank's own rows directly, another rank's rows into a local buffer that copy kernels on a side
        stream carry over NVLink while the next launch probes (row-sized stores from the probing kernel itself use
        the link far worse).  Lookups commute, so the other ranks' rows go first, in at most two launches over several
        slices each; removals are one launch over all slices (equal keys report once; which of them is unspecified,
        across ranks as within a batch)."""
        lib = L.lib()
        p = self._sx
        w, rows, r = p["world"], p["slice_rows"], p["rank"]
        plan = p.setdefault("lookup_plans", {}).get((generation, with_values))
        if plan is None:                                  # views and addresses of a generation never change: build once
            counts = self._region(r, generation, 2)

            def piece(first, n_slices):
                """slices [first, first + n_slices) of the inbox as one launch; answers go to the local buffer, or --
                for this rank's own slice -- straight into its result region"""
                keys = self._region(r, generation, 0, rows=n_slices * rows, row0=first * rows)
                if first == r and n_slices == 1:
                    out_values = self._region(r, generation, 3, rows=rows, row0=r * rows) if with_values else None
                    out_flags = self._region(r, generation, 4, rows=rows, row0=r * rows)
                else:
                    out_values = p["answer_values"][first * rows:(first + n_slices) * rows] if with_values else None
                    out_flags = p["answer_flags"][first * rows:(first + n_slices) * rows]
                copies = []
                for s in range(first, first + n_slices):
                    if s != r:
                        lo = (s - first) * rows
                        copies.append((ctypes.c_void_p(self._region_ptr(s, generation, 3, r * rows)) if with_values else None,
                                       out_values[lo:lo + rows] if with_values else None,
                                       ctypes.c_void_p(self._region_ptr(s, generation, 4, r * rows)), out_flags[lo:lo + rows],
                                       counts[s:s + 1]))
                return (keys, n_slices, counts[first:first + n_slices], out_values, out_flags, copies)

            if with_values:
                # lookups commute: everything the other ranks sent in two or three launches over several slices each
                # (runs of slices below and above this rank's own), then this rank's own rows: the answers of one
                # launch travel while the next one probes
                plan, most = [], max(1, (w - 1 + 1) // 2)
                for first, n_slices in ((0, r), (r + 1, w - r - 1)):
                    while n_slices > 0:                       # no launch over more than half of the other ranks' slices:
                        take = min(n_slices, most)            # its answers travel while the next launch probes
                        plan.append(piece(first, take))
                        first, n_slices = first + take, n_slices - take
                plan.append(piece(r, 1))
            else:
                # removals: ONE launch over everything received.  Equal keys report once, wherever they came from;
                # which of them reports is left to the race, as it is among the rows of one batch on one GPU.  The
                # flags of this rank's own rows take the same way back as the others' (a copy into its result region).
                keys = self._region(r, generation, 0)
                flags = p["answer_flags"]
                copies = [(None, None, ctypes.c_void_p(self._region_ptr(s, generation, 4, r * rows)),
                           flags[s * rows:(s + 1) * rows], counts[s:s + 1]) for s in range(w)]
                plan = [(keys, w, counts, None, flags, copies)]
            p["lookup_plans"][(generation, with_values)] = plan
        for keys, n_slices, count, out_values, out_flags, copies in plan:
            if with_values:
                self.local.get_sliced(keys, n_slices, rows, count, abort, fallback_value, out_values, out_flags)
            else:
                self.local.remove_sliced(keys, n_slices, rows, count, abort, out_flags)
            if not copies:
                continue
            if self._copy_stream is None:
                # high priority: the copy kernels' few blocks must not queue behind the big grid of the next launch,
                # which they are meant to overlap
                self._copy_stream = torch.cuda.Stream(device=self.device, priority=-1)
            answered = torch.cuda.Event()
            answered.record()
            with torch.cuda.stream(self._copy_stream):
                self._copy_stream.wait_event(answered)
                with torch.cuda.device(self.device):
                    for dst_values, src_values, dst_flags, src_flags, one_count in copies:
                        L.check(lib.dok_copy_counted(dst_values, L.ptr(src_values), p["vb"], dst_flags, L.ptr(src_flags), 1, rows,
                                                     L.ptr(one_count), L.ptr(abort), L.stream_ptr(self.device)), "dok_copy_counted")
            self._in_flight.append(True)
        self.answers_delivered()

    def sliced_results(self, generation, dest, with_values, abort=None):
        """Inverse permutation of this rank's result region into the caller's row order (nothing happens when the
        operation was skipped: dest was never written then)."""
        p = self._sx
        values = self._region(p["rank"], generation, 3) if with_values else None
        flags = self._region(p["rank"], generation, 4).view(torch.uint8)
        out_values, out_flags = self.unpermute(values, flags, dest, abort=abort)
        return out_values, out_flags.view(torch.bool)

    def ensure_allocated(self, key_row, value_row):
        """The local shard gets its storage at the first collective set, also on a rank that receives no row, so that
        lookups can run on every rank from then on."""
        if self.local._slots is None:
            self.local._allocate(key_row[0], key_row[1], value_row[0], value_row[1])

    def partition_count(self, keys, world):
        """First pass of the partition -> (owners, tile offsets, counts[2 * world] on the device)."""
        lib = L.lib()
        n = keys.shape[0]
        with torch.cuda.device(self.device):
            offsets = torch.empty(lib.dok_partition_offset_words(n, world), device=self.device, dtype=torch.long)
            counts = torch.empty(2 * world, device=self.device, dtype=torch.long)
            owners = torch.empty(max(n, 1), device=self.device, dtype=torch.uint8)
            L.check(lib.dok_shard_partition_count(self._routing_hash(keys), L.ptr(keys), n, world, L.ptr(owners),
                                                  L.ptr(offsets), L.ptr(counts), L.stream_ptr(self.device)),
                    "dok_shard_partition_count")
        return owners, offsets, counts

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
            cap = lib.dok_partition_capacity(n, world)
            offsets = torch.empty(lib.dok_partition_offset_words(n, world), device=self.device, dtype=torch.long)
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

    def unpermute(self, grouped_values, grouped_flags, dest, out_values=None, out_flags=None, abort=None):
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
                                            L.ptr(out_flags) if grouped_flags is not None else None, L.ptr(abort),
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

    def answers_delivered(self):
        """The current stream waits for the bulk copies of local_answer; their source buffers may then be reused."""
        if self._in_flight:
            done = torch.cuda.Event()
            done.record(self._copy_stream)
            torch.cuda.current_stream(self.device).wait_event(done)
            self._in_flight = []

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
    SEND_STREAM_PRIORITY = -1       # the send stage's stream: high priority (see run())

    KINDS = {"get": 1, "set": 2, "remove": 3}

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
        # Sliced exchange (ranks of ONE node, NVLink): with peer_capacity_rows > 0 (the same on every rank: the largest
        # batch a rank submits) the rows of a batch are stored straight into fixed slices of the owners' memory by the
        # partition kernel, and answers straight into the askers', with every count read on the device: no all-to-all
        # pass, and no host waits anywhere between submission and result.  A batch that does not fit its slices is
        # detected on the device, skipped by every rank, and repeated over the exact all-to-all exchange at wait().
        self._peer_capacity = int(peer_capacity_rows) if (self.world > 1 and self.world <= 16) else 0
        self._sliced_on = False
        self._seq = 0
        self._streams = None
        self._last_applied = None
        self._recent_applied = []     # apply-done events of the last GENERATIONS - 1 operations submitted
        self._pending = []            # submissions whose tokens have not been read yet: (operations, results, tokens)
        self._value_shape = None
        self._value_dtype = None
        self._key_shape = None
        self._key_dtype = None
        self.profile = None           # a list: run() appends (kind, [CUDA events at the stage boundaries]) per operation

    def phase_times(self):
        """Mean milliseconds per stage and operation kind of the operations recorded while `profile` was a list:
        partition+scatter and fence of the SEND stage; table work with answer delivery, fence and inverse permutation
        of the APPLY stage.  Synchronises."""
        torch.cuda.synchronize(self.ops.device)
        names = ("send_partition_scatter", "send_fence", "apply_table_and_answers", "apply_fence", "apply_unpermute")
        acc = {}
        for kind, ev in self.profile or []:
            row = acc.setdefault(kind, [0.0] * len(names) + [0])
            spans = [ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2]), ev[3].elapsed_time(ev[4]), ev[4].elapsed_time(ev[5]),
                     ev[5].elapsed_time(ev[6])]
            for i, ms in enumerate(spans):
                row[i] += ms
            row[-1] += 1
        return {kind: {name: row[i] / row[-1] for i, name in enumerate(names)} for kind, row in acc.items()}

    # ------------------------------------------------------------------ argument checks (before anything is launched)
    def _check_keys(self, keys):
        """Same assertions as the single map (cuda_closed_hashmap.py:397-399 of the reference): a batch whose key
        dtype or row shape differs from the first set would make the routing kernels read past its end."""
        assert isinstance(keys, torch.Tensor) and keys.dim() >= 1, "keys must be a tensor of rows"
        if self._key_shape is not None:
            assert keys.dtype == self._key_dtype, f"key dtype {keys.dtype}, the map holds {self._key_dtype}"
            assert tuple(keys.shape[1:]) == self._key_shape, f"key rows {tuple(keys.shape[1:])}, the map holds {self._key_shape}"

    def _check_values(self, keys, values):
        assert isinstance(values, torch.Tensor) and values.shape[0] == keys.shape[0], "one value row per key row"
        if self._value_shape is not None:
            assert values.dtype == self._value_dtype, f"value dtype {values.dtype}, the map holds {self._value_dtype}"
            assert tuple(values.shape[1:]) == self._value_shape, f"value rows {tuple(values.shape[1:])}, the map holds {self._value_shape}"

    def _check_operation(self, op):
        assert op[0] in self.KINDS, f"unknown operation {op[0]!r}"
        if op[0] != "set" and self._value_shape is None:
            raise RuntimeError("store something first")
        self._check_keys(op[1])
        if op[0] == "set":
            self._check_values(op[1], op[2])

    def _signature(self, kind):
        """What every rank must agree on for one collective operation, as one integer."""
        return self.KINDS[kind]

    # ------------------------------------------------------------------ exchange plumbing
    def _exchange_counts(self, counts, signature=0):
        """counts[2, world] (device; rows and padded rows per owner) -> (send_padded, recv_rows, recv_padded) as host
        lists; one synchronisation per batch.  The operation's signature travels with the counts, so that ranks which
        submitted different operations find out here, on every rank, instead of deadlocking in the row exchange."""
        w = self.world
        send = torch.cat([counts.t().contiguous(), counts.new_full((w, 1), int(signature))], dim=1)   # [world, 3]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        flat = self.ops.to_host(torch.stack([send, recv]))          # [2, world, 3] flattened
        send_h = [flat[3 * i:3 * i + 3] for i in range(w)]
        recv_h = [flat[3 * w + 3 * i:3 * w + 3 * i + 3] for i in range(w)]
        theirs = sorted({int(c[2]) for c in recv_h})
        if theirs != [int(signature)]:
            raise L.DokError(f"ranks submitted different operations to a collective call (signatures {theirs}, "
                             f"rank {self.rank} has {int(signature)})")
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

    def _route(self, keys, values=None, want_dest=True, async_op=False, signature=0):
        """-> (owned_keys, owned_values, segments, dest, send, recv[, works]); segments = [(start, rows)] per source
        rank.  With async_op the key / value exchanges are in flight on return and `works` must be waited for."""
        if self.world == 1:        # one shard owns everything: no partition, no exchange, no permutation
            out = (keys, values, [(0, keys.shape[0])], None, None, None)
            return out + ([],) if async_op else out
        grouped_keys, grouped_values, dest, counts = self.ops.partition(keys, values, self.world, want_dest=want_dest)
        send, recv_rows, recv = self._exchange_counts(counts, signature)
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

    # ------------------------------------------------------------------ sliced exchange: submission without host waits
    def run(self, operations, wait=True, _force_overflow=False):
        """Several operations as one submission: [("get", keys[, fallback_value]), ("set", keys, values[,
        assume_unique]), ("remove", keys)] -> list of results (get: (values, is_found); set: None; remove: flags).
        Collective: every rank passes the same sequence of operation kinds.  The operations are applied in order, as if
        called one after the other.

        Over the sliced exchange an operation has two stages.  SEND (it only reads the caller's batch): partition,
        stores of the rows into the owners' inbox slices over NVLink, a fence.  APPLY: the owner's table work on its
        inbox, answers into the askers' result regions, a fence, the inverse permutation.  The two stages run on two
        streams, so the SEND of operation k + 1 overlaps the APPLY of operation k, and since every row count is read on
        the device the host only enqueues: it never waits for a count, a fence or a kernel.

        Results are ready for the caller's current stream when the call returns -- unless `wait=False`: then the call
        only enqueues, the next submission's first send may overlap this one's last table work, and the caller calls
        `wait()` before it uses results or reuses / frees the input tensors (which must already be complete on the
        current stream at the time of the call).  Without the sliced exchange the operations simply run one after the
        other over the all-to-all exchange."""
        if not operations:
            return []
        for op in operations:
            self._check_operation(op)
        if not self._sliced_on or not self.ops.can_pipeline():
            return [self._run_one(op) for op in operations]
        ops = self.ops
        device = ops.device
        nvtx = torch.cuda.nvtx
        if self._streams is None:
            # the send stage runs at high priority: its kernels are short, and behind the big grids of the table work
            # they would otherwise only start when those have handed out all their blocks
            self._streams = (torch.cuda.Stream(device=device, priority=self.SEND_STREAM_PRIORITY), torch.cuda.Stream(device=device))
        s_send, s_apply = self._streams
        main = torch.cuda.current_stream(device)
        # copies that make the inputs contiguous run on the caller's stream, before the side streams branch off
        prepared = [(op[0], op[1].contiguous(), op[2].contiguous() if op[0] == "set" else None) for op in operations]
        for op, (_, keys, values) in zip(operations, prepared):
            for made, given in ((keys, op[1]), (values, op[2] if op[0] == "set" else None)):
                if made is not None and made is not given:
                    made.record_stream(s_send)            # a copy made here is read on the send stream after we return
        start = torch.cuda.Event()
        start.record(main)
        s_send.wait_event(start)
        s_apply.wait_event(start)
        results = [None] * len(operations)
        with torch.cuda.stream(s_send):
            tokens = torch.zeros((len(operations), 3), device=device, dtype=torch.long)
        n_gen = ops.generations()
        recent = self._recent_applied         # apply-done events of the last operations (also of earlier submissions)
        for i, op in enumerate(operations):
            kind, keys, values = prepared[i]
            generation = self._seq % n_gen
            self._seq += 1
            token = tokens[i]
            marks = [torch.cuda.Event(enable_timing=True) for _ in range(7)] if self.profile is not None else None
            mark = (lambda k, stream: marks[k].record(stream)) if marks else (lambda k, stream: None)
            nvtx.range_push(f"dok.sharded.{kind}.send")
            with torch.cuda.stream(s_send):
                mark(0, s_send)
                dest = ops.sliced_send(keys, values, generation, want_dest=(kind != "set"), force_overflow=_force_overflow,
                                       overlapped=(i > 0 or bool(self._pending)))
                if len(recent) >= n_gen - 1:
                    # the NEXT operation's send overwrites the generation that the apply of n_gen - 1 operations back
                    # reads: the fence below (all ranks) must come after that apply, on every rank
                    s_send.wait_event(recent[-(n_gen - 1)])
                mark(1, s_send)
                ops.sliced_fence(token, self._signature(kind))
                mark(2, s_send)
                sent = torch.cuda.Event()
                sent.record(s_send)
                if dest is not None:
                    # allocated on the send stream, read on the apply stream: the allocator may hand the block out again
                    # only after that read.  Nothing of an operation is held until wait() -- holding it would make every
                    # step of a long submission allocate fresh device memory (a device-wide synchronisation each time).
                    dest.record_stream(s_apply)
            nvtx.range_pop()
            nvtx.range_push(f"dok.sharded.{kind}.apply")
            with torch.cuda.stream(s_apply):
                s_apply.wait_event(sent)
                mark(3, s_apply)
                abort = token[0:1]
                if kind == "set":
                    ops.sliced_apply_set(generation, abort, op[3] if len(op) > 3 else False)
                    mark(4, s_apply)
                    ops.sliced_apply_fence()      # nothing to deliver, but every kind issues the same collectives
                    mark(5, s_apply)
                else:
                    with_values = kind == "get"
                    ops.sliced_apply_lookup(generation, abort, with_values, (op[2] if len(op) > 2 else None) if with_values else None)
                    mark(4, s_apply)
                    ops.sliced_apply_fence()
                    mark(5, s_apply)
                    out_values, out_flags = ops.sliced_results(generation, dest, with_values, abort)
                    results[i] = (out_values, out_flags) if with_values else out_flags
                    for t in (out_values, out_flags):
                        if t is not None:
                            t.record_stream(main)
                mark(6, s_apply)
                applied = torch.cuda.Event()
                applied.record(s_apply)
            recent.append(applied)
            del recent[:-(n_gen - 1)]
            if marks:
                self.profile.append((kind, marks))
            nvtx.range_pop()
        self._last_applied = applied
        self._pending.append((list(operations), results, tokens))
        if wait:
            self.wait()
        return results

    def wait(self):
        """The caller's current stream waits for everything submitted with run(..., wait=False), and the host reads
        the tokens of those submissions (one small copy): operations that some rank could not fit into its slices --
        all ranks skipped them, and everything submitted after them -- are repeated now, in order, over the exact
        all-to-all exchange, and their results are written into the tensors that run() handed out."""
        if self._streams is not None:
            main = torch.cuda.current_stream(self.ops.device)
            for s in self._streams:
                ev = torch.cuda.Event()
                ev.record(s)
                main.wait_event(ev)
        self._last_applied = None
        self._recent_applied = []
        pending, self._pending = self._pending, []
        if not pending:
            return
        flat = torch.cat([t for _, _, t in pending]).cpu().tolist()         # waits for the device
        redo, i = False, 0
        for operations, results, _ in pending:
            for k, op in enumerate(operations):
                flag, sig_max, neg_sig_min = flat[i]
                i += 1
                if sig_max != -neg_sig_min:
                    self.ops.sliced_reset_status()
                    raise L.DokError(f"ranks submitted different operations to a collective call (operation {k}: "
                                     f"signatures {-neg_sig_min} .. {sig_max}, rank {self.rank} has {self._signature(op[0])})")
                if flag and not redo:
                    redo = True
                    self.ops.sliced_reset_status()
                if redo:
                    again = self._run_one(op, sliced=False)
                    if op[0] == "get":
                        results[k][0].copy_(again[0])
                        results[k][1].copy_(again[1])
                    elif op[0] == "remove":
                        results[k].copy_(again)
        maintain = getattr(self.ops.local, "_maintain", None)
        if maintain is not None:
            maintain()              # the sliced removals only counted their tombstones; rebuild here if it is time

    def _settle(self):
        """Anything still in flight from a submission that was not waited for is completed (and, if it overflowed,
        repeated) before an operation that runs on the caller's stream."""
        if self._last_applied is not None or self._pending:
            self.wait()

    def _run_one(self, op, sliced=True):
        kind = op[0]
        saved, self._sliced_on = self._sliced_on, self._sliced_on and sliced
        try:
            if kind == "set":
                return self.set(op[1], op[2], assume_unique=op[3] if len(op) > 3 else False)
            if kind == "get":
                return self.get(op[1], op[2] if len(op) > 2 else None)
            return self.remove(op[1])
        finally:
            self._sliced_on = saved

    # ------------------------------------------------------------------ operations
    def _first_set(self, keys, values):
        self._key_shape, self._key_dtype = tuple(keys.shape[1:]), keys.dtype
        self._value_shape, self._value_dtype = tuple(values.shape[1:]), values.dtype
        if hasattr(self.ops, "ensure_allocated"):
            self.ops.ensure_allocated((self._key_shape, self._key_dtype), (self._value_shape, self._value_dtype))
        self._start_sliced()

    def _start_sliced(self):
        if self._peer_capacity and not self._sliced_on and getattr(self.ops, "supports_sliced", False):
            self._sliced_on = self.ops.sliced_setup(self.group, self.world, self.rank, self._peer_capacity,
                                                    (self._key_shape, self._key_dtype), (self._value_shape, self._value_dtype))

    def set(self, keys, values, assume_unique=False):
        """Collective insert-or-assign.  `assume_unique` promises pairwise different keys across ALL ranks' batches."""
        self._check_keys(keys)
        self._check_values(keys, values)
        self._settle()
        if self._value_shape is None:
            self._first_set(keys, values)
        if self._sliced_on:
            self.run([("set", keys, values, assume_unique)])
            return
        owned_keys, owned_values, segments, _, _, _ = self._route(keys, values, want_dest=False,
                                                                  signature=self._signature("set"))
        self.ops.local_set(owned_keys, owned_values, segments, assume_unique)

    def state_dict(self):
        """This rank's shard (see CudaClosedHashmap.state_dict) plus the sharding it belongs to.  Every rank saves its
        own; a map rebuilt with the same world size and parameters routes every key to the shard that holds it."""
        self._settle()
        return {"world": self.world, "rank": self.rank, "shard": self.ops.local.state_dict(),
                "value_shape": self._value_shape, "value_dtype": self._value_dtype,
                "key_shape": self._key_shape, "key_dtype": self._key_dtype}

    def load_state_dict(self, state):
        """Replaces this rank's shard by a saved one (same world size and rank).  Collective when the sliced exchange
        is configured: it is brought up here if the map has not stored anything yet."""
        assert state["world"] == self.world and state["rank"] == self.rank, "a shard belongs to its rank"
        self._settle()
        self.ops.local = CudaClosedHashmap.from_state_dict(state["shard"], device=self.ops.device)
        self._value_shape, self._value_dtype = state["value_shape"], state["value_dtype"]
        self._key_shape, self._key_dtype = state.get("key_shape"), state.get("key_dtype")
        if self._key_shape is None and self.ops.local._slots is not None:
            self._key_shape, self._key_dtype = tuple(self.ops.local.key_shape), self.ops.local.key_type
        if self._value_shape is not None and self._key_shape is not None:
            if hasattr(self.ops, "ensure_allocated"):
                self.ops.ensure_allocated((self._key_shape, self._key_dtype), (self._value_shape, self._value_dtype))
            self._start_sliced()

    def close(self):
        """Releases the exchange arena (every rank, after the last operation)."""
        self._settle()
        if self._sliced_on:
            self._sliced_on = False
            self.ops.sliced_close()

    def _lookup(self, keys, local_op, with_values, fallback_value=None):
        """Shared body of get and remove over the all-to-all exchange.  For get the batch is cut into
        `pipeline_chunks` pieces that move through partition -> key exchange -> local op -> result exchange -> inverse
        permutation as a software pipeline: the exchanges are enqueued asynchronously, so the key exchange of piece
        i + 1 and the result exchange of piece i - 1 run while the table is probed for piece i.  remove goes through in
        one piece: cutting it would let a later rank's first piece overtake an earlier rank's second, and which of two
        equal keys reports the removal is defined by rank order."""
        n = keys.shape[0]
        out_values = self.ops.empty((n,) + self._value_shape, self._value_dtype) if with_values else None
        out_flags = self.ops.empty((n,), torch.bool)
        bounds = self._chunk_bounds(n, pipelined=with_values)
        signature = self._signature("get" if with_values else "remove")
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
            routed.append(self._route(keys[lo:hi], async_op=True, signature=signature))
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
        self._check_keys(keys)
        self._settle()
        if self.world == 1:
            if not self.ops.ready():
                return self._lookup(keys, None, True, fallback_value)
            return self.ops.local_get(keys, [(0, keys.shape[0])], fallback_value)
        if self._sliced_on:
            return self.run([("get", keys, fallback_value)])[0]
        return self._lookup(keys, lambda k, seg: self.ops.local_get(k, seg, fallback_value), True, fallback_value)

    def remove(self, keys):
        """Collective removal -> is_removed[n] aligned to the caller's rows.  Equal keys -- in one rank's batch or in
        several ranks' batches -- report once; which of them reports is unspecified (over the all-to-all exchange it is
        the first in rank order)."""
        if self._value_shape is None:
            raise RuntimeError("store something first")
        self._check_keys(keys)
        self._settle()
        if self.world == 1 and self.ops.ready():
            return self.ops.local_remove(keys, [(0, keys.shape[0])])
        if self._sliced_on:
            return self.run([("remove", keys)])[0]
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
