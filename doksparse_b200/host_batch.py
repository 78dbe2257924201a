"""Batched map operations on HOST buffers, pipelined over PCIe.

A caller whose keys arrive in (pinned) host memory and whose results must land there again pays, per batch, a
host->device copy, the kernels, and a device->host copy.  Done one after the other these add up; done in chunks on
three streams (copy in | kernels | copy out) the copies of one chunk hide behind the kernels and the opposite-direction
copy of its neighbours, and the batch runs at the speed of the slower PCIe direction.  The reference has no such path:
its callers hand it CUDA tensors (`sparse_dok/components/cuda_closed_hashmap.py:321-454`).

Works on a `CudaClosedHashmap` and on a `ShardedClosedHashmap` (whose calls are collective: every rank must then use
the same chunking, i.e. equal batch sizes).  Chunks are applied in order, so a chunked `set` resolves duplicates like
one big `set` (last row wins).  Staging buffers are allocated once per row shape and reused (two per direction), so
the steady state makes no allocator calls.

The copy-in of a chunk is enqueued one chunk AHEAD of its kernels: map operations may block the host (the sharded map
reads row counts back before each exchange), and a copy that is already queued keeps PCIe busy meanwhile.  `run()`
takes several operations at once so that this look-ahead also bridges the boundary between them.  Calls only enqueue
work; `join()` makes the caller's current stream wait for it.
"""
import torch


class _Ring:
    """Two device staging buffers of one row shape with the event after which each may be overwritten."""

    def __init__(self, rows, row_shape, dtype, device):
        self.buffers = [torch.empty((rows,) + tuple(row_shape), device=device, dtype=dtype) for _ in range(2)]
        self.free_after = [None, None]
        self.turn = 0

    def take(self, stream):
        i = self.turn
        self.turn ^= 1
        if self.free_after[i] is not None:
            stream.wait_event(self.free_after[i])
        return i, self.buffers[i]


class HostBatch:
    def __init__(self, table, device, chunk_rows=1 << 22):
        self.table = table
        self.device = torch.device(device)
        self.chunk_rows = int(chunk_rows)
        with torch.cuda.device(self.device):
            self.s_in, self.s_run, self.s_out = (torch.cuda.Stream() for _ in range(3))
        self._rings = {}
        self._takes_outputs = hasattr(table, "_slots")      # a plain map writes straight into the staging buffers
        self.begin()

    # ------------------------------------------------------------------ stream plumbing
    def begin(self):
        """Side streams start after whatever the caller's current stream has enqueued so far."""
        with torch.cuda.device(self.device):
            ev = torch.cuda.Event()
            ev.record()
            for s in (self.s_in, self.s_run, self.s_out):
                s.wait_event(ev)

    def join(self):
        """The caller's current stream waits for everything enqueued through this object."""
        with torch.cuda.device(self.device):
            cur = torch.cuda.current_stream()
            for s in (self.s_in, self.s_run, self.s_out):
                ev = torch.cuda.Event()
                ev.record(s)
                cur.wait_event(ev)

    def _ring(self, tag, row_shape, dtype):
        key = (tag, tuple(row_shape), dtype)
        if key not in self._rings:
            self._rings[key] = _Ring(self.chunk_rows, row_shape, dtype, self.device)
        return self._rings[key]

    def _stage_in(self, tag, host_slice):
        """host (pinned) rows -> a reused device buffer, on the copy-in stream -> (ring, index, device view)"""
        ring = self._ring(tag, host_slice.shape[1:], host_slice.dtype)
        i, buf = ring.take(self.s_in)
        view = buf[: host_slice.shape[0]]
        with torch.cuda.stream(self.s_in):
            view.copy_(host_slice, non_blocking=True)
        return ring, i, view

    def _copy_out(self, done, pairs, rings):
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(done)
            for host_slice, dev in pairs:
                host_slice.copy_(dev, non_blocking=True)
            copied = torch.cuda.Event()
            copied.record(self.s_out)
        for ring, i in rings:
            ring.free_after[i] = copied

    # ------------------------------------------------------------------ chunk programs
    # A chunk is (inputs, body): inputs = [(tag, pinned host slice)], body(device views) runs on the kernel stream and
    # returns (pairs, rings) for the copy-out: [(host slice, device tensor)], [(ring, index)] of result buffers.
    def _chunks(self, n):
        for lo in range(0, n, self.chunk_rows):
            yield lo, min(n, lo + self.chunk_rows)

    def _get_chunks(self, keys_host, out_values_host, out_found_host, fallback_value=None):
        vr = self._ring("ov", out_values_host.shape[1:], out_values_host.dtype)
        fr = self._ring("of", (), torch.bool)
        for lo, hi in self._chunks(keys_host.shape[0]):
            def body(keys, lo=lo, hi=hi):
                vi, vbuf = vr.take(self.s_run)
                fi, fbuf = fr.take(self.s_run)
                values, found = vbuf[: hi - lo], fbuf[: hi - lo]
                if self._takes_outputs:
                    self.table.get(keys, fallback_value, values=values, is_found=found)
                else:                       # results come back in tensors of the kernel stream's pool: move them over
                    v, f = self.table.get(keys, fallback_value)
                    values.copy_(v)
                    found.copy_(f)
                return [(out_values_host[lo:hi], values), (out_found_host[lo:hi], found)], [(vr, vi), (fr, fi)]
            yield [("k", keys_host[lo:hi])], body

    def _set_chunks(self, keys_host, values_host, assume_unique=False):
        for lo, hi in self._chunks(keys_host.shape[0]):
            def body(keys, values):
                self.table.set(keys, values, assume_unique=assume_unique)
                return [], []
            yield [("k", keys_host[lo:hi]), ("v", values_host[lo:hi])], body

    def _remove_chunks(self, keys_host, out_flags_host=None):
        remove = getattr(self.table, "remove_rows", None) or self.table.remove
        fr = self._ring("rf", (), torch.bool)
        for lo, hi in self._chunks(keys_host.shape[0]):
            def body(keys, lo=lo, hi=hi):
                flags = remove(keys)
                if out_flags_host is None:
                    return [], []
                fi, fbuf = fr.take(self.s_run)
                fbuf[: hi - lo].copy_(flags)
                return [(out_flags_host[lo:hi], fbuf[: hi - lo])], [(fr, fi)]
            yield [("k", keys_host[lo:hi])], body

    def _execute(self, chunks):
        """Copy-in of chunk i + 1 is enqueued before the kernels of chunk i."""
        chunks = iter(chunks)

        def stage(chunk):
            if chunk is None:
                return None
            inputs, body = chunk
            staged = [self._stage_in(tag, host_slice) for tag, host_slice in inputs]
            ready = torch.cuda.Event()
            ready.record(self.s_in)
            return staged, ready, body

        ahead = stage(next(chunks, None))
        while ahead is not None:
            staged, ready, body = ahead
            # a staging buffer is reused every second chunk of its kind, so the copy-in of the NEXT chunk never waits
            # for kernels that are not enqueued yet
            ahead = stage(next(chunks, None))
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(ready)
                pairs, out_rings = body(*[view for _, _, view in staged])
                done = torch.cuda.Event()
                done.record(self.s_run)
            for ring, i, _ in staged:
                ring.free_after[i] = done
            if pairs:
                self._copy_out(done, pairs, out_rings)

    # ------------------------------------------------------------------ public operations
    def get(self, keys_host, out_values_host, out_found_host, fallback_value=None):
        self._execute(self._get_chunks(keys_host, out_values_host, out_found_host, fallback_value))

    def set(self, keys_host, values_host, assume_unique=False):
        self._execute(self._set_chunks(keys_host, values_host, assume_unique))

    def remove_rows(self, keys_host, out_flags_host=None):
        """Kernel-level removal: flags aligned to the rows given (no dedup, no sort)."""
        self._execute(self._remove_chunks(keys_host, out_flags_host))

    def run(self, operations):
        """Several operations as one pipeline: [("get", keys, out_values, out_found[, fallback]),
        ("set", keys, values[, assume_unique]), ("remove_rows", keys[, out_flags]), ...], applied in order."""
        makers = {"get": self._get_chunks, "set": self._set_chunks, "remove_rows": self._remove_chunks}

        def all_chunks():
            for name, *args in operations:
                yield from makers[name](*args)
        self._execute(all_chunks())
