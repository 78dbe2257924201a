"""Batched map operations on HOST buffers, pipelined over PCIe.

A caller whose keys arrive in (pinned) host memory and whose results must land there again pays, per batch, a
host->device copy, the kernels, and a device->host copy.  Done one after the other these add up; done in chunks on
three streams (copy in | kernels | copy out) the copies of one chunk hide behind the kernels and the opposite-direction
copy of its neighbours, and the batch runs at the speed of the slower PCIe direction.  The reference has no such path:
its callers hand it CUDA tensors (`sparse_dok/components/cuda_closed_hashmap.py:321-454`).

Works on a `CudaClosedHashmap` and on a `ShardedClosedHashmap` (whose calls are collective: every rank must then use
the same chunking, i.e. equal batch sizes).  Chunks are applied in order, so a chunked `set` resolves duplicates like
one big `set` (last row wins).  Staging buffers are allocated once per row shape and reused (two per direction), so
the steady state makes no allocator calls.  Calls only enqueue work; `join()` makes the caller's current stream wait.
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
        self.begin()

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

    def _chunks(self, n):
        for lo in range(0, n, self.chunk_rows):
            yield lo, min(n, lo + self.chunk_rows)

    def _ring(self, tag, like_rows, dtype):
        key = (tag, tuple(like_rows), dtype)
        if key not in self._rings:
            self._rings[key] = _Ring(self.chunk_rows, like_rows, dtype, self.device)
        return self._rings[key]

    def _stage_in(self, tag, host_slice):
        """host (pinned) rows -> a reused device buffer, on the copy-in stream -> (ring, index, device view)"""
        ring = self._ring(tag, host_slice.shape[1:], host_slice.dtype)
        i, buf = ring.take(self.s_in)
        view = buf[: host_slice.shape[0]]
        with torch.cuda.stream(self.s_in):
            view.copy_(host_slice, non_blocking=True)
        return ring, i, view

    def _run(self, staged, fn):
        """fn() on the kernel stream once the staged inputs have arrived; marks them reusable afterwards"""
        ready = torch.cuda.Event()
        ready.record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(ready)
            result = fn()
            done = torch.cuda.Event()
            done.record(self.s_run)
        for ring, i, _ in staged:
            ring.free_after[i] = done
        return result, done

    def _copy_out(self, done, pairs, rings):
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(done)
            for host_slice, dev in pairs:
                host_slice.copy_(dev, non_blocking=True)
            copied = torch.cuda.Event()
            copied.record(self.s_out)
        for ring, i in rings:
            ring.free_after[i] = copied

    def get(self, keys_host, out_values_host, out_found_host, fallback_value=None):
        takes_outputs = hasattr(self.table, "_slots")       # a plain map writes straight into the staging buffers
        vr = self._ring("ov", out_values_host.shape[1:], out_values_host.dtype)
        fr = self._ring("of", (), torch.bool)
        for lo, hi in self._chunks(keys_host.shape[0]):
            staged = self._stage_in("k", keys_host[lo:hi])
            keys = staged[2]
            vi, vbuf = vr.take(self.s_run)
            fi, fbuf = fr.take(self.s_run)
            values, found = vbuf[: hi - lo], fbuf[: hi - lo]

            def lookup():
                if takes_outputs:
                    self.table.get(keys, fallback_value, values=values, is_found=found)
                else:                       # results come back in tensors of the kernel stream's pool: move them over
                    v, f = self.table.get(keys, fallback_value)
                    values.copy_(v)
                    found.copy_(f)

            _, done = self._run([staged], lookup)
            self._copy_out(done, [(out_values_host[lo:hi], values), (out_found_host[lo:hi], found)], [(vr, vi), (fr, fi)])

    def set(self, keys_host, values_host, assume_unique=False):
        for lo, hi in self._chunks(keys_host.shape[0]):
            sk = self._stage_in("k", keys_host[lo:hi])
            sv = self._stage_in("v", values_host[lo:hi])
            self._run([sk, sv], lambda: self.table.set(sk[2], sv[2], assume_unique=assume_unique))

    def remove_rows(self, keys_host, out_flags_host=None):
        """Kernel-level removal: flags aligned to the rows given (no dedup, no sort)."""
        remove = getattr(self.table, "remove_rows", None) or self.table.remove
        fr = self._ring("rf", (), torch.bool)
        for lo, hi in self._chunks(keys_host.shape[0]):
            staged = self._stage_in("k", keys_host[lo:hi])
            if out_flags_host is None:
                self._run([staged], lambda: remove(staged[2]))
                continue
            fi, fbuf = fr.take(self.s_run)
            _, done = self._run([staged], lambda: fbuf[: hi - lo].copy_(remove(staged[2])))
            self._copy_out(done, [(out_flags_host[lo:hi], fbuf[: hi - lo])], [(fr, fi)])
