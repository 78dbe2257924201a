#!/usr/bin/env python
"""Benchmark of the hash-map hot path: batched get + set (+ remove of the rows the set inserted) on a
hash-sharded CudaClosedHashmap.

Workload (BASELINE.json configs[4], per-GPU shard, weak scaling): every GPU holds 2^28 int64 keys drawn
uniformly from [0, 2^62) mapped to float32[2] values in a shard of 447,392,427 buckets (load 0.6); a step is,
per GPU, a get of 32 Mi queries (80 % stored keys of ANY shard, 20 % absent), a set of 32 Mi rows (80 %
stored keys -> overwrite, 20 % new keys) and the removal of the rows that set inserted, which keeps the load
stationary.  With N GPUs the table has N * 2^28 keys and each rank routes its batch to the owning shards
(stable partition + NCCL all-to-all) and gets the results back; N = 8 is exactly the 2^31-key configuration.

  python bench.py [--gpus N] [--steps K] [--warmup W]            candidate (CUDA), one process per GPU
  python bench.py --impl reference ...                            the reference's own kernels on the host cores

One JSON line on stdout (rank 0).  Inputs are seeded and synthetic; nothing is read from disk except
MEASURED_PEAKS.json (the roofline denominator).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M62 = (1 << 62) - 1
KEY_BYTES, VALUE_BYTES = 8, 8
HIT_FRACTION = 0.8
LOAD_FACTOR = 0.6
N_BATCHES = 4          # distinct query/update batches rotated over the steps (each is larger than L2)
# DRAM bytes per operation of the kernels, dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture divided by
# the rows of the launch (profiles/k_*_c5_shard_2e26keys.md; the capture ran at 2^26 keys and 2^24 rows, traffic per row
# does not depend on the size once the table is much larger than L2)
TRAFFIC_BYTES_PER_OP = {"get": 171.5, "set": 210.4, "remove": 230.3}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["candidate", "reference"], default="candidate")
    ap.add_argument("--keys-log2", type=int, default=28, help="stored keys per GPU (default 2^28)")
    ap.add_argument("--batch-log2", type=int, default=25, help="queries per GPU and step (default 2^25 = 32 Mi)")
    ap.add_argument("--no-ref-gpu", action="store_true",
                    help="reference arm: skip the extra leg that runs the reference's kernels on the GPU")
    ap.add_argument("--no-peer", action="store_true",
                    help="multi-GPU: exchange rows with NCCL all-to-all instead of stores into the peers' memory")
    ap.add_argument("--no-pipeline", action="store_true",
                    help="multi-GPU: call get / set / remove one after the other instead of one pipelined submission")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer (end-to-end) measurement")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


# ---------------------------------------------------------------------------------------------------------------
# byte model and peaks
# ---------------------------------------------------------------------------------------------------------------

def algorithmic_bytes(op, kb=KEY_BYTES, vb=VALUE_BYTES, hit=HIT_FRACTION):
    """Bytes one operation must move with the ideal layout (tag and value in one 32-byte sector)."""
    sectors = -(-(8 + vb) // 32)
    if op == "get":       # key in, value + flag out, one sector read per probe chain (hit: the bucket row, miss: one tag)
        return kb + vb + 1 + 32 * (hit * sectors + (1 - hit))
    if op == "set":       # key + value in, the bucket sector(s) and the key-row sector read and written back
        return kb + vb + 2 * 32 * -(-(8 + vb + kb) // 32)
    if op == "remove":    # key in, flag out, the tag sector read and written back
        return kb + 1 + 2 * 32
    raise ValueError(op)


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


# ---------------------------------------------------------------------------------------------------------------
# synthetic keys: a bijection of [0, 2^62) makes every key index a distinct, uniformly spread key
# ---------------------------------------------------------------------------------------------------------------

def mix62_torch(x):
    x = (x * 0x2545F4914F6CDD1D) & M62
    x = x ^ (x >> 29)
    x = (x * 0x1B03738712FAD5C9) & M62
    x = x ^ (x >> 32)
    return x


def mix62_numpy(x):
    x = x.astype(np.uint64)
    m = np.uint64(M62)
    x = (x * np.uint64(0x2545F4914F6CDD1D)) & m
    x = x ^ (x >> np.uint64(29))
    x = (x * np.uint64(0x1B03738712FAD5C9)) & m
    x = x ^ (x >> np.uint64(32))
    return x.astype(np.int64)


def value_of_index(idx, xp):
    """float32[2] value stored for key index idx (lets the bench verify what a get returns)"""
    a = (idx & 0xFFFF)
    b = ((idx >> 16) & 0xFF)
    if xp is np:
        return np.stack([a, b], axis=1).astype(np.float32)
    return xp.stack([a, b], dim=1).float()


def fixed_parameters():
    """Explicit hash parameters, identical on every rank: one draw of the reference's generator (numpy seed 2024)
    for a table of 2^28 / 0.6 buckets."""
    return dict(prime1=[825411893], prime2=[131956765728754273], alpha1=[808106522], alpha2=[408516131],
                beta1=[188156349], beta2=[614383798])


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.thread = [], None, None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "25"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
                for name, cell in zip(names, r[4:8]):
                    if cell.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                pass
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------------------
# CPU arm: the reference's own kernels compiled for the host (oracle/_ref), else the C restatement
# ---------------------------------------------------------------------------------------------------------------

def cpu_arm(steps, warmup, sample_keys_log2=24, sample_batch_log2=22, budget_s=None):
    """One step = get(q) + set(q) + remove(inserted) on a table of 2^sample_keys_log2 keys at load 0.6, all host
    threads.  Returns (Mops/s over get+set rows, description dict)."""
    from oracle import port, ref
    cores = len(os.sched_getaffinity(0))
    n_keys, q = 1 << sample_keys_log2, 1 << sample_batch_log2
    nb = int(n_keys / LOAD_FACTOR)
    params = {k: np.asarray(v, dtype=np.int64) for k, v in fixed_parameters().items()}
    params["key_perm"] = np.zeros(1, dtype=np.int64)
    use_ref = os.path.exists(ref.map_lib_path("i64x1_f32x2"))
    if use_ref:
        table = ref.RefMap(nb, np.int64, 1, np.float32, 2, params, n_threads=cores)
        do_set, do_get, do_remove = table.set, table.get, table.remove
        kind = "reference"
    else:
        table = port.OracleHashmap(n_buckets=nb, n_threads=cores, **{k: v for k, v in params.items() if k != "key_perm"})
        table._keys, table._values = np.zeros((nb, 1), np.int64), np.zeros((nb, 2), np.float32)
        do_set, do_get, do_remove = table.set_rows, table._kernel_get, table.remove_rows
        kind = "port"
    idx = np.arange(n_keys, dtype=np.int64)
    for lo in range(0, n_keys, 1 << 22):
        part = idx[lo:lo + (1 << 22)]
        do_set(mix62_numpy(part)[:, None], value_of_index(part, np))
    n_hit = int(q * HIT_FRACTION)
    batches = []
    for b in range(2):
        rng = np.random.default_rng(b)
        hit_idx = (np.arange(n_hit, dtype=np.int64) * 7919 + 104729 * (b + 1)) % n_keys
        miss_idx = (1 << 40) + (b << 32) + np.arange(q - n_hit, dtype=np.int64)
        new_idx = (1 << 41) + (b << 32) + np.arange(q - n_hit, dtype=np.int64)
        perm = rng.permutation(q)
        gq = mix62_numpy(np.concatenate([hit_idx, miss_idx]))[perm][:, None]
        sk_idx = np.concatenate([hit_idx, new_idx])[perm]
        batches.append((gq, mix62_numpy(sk_idx)[:, None], value_of_index(sk_idx, np), mix62_numpy(new_idx)[:, None]))

    def step(b):
        gq, sk, sv, fresh = batches[b % 2]
        do_get(gq)
        do_set(sk, sv)
        do_remove(fresh)

    for s in range(warmup):
        step(s)
    t0 = time.perf_counter()
    done = 0
    for s in range(steps):
        step(s)
        done += 1
        if budget_s is not None and time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    mops = done * 2 * q / dt / 1e6
    desc = {"value": mops, "unit": "Mops/s", "cores": cores, "kind": kind,
            "sample": f"table of 2^{sample_keys_log2} keys at load {LOAD_FACTOR}, {done} steps of get 2^{sample_batch_log2} + "
                      f"set 2^{sample_batch_log2} + remove of the inserted 20 %, kernels only (no Python-side pre-get / unique)"}
    return mops, dt / max(done, 1) * 1e3, desc


def reference_kernels_on_gpu(args, steps=5, warmup=3):
    """The reference's own get / set / remove kernels (its kernel text compiled ahead of time by nvcc, since CuPy is
    not available) on cuda:0, on this bench's per-GPU workload: same table size and load, same batch construction,
    same operation order.  Kernels only -- the reference's Python bookkeeping around them (a pre-get, a row-sort
    unique and host synchronisations per set; a unique per remove) is left out, which favours the reference.
    Returns a dict for the JSON line, or a reason string when it cannot run here."""
    try:
        import torch
        from oracle import ref_gpu
    except Exception as exc:                                    # pragma: no cover
        return f"import failed: {exc}"
    if not torch.cuda.is_available():
        return "no GPU"
    if not ref_gpu.available(torch.int64, 1, torch.float32, 2):
        return "oracle/_ref/refgpu_map_i64x1_f32x2.so not built"
    device = torch.device("cuda", 0)
    n_keys, q = 1 << args.keys_log2, 1 << args.batch_log2
    nb = int(n_keys / LOAD_FACTOR)
    if nb * 2 > ref_gpu.RefGpuMap.MAX_ELEMENTS:
        return "table beyond the reference's 32-bit bucket indices"
    table = ref_gpu.RefGpuMap(nb, torch.int64, 1, torch.float32, 2, dict(fixed_parameters(), key_perm=[0]), device)
    chunk = min(n_keys, 1 << 25)
    for lo in range(0, n_keys, chunk):
        idx = torch.arange(lo, lo + chunk, device=device, dtype=torch.long)
        table.set(mix62_torch(idx)[:, None].contiguous(), value_of_index(idx, torch).contiguous())
    n_hit = int(q * HIT_FRACTION)
    g = torch.Generator(device=device).manual_seed(1234)
    batches = []
    for b in range(N_BATCHES):
        j = torch.arange(n_hit, device=device, dtype=torch.long)
        hit_idx = (j * 7919 + 104729 * (b + 1)) % n_keys
        miss_idx = (1 << 40) + (b << 32) + torch.arange(q - n_hit, device=device, dtype=torch.long)
        new_idx = (1 << 41) + (b << 32) + torch.arange(q - n_hit, device=device, dtype=torch.long)
        perm = torch.randperm(q, device=device, generator=g)
        get_idx, set_idx = torch.cat([hit_idx, miss_idx])[perm], torch.cat([hit_idx, new_idx])[perm]
        batches.append((mix62_torch(get_idx)[:, None].contiguous(), get_idx, mix62_torch(set_idx)[:, None].contiguous(),
                        value_of_index(set_idx, torch).contiguous(), mix62_torch(new_idx)[:, None].contiguous()))

    def step(b, events=None):
        gk, _, sk, sv, fk = batches[b % N_BATCHES]
        marks = []
        for fn in (lambda: table.get(gk), lambda: table.set(sk, sv), lambda: table.remove(fk), None):
            if events is not None:
                marks.append(torch.cuda.Event(enable_timing=True)); marks[-1].record()
            if fn is not None:
                fn()
        if events is not None:
            events.append(marks)

    values, found = table.get(batches[0][0])
    expect = batches[0][1] < (1 << 40)
    ok = bool(torch.equal(found, expect)) and bool(torch.equal(values[expect], value_of_index(batches[0][1][expect], torch)))
    for s in range(warmup):
        step(s)
    torch.cuda.synchronize()
    events = []
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for s in range(steps):
        step(warmup + s, events)
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / steps
    phase = [sum(m[i].elapsed_time(m[i + 1]) for m in events) / steps for i in range(3)]

    # the same step the way a user of the reference calls it: with the Python bookkeeping of its set / remove
    # (pre-get, row-wise unique, host read of n_elements) around the kernels
    def api_step(b):
        gk, _, sk, sv, fk = batches[b % N_BATCHES]
        table.get(gk)
        table.api_set(sk, sv, rehash_threshold=0.95)
        table.api_remove(fk)

    table.n_elements = torch.tensor(n_keys, device=device)
    api_step(0)
    torch.cuda.synchronize()
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    api_steps = 3
    a0.record()
    for s in range(api_steps):
        api_step(1 + s)
    a1.record()
    torch.cuda.synchronize()
    api_ms = a0.elapsed_time(a1) / api_steps
    live = int(((table.all_uuids != -1) & (table.all_uuids != -3)).sum().item())
    return {"value": 2 * q / (ms * 1e-3) / 1e6, "unit": "Mops/s", "ms_per_step": ms,
            "get_ms": phase[0], "set_ms": phase[1], "remove_ms": phase[2], "steps": steps, "results_ok": ok,
            "live_keys_after": live, "live_keys_expected": n_keys,
            "api_path": {"value": 2 * q / (api_ms * 1e-3) / 1e6, "unit": "Mops/s", "ms_per_step": api_ms, "steps": api_steps,
                         "what": "the same kernels with the reference's Python bookkeeping restated around them "
                                 "(cuda_closed_hashmap.py:321-384, 423-454: pre-get + unique(dim=0) + n_elements.item() "
                                 "per set, unique(dim=0) per remove), i.e. what a caller of the reference API pays"},
            "what": "the reference's closed_hashmap_get/set/remove kernels (closed_hashmap_impl.cu), nvcc -O3 for sm_100a, "
                    "launched like closed_hashmap_impl.py does, incl. its output allocation and fallback fill; "
                    "no Python-side pre-get / unique / rehash logic"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    mops, ms, desc = cpu_arm(args.steps, args.warmup)
    gpu_leg = None if args.no_ref_gpu else reference_kernels_on_gpu(args)
    line = {
        "impl": "reference", "metric": "hashmap get/set Mops/s", "value": mops, "unit": "Mops/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int64", "data": "synthetic",
        "config": workload_config(args, world=args.gpus),
        "cpu_baseline": desc,
        "e2e": {"value": mops, "unit": "Mops/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        # extra: the same reference kernel text run on this box's GPU (kernel-only, 1 GPU); not the line's value
        "reference_kernels_gpu": gpu_leg,
    }
    print(json.dumps(line))


def workload_config(args, world):
    return {
        "workload": "BASELINE configs[4]: hash-sharded CudaClosedHashmap, int64 keys uniform in [0,2^62) -> float32[2], "
                    f"2^{args.keys_log2} keys per GPU at load {LOAD_FACTOR}, per GPU and step: get 2^{args.batch_log2} "
                    f"(80% hits) + set 2^{args.batch_log2} (80% overwrite, 20% insert) + remove of the inserted rows",
        "keys_per_gpu": 1 << args.keys_log2, "buckets_per_gpu": int((1 << args.keys_log2) / LOAD_FACTOR),
        "batch_per_gpu": 1 << args.batch_log2, "shards": world,
        "l2_policy": f"inputs larger than L2: {N_BATCHES} rotating batches of {(1 << args.batch_log2) * 8 >> 20} MiB keys, "
                     f"table {(int((1 << args.keys_log2) / LOAD_FACTOR) * 32) >> 20} MiB per GPU",
        "parallelism": ("single GPU" if world == 1 else
                        f"hash-sharded x{world}, " + ("NCCL all-to-all" if getattr(args, "no_peer", False) else
                                                      "rows stored into the owners' memory over NVLink (peer exchange)")),
    }


# ---------------------------------------------------------------------------------------------------------------
# candidate arm
# ---------------------------------------------------------------------------------------------------------------

def run_candidate(args):
    import torch
    import torch.distributed as dist
    from doksparse_b200 import _lib as L
    from doksparse_b200.sharded import ShardedClosedHashmap

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"        # keep NCCL's banner off stdout: one JSON line only
        # the small collectives of the exchange (count gather, fences) must not queue behind the big probing grids
        os.environ.setdefault("TORCH_NCCL_HIGH_PRIORITY", "1")
        dist.init_process_group("nccl", device_id=device)
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run"

    n_keys, q = 1 << args.keys_log2, 1 << args.batch_log2
    total_keys = n_keys * world
    nb = int(n_keys / LOAD_FACTOR)
    # rows of a batch go straight into the owners' memory over NVLink (sized for a batch plus skew and padding);
    # --no-peer keeps the NCCL all-to-all exchange
    peer_rows = 0 if (world == 1 or args.no_peer) else int(q * 1.25) + 16 * world
    table = ShardedClosedHashmap(nb, device=device, rehash_threshold=0.95, peer_capacity_rows=peer_rows, **fixed_parameters())

    # ---- build (untimed): rank r inserts key indices [r * n_keys, (r + 1) * n_keys), routed to their owners
    chunk = min(n_keys, 1 << 25)
    for lo in range(rank * n_keys, (rank + 1) * n_keys, chunk):
        idx = torch.arange(lo, lo + chunk, device=device, dtype=torch.long)
        table.set(mix62_torch(idx)[:, None], value_of_index(idx, torch), assume_unique=True)
    del idx
    assert table.n_elements == total_keys, "build lost keys"

    # ---- batches
    n_hit = int(q * HIT_FRACTION)
    g = torch.Generator(device=device).manual_seed(1234 + rank)
    batches = []
    for b in range(N_BATCHES):
        j = torch.arange(n_hit, device=device, dtype=torch.long)
        hit_idx = (j * 7919 + 104729 * (b + 1) + 15485863 * rank) % total_keys
        base = (b << 32) + (rank << 28)
        miss_idx = (1 << 40) + base + torch.arange(q - n_hit, device=device, dtype=torch.long)
        new_idx = (1 << 41) + base + torch.arange(q - n_hit, device=device, dtype=torch.long)
        perm = torch.randperm(q, device=device, generator=g)
        get_idx = torch.cat([hit_idx, miss_idx])[perm]
        set_idx = torch.cat([hit_idx, new_idx])[perm]
        batches.append({
            "get_keys": mix62_torch(get_idx)[:, None].contiguous(), "get_idx": get_idx,
            "set_keys": mix62_torch(set_idx)[:, None].contiguous(), "set_values": value_of_index(set_idx, torch).contiguous(),
            "fresh_keys": mix62_torch(new_idx)[:, None].contiguous(),
        })
    del j, hit_idx, miss_idx, new_idx, perm, set_idx

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    pipelined = world > 1 and not args.no_peer and not args.no_pipeline

    def step(b, events=None):
        d = batches[b % N_BATCHES]
        if pipelined and events is None:
            # one submission: the send stage of each operation overlaps the table work of the one before
            # (wait=False: the first send of the next step may overlap this step's last table work; the timed loop
            # and the check wait once, at their end)
            (values, found), _, _ = table.run([("get", d["get_keys"]), ("set", d["set_keys"], d["set_values"]),
                                               ("remove", d["fresh_keys"])], wait=False)
            return values, found
        if events is not None:
            events.append(torch.cuda.Event(enable_timing=True)); events[-1].record()
        values, found = table.get(d["get_keys"])
        if events is not None:
            events.append(torch.cuda.Event(enable_timing=True)); events[-1].record()
        table.set(d["set_keys"], d["set_values"])
        if events is not None:
            events.append(torch.cuda.Event(enable_timing=True)); events[-1].record()
        table.remove(d["fresh_keys"])
        if events is not None:
            events.append(torch.cuda.Event(enable_timing=True)); events[-1].record()
        return values, found

    # ---- correctness of what is being timed (first batch, before any timing)
    values, found = step(0)
    if pipelined:
        table.wait()
    d0 = batches[0]
    expect_found = d0["get_idx"] < (1 << 40)
    checks = {"found_flags_ok": bool(torch.equal(found, expect_found)),
              "hit_values_ok": bool(torch.equal(values[expect_found], value_of_index(d0["get_idx"][expect_found], torch))),
              "miss_values_zero": bool((values[~expect_found] == 0).all()),
              "n_elements_stationary": table.n_elements == total_keys}
    del values, found, expect_found

    sampler = ClockSampler(local_rank) if rank == 0 else None      # started early: its start-up must not fall into the timed region
    for s in range(1, args.warmup):
        step(s)
    if pipelined:
        table.wait()
    if sampler:
        time.sleep(0.5)
        sampler.rows.clear()

    # ---- timed region: exactly K steps, device-resident inputs
    launches0 = L.lib().dok_launch_count()
    events = []
    barrier()
    t_start, t_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    for s in range(args.steps):
        step(s + args.warmup, None if pipelined else events)
    if pipelined:
        table.wait()
    t_stop.record()
    barrier()
    launches = L.lib().dok_launch_count() - launches0
    clocks = sampler.stop() if sampler else None
    elapsed_ms = torch.tensor([t_start.elapsed_time(t_stop)], device=device)
    phase_steps = args.steps
    if pipelined:
        # the timed steps were single pipelined submissions; the per-operation times come from a short separate
        # pass that calls the operations one after the other (they add up to more than a pipelined step)
        phase_steps = 3
        step(0, [])                                   # warm the sequential path (allocator pools of the main stream)
        barrier()
        for s in range(phase_steps):
            step(s + 1, events)
        barrier()
    phase = torch.zeros(3, device=device)
    for s in range(phase_steps):
        e = events[4 * s: 4 * s + 4]
        phase += torch.tensor([e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2]), e[2].elapsed_time(e[3])], device=device)
    phase /= phase_steps
    if world > 1:
        dist.all_reduce(elapsed_ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(phase, op=dist.ReduceOp.MAX)
    elapsed_ms = float(elapsed_ms.item())
    get_ms, set_ms, remove_ms = (float(x) for x in phase.tolist())
    ms_per_step = elapsed_ms / args.steps
    ops_per_step = 2 * q * world                         # get rows + set rows over all GPUs
    value = ops_per_step / (ms_per_step * 1e-3) / 1e6

    # ---- end to end: host (pinned) buffers in, host buffers out, through the public API
    e2e = None
    if not args.no_e2e:
        host = [{k: v.cpu().pin_memory() for k, v in d.items() if k != "get_idx"} for d in batches[:2]]
        out_values = torch.empty(q, 2, dtype=torch.float32).pin_memory()
        out_found = torch.empty(q, dtype=torch.bool).pin_memory()
        h2d = sum(host[0][k].numel() * host[0][k].element_size() for k in ("get_keys", "set_keys", "set_values", "fresh_keys"))
        d2h = out_values.numel() * 4 + out_found.numel()

        # what the host link gives when every rank copies at once and nothing else runs: the bound of the e2e leg
        probe_src, probe_dst = host[0]["get_keys"], torch.empty_like(batches[0]["get_keys"])
        probe_dst.copy_(probe_src, non_blocking=True)
        barrier()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        for _ in range(4):
            probe_dst.copy_(probe_src, non_blocking=True)
        p1.record()
        torch.cuda.synchronize()
        probe_gbs = torch.tensor([4 * probe_src.numel() * 8 / (p0.elapsed_time(p1) * 1e-3) / 1e9], device=device)
        if world > 1:
            dist.all_reduce(probe_gbs, op=dist.ReduceOp.MIN)
        del probe_dst

        from doksparse_b200.host_batch import HostBatch
        # chunks of 4 Mi rows on three streams (copy in | kernels | copy out); routed batches use larger chunks
        pipe = HostBatch(table, device, chunk_rows=(1 << 22) if world == 1 else (1 << 23))

        def e2e_step(b):
            h = host[b % 2]
            pipe.run([("get", h["get_keys"], out_values, out_found), ("set", h["set_keys"], h["set_values"]),
                      ("remove_rows", h["fresh_keys"])])

        e2e_steps = max(3, min(args.steps, 10))
        e2e_step(0)
        pipe.join()
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        pipe.begin()
        for s in range(e2e_steps):
            e2e_step(s + 1)
        pipe.join()
        t1.record()
        barrier()
        e2e_checks = {"e2e_found_ok": bool(torch.equal(out_found.to(device), batches[e2e_steps % 2]["get_idx"] < (1 << 40)))}
        e_ms = torch.tensor([t0.elapsed_time(t1)], device=device)
        if world > 1:
            dist.all_reduce(e_ms, op=dist.ReduceOp.MAX)
        e2e = {"value": ops_per_step / (float(e_ms.item()) / e2e_steps * 1e-3) / 1e6, "unit": "Mops/s",
               "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world, "steps": e2e_steps,
               "how": "HostBatch: pinned host buffers in and out, chunked over copy-in / kernel / copy-out streams",
               "ms_per_step": float(e_ms.item()) / e2e_steps,
               "h2d_gbs_per_gpu": h2d / (float(e_ms.item()) / e2e_steps * 1e-3) / 1e9,
               "h2d_copy_only_gbs_per_gpu": float(probe_gbs.item()),   # all ranks copying at once, slowest rank
               **e2e_checks}

    # ---- what the hardware gives a probing kernel: independent random 16-byte reads over this GPU's slot array
    slots = table.ops.local._slots
    n_reads = 1 << 26
    lib = L.lib()
    lib.dok_diag_random_reads(L.ptr(slots), slots.numel(), n_reads, 1, None, L.stream_ptr(device))
    r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    r0.record()
    for rep in range(3):
        lib.dok_diag_random_reads(L.ptr(slots), slots.numel(), n_reads, 100 + rep, None, L.stream_ptr(device))
    r1.record()
    torch.cuda.synchronize()
    request_ceiling = 3 * n_reads / (r0.elapsed_time(r1) * 1e-3) / 1e9          # G requests/s, this GPU

    # ---- roofline of the dominant kernel and of the other two
    peak, peak_source = measured_peak_gbs()
    local_rows = {"get": q, "set": q, "remove": q - n_hit}       # rows each GPU processes per step (weak scaling)
    kernel_ms = {"get": get_ms, "set": set_ms, "remove": remove_ms}
    per_kernel = {}
    for op in ("get", "set", "remove"):
        achieved = algorithmic_bytes(op) * local_rows[op] / (kernel_ms[op] * 1e-3) / 1e9
        gops = local_rows[op] / (kernel_ms[op] * 1e-3) / 1e9
        per_kernel[op] = {"ms": kernel_ms[op], "mops_per_gpu": gops * 1e3, "bytes_per_op": algorithmic_bytes(op),
                          "achieved_gbs": achieved, "frac": achieved / peak,
                          "frac_of_random_request_ceiling": gops / request_ceiling}
        if TRAFFIC_BYTES_PER_OP.get(op) and world == 1:
            # what DRAM really moves (ncu: whole 128-byte lines per probed group), as a rate and against the peak
            dram = TRAFFIC_BYTES_PER_OP[op] * local_rows[op] / (kernel_ms[op] * 1e-3) / 1e9
            per_kernel[op].update({"dram_traffic_gbs": dram, "dram_traffic_frac": dram / peak})
    top = max(kernel_ms, key=kernel_ms.get)
    roofline = {"bound": "hbm", "kernel": {"get": "k_get", "set": "k_set_claim (+ k_set_resolve, idle without duplicates)",
                                           "remove": "k_find<remove>"}[top],
                "achieved": per_kernel[top]["achieved_gbs"], "peak": peak, "unit": "GB/s", "frac": per_kernel[top]["frac"],
                "traffic": TRAFFIC_BYTES_PER_OP.get(top, 0) * local_rows[top] if TRAFFIC_BYTES_PER_OP.get(top) else None,
                "peak_source": peak_source,
                "random_request_ceiling_greq_s": request_ceiling,
                "note": ("phase time includes routing and exchange when shards > 1" +
                         (", measured with the operations called one after the other (the timed steps pipeline them); "
                          if pipelined else "; ") if world > 1 else "") +
                        "DRAM serves a random access with a whole 128-byte line (~48 G lines/s = the HBM bandwidth), "
                        "so a probing kernel is bound by lines touched per operation, not by the bytes it needs: "
                        "see kernels.*.dram_traffic_frac for the share of the HBM peak each kernel really moves"}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        _, _, cpu_baseline = cpu_arm(steps=4, warmup=1, budget_s=25.0)

    if rank == 0:
        line = {
            "metric": "hashmap get/set Mops/s", "value": value, "unit": "Mops/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int64", "data": "synthetic", "config": workload_config(args, world),
            "roofline": roofline, "kernels": per_kernel, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_launches": int(launches), "clocks": clocks, "checks": checks,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_candidate(args)


if __name__ == "__main__":
    main()
